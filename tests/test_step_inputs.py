"""Host-side planning of a step's attention work and of step programs (no GPU needed)."""

from __future__ import annotations

import numpy as np
import torch

from tokenmill_b200.parts.attention_plan import PREFILL_CHUNK, choose_chunk, packed_units


def _keys_per_tile(q_lens, starts, G, tile):
    out = []
    for n, s in zip(q_lens, starts):
        rows = n * G
        for r0 in range(0, rows, tile):
            out.append(s + (min(r0 + tile, rows) - 1) // G + 1)
    return out


def test_chunk_choice_is_a_power_of_two_multiple_of_512_and_follows_the_step():
    G, nkv = 7, 2
    picks = {}
    for T in (1024, 2048, 4096, 8192):
        for tile in (64, 128):
            c = choose_chunk(np.array([T]), np.array([0]), G, nkv, tile=tile)
            assert c % PREFILL_CHUNK == 0 and (c // PREFILL_CHUNK) & (c // PREFILL_CHUNK - 1) == 0
            picks[T, tile] = c
    # a short prompt keeps short chunks (few tiles: they must spread), long prompts take long ones
    assert picks[1024, 128] == 512 and picks[2048, 128] == 1024 and picks[8192, 128] == 8192
    assert picks[1024, 64] == 512 and picks[8192, 64] >= 4096
    # a late portion of a long prompt: few tiles, every one with thousands of keys -> cut, but not finely
    assert choose_chunk(np.array([1024]), np.array([3072]), G, nkv, tile=128) == 2048
    # nothing but single tokens and a tiny prompt: the base size
    assert choose_chunk(np.array([1, 1, 5]), np.array([900, 30, 0]), G, nkv, tile=128) == PREFILL_CHUNK
    assert choose_chunk(np.zeros(0, dtype=np.int64), np.zeros(0, dtype=np.int64), G, nkv) == PREFILL_CHUNK


def test_units_cover_every_tile_s_keys_once_for_any_chunk():
    rng = np.random.default_rng(0)
    for _ in range(20):
        S = int(rng.integers(1, 5))
        q_lens = rng.integers(1, 400, S)
        starts = rng.integers(0, 3000, S)
        G = int(rng.choice([1, 3, 7]))
        tile = int(rng.choice([64, 128]))
        chunk = int(rng.choice([128, 512, 1024, 4096]))
        rec, n_tiles, n_slots = packed_units(q_lens, starts, G, tile=tile, chunk=chunk)
        keys = _keys_per_tile(q_lens.tolist(), starts.tolist(), G, tile)
        assert n_tiles == len(keys)
        covered = {}
        for seq, row0, packed, slot0, t, q_start, q_len, before in rec.tolist():
            c, n = packed & 0xffff, packed >> 16
            assert n == -(-keys[t] // chunk) and 0 <= c < n and q_len == q_lens[seq] and before == starts[seq]
            assert (slot0 == -1) == (n == 1)
            covered.setdefault(t, []).append(c)
        assert all(sorted(v) == list(range(len(v))) for v in covered.values()) and len(covered) == n_tiles
        assert n_slots == sum(len(v) for v in covered.values() if len(v) > 1)
        # heaviest first
        work = [min(chunk, keys[t] - (p & 0xffff) * chunk) for _, _, p, _, t, _, _, _ in rec.tolist()]
        assert work == sorted(work, reverse=True)


def test_program_builder_shares_parameters_and_buffers_by_name():
    from tokenmill_b200.kernels.program import OP_SWIGLU, Buffer, Param, ProgramBuilder
    b = ProgramBuilder(torch.device("cpu"), torch.bfloat16)
    t1, t2 = b.tokens(), b.tokens()
    assert t1 == t2 == Param(0) and len(b.providers) == 1
    p = b.param("n_want", lambda s: s.n_want)
    assert p == Param(1) and b.param("n_want", lambda s: -1) == p and len(b.providers) == 2
    x = b.buffer("act", 64)
    y = b.buffer("act", 128)            # the same buffer, grown to the larger row
    assert x.tag == y.tag == "act" and b.buffers["act"] == Buffer("act", 128)
    b.emit(OP_SWIGLU, [2, x, y, t1, 32], cond=p)
    assert b.ops == [(OP_SWIGLU, p, [2, x, y, t1, 32])]
    try:
        b.emit(OP_SWIGLU, list(range(25)))
        assert False, "a record of 25 values must be refused"
    except ValueError:
        pass


def test_short_prompts_are_cut_into_pieces_an_attention_unit_holds():
    from types import SimpleNamespace

    from tokenmill_b200.engine.batch import StepEntry
    from tokenmill_b200.engine.runner import ModelRunner

    def pieces(entries, nh, nkv):
        me = SimpleNamespace(fused=SimpleNamespace(nh=nh, nkv=nkv))
        return ModelRunner._pieces_for_fused(me, entries)

    h1, h2 = object(), object()
    # 7 heads per kv head: 2 tokens per piece; the wanted places move with their piece
    got = pieces([StepEntry(h1, [10, 11, 12, 13, 14], 100, [0, 3, 4]), StepEntry(h2, [7], 5, [0])], 14, 2)
    assert [(p.handle, p.tokens, p.start, p.want) for p in got] == [
        (h1, [10, 11], 100, [0]), (h1, [12, 13], 102, [1]), (h1, [14], 104, [0]), (h2, [7], 5, [0])]
    # nothing to cut: every entry already fits
    assert pieces([StepEntry(h1, [1, 2], 0, [1]), StepEntry(h2, [3], 9, [0])], 14, 2) is None
    # 3 heads per kv head: 5 tokens per piece
    got = pieces([StepEntry(h1, list(range(12)), 0, [11])], 6, 2)
    assert [(p.tokens, p.start, p.want) for p in got] == [(list(range(5)), 0, []), (list(range(5, 10)), 5, []),
                                                           ([10, 11], 10, [1])]
    # wanted places out of order, more heads per kv head than rows, or too many pieces: not cut
    assert pieces([StepEntry(h1, [1, 2, 3, 4], 0, [3, 0])], 14, 2) is None
    assert pieces([StepEntry(h1, [1, 2, 3], 0, [2])], 32, 1) is None
    assert pieces([StepEntry(h1, list(range(34)), 0, [33])], 14, 2) is None


def test_decode_units_cover_every_stage_once_and_fill_the_slots():
    """The decode kernel's plan: every request's stages (from its window's start to its last key) lie in exactly
    one unit, parts are numbered 0 .. parts - 1, no unit is longer than the kernel takes, no request has more
    parts than the cap; the list is sorted longest first and padded with empty rows when asked."""
    import numpy as np
    from tokenmill_b200.parts.attention_plan import DECODE_MAX_UNIT_STAGES, decode_parts_cap, decode_units
    rng = np.random.default_rng(0)
    for trial in range(50):
        S = int(rng.integers(1, 40))
        q_lens = rng.integers(1, 3, S)
        starts = rng.integers(0, int(rng.choice([100, 3000, 40000])), S)
        window = int(rng.choice([0, 0, 70, 1000]))
        cap = int(rng.choice([decode_parts_cap(int(starts.max()) + 2), 64]))
        slots = int(rng.choice([3, 444, 592]))
        rows = S * cap if trial % 2 else None
        rec, n, max_parts = decode_units(q_lens, starts, window, kv_heads=2, slots=slots, cap=cap, rows=rows)
        assert max_parts <= cap and rec.shape[0] == (rows if rows else n)
        assert not rec[n:].any()
        sizes = rec[:n, 2] - rec[:n, 1]
        assert (sizes >= 1).all() and (sizes <= DECODE_MAX_UNIT_STAGES).all() and (np.diff(sizes) <= 0).all()
        for s in range(S):
            mine = rec[:n][rec[:n, 0] == s]
            mine = mine[np.argsort(mine[:, 3] & 0xffff)]
            parts = int(mine[0, 3]) >> 16
            assert len(mine) == parts and (mine[:, 3] >> 16 == parts).all()
            assert (mine[:, 3] & 0xffff).tolist() == list(range(parts))
            lo = max(0, int(starts[s]) - window + 1) if window else 0
            assert mine[0, 1] == lo // 64 and mine[-1, 2] == (int(starts[s]) + int(q_lens[s]) - 1) // 64 + 1
            assert (mine[1:, 1] == mine[:-1, 2]).all()
    # the example of the docstring: two rounds, not three
    rec, n, _ = decode_units(np.ones(27, int), np.full(27, 4400), 0, kv_heads=4, slots=444, cap=16)
    assert n * 4 <= 2 * 444


def test_the_whole_step_kernels_key_split_weighs_unit_length_against_the_merge():
    """Keys per attention unit of the whole-step kernel: a multiple of 64 that keeps the blocks evenly loaded
    (several rounds of short units may beat one round of long ones); one short request is not cut into 64-key units (their merge costs more than a
    warp's second 16 keys would), and many requests get units long enough for one round."""
    from types import SimpleNamespace
    from tokenmill_b200.kernels.fused import SPLIT_KEYS, FusedDecoder
    for D, nkv, n_sm in [(64, 2, 148), (128, 4, 148), (80, 3, 132)]:
        me = SimpleNamespace(nkv=nkv, n_sm=n_sm, D=D, _split_cache={})
        for n_seqs in (1, 2, 3, 8, 16):
            for kv in (1, 63, 64, 65, 770, 2256, 4256, 8256, 16256, 32256, 131072):
                split = FusedDecoder.split_for(me, n_seqs, kv)
                assert split % SPLIT_KEYS == 0 and split >= SPLIT_KEYS
                # the work of the slowest block stays within twice an even spread of 16-key rounds over the warps
                units = n_seqs * nkv * -(-kv // split)
                per_block = -(-units // n_sm) * -(-split // 128)
                assert per_block <= 2 * max(1, -(-n_seqs * nkv * -(-kv // 64) // (2 * n_sm))) + 1, (n_seqs, kv, split)
    me = SimpleNamespace(nkv=2, n_sm=148, D=64, _split_cache={})
    assert FusedDecoder.split_for(me, 1, 770) == 128 and FusedDecoder.split_for(me, 1, 4256) in (128, 256)
    assert FusedDecoder.split_for(me, 8, 770) == 128 and FusedDecoder.split_for(me, 8, 4256) == 512


def test_small_steps_of_wide_heads_keep_the_fixed_key_split():
    """... outside captured graphs and at short contexts only: a graph serves every context with one kernel."""
    from tokenmill_b200.parts.attention_plan import decode_units_pay
    assert not decode_units_pay(1, 2, 128, 800, False) and not decode_units_pay(8, 2, 128, 1024, False)
    assert not decode_units_pay(4, 4, 128, 64, False)
    assert decode_units_pay(9, 2, 128, 800, False) and decode_units_pay(5, 4, 128, 800, False)
    assert decode_units_pay(1, 2, 128, 1025, False) and decode_units_pay(1, 2, 128, 800, True)
    assert decode_units_pay(1, 2, 64, 100, False) and decode_units_pay(1, 1, 16, 100, False)
