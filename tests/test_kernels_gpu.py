"""Each kernel alone against its plain float32 reference, at sizes other than the engine tests use:
odd widths, head sizes in steps of 16, many groupings, several page sizes, float32 and bfloat16."""

from __future__ import annotations

import math

import pytest
import torch

from plain_qwen2 import (plain_apply_rope, plain_causal_attention, plain_filtered_probs, plain_inverse_cdf,
                         plain_rmsnorm, plain_rope_tables, plain_silu)

from kernel_cases import paged_case as _paged_case

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, ref, f32=2e-5, bf16=1.5e-2):
    return (f32 if dtype == torch.float32 else bf16) * max(1e-6, float(ref.abs().max()))


def _ops():
    from tokenmill_b200.kernels import ops
    return ops


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H", [(1, 16), (7, 100), (33, 896), (5, 3000), (3, 12288)])
def test_add_rmsnorm(dtype, T, H):
    ops = _ops()
    g = torch.Generator().manual_seed(T * 1000 + H)
    resid = torch.randn(T, H, generator=g)
    branch = torch.randn(T, H, generator=g).to(dtype)
    w = 1 + 0.1 * torch.randn(H, generator=g)
    eps = 1e-5
    d_res = resid.to(DEV)
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(d_res, w.to(DEV), eps, out, branch=branch.to(DEV))
    x = resid + branch.float()
    assert torch.equal(d_res.cpu(), x)                           # the 32-bit sum is stored back
    ref = plain_rmsnorm(x, w, eps)
    assert (out.float().cpu() - ref).abs().max() <= tol(dtype, ref)
    # norm only, selected rows, the stream untouched
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
    out2 = torch.empty(2, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(d_res, w.to(DEV), eps, out2, rows=rows)
    assert torch.equal(d_res.cpu(), x)
    assert (out2.float().cpu() - ref[[T - 1, 0]]).abs().max() <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_gather_and_partials(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    V, H, T = 301, 72, 9
    table = torch.randn(V, H, generator=g).to(dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    w = torch.rand(H, generator=g) + 0.5
    resid = torch.full((T, H), 7.0, device=DEV)                  # stale content must be overwritten
    out = torch.empty(T, H, dtype=dtype, device=DEV)
    ops.add_rmsnorm(resid, w.to(DEV), 1e-6, out, ids=ids.to(DEV), table=table.to(DEV))
    x = table.float()[ids.long()]
    assert torch.equal(resid.cpu(), x)
    ref = plain_rmsnorm(x, w, 1e-6)
    assert (out.float().cpu() - ref).abs().max() <= tol(dtype, ref)
    parts = torch.randn(3, T, H, generator=g)
    ops.add_rmsnorm(resid, w.to(DEV), 1e-6, out, partials=parts.to(DEV))
    x2 = x + ((parts[0] + parts[1]) + parts[2])
    assert (resid.cpu() - x2).abs().max() <= 1e-6
    assert (out.float().cpu() - plain_rmsnorm(x2, w, 1e-6)).abs().max() <= tol(dtype, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,D,page", [(4, 2, 16, 16), (3, 1, 32, 8), (14, 2, 64, 16), (5, 5, 48, 4), (8, 1, 128, 32)])
def test_qkv_rope_write(dtype, nh, nkv, D, page):
    ops = _ops()
    g = torch.Generator().manual_seed(nh * 100 + D)
    T, P, pages = 11, 300, 6
    width = (nh + 2 * nkv) * D
    qkv = torch.randn(T, width, generator=g).to(dtype)
    bias = 0.3 * torch.randn(width, generator=g)
    pos = torch.tensor([0, 1, 2, 3, 299, 17, 18, 19, 100, 101, 255], dtype=torch.int32)
    cos, sin = plain_rope_tables(P, D, 10000.0)
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, page, nkv, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, nh, D, dtype=dtype, device=DEV)
    ops.qkv_rope_write(qkv.to(DEV), bias.to(DEV), pos.to(DEV), cos[:, :D // 2].contiguous().to(DEV),
                       sin[:, :D // 2].contiguous().to(DEV), slots.to(DEV), q_out, kc, vc, nh, nkv, D)
    x = qkv.float() + bias
    q = plain_apply_rope(x[:, :nh * D].view(T, nh, D), cos, sin, pos)
    k = plain_apply_rope(x[:, nh * D:(nh + nkv) * D].view(T, nkv, D), cos, sin, pos)
    v = x[:, (nh + nkv) * D:].view(T, nkv, D)
    f32 = 0 if dtype == torch.float32 else None
    def close(a, b):
        d = (a.float().cpu() - b).abs().max()
        return d == 0 if f32 == 0 else d <= tol(dtype, b)
    assert close(q_out, q)                                        # float32: bit-equal, products not fused
    flat_k, flat_v = kc.view(-1, nkv, D), vc.view(-1, nkv, D)
    assert close(flat_k[slots.long().to(DEV)], k) and close(flat_v[slots.long().to(DEV)], v)
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[slots.long()] = False
    assert float(flat_k[untouched.to(DEV)].abs().max()) == 0      # nothing written elsewhere


ATTN_SHAPES = [(4, 2, 16, 16), (3, 1, 32, 8), (14, 2, 64, 16), (6, 3, 48, 5), (12, 2, 128, 32), (40, 1, 16, 16),
               (2, 2, 256, 16), (5, 1, 80, 1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,D,page", ATTN_SHAPES)
def test_paged_attention_mixed_batch(dtype, nh, nkv, D, page):
    """Prompt portions beside decoded tokens: whole prompts, later portions, single tokens."""
    ops = _ops()
    c = _paged_case(nh, nkv, D, page, q_lens=[37, 1, 5, 1, 64, 2], befores=[0, 130, 59, 0, 31, 300], dtype=dtype,
                    seed=nh + D)
    out = torch.empty_like(c["q"])
    ops.paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], c["tile_seq"], c["tile_row0"],
                        c["n_tiles"], out, scale=D ** -0.5)
    diff = (out.float().cpu() - c["ref"]).abs().max()
    assert diff <= tol(dtype, c["ref"], f32=1e-5, bf16=1e-2), diff


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,D,page", [(14, 2, 64, 16), (3, 1, 32, 8), (8, 8, 16, 4), (6, 1, 128, 16)])
def test_paged_attention_split_keys_decode(dtype, nh, nkv, D, page):
    """Decoded tokens over long contexts, keys cut at multiples of 256 and merged by the second kernel;
    lengths sit on and around the cuts."""
    ops = _ops()
    befores = [0, 255, 256, 257, 511, 1000, 31]
    c = _paged_case(nh, nkv, D, page, q_lens=[1] * len(befores), befores=befores, dtype=dtype, seed=D)
    T = len(befores)
    max_splits = -(-1001 // 256)
    part_acc = torch.full((T * nh * max_splits * D,), float("nan"), device=DEV)
    part_ml = torch.full((T * nh * max_splits * 2,), float("nan"), device=DEV)
    out = torch.empty_like(c["q"])
    ops.paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], c["tile_seq"], c["tile_row0"],
                        c["n_tiles"], out, scale=D ** -0.5, split_keys=256, max_splits=max_splits,
                        part_acc=part_acc, part_ml=part_ml, seq_of_token=c["seq_of"])
    diff = (out.float().cpu() - c["ref"]).abs().max()
    assert diff <= tol(dtype, c["ref"], f32=1e-5, bf16=1e-2), diff


@pytest.mark.parametrize("nh,nkv,D,page,q_lens,window", [
    (14, 2, 64, 16, [1] * 7, 0), (12, 2, 128, 16, [1] * 7, 0), (16, 1, 64, 8, [1] * 7, 0), (4, 4, 128, 1, [1] * 7, 0),
    (14, 2, 64, 16, [2, 1, 2, 1, 1, 2, 1], 0), (8, 4, 64, 5, [8, 1, 3, 1, 1, 2, 5], 0), (14, 2, 64, 16, [1] * 7, 100),
    (6, 2, 128, 32, [4, 1, 1, 5, 1, 2, 1], 300),
])
def test_decode_attention_tensor_core_kernel(nh, nkv, D, page, q_lens, window):
    """The bfloat16 decode kernel: few query rows per request, long contexts on and around the key cuts,
    one far key that dominates, windows, odd page sizes."""
    ops = _ops()
    befores = [0, 255, 256, 257, 511, 1000, 63]
    c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=D + nh, window=window)
    T = sum(q_lens)
    max_splits = -(-(1000 + max(q_lens)) // 256)
    part_acc = torch.full((T * nh * max_splits * D,), float("nan"), device=DEV)
    part_ml = torch.full((T * nh * max_splits * 2,), float("nan"), device=DEV)
    out = torch.empty_like(c["q"])
    ops.decode_attention_bf16(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], len(q_lens), out,
                              scale=D ** -0.5, window=window, split_keys=256, max_splits=max_splits,
                              part_acc=part_acc, part_ml=part_ml)
    diff = (out.float().cpu() - c["ref"]).abs().max()
    assert diff <= tol(torch.bfloat16, c["ref"], bf16=1e-2), diff


@pytest.mark.parametrize("nh,nkv,D,page,q_lens,window,cap,slots", [
    (14, 2, 64, 16, [1] * 8, 0, 16, 592), (12, 2, 128, 16, [1] * 8, 0, 16, 444), (16, 1, 64, 8, [1] * 8, 0, 16, 5),
    (4, 4, 128, 64, [1] * 8, 0, 3, 7), (14, 2, 64, 32, [2, 1, 2, 1, 1, 2, 1, 2], 0, 16, 592),
    (8, 4, 64, 8, [4, 1, 3, 1, 1, 2, 4, 1], 0, 4, 3), (14, 2, 64, 16, [1] * 8, 100, 16, 592),
    (6, 2, 128, 32, [4, 1, 1, 5, 1, 2, 1, 1], 300, 16, 11), (28, 4, 128, 16, [1] * 8, 0, 16, 444),
])
def test_decode_attention_by_units_kernel(nh, nkv, D, page, q_lens, window, cap, slots):
    """The persistent decode kernel with its host-made list of units: contexts on and around the stage and page
    edges and one of thousands of keys, one far key that dominates, windows, several query tokens a request; few
    slots and a low cap so that blocks take several units each and units are long; the list padded as a captured
    graph pads it. Twice: the second launch finds the counters at zero."""
    import numpy as np
    from tokenmill_b200.parts.attention_plan import decode_units
    ops = _ops()
    befores = [0, 63, 64, 255, 256, 1000, 5000, 127]
    c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=D + nh, window=window)
    T, S = sum(q_lens), len(q_lens)
    for rows in (None, S * 32):
        rec, n_units, max_parts = decode_units(np.array(q_lens), np.array(befores), window, kv_heads=nkv, slots=slots,
                                               cap=cap, head_dim=D, rows=rows)
        assert max_parts <= cap and int((rec[:, 2] - rec[:, 1]).max()) <= 32
        units = torch.from_numpy(rec).to(DEV)
        n_work = torch.tensor([n_units * nkv], dtype=torch.int32, device=DEV)
        part_acc = torch.full((T * nh * max_parts * D,), float("nan"), device=DEV)
        part_ml = torch.full((T * nh * max_parts * 2,), float("nan"), device=DEV)
        done = torch.zeros(S * nkv, dtype=torch.int32, device=DEV)
        for _ in range(2):
            out = torch.full_like(c["q"], float("nan"))
            ops.decode_attention_units_bf16(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], units, n_work, out,
                                            scale=D ** -0.5, window=window, max_parts=max_parts,
                                            grid=min(slots, rec.shape[0] * nkv), part_acc=part_acc, part_ml=part_ml,
                                            done=done)
            ops.tc_check(torch.device(DEV))
            diff = (out.float().cpu() - c["ref"]).abs().max()
            assert diff <= tol(torch.bfloat16, c["ref"], bf16=1e-2), diff
            assert int(done.abs().sum()) == 0


@pytest.mark.parametrize("nh,nkv,D,page,q_lens,window,bias", [
    (14, 2, 64, 16, [1] * 8, 0, True), (12, 2, 128, 16, [1] * 8, 0, True), (28, 4, 128, 8, [1] * 8, 0, False),
    (8, 4, 64, 32, [2, 1, 3, 1, 1, 2, 4, 1], 0, True), (6, 2, 128, 64, [1, 1, 2, 5, 1, 2, 1, 1], 300, True),
    (16, 1, 64, 16, [1] * 8, 90, False),
])
def test_decode_attention_by_units_finishing_the_projection_itself(nh, nkv, D, page, q_lens, window, bias):
    """The unit-driven decode kernel fed with the RAW q/k/v product (bias not added, nothing rotated, nothing in
    the cache yet) against the two kernels it replaces (rotation + cache write, then attention): the same
    arithmetic in the same order, so the outputs and the cache are EQUAL, bit for bit. New tokens on a stage's
    first and last row, several new tokens a request, a window, few slots so that blocks take several units."""
    import numpy as np
    from tokenmill_b200.parts.attention_plan import decode_units
    ops = _ops()
    befores = [0, 63, 64, 255, 256, 1000, 2047, 127]
    c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=D + nh, window=window)
    T, S = sum(q_lens), len(q_lens)
    g = torch.Generator().manual_seed(nh * D + page)
    qkv = torch.randn(T, (nh + 2 * nkv) * D, generator=g).bfloat16().to(DEV)
    b = torch.randn((nh + 2 * nkv) * D, generator=g).to(DEV) if bias else None
    n_pos = 2100
    ang = torch.arange(n_pos)[:, None] * (10000.0 ** (-torch.arange(D // 2) / (D // 2)))[None, :]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    positions, slots = [], []
    table = c["table"].cpu()
    for s_i, (n, before) in enumerate(zip(q_lens, befores)):
        for j in range(n):
            positions.append(before + j)
            slots.append(int(table[s_i, (before + j) // page]) * page + (before + j) % page)
    positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slot_map = torch.tensor(slots, dtype=torch.int32, device=DEV)
    rec, n_units, max_parts = decode_units(np.array(q_lens), np.array(befores), window, kv_heads=nkv, slots=9, cap=16,
                                           head_dim=D)
    units = torch.from_numpy(rec).to(DEV)
    n_work = torch.tensor([n_units * nkv], dtype=torch.int32, device=DEV)
    scratch = dict(part_acc=torch.empty(T * nh * max_parts * D, device=DEV), part_ml=torch.empty(T * nh * max_parts * 2, device=DEV),
                   done=torch.zeros(S * nkv, dtype=torch.int32, device=DEV))
    common = dict(scale=D ** -0.5, window=window, max_parts=max_parts, grid=min(9, n_units * nkv))
    # the two kernels
    kc_a, vc_a = c["kc"].clone(), c["vc"].clone()
    q = torch.empty(T, nh, D, dtype=torch.bfloat16, device=DEV)
    ops.qkv_rope_write(qkv, b, positions, cos, sin, slot_map, q, kc_a, vc_a, nh, nkv, D)
    out_a = torch.full_like(q, float("nan"))
    ops.decode_attention_units_bf16(q, kc_a, vc_a, c["table"], c["cu"], c["before"], units, n_work, out_a, **common, **scratch)
    # the one kernel
    kc_b, vc_b = c["kc"].clone(), c["vc"].clone()
    out_b = torch.full_like(q, float("nan"))
    ops.decode_attention_units_rope_bf16(qkv, b, positions, cos, sin, slot_map, kc_b, vc_b, c["table"], c["cu"], c["before"],
                                         units, n_work, out_b, **common, **scratch)
    ops.tc_check(torch.device(DEV))
    assert torch.isfinite(out_a.float()).all()
    assert torch.equal(kc_a, kc_b) and torch.equal(vc_a, vc_b)
    assert torch.equal(out_a, out_b)


def test_decode_attention_finishing_the_projection_reports_a_position_outside_the_tables():
    """A position beyond the rotation tables is never used to index them: the row is clamped and the error word
    raised, which the next check turns into an exception."""
    import numpy as np
    from tokenmill_b200.kernels import lib
    from tokenmill_b200.parts.attention_plan import decode_units
    ops = _ops()
    nh, nkv, D, page = 4, 2, 64, 16
    c = _paged_case(nh, nkv, D, page, q_lens=[1, 1], befores=[10, 130], dtype=torch.bfloat16, seed=3)
    qkv = torch.randn(2, (nh + 2 * nkv) * D).bfloat16().to(DEV)
    n_pos = 100                                                           # the second token stands at 130
    ang = torch.arange(n_pos)[:, None] * torch.ones(D // 2)[None, :]
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    table = c["table"].cpu()
    positions = torch.tensor([10, 130], dtype=torch.int32, device=DEV)
    slot_map = torch.tensor([int(table[0, 0]) * page + 10, int(table[1, 130 // page]) * page + 130 % page],
                            dtype=torch.int32, device=DEV)
    rec, n_units, max_parts = decode_units(np.array([1, 1]), np.array([10, 130]), 0, kv_heads=nkv, slots=8, cap=16, head_dim=D)
    out = torch.empty(2, nh, D, dtype=torch.bfloat16, device=DEV)
    ops.tc_check(torch.device(DEV))
    ops.decode_attention_units_rope_bf16(
        qkv, None, positions, cos, sin, slot_map, c["kc"], c["vc"], c["table"], c["cu"], c["before"],
        torch.from_numpy(rec).to(DEV), torch.tensor([n_units * nkv], dtype=torch.int32, device=DEV), out,
        scale=D ** -0.5, window=0, max_parts=max_parts, grid=4, part_acc=torch.empty(2 * nh * max_parts * D, device=DEV),
        part_ml=torch.empty(2 * nh * max_parts * 2, device=DEV), done=torch.zeros(2 * nkv, dtype=torch.int32, device=DEV))
    with pytest.raises(lib.KernelError, match="position"):
        ops.tc_check(torch.device(DEV))
    ops.tc_check(torch.device(DEV))                                        # (the word is cleared by the check)
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("nh,nkv,D,page,window", [
    (14, 2, 64, 16, 0), (12, 2, 128, 16, 0), (3, 3, 64, 1, 0), (4, 1, 128, 7, 0), (14, 2, 64, 16, 70), (4, 2, 64, 8, 1),
    (6, 2, 128, 32, 200),
])
def test_prefill_attention_tensor_core_kernel(nh, nkv, D, page, window):
    """The bfloat16 prompt kernel: whole prompts, later portions that start off a tile or page edge, short
    portions and single tokens in the same launch; tiles that end inside a key block; windows."""
    from tokenmill_b200.parts.attention_plan import packed_units
    from tokenmill_b200.parts.base import PrefillUnits
    import numpy as np
    ops = _ops()
    q_lens, befores = [200, 1, 64, 3, 129, 65, 17], [0, 300, 64, 5, 77, 191, 1000]
    c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=D + nh + window,
                    window=window)
    G = nh // nkv
    counters = torch.zeros(2, dtype=torch.int32, device=DEV)
    for chunk in (512, 64, 128):       # the engine's chunk; then chunks so short that most tiles have several
        rec, n_tiles, n_slots = packed_units(np.array(q_lens, dtype=np.int32), np.array(befores, dtype=np.int32), G,
                                             chunk=chunk)
        assert n_tiles == sum(-(-n * G // 64) for n in q_lens)
        assert len({(r[4], r[2] & 0xffff) for r in rec.tolist()}) == len(rec)          # every (tile, chunk) once
        units = PrefillUnits(torch.from_numpy(rec).to(DEV), len(rec), n_tiles, n_slots, chunk)
        part_acc = torch.full((max(1, n_slots) * nkv * 64 * D,), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((max(1, n_slots) * nkv * 64 * 2,), float("nan"), dtype=torch.float32, device=DEV)
        tile_done = torch.zeros(n_tiles * nkv, dtype=torch.int32, device=DEV)
        for _ in range(2):                                          # the second launch finds the counters at zero
            out = torch.full_like(c["q"], float("nan"))
            ops.prefill_attention_bf16(c["q"], c["kc"], c["vc"], c["table"], units, counters, out, scale=D ** -0.5,
                                       window=window, part_acc=part_acc, part_ml=part_ml, tile_done=tile_done)
            diff = (out.float().cpu() - c["ref"]).abs().max()
            assert diff <= tol(torch.bfloat16, c["ref"], bf16=1e-2), (chunk, diff)
            assert counters.tolist() == [0, 0] and int(tile_done.abs().sum()) == 0


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("nh,nkv,page,window", [(14, 2, 16, 0), (3, 3, 1, 0), (8, 1, 7, 0), (14, 2, 16, 70), (4, 2, 8, 1)])
def test_prefill_attention_tcgen05_kernel(nh, nkv, page, window, D):
    """The tcgen05 prompt kernel (heads of 64 on blocks of 128 keys, heads of 128 on blocks of 64; 128-row
    tiles, scores and outputs in tensor memory): whole
    prompts, later portions that start off a tile or page edge, short portions and single tokens in the same
    launch; tiles that end inside a key block; key chunks so short that most tiles have several; windows."""
    from tokenmill_b200.parts.attention_plan import packed_units
    from tokenmill_b200.parts.base import PrefillUnits
    import numpy as np
    ops = _ops()
    q_lens, befores = [200, 1, 64, 3, 129, 65, 17, 300], [0, 300, 64, 5, 77, 191, 1000, 131]
    c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=nh + window,
                    window=window)
    G = nh // nkv
    counters = torch.zeros(2, dtype=torch.int32, device=DEV)
    for chunk in (512, 128, 256):
        rec, n_tiles, n_slots = packed_units(np.array(q_lens, dtype=np.int32), np.array(befores, dtype=np.int32), G,
                                             tile=128, chunk=chunk)
        assert n_tiles == sum(-(-n * G // 128) for n in q_lens)
        units = PrefillUnits(torch.from_numpy(rec).to(DEV), len(rec), n_tiles, n_slots, chunk, 128)
        part_acc = torch.full((max(1, n_slots) * nkv * 128 * D,), float("nan"), dtype=torch.float32, device=DEV)
        part_ml = torch.full((max(1, n_slots) * nkv * 128 * 2,), float("nan"), dtype=torch.float32, device=DEV)
        tile_done = torch.zeros(n_tiles * nkv, dtype=torch.int32, device=DEV)
        for _ in range(2):                                          # the second launch finds the counters at zero
            out = torch.full_like(c["q"], float("nan"))
            ops.prefill_attention_tc_bf16(c["q"], c["kc"], c["vc"], c["table"], units, counters, out, scale=D ** -0.5,
                                          window=window, part_acc=part_acc, part_ml=part_ml, tile_done=tile_done)
            ops.tc_check(torch.device(DEV))
            diff = (out.float().cpu() - c["ref"]).abs().max()
            assert diff <= tol(torch.bfloat16, c["ref"], bf16=1e-2), (chunk, diff)
            assert counters.tolist() == [0, 0] and int(tile_done.abs().sum()) == 0


def test_prefill_attention_tcgen05_kernel_merges_more_chunks_than_fit_shared_memory():
    """A row tile whose keys make so many chunks (57 of 128 keys) that not even 8 rows of all of them fit in
    shared memory is merged piece by piece from the L2 instead; a tile with 29 chunks takes several passes."""
    from tokenmill_b200.parts.attention_plan import packed_units
    from tokenmill_b200.parts.base import PrefillUnits
    import numpy as np
    ops = _ops()
    nh, nkv, D, page = 2, 1, 64, 32
    q_lens, befores = [3, 70], [7290, 3600]
    c = _paged_case(nh, nkv, D, page, q_lens=q_lens, befores=befores, dtype=torch.bfloat16, seed=11)
    counters = torch.zeros(2, dtype=torch.int32, device=DEV)
    rec, n_tiles, n_slots = packed_units(np.array(q_lens, dtype=np.int32), np.array(befores, dtype=np.int32), nh // nkv,
                                         tile=128, chunk=128)
    assert (rec[:, 2] >> 16).max() >= 57
    units = PrefillUnits(torch.from_numpy(rec).to(DEV), len(rec), n_tiles, n_slots, 128, 128)
    part_acc = torch.full((n_slots * nkv * 128 * D,), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((n_slots * nkv * 128 * 2,), float("nan"), dtype=torch.float32, device=DEV)
    tile_done = torch.zeros(n_tiles * nkv, dtype=torch.int32, device=DEV)
    out = torch.full_like(c["q"], float("nan"))
    ops.prefill_attention_tc_bf16(c["q"], c["kc"], c["vc"], c["table"], units, counters, out, scale=D ** -0.5,
                                  part_acc=part_acc, part_ml=part_ml, tile_done=tile_done)
    ops.tc_check(torch.device(DEV))
    diff = (out.float().cpu() - c["ref"]).abs().max()
    assert diff <= tol(torch.bfloat16, c["ref"], bf16=1e-2), diff


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 32, 33, 100])
def test_paged_attention_window_edge(dtype, window):
    """A key exactly at the window's edge counts, the one before it does not."""
    ops = _ops()
    nh, nkv, D, page = 4, 2, 32, 8
    c = _paged_case(nh, nkv, D, page, q_lens=[50, 1, 3], befores=[20, 140, 64], dtype=dtype, seed=window, window=window)
    out = torch.empty_like(c["q"])
    ops.paged_attention(c["q"], c["kc"], c["vc"], c["table"], c["cu"], c["before"], c["tile_seq"], c["tile_row0"],
                        c["n_tiles"], out, scale=D ** -0.5, window=window)
    diff = (out.float().cpu() - c["ref"]).abs().max()
    assert diff <= tol(dtype, c["ref"], f32=1e-5, bf16=1e-2), diff


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(1, 16), (9, 160), (4, 4864), (130, 77)])
def test_swiglu(dtype, T, I):
    ops = _ops()
    gu = (3 * torch.randn(T, 2 * I, generator=torch.Generator().manual_seed(I))).to(dtype)
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    ops.swiglu(gu.to(DEV), out)
    ref = plain_silu(gu.float()[:, :I]) * gu.float()[:, I:]
    assert (out.float().cpu() - ref).abs().max() <= tol(dtype, ref, f32=1e-6, bf16=8e-3)


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 70, 33), (64, 64, 16), (130, 257, 896), (3, 1000, 4864)])
def test_gemm_f32(M, N, K):
    ops = _ops()
    g = torch.Generator().manual_seed(M + N + K)
    a, w, b = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g), torch.randn(N, generator=g)
    ref = (a.double() @ w.double().T + b.double()).float()
    out = torch.empty(M, N, device=DEV)
    ops.linear(a.to(DEV), w.to(DEV), bias=b.to(DEV), out=out)
    assert (out.cpu() - ref).abs().max() <= 3e-6 * math.sqrt(K) * max(1.0, float(ref.abs().max()))
    # a row's result does not depend on the rows beside it
    one = ops.linear(a[:1].contiguous().to(DEV), w.to(DEV))
    many = ops.linear(a.to(DEV), w.to(DEV))
    assert torch.equal(one[0], many[0])


def test_linear_bf16_library_product_keeps_fp32_accumulation():
    ops = _ops()
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(9, 896, generator=g).bfloat16(), torch.randn(301, 896, generator=g).bfloat16()
    ref = x.float() @ w.float().T
    out32 = ops.linear(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert out32.dtype == torch.float32 and (out32.cpu() - ref).abs().max() <= 2e-4 * ref.abs().max()
    out16 = ops.linear(x.to(DEV), w.to(DEV))
    assert out16.dtype == torch.bfloat16 and (out16.float().cpu() - ref).abs().max() <= 6e-3 * ref.abs().max()


@pytest.mark.parametrize("T,N,K,rows,splits", [
    (1, 896, 896, 8, 1), (8, 904, 896, 8, 1), (17, 1000, 4864, 8, 2), (64, 896, 4864, 8, 4), (5, 3000, 200, 64, 1),
    (33, 151936, 896, 64, 1), (64, 72, 40, 16, 1), (3, 100, 1536, 32, 3),
])
def test_skinny_linear(T, N, K, rows, splits):
    """The decode-step product: plain store in either dtype, bias, K-range partial products."""
    ops = _ops()
    g = torch.Generator().manual_seed(T + N + K)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    b = torch.randn(N, generator=g)
    ref = x.float() @ w.float().T
    dx, dw = x.to(DEV), w.to(DEV)
    assert ops.skinny_ok(dx, dw, allow_split=True) == (T <= ops.SKINNY_MAX_TOKENS)    # the engine's own policy
    if splits > 1:
        parts = ops.skinny_linear(dx, dw, k_splits=splits, rows_per_block=rows)
        assert parts.shape == (splits, T, N) and parts.dtype == torch.float32
        assert (parts.sum(0).cpu() - ref).abs().max() <= 2e-5 * K ** 0.5 * max(1.0, float(ref.abs().max()))
    else:
        out32 = ops.skinny_linear(dx, dw, bias=b.to(DEV), out_dtype=torch.float32, rows_per_block=rows)
        assert (out32.cpu() - (ref + b)).abs().max() <= 2e-5 * K ** 0.5 * max(1.0, float(ref.abs().max()))
        out16 = ops.skinny_linear(dx, dw, rows_per_block=rows)
        assert out16.dtype == torch.bfloat16 and (out16.float().cpu() - ref).abs().max() <= 1e-2 * float(ref.abs().max())


@pytest.mark.parametrize("T,H,nh,nkv,D", [(1, 896, 14, 2, 64), (8, 896, 14, 2, 64), (40, 1536, 12, 2, 128), (7, 72, 3, 1, 32),
                                          (64, 264, 5, 5, 48), (2, 64, 4, 2, 16)])
def test_skinny_qkv_with_rope_and_cache_write(T, H, nh, nkv, D):
    ops = _ops()
    g = torch.Generator().manual_seed(T + H + D)
    width = (nh + 2 * nkv) * D
    x = torch.randn(T, H, generator=g).bfloat16()
    w = (torch.randn(width, H, generator=g) / H ** 0.5).bfloat16()
    bias = 0.3 * torch.randn(width, generator=g)
    pos = torch.randint(0, 500, (T,), generator=g, dtype=torch.int32)
    cos, sin = plain_rope_tables(500, D, 1e6)
    page, pages = 8, 20
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, page, nkv, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, nh, D, dtype=torch.bfloat16, device=DEV)
    dx, dw = x.to(DEV), w.to(DEV)
    ops.skinny_qkv_rope_write(dx, dw, bias.to(DEV), pos.to(DEV), cos[:, :D // 2].contiguous().to(DEV),
                              sin[:, :D // 2].contiguous().to(DEV), slots.to(DEV), q_out, kc, vc, nh, nkv, D)
    y = x.float() @ w.float().T + bias
    q = plain_apply_rope(y[:, :nh * D].view(T, nh, D), cos, sin, pos)
    k = plain_apply_rope(y[:, nh * D:(nh + nkv) * D].view(T, nkv, D), cos, sin, pos)
    v = y[:, (nh + nkv) * D:].view(T, nkv, D)
    t = 1e-2 * float(y.abs().max())
    assert (q_out.float().cpu() - q).abs().max() <= t
    assert (kc.view(-1, nkv, D)[slots.long().to(DEV)].float().cpu() - k).abs().max() <= t
    assert (vc.view(-1, nkv, D)[slots.long().to(DEV)].float().cpu() - v).abs().max() <= t
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[slots.long()] = False
    assert float(kc.view(-1, nkv, D)[untouched.to(DEV)].abs().max()) == 0


@pytest.mark.parametrize("T,H,I", [(1, 896, 4864), (8, 896, 4864), (64, 1536, 8960), (9, 96, 160), (20, 64, 100)])
def test_skinny_gate_up_swiglu(T, H, I):
    ops = _ops()
    g = torch.Generator().manual_seed(T + H + I)
    x = torch.randn(T, H, generator=g).bfloat16()
    w = (2 * torch.randn(2 * I, H, generator=g) / H ** 0.5).bfloat16()
    out = torch.empty(T, I, dtype=torch.bfloat16, device=DEV)
    ops.skinny_gate_up_swiglu(x.to(DEV), w.to(DEV), out)
    y = x.float() @ w.float().T
    ref = plain_silu(y[:, :I]) * y[:, I:]
    assert (out.float().cpu() - ref).abs().max() <= 1e-2 * float(ref.abs().max())


@pytest.mark.parametrize("T,N,K", [(128, 256, 64), (2048, 896, 896), (300, 904, 4864), (129, 1152, 200), (1000, 72, 1536)])
def test_tcgen05_linear(T, N, K):
    ops = _ops()
    g = torch.Generator().manual_seed(T + N + K)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    ref = x.float() @ w.float().T
    dx, dw = x.to(DEV), w.to(DEV)
    out = ops.tc_linear(dx, dw)
    ops.tc_check(dx.device)
    assert (out.float().cpu() - ref).abs().max() <= 1e-2 * float(ref.abs().max())


@pytest.mark.parametrize("T,N,K", [(64, 896, 4864), (17, 896, 896), (100, 1536, 8960), (128, 3584, 18944), (33, 100, 72),
                                   (64, 132, 200), (48, 896, 64), (1, 1536, 8960), (8, 3584, 18944)])
def test_tcgen05_linear_added_into_a_float32_stream(T, N, K):
    """The product of a step of a few dozen tokens, its K range cut over the chip and every piece added into the
    32-bit stream: the stream's own values stay, rows beyond T stay untouched, twice in a row adds twice."""
    ops = _ops()
    g = torch.Generator().manual_seed(T + N + K)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) / K ** 0.5).bfloat16()
    base = torch.randn(T + 3, N, generator=g)
    ref = base[:T] + x.float() @ w.float().T
    stream = base.to(DEV)
    assert ops.tc_add_ok(x.to(DEV), w.to(DEV), stream[:T]) == (K >= ops.TC_ADD_MIN_K)    # (the kernel takes short rows too)
    ops.tc_linear_add(x.to(DEV), w.to(DEV), stream[:T])
    ops.tc_check(stream.device)
    got = stream.cpu()
    assert (got[:T] - ref).abs().max() <= 1e-3 * float(ref.abs().max()) + 1e-5
    assert torch.equal(got[T:], base[T:])
    ops.tc_linear_add(x.to(DEV), w.to(DEV), stream[:T])
    ops.tc_check(stream.device)
    twice = base[:T] + 2 * (x.float() @ w.float().T)
    assert (stream[:T].cpu() - twice).abs().max() <= 2e-3 * float(twice.abs().max()) + 1e-5


@pytest.mark.parametrize("T,H,I", [(128, 64, 128), (2048, 896, 4864), (333, 1536, 8960), (200, 96, 160), (130, 72, 1000),
                                   (64, 896, 4864), (17, 1536, 8960), (100, 3584, 18944), (33, 72, 200), (128, 96, 40)])
def test_tcgen05_gate_up_swiglu(T, H, I):
    ops = _ops()
    g = torch.Generator().manual_seed(T + H + I)
    x = torch.randn(T, H, generator=g).bfloat16()
    w = (2 * torch.randn(2 * I, H, generator=g) / H ** 0.5).bfloat16()
    out = torch.full((T, I), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.tc_gate_up_swiglu(x.to(DEV), w.to(DEV), out)
    ops.tc_check(out.device)
    y = x.float() @ w.float().T
    ref = plain_silu(y[:, :I]) * y[:, I:]
    assert (out.float().cpu() - ref).abs().max() <= 1e-2 * float(ref.abs().max())


@pytest.mark.parametrize("T,H,nh,nkv,D", [(128, 896, 14, 2, 64), (2048, 896, 14, 2, 64), (300, 1536, 12, 2, 128),
                                          (129, 264, 5, 5, 64), (200, 128, 3, 1, 256)])
def test_tcgen05_qkv_with_rope_and_cache_write(T, H, nh, nkv, D):
    ops = _ops()
    g = torch.Generator().manual_seed(T + H + D)
    width = (nh + 2 * nkv) * D
    x = torch.randn(T, H, generator=g).bfloat16()
    w = (torch.randn(width, H, generator=g) / H ** 0.5).bfloat16()
    bias = 0.3 * torch.randn(width, generator=g)
    pos = torch.randint(0, 3000, (T,), generator=g, dtype=torch.int32)
    cos, sin = plain_rope_tables(3000, D, 1e6)
    page = 8
    pages = -(-T // page) + 3
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, page, nkv, D, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.full((T, nh, D), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.tc_qkv_rope_write(x.to(DEV), w.to(DEV), bias.to(DEV), pos.to(DEV), cos[:, :D // 2].contiguous().to(DEV),
                          sin[:, :D // 2].contiguous().to(DEV), slots.to(DEV), q_out, kc, vc, nh, nkv, D)
    ops.tc_check(q_out.device)
    y = x.float() @ w.float().T + bias
    q = plain_apply_rope(y[:, :nh * D].view(T, nh, D), cos, sin, pos)
    k = plain_apply_rope(y[:, nh * D:(nh + nkv) * D].view(T, nkv, D), cos, sin, pos)
    v = y[:, (nh + nkv) * D:].view(T, nkv, D)
    t = 1e-2 * float(y.abs().max())
    assert (q_out.float().cpu() - q).abs().max() <= t
    assert (kc.view(-1, nkv, D)[slots.long().to(DEV)].float().cpu() - k).abs().max() <= t
    assert (vc.view(-1, nkv, D)[slots.long().to(DEV)].float().cpu() - v).abs().max() <= t
    untouched = torch.ones(pages * page, dtype=torch.bool)
    untouched[slots.long()] = False
    assert float(kc.view(-1, nkv, D)[untouched.to(DEV)].abs().max()) == 0


@pytest.mark.parametrize("n,V", [(1, 5), (3, 1000), (2, 151936), (4, 1025), (64, 151936), (3, 4097)])
def test_argmax_lowest_index_on_ties(n, V):
    ops = _ops()
    logits = torch.randn(n, V, generator=torch.Generator().manual_seed(V))
    logits[0, V // 2] = 50.0
    logits[0, V - 1] = 50.0                                        # a tie: the lower index wins
    got = ops.argmax(logits.to(DEV)).cpu()
    assert got.tolist() == logits.argmax(-1).tolist() and got[0] == V // 2


@pytest.mark.parametrize("V", [7, 1000, 8195, 151936, 300000])
def test_sampling_matches_the_plain_rules(V):
    ops = _ops()
    g = torch.Generator().manual_seed(V)
    n = 12
    logits = 3 * torch.randn(n, V, generator=g)
    temps = torch.tensor([1.0, 0.7, 1.3, 0.8] * 3)
    top_k = torch.tensor([-1, 5, -1, 3, 0, 50, -1, 2, 1000000, 4, -1, 6], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.5, 0.3, 0.95, 0.01, 1.0, 1.0, 0.7, 0.6, 0.99])
    u = torch.rand(n, generator=g)
    u[0], u[1] = 0.0, 0.999999
    got = ops.sample(logits.to(DEV), temps.to(DEV), top_k.to(DEV), top_p.to(DEV), u.to(DEV)).cpu().tolist()
    for i in range(n):
        probs = plain_filtered_probs(logits[i], float(temps[i]), int(top_k[i]), float(top_p[i]))
        assert probs[got[i]] > 0, f"row {i}: token {got[i]} lies outside the kept set"
        cdf = probs.cumsum(0)
        lo = float(cdf[got[i]] - probs[got[i]])
        assert lo - 1e-5 <= float(u[i]) <= float(cdf[got[i]]) + 1e-5, (i, got[i], plain_inverse_cdf(probs, float(u[i])))
    # rows indirection: draw i reads row rows[i]
    rows = torch.tensor([3, 3, 0], dtype=torch.int32)
    again = ops.sample(logits.to(DEV), temps[[3, 3, 0]].to(DEV), top_k[[3, 3, 0]].to(DEV), top_p[[3, 3, 0]].to(DEV),
                       u[[3, 3, 0]].to(DEV), rows=rows.to(DEV)).cpu().tolist()
    assert again == [got[3], got[3], got[0]]
    # ... and lands where the row lies when asked to scatter; the other entries stay
    out = torch.full((n,), -5, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), temps[[3, 0]].to(DEV), top_k[[3, 0]].to(DEV), top_p[[3, 0]].to(DEV), u[[3, 0]].to(DEV),
               rows=torch.tensor([3, 0], dtype=torch.int32, device=DEV), out=out, scatter=True)
    assert out.cpu().tolist() == [got[0], -5, -5, got[3]] + [-5] * (n - 4)
    ops.tc_check(torch.device(DEV))                                # no block of a cluster gave up waiting


@pytest.mark.parametrize("V,scale", [(151936, 0.5), (151936, 3.0), (151936, 12.0), (5000, 3.0), (33, 1.0),
                                     (8192, 3.0), (20001, 12.0), (20001, 0.5)])
def test_sampling_cuts_inside_and_outside_the_band_of_candidates(V, scale):
    """(Rows of 8,192 logits and more are sampled by a cluster of eight blocks, narrower ones by one block.)
    Top-k and top-p over flat rows (the cut reaches far below the maximum: the kernel reads the whole row pass by
    pass), ordinary and peaked rows (the cut lies among the few thousand tokens next to the maximum, which the
    kernel copies to shared memory), with exact ties at the cut: whichever way the kernel takes, the token lies in
    the kept set of the plain rules and the uniform number falls into its interval of the kept distribution."""
    ops = _ops()
    g = torch.Generator().manual_seed(V + int(scale * 10))
    ks = [0, 1, 2, 40, 1000, 5000, 0, 0, 40, 3, 0, 200]
    ps = [0.9, 1.0, 0.5, 0.95, 0.999, 1.0, 0.1, 0.999, 0.2, 0.99, 0.5, 0.7]
    n = len(ks)
    logits = scale * torch.randn(n, V, generator=g)
    top = logits.topk(min(V, 60), dim=-1).indices
    for i in range(n):                                             # ties: the 3rd to 6th largest are equal, and a far run too
        logits[i, top[i, 3:6]] = float(logits[i, top[i, 2]])
        if V > 50:
            logits[i, top[i, 45:50]] = float(logits[i, top[i, 44]])
    temps = torch.tensor([1.0, 0.7, 1.3, 0.8] * 3)
    top_k = torch.tensor([k if k < V else 0 for k in ks], dtype=torch.int32)
    top_p = torch.tensor(ps)
    for trial in range(3):
        u = torch.rand(n, generator=g)
        if trial == 0:
            u[:] = 0.0
        elif trial == 1:
            u[:] = 0.9999999
        got = ops.sample(logits.to(DEV), temps.to(DEV), top_k.to(DEV), top_p.to(DEV), u.to(DEV)).cpu().tolist()
        for i in range(n):
            probs = plain_filtered_probs(logits[i], float(temps[i]), int(top_k[i]), float(top_p[i]))
            if probs[got[i]] == 0:
                # The one difference from the plain rules, by design: tokens tied exactly at a cut value are all
                # kept (a sort keeps as many of them as fit and drops the rest in no particular order).
                assert float(logits[i, got[i]]) == float(logits[i][probs > 0].min()), \
                    f"row {i}: token {got[i]} lies outside the kept set"
                continue
            tied = int((logits[i] == logits[i][probs > 0].min()).sum()) > int(((logits[i] == logits[i][probs > 0].min()) & (probs > 0)).sum())
            if tied:
                continue                                           # (the kept set is larger by the ties: other intervals)
            cdf = probs.cumsum(0)
            lo = float(cdf[got[i]] - probs[got[i]])
            assert lo - 1e-5 <= float(u[i]) <= float(cdf[got[i]]) + 1e-5, (i, got[i], plain_inverse_cdf(probs, float(u[i])))


def test_sampling_frequencies_follow_the_distribution():
    ops = _ops()
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 0.5]]).repeat(4000, 1)
    u = torch.rand(4000, generator=torch.Generator().manual_seed(1))
    t = torch.full((4000,), 0.8)
    got = ops.sample(logits.to(DEV), t.to(DEV), torch.full((4000,), -1, dtype=torch.int32, device=DEV),
                     torch.ones(4000, device=DEV), u.to(DEV)).cpu()
    freq = torch.bincount(got.long(), minlength=5).float() / 4000
    assert (freq - torch.softmax(logits[0] / 0.8, 0)).abs().max() < 0.03


def test_kernels_refuse_what_they_cannot_do():
    from tokenmill_b200.kernels.lib import KernelError
    ops = _ops()
    q = torch.zeros(1, 2, 24, device=DEV)                            # head size 24 is no multiple of 16
    kc = torch.zeros(2, 4, 1, 24, device=DEV)
    z = torch.zeros(2, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="unsupported shape"):
        ops.paged_attention(q, kc, kc.clone(), z.view(1, 2), z, z[:1], z[:1], z[:1], 1, torch.empty_like(q), scale=1.0)
    with pytest.raises(KernelError, match="CPU"):
        ops.swiglu(torch.zeros(2, 4), torch.zeros(2, 2))
    with pytest.raises(KernelError, match="float32 or bfloat16"):
        ops.swiglu(torch.zeros(2, 4, device=DEV, dtype=torch.float16), torch.zeros(2, 2, device=DEV, dtype=torch.float16))


@pytest.mark.parametrize("T", [1, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(1000, 896), (151, 64), (4099, 136), (33000, 1024), (16, 32)])
def test_output_matrix_streaming_kernel(T, N, K):
    """The decode step's output matrix product from the packed copy of the matrix: vocabularies that are no
    multiple of 8 or 16 rows, widths that are no multiple of 32, more row-group pairs than blocks and fewer;
    rows 8..15 of the token tile unused or used. One weight row is made to stand out for one token."""
    from tokenmill_b200.kernels.fused import pack_rows
    ops = _ops()
    g = torch.Generator().manual_seed(N + T)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    w[N - 1] = (x[T - 1].float() * 0.5).bfloat16()                      # the last row answers the last token
    ref = x.float() @ w.float().t()
    out = ops.lm_head(x.to(DEV), pack_rows(w.to(DEV)), N)
    ops.tc_check(torch.device(DEV))
    assert out.shape == (T, N) and out.dtype == torch.float32
    diff = (out.cpu() - ref).abs().max()
    assert diff <= 1e-5 * max(1.0, float(ref.abs().max())), diff
    assert int(out[T - 1].argmax()) == N - 1


@pytest.mark.parametrize("T", [1, 5, 8, 16])
@pytest.mark.parametrize("N,K", [(1000, 896), (151, 64), (4099, 136), (151936, 896), (16, 32)])
def test_output_matrix_kernel_finds_the_arg_max_in_its_epilogue(T, N, K):
    """The same product with each token's arg-max taken in the epilogue, three calls in a row on the same
    scratch (the arrival counter must end at zero): with and without the logits being written; equal logits
    (exact ties) at several indices must give the lowest of them, in the same block and across blocks; one
    token's winner is made to sit in the last, partly filled row group."""
    from tokenmill_b200.kernels.fused import pack_rows
    ops = _ops()
    g = torch.Generator().manual_seed(N * 3 + T)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    if T > 1:
        w[N - 1] = (x[T - 1].float() * 0.5).bfloat16()                  # the last row answers the last token
    if N > 600:                                                          # identical rows: identical logits
        w[17] = w[577] = w[N // 2 + 3] = (x[0].float() * 0.7).bfloat16()  # ... that win for token 0
    packed = pack_rows(w.to(DEV))
    logits = ops.lm_head(x.to(DEV), packed, N)
    want = logits.argmax(-1).to(torch.int32)
    if N > 600:
        assert float(logits[0, 17]) == float(logits[0, 577]) == float(logits[0, N // 2 + 3]) and int(want[0]) == 17
    if T > 1:
        assert int(want[T - 1]) == N - 1
    for call in range(3):
        tokens = torch.full((16,), -7, dtype=torch.int32, device=DEV)
        out = torch.full((T, N), float("nan"), device=DEV) if call == 1 else None
        ops.lm_head_argmax(x.to(DEV), packed, N, tokens, logits=out)
        ops.tc_check(torch.device(DEV))
        assert torch.equal(tokens[:T], want), (call, tokens[:T].tolist(), want.tolist())
        assert int((tokens[T:] == -7).sum()) == 16 - T
        if out is not None:
            assert torch.equal(out, logits)


@pytest.mark.parametrize("T", [1, 8, 13, 16])
@pytest.mark.parametrize("N,K", [(1536, 8960), (3584, 18944), (17920, 1536), (200, 1032), (24, 4104)])
def test_streaming_product_with_a_cut_k_range(T, N, K):
    """The streaming product for K beyond what a warp's registers hold of the activations: the K range is cut
    into slices of at most 1024 columns (the last shorter, or ending inside a 32-column chunk), every slice's
    sums come back separately, and their sum in index order is the product."""
    from tokenmill_b200.kernels.fused import pack_rows
    ops = _ops()
    g = torch.Generator().manual_seed(N + K + T)
    x = torch.randn(T, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.03).bfloat16()
    ref = x.double() @ w.double().t()
    parts = ops.stream_linear(x.to(DEV), pack_rows(w.to(DEV)), N)
    ops.tc_check(torch.device(DEV))
    S = -(-(-(-K // 32)) // 32)
    assert parts.shape == (S, T, N) and parts.dtype == torch.float32
    total = parts[0].clone()
    for s in range(1, S):
        total += parts[s]
    assert (total.cpu().double() - ref).abs().max() <= 2e-5 * max(1.0, float(ref.abs().max()))
    # a slice holds its own columns only: slice 0 is the product over the first columns
    if S > 1:
        width = -(-(-(-K // 32)) // S) * 32
        first = x[:, :width].double() @ w[:, :width].double().t()
        assert (parts[0].cpu().double() - first).abs().max() <= 2e-5 * max(1.0, float(first.abs().max()))


@pytest.mark.parametrize("S,T,I", [(1, 3, 160), (9, 8, 8960), (4, 16, 44)])
def test_swiglu_over_partial_sums(S, T, I):
    ops = _ops()
    g = torch.Generator().manual_seed(S + I)
    parts = torch.randn(S, T, 2 * I, generator=g)
    total = parts[0].clone()
    for s in range(1, S):
        total += parts[s]
    gate, up = total[:, :I].bfloat16().float(), total[:, I:].bfloat16().float()
    ref = (gate * torch.sigmoid(gate) * up)
    out = ops.swiglu_partials(parts.to(DEV), torch.empty(T, I, dtype=torch.bfloat16, device=DEV))
    assert (out.float().cpu() - ref).abs().max() <= 1e-2 * max(1.0, float(ref.abs().max()))
