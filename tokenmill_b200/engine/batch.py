"""Turn a step's entries into device metadata: one packed int32 buffer, one host-to-device copy.

The reference builds five int64 tensors from Python lists over every token and copies each
(src/infer/engine/model_runner.py:30-32,40-74). Here the same information (token ids, absolute
positions, cache slots, block tables, per-request offsets, rows whose logits are wanted) is laid out
with numpy in a single pinned buffer; the device tensors the kernels read are views of one
allocation.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheHandle, CacheManager
from ..parts.base import PrefillUnits, StepInputs

TILE_ROWS = 32       # rows of (token, head-in-group) one attention tile covers


@dataclass
class StepEntry:
    """One request's share of a step: ``tokens`` continue the request at position ``start``;
    ``want`` lists the places among these tokens whose logits are asked for."""

    handle: CacheHandle
    tokens: list[int]
    start: int
    want: list[int] = field(default_factory=list)


class Layout:
    """Offsets of every section inside the packed buffer, for given sizes."""

    def __init__(self, T: int, S: int, n_want: int, widths: list[int], tiles: dict[int, int],
                 units: dict[int, int] | None = None):
        self.T, self.S, self.n_want, self.widths, self.tiles = T, S, n_want, widths, tiles
        off = 0

        def take(n: int) -> slice:
            nonlocal off
            s = slice(off, off + n)
            off += (n + 3) // 4 * 4          # keep every section 16-byte aligned
            return s

        self.token_ids, self.positions, self.seq_of_token = take(T), take(T), take(T)
        self.cu_q, self.kv_before, self.state_slots = take(S + 1), take(S), take(S)
        self.want_rows = take(n_want)
        self.slot_maps = [take(T) for _ in widths]
        self.block_tables = [take(S * w) for w in widths]
        self.tile_seq = {g: take(n) for g, n in tiles.items()}
        self.tile_row0 = {g: take(n) for g, n in tiles.items()}
        # prompt-attention unit records per group size
        self.prefill = {g: take(n_units * UNIT_FIELDS) for g, n_units in (units or {}).items()}
        self.total = off


def tiles_for(q_lens: np.ndarray, group_size: int) -> tuple[np.ndarray, np.ndarray]:
    per_seq = (q_lens * group_size + TILE_ROWS - 1) // TILE_ROWS
    tile_seq = np.repeat(np.arange(len(q_lens), dtype=np.int32), per_seq)
    first = np.cumsum(per_seq) - per_seq
    tile_row0 = (np.arange(tile_seq.size, dtype=np.int32) - np.repeat(first, per_seq).astype(np.int32)) * TILE_ROWS
    return tile_seq.astype(np.int32), tile_row0.astype(np.int32)


last_h2d_bytes = 0    # bytes of the most recent step's host-to-device copy (read by the runner's statistics)

PACKED_TILE = 64        # rows of the tensor-core prompt attention's row tile
PREFILL_CHUNK = 512     # keys of one work unit of that kernel (a multiple of its 64-key blocks)

UNIT_FIELDS = 8         # ints of one unit record


def packed_units(q_lens: np.ndarray, starts: np.ndarray, group_size: int, tile: int = PACKED_TILE,
                 chunk: int = PREFILL_CHUNK) -> tuple[np.ndarray, int, int]:
    """Work units of the tensor-core prompt attention. A ROW TILE is ``tile`` consecutive (token,
    head-in-group) rows of one request; it sees keys 0 .. the position of its last row. A causal prompt's
    last tile has many times the keys of its first, so a tile's keys are cut at absolute multiples of
    ``chunk`` and every (tile, chunk) is a UNIT of its own, handed out heaviest first. A tile with one chunk
    writes its output itself (slot0 -1); the chunks of the others write partial results into slots
    slot0 .. slot0 + nchunks - 1, which the last of them to finish merges.

    Returns (records, n_tiles, n_slots); records is int32 [n_units, 8]: request, first row, chunk,
    number of chunks of the tile, slot0, tile index, first flat row of the request, tokens of the request
    in this step, tokens of it already in the cache. Everything the kernel needs to start a unit is in its
    record: one load instead of a chain of lookups."""
    per_seq = (q_lens * group_size + tile - 1) // tile
    n_tiles = int(per_seq.sum())
    tile_seq = np.repeat(np.arange(len(q_lens), dtype=np.int64), per_seq)
    first = np.cumsum(per_seq) - per_seq
    row0 = (np.arange(n_tiles, dtype=np.int64) - np.repeat(first, per_seq)) * tile
    last_pos = starts[tile_seq] + np.minimum(row0 + tile - 1, q_lens[tile_seq] * group_size - 1) // group_size
    n_chunks = last_pos // chunk + 1
    multi = n_chunks > 1
    counted = np.where(multi, n_chunks, 0)
    slot0 = np.where(multi, np.cumsum(counted) - counted, -1)
    unit_tile = np.repeat(np.arange(n_tiles, dtype=np.int64), n_chunks)
    cfirst = np.cumsum(n_chunks) - n_chunks
    unit_chunk = np.arange(unit_tile.size, dtype=np.int64) - np.repeat(cfirst, n_chunks)
    work = np.minimum(chunk, last_pos[unit_tile] + 1 - unit_chunk * chunk)
    order = np.argsort(-work, kind="stable")
    t, c = unit_tile[order], unit_chunk[order]
    cu_q = np.cumsum(q_lens) - q_lens
    sq = tile_seq[t]
    rec = np.stack([sq, row0[t], c, n_chunks[t], slot0[t], t, cu_q[sq], q_lens[sq], starts[sq]], axis=1)
    assert rec.shape[1] == UNIT_FIELDS + 1
    # chunk and number of chunks share one int (both far below 2^16: a chunk is hundreds of keys)
    packed = np.concatenate([rec[:, :2], (rec[:, 2] | (rec[:, 3] << 16))[:, None], rec[:, 4:]], axis=1)
    return np.ascontiguousarray(packed, dtype=np.int32), n_tiles, int(counted.sum())


def choose_chunk(q_lens: np.ndarray, starts: np.ndarray, group_size: int, kv_heads: int, tile: int = 128,
                 key_block: int = 128, n_sm: int = 148) -> int:
    """Keys per work unit of the prompt attention kernels, chosen for the step at hand. For the tcgen05 kernel
    (128-row tiles): Long units spare the
    per-unit costs (ticket, queries, first tile, writing and merging partial results: about 4 us of an SM's time
    against 1.4 us per block of 128 keys, two blocks of threads sharing the SM), short ones spread a few heavy
    tiles over the chip; the estimate is the larger of the work divided over the SMs and the longest unit running
    alone (1.8 us a block plus 8 us), over chunks of 512, 1024, 2048, ... keys. Measured at 14 query heads
    over 2 kv heads of 64 against a fixed 512: 2,048-token prompt 3.92 vs 4.21 ms for 24 layers, 4,096 tokens
    6.97 vs 8.38 ms, 8,192 tokens 15.7 vs 20.4 ms, 1,024 tokens behind 3,072 cached 3.70 vs 4.01 ms."""
    per_seq = (q_lens * group_size + tile - 1) // tile
    rows_end = np.minimum((np.concatenate([np.arange(n) for n in per_seq]) + 1) * tile,
                          np.repeat(q_lens * group_size, per_seq)) if len(per_seq) else np.zeros(0, dtype=np.int64)
    keys = np.repeat(starts, per_seq) + (rows_end - 1) // group_size + 1        # keys each row tile sees
    if keys.size == 0:
        return PREFILL_CHUNK
    longest = int(keys.max())
    if tile != 128:
        # The mma.sync kernel (64-row tiles, three blocks of threads per SM): the longest chunk that still leaves
        # three units per SM. Measured at 12 query heads over 2 kv heads of 128 against a fixed 512: 4,096-token
        # prompt 6.37 vs 6.94 ms for 8 layers, 8,192 tokens 17.2 vs 19.6 ms, 1,024 and 2,048 tokens unchanged.
        best, chunk = PREFILL_CHUNK, PREFILL_CHUNK
        while chunk < longest and chunk < (1 << 15):
            chunk *= 2
            if float(np.sum((keys + chunk - 1) // chunk)) * kv_heads >= 3 * n_sm:
                best = chunk
        return best
    blocks = float(np.sum((keys + key_block - 1) // key_block))
    best, best_cost, chunk = PREFILL_CHUNK, None, PREFILL_CHUNK
    while True:
        units = float(np.sum((keys + chunk - 1) // chunk))
        spread = (blocks * 1.37 + units * 4.0) * kv_heads / n_sm
        alone = -(-min(chunk, longest) // key_block) * 1.8 + 8.0
        cost = max(spread, alone)
        if best_cost is None or cost <= best_cost:
            best, best_cost = chunk, cost
        if chunk >= longest or chunk >= (1 << 15):
            return best
        chunk *= 2


def build_step_inputs(entries: list[StepEntry], cache: CacheManager, device: torch.device,
                      group_sizes: list[int], *, scratch=None, split_keys: int = 0,
                      min_table_width: int = 0, prefill_tile: int = PACKED_TILE,
                      prefill_chunk: int = PREFILL_CHUNK, kv_heads_of: dict[int, int] | None = None) -> StepInputs:
    S = len(entries)
    ps = cache.page_size
    q_lens = np.array([len(e.tokens) for e in entries], dtype=np.int32)
    if S == 0 or (q_lens <= 0).any():
        raise ValueError("a step needs at least one entry, and every entry at least one token")
    starts = np.array([e.start for e in entries], dtype=np.int32)
    T = int(q_lens.sum())
    cu_q = np.zeros(S + 1, dtype=np.int32)
    np.cumsum(q_lens, out=cu_q[1:])
    kv_after = starts + q_lens
    max_kv = int(kv_after.max())
    widths = [max(min_table_width, -(-max_kv // ps)) for _ in range(cache.num_groups)]
    want_rows = [int(cu_q[i]) + w for i, e in enumerate(entries) for w in e.want]
    for i, e in enumerate(entries):
        if any(not (0 <= w < len(e.tokens)) for w in e.want):
            raise ValueError(f"entry {i}: a wanted place lies outside its {len(e.tokens)} tokens")
    tile_arrays = {g: tiles_for(q_lens, g) for g in group_sizes}
    # keys per work unit: the given number, or (0) chosen for this step's shape
    # (A step in which every request brings so few rows that the decode kernel takes it needs no prompt units.)
    unit_groups = [g for g in group_sizes if not (split_keys and int(q_lens.max()) * g <= 16)]
    chunks = {g: prefill_chunk or choose_chunk(q_lens, starts, g, (kv_heads_of or {}).get(g, 1), tile=prefill_tile)
              for g in unit_groups}
    unit_arrays = {g: packed_units(q_lens, starts, g, tile=prefill_tile, chunk=chunks[g]) for g in unit_groups}
    lay = Layout(T, S, len(want_rows), widths, {g: a[0].size for g, a in tile_arrays.items()},
                 {g: u[0].shape[0] for g, u in unit_arrays.items()})

    host = torch.empty(lay.total, dtype=torch.int32, pin_memory=device.type == "cuda")
    buf = host.numpy()
    buf[lay.token_ids] = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
    seq_of_token = np.repeat(np.arange(S, dtype=np.int32), q_lens)
    positions = np.arange(T, dtype=np.int32) - np.repeat(cu_q[:-1], q_lens) + np.repeat(starts, q_lens)
    buf[lay.positions] = positions
    buf[lay.seq_of_token] = seq_of_token
    buf[lay.cu_q] = cu_q
    buf[lay.kv_before] = starts
    buf[lay.state_slots] = [e.handle.state_slot for e in entries]
    buf[lay.want_rows] = want_rows
    cu_list = cu_q.tolist()
    for g in range(cache.num_groups):
        w = widths[g]
        table = np.zeros((S, w), dtype=np.int32)
        slots = np.empty(T, dtype=np.int32)
        for i, e in enumerate(entries):
            pages_of = e.handle.tables[g]
            have, start, n_new = len(pages_of), e.start, len(e.tokens)
            need = -(-(start + n_new) // ps)
            if have < need:
                raise RuntimeError(f"entry {i} holds {have} pages in group {g}, its {start + n_new} tokens need {need}")
            table[i, :min(have, w)] = pages_of[:w]
            if n_new == 1:                       # a decoded token: no arrays for one slot
                page = pages_of[start // ps]
                if page < 0:
                    raise RuntimeError(f"entry {i} writes into a page it has already given back")
                slots[cu_list[i]] = page * ps + start % ps
                continue
            row = np.asarray(pages_of, dtype=np.int32)
            p = positions[cu_list[i]:cu_list[i + 1]]
            pages = row[p // ps]
            if (pages < 0).any():
                raise RuntimeError(f"entry {i} writes into a page it has already given back")
            slots[cu_list[i]:cu_list[i + 1]] = pages * ps + p % ps
        buf[lay.block_tables[g]] = table.reshape(-1)
        buf[lay.slot_maps[g]] = slots
    for g, (tile_seq, tile_row0) in tile_arrays.items():
        buf[lay.tile_seq[g]] = tile_seq
        buf[lay.tile_row0[g]] = tile_row0
    for g, (records, _, _) in unit_arrays.items():
        buf[lay.prefill[g]] = records.reshape(-1)

    dev = host.to(device, non_blocking=True)
    global last_h2d_bytes
    last_h2d_bytes = lay.total * 4
    max_q = int(q_lens.max())
    use_split = split_keys
    return StepInputs(
        n_tokens=T, n_seqs=S, token_ids=dev[lay.token_ids], positions=dev[lay.positions],
        seq_of_token=dev[lay.seq_of_token], cu_q=dev[lay.cu_q], kv_before=dev[lay.kv_before],
        state_slots=dev[lay.state_slots],
        block_tables=[dev[lay.block_tables[g]].view(S, widths[g]) for g in range(cache.num_groups)],
        slot_maps=[dev[lay.slot_maps[g]] for g in range(cache.num_groups)],
        want_rows=dev[lay.want_rows], n_want=len(want_rows), max_q_len=max_q, max_kv_len=max_kv,
        q_lens=q_lens.tolist(), kv_befores=starts.tolist(),
        tiles={g: (dev[lay.tile_seq[g]], dev[lay.tile_row0[g]], a[0].size) for g, a in tile_arrays.items()},
        prefill={g: PrefillUnits(dev[lay.prefill[g]], records.shape[0], n_tiles, n_slots, chunks[g], prefill_tile)
                 for g, (records, n_tiles, n_slots) in unit_arrays.items()},
        scratch=scratch, split_keys=use_split, max_splits=-(-max_kv // use_split) if use_split else 0)
