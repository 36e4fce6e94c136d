"""Host-side planning of a step's attention work: which (request, rows, keys) pieces the attention
kernels of parts/attention.py take, as integer arrays. Pure numpy; no GPU needed.

The grouped-query attention mixer returns these arrays from its ``step_metadata`` hook, and the engine
packs them into the step's single host-to-device copy.
"""

from __future__ import annotations

import numpy as np

TILE_ROWS = 32       # rows of (token, head-in-group) one tile of the shape-generic kernel covers


def tiles_for(q_lens: np.ndarray, group_size: int) -> tuple[np.ndarray, np.ndarray]:
    per_seq = (q_lens * group_size + TILE_ROWS - 1) // TILE_ROWS
    tile_seq = np.repeat(np.arange(len(q_lens), dtype=np.int32), per_seq)
    first = np.cumsum(per_seq) - per_seq
    tile_row0 = (np.arange(tile_seq.size, dtype=np.int32) - np.repeat(first, per_seq).astype(np.int32)) * TILE_ROWS
    return tile_seq.astype(np.int32), tile_row0.astype(np.int32)


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


# --- decode: units of whole 64-key stages for the persistent kernel ------------------------------------------------

DECODE_STAGE_KEYS = 64          # keys of a stage of the decode kernel
DECODE_MAX_UNIT_STAGES = 32     # most stages the kernel takes in one unit
DECODE_MIN_PARTS = 64           # partial results a request may have at least (the scratch is sized by the cap)
_UNIT_CANDIDATES = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 12, 14, 16, 20, 24, 28, 32], dtype=np.int64)


def decode_units_pay(n_seqs: int, kv_heads: int, head_dim: int, max_kv_len: int, for_graph: bool) -> bool:
    """Whether a decode step of this many requests goes to the unit-driven kernel. Not with heads of 128, at most
    16 (request, kv head) pairs and contexts of at most 1,024 keys: a unit's one consumer warp takes 2 us a stage
    of 64 keys there and the merge 0.75 us a part, and the kernel with one block of four warps per fixed key split
    is ahead. Measured with the unit-driven kernel switched off altogether against on (1.5B sizes, context 768):
    1 / 2 / 4 requests 1.48 / 1.45 / 1.45 ms a step against 1.54 / 1.52 / 1.55; 8 requests 1.49 either way; 16
    requests 1.57 against 1.55; 7B sizes, 8 layers: 1 / 2 / 4 requests 1.16 / 1.19 / 1.15 against 1.22 / 1.25 /
    1.17. At context 3,328 it is the other way round (1.5B sizes, 4 / 8 requests: 1.75 / 1.82 ms by splits, 1.65 /
    1.70 by units), and a captured graph serves every context with the kernel it was captured with: graphs
    therefore always take the unit-driven kernel, and this rule is for steps outside graphs."""
    return for_graph or not (head_dim >= 128 and n_seqs * kv_heads <= 16 and max_kv_len <= 1024)


def decode_parts_cap(max_kv_len: int) -> int:
    """The most units a request of up to ``max_kv_len`` keys is ever cut into: what the scratch for the partial
    results is sized by where it cannot follow the step (a captured graph)."""
    stages = -(-max(int(max_kv_len), 1) // DECODE_STAGE_KEYS)
    return max(DECODE_MIN_PARTS, -(-stages // DECODE_MAX_UNIT_STAGES))


def decode_units(q_lens: np.ndarray, starts: np.ndarray, window: int, *, kv_heads: int, slots: int, cap: int,
                 head_dim: int = 128, rows: int | None = None) -> tuple[np.ndarray, int, int]:
    """Cut every request's keys into units for the persistent decode kernel. Returns (records, n_units, max_parts):
    records int32 [n, 4] = {request, first stage, end stage, part | parts << 16}, longest first, padded with zero
    rows to ``rows`` when given.

    A request whose rows see keys lo .. p (lo the window's start) has the stages lo // 64 .. p // 64; they are
    divided evenly among ``parts`` units. The unit length is the one (of a short list) for which the step takes
    the least time by this model: the grid's ``slots`` blocks take the (unit, kv head) items round-robin, so a
    step of ``items`` takes ceil(items / slots) rounds of the longest unit's stages (2 us a stage of 128-wide
    heads) plus a fixed cost per unit (its first copies' latency and its partial result: about 3 us), and the
    merge of a request's partials at the end costs 1.5 us and 0.75 us a part (measured: 4 parts 4.5 us, 7 parts
    6.7 us; a request in one unit writes its result itself). Short units fill the last
    round better and cost more partials; the model picks between them (27 requests of 4,400 keys,
    4 kv heads, 444 slots: 9 stages a unit, 864 items in 2 rounds, where 8 stages would need 3)."""
    q_lens = np.asarray(q_lens, dtype=np.int64)
    starts = np.asarray(starts, dtype=np.int64)
    S = int(q_lens.size)
    p_max = starts + np.maximum(q_lens, 1) - 1
    lo = np.maximum(0, starts - window + 1) if window > 0 else np.zeros(S, dtype=np.int64)
    first = lo // DECODE_STAGE_KEYS
    n = p_max // DECODE_STAGE_KEYS + 1 - first
    n_max = int(n.max()) if S else 1
    u_min = max(1, -(-n_max // cap))
    if u_min > DECODE_MAX_UNIT_STAGES:
        raise ValueError(f"a request of {n_max} stages of keys does not fit {cap} units of {DECODE_MAX_UNIT_STAGES} stages")
    stage_us = 2.0 * head_dim / 128          # a stage of 64 keys when every block of a multiprocessor streams
    cand = _UNIT_CANDIDATES[(_UNIT_CANDIDATES >= u_min) & (_UNIT_CANDIDATES < n_max)]
    cand = np.append(cand, min(max(n_max, u_min), DECODE_MAX_UNIT_STAGES))          # (one unit a request, if it may be)
    parts_c = -(-n[None, :] // cand[:, None])                                       # [candidates, requests]
    items = parts_c.sum(axis=1) * kv_heads
    longest = (-(-n[None, :] // parts_c)).max(axis=1)
    most = parts_c.max(axis=1)
    merge_us = np.where(most > 1, 1.5 + (0.4 if head_dim <= 64 else 0.75) * most, 0.0)   # the last unit counts and merges
    cost = -(-items // slots) * (longest * stage_us + 3.0) + merge_us
    best_u = int(cand[len(cost) - 1 - int(np.argmin(cost[::-1]))])                  # (ties: the longer unit)
    parts = -(-n // best_u)
    total = int(parts.sum())
    req = np.repeat(np.arange(S, dtype=np.int64), parts)
    j = np.arange(total, dtype=np.int64) - np.repeat(np.cumsum(parts) - parts, parts)
    base, extra = (n // parts)[req], (n % parts)[req]
    begin = first[req] + j * base + np.minimum(j, extra)
    size = base + (j < extra)
    records = np.stack([req, begin, begin + size, j | (parts[req] << 16)], axis=1).astype(np.int32)
    records = records[np.argsort(-size, kind="stable")]
    max_parts = int(parts.max()) if S else 1
    if rows is not None:
        if total > rows:
            raise ValueError(f"{total} units, room for {rows}")
        padded = np.zeros((rows, 4), dtype=np.int32)
        padded[:total] = records
        records = padded
    return records, total, max_parts
