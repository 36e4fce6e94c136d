"""Turn a step's entries into device metadata: one packed int32 buffer, one host-to-device copy.

The reference builds five int64 tensors from Python lists over every token and copies each
(src/infer/engine/model_runner.py:30-32,40-74). Here the same information (token ids, absolute
positions, cache slots, block tables, per-request offsets, rows whose logits are wanted) is laid out
with numpy in a single pinned buffer; the device tensors the kernels read are views of one
allocation. The parts of the model add their own sections to that buffer: each part that has a
``step_metadata`` hook is asked once per step (parts with the same ``metadata_key()`` share one answer),
and its integer arrays travel in the same copy (``StepInputs.meta``). The engine does not know what
they mean.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable

import numpy as np
import torch

from ..cache.manager import CacheHandle, CacheManager
from ..parts.base import PartMeta, StepInputs, StepMetadata, StepShape, part_metadata_key


@dataclass
class StepEntry:
    """One request's share of a step: ``tokens`` continue the request at position ``start``;
    ``want`` lists the places among these tokens whose logits are asked for."""

    handle: CacheHandle
    tokens: list[int]
    start: int
    want: list[int] = field(default_factory=list)


def metadata_providers(parts) -> dict[Hashable, object]:
    """The parts that ask for step metadata, one per distinct key, in first-seen order."""
    out: dict[Hashable, object] = {}
    for p in parts:
        key = part_metadata_key(p)
        if key is not None and key not in out:
            out[key] = p
    return out


def collect_metadata(providers: dict[Hashable, object], shape: StepShape) -> dict[Hashable, StepMetadata]:
    """Ask every provider for its arrays and numbers for this step."""
    out = {}
    for key, part in providers.items():
        md = part.step_metadata(shape)
        if md is None:
            md = StepMetadata()
        for name, arr in md.arrays.items():
            if not isinstance(arr, np.ndarray) or arr.dtype != np.int32:
                raise TypeError(f"step metadata {key!r}/{name}: arrays are int32 numpy arrays, got "
                                f"{getattr(arr, 'dtype', type(arr))}")
        out[key] = md
    return out


class Layout:
    """Offsets of every section inside the packed buffer, for given sizes. ``extra`` names the parts'
    own sections: {(key, name): number of ints}."""

    def __init__(self, T: int, S: int, n_want: int, widths: list[int],
                 extra: dict[tuple[Hashable, str], int] | None = None):
        self.T, self.S, self.n_want, self.widths = T, S, n_want, widths
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
        self.extra = {k: take(n) for k, n in (extra or {}).items()}
        self.total = off


def extra_sizes(metadata: dict[Hashable, StepMetadata]) -> dict[tuple[Hashable, str], int]:
    return {(key, name): int(arr.size) for key, md in metadata.items() for name, arr in md.arrays.items()}


def write_extra(buf: np.ndarray, lay: Layout, metadata: dict[Hashable, StepMetadata]) -> None:
    for key, md in metadata.items():
        for name, arr in md.arrays.items():
            sl = lay.extra[(key, name)]
            if sl.stop - sl.start != arr.size:
                raise RuntimeError(f"step metadata {key!r}/{name} changed its size ({arr.size} ints, the buffer "
                                   f"has room for {sl.stop - sl.start})")
            buf[sl] = arr.reshape(-1)


def device_meta(dev: torch.Tensor, lay: Layout, metadata: dict[Hashable, StepMetadata]) -> dict[Hashable, PartMeta]:
    """The parts' sections as views of the device buffer, shaped as the parts shaped them."""
    return {key: PartMeta({name: dev[lay.extra[(key, name)]].view(arr.shape) for name, arr in md.arrays.items()},
                          dict(md.host))
            for key, md in metadata.items()}


last_h2d_bytes = 0    # bytes of the most recent step's host-to-device copy (read by the runner's statistics)


def build_step_inputs(entries: list[StepEntry], cache: CacheManager, device: torch.device,
                      providers: dict[Hashable, object] | None = None, *, workspace=None,
                      min_table_width: int = 0) -> StepInputs:
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
    metadata = collect_metadata(providers or {}, StepShape(q_lens, starts, ps, max_kv))
    lay = Layout(T, S, len(want_rows), widths, extra_sizes(metadata))

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
    write_extra(buf, lay, metadata)

    dev = host.to(device, non_blocking=True)
    global last_h2d_bytes
    last_h2d_bytes = lay.total * 4
    return StepInputs(
        n_tokens=T, n_seqs=S, token_ids=dev[lay.token_ids], positions=dev[lay.positions],
        seq_of_token=dev[lay.seq_of_token], cu_q=dev[lay.cu_q], kv_before=dev[lay.kv_before],
        state_slots=dev[lay.state_slots],
        block_tables=[dev[lay.block_tables[g]].view(S, widths[g]) for g in range(cache.num_groups)],
        slot_maps=[dev[lay.slot_maps[g]] for g in range(cache.num_groups)],
        want_rows=dev[lay.want_rows], n_want=len(want_rows), max_q_len=int(q_lens.max()), max_kv_len=max_kv,
        q_lens=q_lens.tolist(), kv_befores=starts.tolist(), meta=device_meta(dev, lay, metadata),
        workspace=workspace)
