"""Tensor-level wrappers over the kernel entry points.

Each wrapper checks what the kernel assumes (device, dtype, contiguity, shapes) and launches on the
current CUDA stream. None of them has a fallback: a tensor on the CPU or a missing library raises.
"""

from __future__ import annotations

import os

import torch

from . import lib

F32, BF16 = 0, 1


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise lib.KernelError(f"kernels run in float32 or bfloat16, got {dtype}")


dtype_code = _code


def _stream() -> int:
    """The raw handle of the stream torch launches on right now (captured graphs included). The private
    C call is a fraction of a microsecond; the public ``torch.cuda.current_stream()`` builds objects on
    the way and costs ten times that, once per kernel launch."""
    return _raw_stream(torch.cuda.current_device())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None) or \
    (lambda device: torch.cuda.current_stream(device).cuda_stream)


def _req(t: torch.Tensor, name: str, dtype: torch.dtype | None = None) -> int:
    if not t.is_cuda:
        raise lib.KernelError(f"{name} is on {t.device}; the kernels have no CPU path")
    if not t.is_contiguous():
        raise lib.KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise lib.KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return t.data_ptr()


def _opt(t: torch.Tensor | None, name: str, dtype: torch.dtype | None = None) -> int | None:
    return None if t is None else _req(t, name, dtype)


def add_rmsnorm(resid: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
                branch: torch.Tensor | None = None, partials: torch.Tensor | None = None,
                ids: torch.Tensor | None = None, table: torch.Tensor | None = None,
                rows: torch.Tensor | None = None) -> torch.Tensor:
    """resid [T, H] float32 (updated in place unless ``rows``); out [n, H] in the activation dtype.
    ids + table: the stream starts as table[ids]. branch [T, H]: added to the stream. partials
    [n, T, H] float32: summed in index order and added. rows [n] int32: norm only these rows."""
    H = resid.shape[-1]
    n_rows = rows.numel() if rows is not None else resid.shape[0]
    if out.shape[0] < n_rows or out.shape[-1] != H or weight.numel() != H:
        raise lib.KernelError(f"add_rmsnorm: out {tuple(out.shape)} / weight {tuple(weight.shape)} do not fit "
                              f"{n_rows} rows of width {H}")
    if (ids is None) != (table is None):
        raise lib.KernelError("add_rmsnorm: ids and table come together")
    n_part, part_stride = 0, 0
    if partials is not None:
        n_part, part_stride = partials.shape[0], partials.stride(0)
    dt = out.dtype
    lib.call("tm_add_rmsnorm", _code(dt), _req(resid, "resid", torch.float32), _opt(branch, "branch", dt),
             _opt(partials, "partials", torch.float32), n_part, part_stride, _opt(ids, "ids", torch.int32),
             _opt(table, "table", dt), _opt(rows, "rows", torch.int32), _req(weight, "weight", torch.float32),
             float(eps), _req(out, "out"), n_rows, H, _stream())
    return out


def qkv_rope_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, cos: torch.Tensor | None,
                   sin: torch.Tensor | None, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                   kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, D: int) -> None:
    """qkv [T, (nh + 2 nkv) D]; cos/sin [P, D/2] float32 (both None: no rotation); q_out [T, nh, D]; caches
    [pages, page, nkv, D]. Without a slot map but with "caches" of T rows, token t's k and v go to row t. A
    position outside the tables raises the device error word (``position_check``) instead of reading them."""
    T = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * D or positions.numel() < T or (cos is None) != (sin is None) or \
            (cos is not None and cos.shape[1] * 2 != D):
        raise lib.KernelError(f"qkv_rope_write: shapes do not fit (qkv {tuple(qkv.shape)}, nh {nh}, nkv {nkv}, D {D})")
    if slot_map is not None and (kcache is None or vcache is None):
        raise lib.KernelError("qkv_rope_write: a slot map needs both caches")
    if slot_map is None and kcache is not None and (kcache.numel() < T * nkv * D or vcache is None
                                                    or vcache.numel() < T * nkv * D):
        raise lib.KernelError("qkv_rope_write: dense k / v outputs need a row per token")
    dt = q_out.dtype
    lib.call("tm_qkv_rope_write", _code(qkv.dtype), _code(dt), _req(qkv, "qkv"), _opt(bias, "bias", torch.float32),
             _req(positions, "positions", torch.int32), _opt(cos, "cos", torch.float32),
             _opt(sin, "sin", torch.float32), _opt(slot_map, "slot_map", torch.int32), _req(q_out, "q_out"),
             _opt(kcache, "kcache", dt), _opt(vcache, "vcache", dt), T, nh, nkv, D, cos.shape[0] if cos is not None else 1,
             _tc_flag(qkv.device).data_ptr(), _stream())


def kv_cache_write(k: torch.Tensor, v: torch.Tensor, slot_map: torch.Tensor, kcache: torch.Tensor,
                   vcache: torch.Tensor) -> None:
    """k, v [T, nkv, D] -> rows slot_map[t] of the caches [pages, page, nkv, D] (negative slots are skipped)."""
    T = k.shape[0]
    width = k.numel() // max(T, 1)
    if v.shape != k.shape or kcache.shape[2:] != k.shape[1:] or vcache.shape != kcache.shape or slot_map.numel() < T:
        raise lib.KernelError("kv_cache_write: k / v / cache shapes disagree")
    dt = kcache.dtype
    lib.call("tm_kv_cache_write", _code(dt), _req(k, "k", dt), _req(v, "v", dt), _req(slot_map, "slot_map", torch.int32),
             _req(kcache, "kcache"), _req(vcache, "vcache", dt), T, width, _stream())


def paged_attention(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                    cu_q: torch.Tensor, kv_before: torch.Tensor, tile_seq: torch.Tensor, tile_row0: torch.Tensor,
                    n_tiles: int, out: torch.Tensor, *, scale: float, window: int = 0, split_keys: int = 0,
                    max_splits: int = 0, part_acc: torch.Tensor | None = None,
                    part_ml: torch.Tensor | None = None, seq_of_token: torch.Tensor | None = None) -> torch.Tensor:
    """q, out [T, nh, D]; caches [pages, page_size, nkv, D]; block_table [S, W] int32. With split_keys
    the partial results go through part_acc / part_ml and are merged into out by a second launch."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("paged_attention: q / cache / out shapes disagree")
    dt = q.dtype
    if split_keys:
        need = T * nh * max_splits
        if part_acc is None or part_ml is None or seq_of_token is None or part_acc.numel() < need * D \
                or part_ml.numel() < need * 2:
            raise lib.KernelError("paged_attention: split mode needs part_acc, part_ml and seq_of_token of full size")
    lib.call("tm_paged_attention", _code(dt), _req(q, "q"), _req(kcache, "kcache", dt), _req(vcache, "vcache", dt),
             _req(block_table, "block_table", torch.int32), block_table.stride(0),
             _req(cu_q, "cu_q", torch.int32), _req(kv_before, "kv_before", torch.int32),
             _req(tile_seq, "tile_seq", torch.int32), _req(tile_row0, "tile_row0", torch.int32), n_tiles,
             _req(out, "out", dt), _opt(part_acc, "part_acc", torch.float32), _opt(part_ml, "part_ml", torch.float32),
             nh, nkv, D, page_size, float(scale), int(window), int(split_keys), int(max_splits), _stream())
    if split_keys:
        lib.call("tm_attention_combine", _code(dt), part_acc.data_ptr(), part_ml.data_ptr(), cu_q.data_ptr(),
                 kv_before.data_ptr(), _req(seq_of_token, "seq_of_token", torch.int32), out.data_ptr(), T, nh, D,
                 int(window), int(split_keys), int(max_splits), _stream())
    return out


def decode_attention_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                          cu_q: torch.Tensor, kv_before: torch.Tensor, n_seqs: int, out: torch.Tensor, *, scale: float,
                          window: int, split_keys: int, max_splits: int, part_acc: torch.Tensor, part_ml: torch.Tensor,
                          done: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core attention for steps whose requests bring at most 16 / (nh / nkv) tokens each
    (decoding). bfloat16, head size 64 or 128; per-split partials through part_acc / part_ml, merged by the
    last block of each (request, kv head); ``done``: n_seqs * kv_heads int32 zeros (left zero), made here when
    not given."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf = torch.bfloat16
    need = T * nh * max_splits
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise lib.KernelError("decode_attention_bf16: scratch too small")
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("decode_attention_bf16: q / cache / out shapes disagree")
    if done is None:
        done = torch.zeros(n_seqs * nkv, dtype=torch.int32, device=q.device)
    elif done.numel() < n_seqs * nkv:
        raise lib.KernelError("decode_attention_bf16: too few arrival counters")
    lib.call("tm_decode_attention_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             _req(block_table, "block_table", torch.int32), block_table.stride(0), _req(cu_q, "cu_q", torch.int32),
             _req(kv_before, "kv_before", torch.int32), n_seqs, _req(part_acc, "part_acc", torch.float32),
             _req(part_ml, "part_ml", torch.float32), _req(out, "out", bf), _req(done, "done", torch.int32), nh, nkv, D,
             page_size, float(scale), int(window), int(split_keys), int(max_splits), _tc_flag(q.device).data_ptr(),
             _stream())
    return out


_DECODE_UNITS = os.environ.get("TOKENMILL_DECODE_UNITS", "1") != "0"


def decode_units_ok(page_size: int, head_dim: int) -> bool:
    """Whether decode attention runs as a persistent grid over a host-made list of units, with the keys and values
    brought in by tensor-map copies (attention_decode_tma_bf16.cu: pages of 8, 16, 32 or 64 tokens, heads of 64 or
    128). TOKENMILL_DECODE_UNITS=0 keeps the kernel with one block per (request, kv head, fixed split)."""
    return _DECODE_UNITS and page_size in (8, 16, 32, 64) and head_dim in (64, 128)


_units_slots: dict[tuple[int, int], int] = {}


def decode_units_slots(head_dim: int, device: torch.device | None = None) -> int:
    """Blocks of the unit-driven decode attention that are resident at once: what a plan of units should fill
    evenly (multiprocessors of the device; 148 where there is none to ask)."""
    sms = 148
    if device is not None and device.type == "cuda":
        sms = torch.cuda.get_device_properties(device).multi_processor_count
    key = (head_dim, sms)
    if key not in _units_slots:
        _units_slots[key] = sms * (4 if head_dim == 64 else 3)
    return _units_slots[key]


def decode_attention_units_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                                cu_q: torch.Tensor, kv_before: torch.Tensor, units: torch.Tensor, n_work: torch.Tensor,
                                out: torch.Tensor, *, scale: float, window: int, max_parts: int, grid: int,
                                part_acc: torch.Tensor, part_ml: torch.Tensor, done: torch.Tensor) -> torch.Tensor:
    """Tensor-core attention for steps whose requests bring at most 16 / (nh / nkv) tokens each (decoding), by a
    list of units (parts/attention_plan.py decode_units): ``units`` int32 [rows, 4] on the device, of which
    ``n_work`` (one int32 on the device) / kv_heads are valid; per-unit partials through part_acc / part_ml
    (``max_parts`` a request), merged by the block that writes a (request, kv head)'s last; ``done``:
    n_seqs * kv_heads int32 zeros (left zero); ``grid``: blocks to launch."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32 = torch.bfloat16, torch.int32
    n_seqs = kv_before.numel()
    need = T * nh * max_parts
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise lib.KernelError("decode_attention_units_bf16: scratch too small")
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("decode_attention_units_bf16: q / cache / out shapes disagree")
    if done.numel() < n_seqs * nkv:
        raise lib.KernelError("decode_attention_units_bf16: too few arrival counters")
    if units.dim() != 2 or units.shape[1] != 4 or units.data_ptr() % 16:
        raise lib.KernelError("decode_attention_units_bf16: units must be 16-byte aligned int32 records of 4")
    lib.call("tm_decode_attention_units_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             kcache.shape[0], _req(block_table, "block_table", i32), block_table.stride(0), _req(cu_q, "cu_q", i32),
             _req(kv_before, "kv_before", i32), _req(units, "units", i32), _req(n_work, "n_work", i32),
             units.shape[0] * nkv, int(grid), _req(part_acc, "part_acc", torch.float32),
             _req(part_ml, "part_ml", torch.float32), _req(out, "out", bf), _req(done, "done", i32), nh, nkv, D, page_size,
             float(scale), int(window), int(max_parts), _tc_flag(q.device).data_ptr(), _stream())
    return out


_DECODE_ROPE = os.environ.get("TOKENMILL_DECODE_ROPE", "1") != "0"


def decode_rope_fused_ok() -> bool:
    """Whether the unit-driven decode attention finishes the q/k/v projection itself (bias, rotation, cache
    write) instead of the kernel that otherwise stands between the two. TOKENMILL_DECODE_ROPE=0 keeps that kernel."""
    return _DECODE_ROPE


def decode_attention_units_rope_bf16(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                                     cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor, kcache: torch.Tensor,
                                     vcache: torch.Tensor, block_table: torch.Tensor, cu_q: torch.Tensor,
                                     kv_before: torch.Tensor, units: torch.Tensor, n_work: torch.Tensor,
                                     out: torch.Tensor, *, scale: float, window: int, max_parts: int, grid: int,
                                     part_acc: torch.Tensor, part_ml: torch.Tensor, done: torch.Tensor) -> torch.Tensor:
    """``decode_attention_units_bf16`` straight from the raw q/k/v product ``qkv`` [T, (nh + 2 nkv) D]: the kernel
    adds the bias, rotates queries and the new keys (rotate-half tables ``cos`` / ``sin`` [n_pos, D / 2]), writes
    each token's key and value to cache slot ``slot_map[t]`` and attends. ``out``: [T, nh, D]."""
    T, nh, D = out.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32, f32 = torch.bfloat16, torch.int32, torch.float32
    n_seqs = kv_before.numel()
    need = T * nh * max_parts
    if part_acc.numel() < need * D or part_ml.numel() < need * 2:
        raise lib.KernelError("decode_attention_units_rope_bf16: scratch too small")
    if qkv.shape != (T, (nh + 2 * nkv) * D) or not qkv.is_contiguous() or kcache.shape[3] != D or vcache.shape != kcache.shape:
        raise lib.KernelError("decode_attention_units_rope_bf16: qkv / cache / out shapes disagree")
    if cos.shape != sin.shape or cos.shape[1] != D // 2 or not cos.is_contiguous() or not sin.is_contiguous():
        raise lib.KernelError("decode_attention_units_rope_bf16: rotation tables of [positions, head_dim / 2] wanted")
    if done.numel() < n_seqs * nkv:
        raise lib.KernelError("decode_attention_units_rope_bf16: too few arrival counters")
    if units.dim() != 2 or units.shape[1] != 4 or units.data_ptr() % 16:
        raise lib.KernelError("decode_attention_units_rope_bf16: units must be 16-byte aligned int32 records of 4")
    lib.call("tm_decode_attention_units_rope_bf16", _req(qkv, "qkv", bf), _opt(bias, "bias", f32),
             _req(positions, "positions", i32), _req(cos, "cos", f32), _req(sin, "sin", f32), cos.shape[0],
             _req(slot_map, "slot_map", i32), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf), kcache.shape[0],
             _req(block_table, "block_table", i32), block_table.stride(0), _req(cu_q, "cu_q", i32),
             _req(kv_before, "kv_before", i32), _req(units, "units", i32), _req(n_work, "n_work", i32),
             units.shape[0] * nkv, int(grid), _req(part_acc, "part_acc", f32), _req(part_ml, "part_ml", f32),
             _req(out, "out", bf), _req(done, "done", i32), nh, nkv, D, page_size, float(scale), int(window),
             int(max_parts), _tc_flag(out.device).data_ptr(), _stream())
    return out


def prefill_attention_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                           units, counters: torch.Tensor, out: torch.Tensor, *, scale: float, window: int = 0,
                           part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                           tile_done: torch.Tensor | None = None) -> torch.Tensor:
    """Tensor-core causal attention for prompt portions (bfloat16, head size 64 or 128). ``units``: the
    step's PrefillUnits for this group size (records of row tiles of 64 (token, head-in-group) rows cut into
    key chunks of units.chunk_keys, heaviest first); part_acc / part_ml: float32 scratch for the tiles with
    several chunks, at least n_slots * kv_heads * 64 * (head_dim | 2) elements, and tile_done, n_tiles *
    kv_heads int32 zeros (left zero); counters: two int32 zeros the kernel uses as work ticket and leaves zero."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32 = torch.bfloat16, torch.int32
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("prefill_attention_bf16: q / cache / out shapes disagree")
    if scale <= 0:
        raise lib.KernelError("prefill_attention_bf16: the score scale must be positive")
    if units.tile_rows != 64:
        raise lib.KernelError("prefill_attention_bf16: units of 64-row tiles only")
    if units.n_slots and (part_acc is None or part_ml is None or tile_done is None
                          or part_acc.numel() < units.n_slots * nkv * 64 * D
                          or part_ml.numel() < units.n_slots * nkv * 64 * 2 or tile_done.numel() < units.n_tiles * nkv):
        raise lib.KernelError("prefill_attention_bf16: scratch for the partial results is missing or too small")
    lib.call("tm_prefill_attention_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             _req(block_table, "block_table", i32), block_table.stride(0), _req(units.records, "unit records", i32),
             units.n_units, int(units.chunk_keys),
             _req(part_acc, "part_acc", torch.float32) if units.n_slots else None,
             _req(part_ml, "part_ml", torch.float32) if units.n_slots else None,
             _req(tile_done, "tile_done", i32) if units.n_slots else None,
             _req(counters, "counters", i32), _req(out, "out", bf), nh, nkv, D, page_size, float(scale), int(window),
             _stream())
    return out


def tc_attention_enabled() -> bool:
    """The tcgen05 prompt-attention kernel is used where it applies unless TOKENMILL_TC_ATTENTION=0."""
    return os.environ.get("TOKENMILL_TC_ATTENTION", "1") != "0"


def prefill_attention_tc_bf16(q: torch.Tensor, kcache: torch.Tensor, vcache: torch.Tensor, block_table: torch.Tensor,
                              units, counters: torch.Tensor, out: torch.Tensor, *, scale: float, window: int = 0,
                              part_acc: torch.Tensor | None = None, part_ml: torch.Tensor | None = None,
                              tile_done: torch.Tensor | None = None) -> torch.Tensor:
    """As prefill_attention_bf16, on tcgen05 with the scores and outputs in tensor memory: head size 64 or 128, units of
    128-row tiles (units.tile_rows == 128; the scratch holds 128 rows per slot). A block that gives up on a
    bounded wait raises the device error word that tc_check reads."""
    T, nh, D = q.shape
    page_size, nkv = kcache.shape[1], kcache.shape[2]
    bf, i32 = torch.bfloat16, torch.int32
    if D not in (64, 128) or units.tile_rows != 128:
        raise lib.KernelError("prefill_attention_tc_bf16: head size 64 or 128 and 128-row tiles only")
    if kcache.shape[3] != D or vcache.shape != kcache.shape or out.shape != q.shape:
        raise lib.KernelError("prefill_attention_tc_bf16: q / cache / out shapes disagree")
    if scale <= 0:
        raise lib.KernelError("prefill_attention_tc_bf16: the score scale must be positive")
    if units.n_slots and (part_acc is None or part_ml is None or tile_done is None
                          or part_acc.numel() < units.n_slots * nkv * 128 * D
                          or part_ml.numel() < units.n_slots * nkv * 128 * 2 or tile_done.numel() < units.n_tiles * nkv):
        raise lib.KernelError("prefill_attention_tc_bf16: scratch for the partial results is missing or too small")
    lib.call("tm_prefill_attention_tc_bf16", _req(q, "q", bf), _req(kcache, "kcache", bf), _req(vcache, "vcache", bf),
             _req(block_table, "block_table", i32), block_table.stride(0), _req(units.records, "unit records", i32),
             units.n_units, int(units.chunk_keys),
             _req(part_acc, "part_acc", torch.float32) if units.n_slots else None,
             _req(part_ml, "part_ml", torch.float32) if units.n_slots else None,
             _req(tile_done, "tile_done", i32) if units.n_slots else None,
             _req(counters, "counters", i32), _req(out, "out", bf), nh, nkv, D, page_size, float(scale), int(window),
             _tc_flag(q.device).data_ptr(), _stream())
    return out


def swiglu(gu: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """gu [T, 2 I] (gate columns first) -> out [T, I] = silu(gate) * up."""
    T, two_i = gu.shape
    if two_i % 2 or out.shape[0] < T or out.shape[1] * 2 != two_i:
        raise lib.KernelError(f"swiglu: gu {tuple(gu.shape)} and out {tuple(out.shape)} do not fit")
    lib.call("tm_swiglu", _code(gu.dtype), _req(gu, "gu"), _req(out, "out", gu.dtype), T, two_i // 2, _stream())
    return out


def linear(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
           out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """x [T, K] . w [N, K]^T -> [T, N].

    float32: this library's own CUDA-core kernel (true 32-bit, k-ordered accumulation).
    bfloat16: the library matrix product (cuBLAS through torch.mm), as the reference uses a library
    for its projections (src/infer/model/layers.py:144,150,163,164); fp32 accumulation, output in
    ``out_dtype`` (bfloat16 or float32)."""
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise lib.KernelError(f"linear: x {tuple(x.shape)} and w {tuple(w.shape)} do not fit")
    if x.dtype == torch.float32:
        if out is None:
            out = torch.empty((T, N), dtype=torch.float32, device=x.device)
        lib.call("tm_gemm_f32_nt", _req(x, "x", torch.float32), x.stride(0), _req(w, "w", torch.float32),
                 _opt(bias, "bias", torch.float32), _req(out, "out", torch.float32), out.stride(0), T, N, K,
                 _stream())
        return out
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_cuda:
        raise lib.KernelError(f"linear: unsupported operands {x.dtype} / {w.dtype} on {x.device}")
    if bias is not None:
        raise lib.KernelError("linear: the bfloat16 product takes no bias (it is added by the kernel that follows)")
    want = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    if want == torch.float32:
        res = torch.mm(x, w.t(), out_dtype=torch.float32)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is not None:
        return torch.mm(x, w.t(), out=out)
    return torch.mm(x, w.t())


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """logits [n, V] float32 -> [n] int32, lowest index on ties."""
    n, V = logits.shape
    if logits.stride(1) != 1:
        raise lib.KernelError("argmax: rows must be contiguous")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    if not logits.is_cuda or logits.dtype != torch.float32:
        raise lib.KernelError("argmax: float32 logits on the GPU")
    chunks = lib.load().tm_argmax_chunks(V)
    sval = sidx = None
    if chunks > 1:                      # wide vocabulary: per-chunk winners, then a final pick
        sval = torch.empty(n * chunks, dtype=torch.float32, device=logits.device)
        sidx = torch.empty(n * chunks, dtype=torch.int32, device=logits.device)
    lib.call("tm_argmax", logits.data_ptr(), n, V, logits.stride(0), _req(out, "out", torch.int32),
             _opt(sval, "scratch"), _opt(sidx, "scratch"), _stream())
    return out


# TOKENMILL_SAMPLE_CLUSTER=0: every row sampled by one block (else rows of 8,192 logits and more go over a cluster
# of eight blocks, an eighth of the row in each block's shared memory).
_SAMPLE_CLUSTER = os.environ.get("TOKENMILL_SAMPLE_CLUSTER", "1") != "0"


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           uniform: torch.Tensor, rows: torch.Tensor | None = None, out: torch.Tensor | None = None,
           scatter: bool = False) -> torch.Tensor:
    """One draw per entry: entry i reads row rows[i] (default i) of logits [*, V] float32.
    temperature/top_p/uniform float32 [n], top_k int32 [n]; returns int32 [n]. With ``scatter`` (and rows and
    out given) draw i is written to out[rows[i]], so the draws land in an array indexed like the logits rows."""
    V = logits.shape[1]
    n = temperature.numel()
    if not logits.is_cuda or logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise lib.KernelError("sample: float32 logits with contiguous rows on the GPU")
    if rows is None and logits.shape[0] < n:
        raise lib.KernelError("sample: fewer logits rows than draws")
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=logits.device)
    lib.call("tm_sample", logits.data_ptr(), n, V, logits.stride(0), _req(temperature, "temperature", torch.float32),
             _req(top_k, "top_k", torch.int32), _req(top_p, "top_p", torch.float32),
             _req(uniform, "uniform", torch.float32), _opt(rows, "rows", torch.int32),
             _req(out, "out", torch.int32), int(bool(scatter and rows is not None)),
             _tc_flag(logits.device).data_ptr() if _SAMPLE_CLUSTER else None, _stream())
    return out


# --- weight-streaming products for decode steps (bfloat16, at most 64 tokens) -------------------------

SKINNY_MAX_TOKENS = 16             # the kernel takes up to 64; beyond 16 the library product is faster today
# Matrices beyond this size go to the library product at every token count: the weight-streaming kernel tops out
# near 1.2 to 2.1 TB/s, which is what a small matrix gets anyway (its time is latency) but half of what the
# library reaches on a large one (7B layer sizes, 8 tokens: gate/up 127 vs 66 us, down 116 vs 42 us).
SKINNY_MAX_WEIGHT_BYTES = 20 << 20
_SKINNY_X_BYTES = 200 * 1024       # shared memory the staged activations may take


def _padded_tokens(T: int) -> int:
    return 16 if T <= 16 else (32 if T <= 32 else 64)


def skinny_ok(x: torch.Tensor, w: torch.Tensor, allow_split: bool = False) -> bool:
    """Whether the weight-streaming kernel takes this product (else the library product does).
    A product with a fused epilogue cannot cut its K range, so its activations must fit shared memory."""
    if not (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2
            and x.shape[0] <= SKINNY_MAX_TOKENS and w.numel() * 2 <= SKINNY_MAX_WEIGHT_BYTES
            and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()):
        return False
    return allow_split or _padded_tokens(x.shape[0]) * (x.shape[1] + 64) * 2 <= _SKINNY_X_BYTES


def skinny_k_splits(T: int, K: int) -> int:
    """Cuts of the K range so that the staged activations fit shared memory."""
    return max(1, -(-(_padded_tokens(T) * K * 2) // _SKINNY_X_BYTES))


def skinny_linear(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None,
                  out_dtype: torch.dtype = torch.bfloat16, k_splits: int = 1, rows_per_block: int = 8) -> torch.Tensor:
    """x [T, K] . w [N, K]^T for T <= 64. k_splits == 1: returns [T, N] in out_dtype. k_splits > 1:
    returns float32 partial products [k_splits, T, N] for the add+norm kernel to sum."""
    T, K = x.shape
    N = w.shape[0]
    ng = rows_per_block // 8
    if k_splits > 1:
        partials = torch.empty((k_splits, T, N), dtype=torch.float32, device=x.device)
        lib.call("tm_skinny_linear", x.data_ptr(), x.stride(0), w.data_ptr(), None, None, 0, 0, partials.data_ptr(),
                 k_splits, T, N, K, ng, _stream())
        return partials
    out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    lib.call("tm_skinny_linear", x.data_ptr(), x.stride(0), w.data_ptr(), _opt(bias, "bias", torch.float32),
             out.data_ptr(), N, 1 if out_dtype == torch.float32 else 0, None, 1, T, N, K, ng, _stream())
    return out


LM_HEAD_MAX_TOKENS, LM_HEAD_MAX_K = 16, 1024


def lm_head_ok(T: int, K: int) -> bool:
    """Whether the streaming output-matrix kernel takes a product of T tokens over K columns."""
    return 0 < T <= LM_HEAD_MAX_TOKENS and K % 8 == 0 and K <= LM_HEAD_MAX_K


def lm_head(x: torch.Tensor, w_packed: torch.Tensor, n_rows: int, error: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] bfloat16 (T <= 16) times the output matrix, given as its packed copy (kernels/fused.py
    pack_rows of w [n_rows, K]) -> logits [T, n_rows] float32. The weights stream through shared memory at
    memory speed; the kernel's waits are bounded and report (code 21) through ``error``, an int32 device word
    that is zero, by default the word that tc_check reads."""
    T, K = x.shape
    if not lm_head_ok(T, K) or x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise lib.KernelError(f"lm_head: {T} tokens of {K} columns in {x.dtype} are not taken")
    if w_packed.dim() != 5 or w_packed.shape[0] * 8 < n_rows or w_packed.shape[1] * 32 < K or not w_packed.is_contiguous():
        raise lib.KernelError("lm_head: the packed matrix does not fit the sizes given")
    out = torch.empty((T, n_rows), dtype=torch.float32, device=x.device)
    lib.call("tm_lm_head_bf16", _req(x, "x", torch.bfloat16), w_packed.data_ptr(), out.data_ptr(), T, n_rows, K,
             (error if error is not None else _tc_flag(x.device)).data_ptr(), _stream())
    return out


_lm_head_scratch: dict[torch.device, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def lm_head_argmax(x: torch.Tensor, w_packed: torch.Tensor, n_rows: int, tokens: torch.Tensor,
                   logits: torch.Tensor | None = None, error: torch.Tensor | None = None) -> torch.Tensor:
    """``lm_head`` with the arg-max found in its epilogue: tokens[:T] (int32, on the device) receives the index
    of each token's largest logit, the lowest index on ties. ``logits`` [T, n_rows] float32 is written as well
    when given; without it no logits reach memory at all."""
    T, K = x.shape
    if not lm_head_ok(T, K) or x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise lib.KernelError(f"lm_head_argmax: {T} tokens of {K} columns in {x.dtype} are not taken")
    if w_packed.dim() != 5 or w_packed.shape[0] * 8 < n_rows or w_packed.shape[1] * 32 < K or not w_packed.is_contiguous():
        raise lib.KernelError("lm_head_argmax: the packed matrix does not fit the sizes given")
    if tokens.dtype != torch.int32 or tokens.numel() < T or (logits is not None and logits.shape != (T, n_rows)):
        raise lib.KernelError("lm_head_argmax: tokens are int32 [T], logits float32 [T, rows]")
    if x.device not in _lm_head_scratch:       # per-block winners (one row of 16 per block) and the arrival counter
        n_blocks = torch.cuda.get_device_properties(x.device).multi_processor_count
        _lm_head_scratch[x.device] = (torch.empty(n_blocks * 16, dtype=torch.float32, device=x.device),
                                      torch.empty(n_blocks * 16, dtype=torch.int32, device=x.device),
                                      torch.zeros(1, dtype=torch.int32, device=x.device))
    best_val, best_idx, done = _lm_head_scratch[x.device]
    lib.call("tm_lm_head_argmax_bf16", _req(x, "x", torch.bfloat16), w_packed.data_ptr(),
             _opt(logits, "logits", torch.float32), _req(tokens, "tokens", torch.int32), best_val.data_ptr(),
             best_idx.data_ptr(), done.data_ptr(), T, n_rows, K,
             (error if error is not None else _tc_flag(x.device)).data_ptr(), _stream())
    return tokens


def stream_linear_ok(T: int, K: int) -> bool:
    """Whether the streaming kernel takes a product of T tokens over K columns (any number of rows)."""
    return 0 < T <= LM_HEAD_MAX_TOKENS and K % 8 == 0 and -(-K // 1024) <= 128


def stream_linear(x: torch.Tensor, w_packed: torch.Tensor, n_rows: int, error: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] bfloat16 (T <= 16) times a matrix given as its packed copy (kernels/fused.py pack_rows of
    w [n_rows, K]) -> float32 partial products [S, T, n_rows], one per slice of at most 1024 columns of K
    (S = 1 for K <= 1024): the weights stream through shared memory at the memory's rate. The norm kernel adds
    such slices in index order (``Pending.partials``), ``swiglu_partials`` does for a gate/up product."""
    T, K = x.shape
    if not stream_linear_ok(T, K) or x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise lib.KernelError(f"stream_linear: {T} tokens of {K} columns in {x.dtype} are not taken")
    if w_packed.dim() != 5 or w_packed.shape[0] * 8 < n_rows or w_packed.shape[1] * 32 < K or not w_packed.is_contiguous():
        raise lib.KernelError("stream_linear: the packed matrix does not fit the sizes given")
    S = int(lib.load().tm_stream_linear_slices(K))
    out = torch.empty((S, T, n_rows), dtype=torch.float32, device=x.device)
    lib.call("tm_stream_linear_bf16", _req(x, "x", torch.bfloat16), w_packed.data_ptr(), out.data_ptr(), T, n_rows, K,
             (error if error is not None else _tc_flag(x.device)).data_ptr(), _stream())
    return out


def swiglu_partials(parts: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """parts [S, T, 2 I] float32 partial gate/up products -> out [T, I] bfloat16 = silu(gate) * up."""
    S, T, two_i = parts.shape
    if two_i % 8 or out.shape != (T, two_i // 2) or out.dtype != torch.bfloat16:
        raise lib.KernelError(f"swiglu_partials: parts {tuple(parts.shape)} and out {tuple(out.shape)} do not fit")
    lib.call("tm_swiglu_partials", _req(parts, "parts", torch.float32), S, parts.stride(0), _req(out, "out", torch.bfloat16),
             T, two_i // 2, _stream())
    return out


def skinny_qkv_rope_write(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                          cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                          kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, D: int) -> None:
    """The fused q/k/v projection of a decode step with its whole epilogue: bias, position encoding,
    q to q_out, k and v to their cache slots."""
    T, K = x.shape
    if w.shape != ((nh + 2 * nkv) * D, K) or cos.shape[1] * 2 != D:
        raise lib.KernelError("skinny_qkv_rope_write: shapes do not fit")
    bf = torch.bfloat16
    lib.call("tm_skinny_qkv_rope_write", x.data_ptr(), x.stride(0), _req(w, "w", bf), _opt(bias, "bias", torch.float32),
             _req(positions, "positions", torch.int32), _req(cos, "cos", torch.float32),
             _req(sin, "sin", torch.float32), _opt(slot_map, "slot_map", torch.int32), _req(q_out, "q_out", bf),
             _opt(kcache, "kcache", bf), _opt(vcache, "vcache", bf), T, K, nh, nkv, D, cos.shape[0],
             _tc_flag(x.device).data_ptr(), _stream())


def skinny_gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [T, I] = silu(x . gate^T) * (x . up^T), w_gate_up [2 I, K] with the gate rows first."""
    T, K = x.shape
    inter = w_gate_up.shape[0] // 2
    lib.call("tm_skinny_gate_up_swiglu", x.data_ptr(), x.stride(0), _req(w_gate_up, "w_gate_up", torch.bfloat16),
             _req(out, "out", torch.bfloat16), out.stride(0), T, K, inter, _stream())
    return out


# --- prompt-step products on tcgen05 tensor cores (bfloat16) ------------------------------------------

TC_MIN_TOKENS = 128                # below this the 128-token tiles are mostly padding
# Which prompt-step products run on this library's tcgen05 kernels (TOKENMILL_TC_GEMM): "0" (default) none: they
# go to the library product, as in the reference; "qkv": the q/k/v projection with bias, rotation and cache write in
# its epilogue, and narrow plain products (o_proj), both while tiles of 128 columns fill the chip in one wave; "1"
# every prompt product. Measured inside the prompt step at the 0.5B layer sizes (24 layers, 2,048 tokens): 3.83 ms
# with "0", 4.07 ms with "qkv" (at 512 tokens 2.16 against 2.45 ms; 1.5B sizes, 8 layers: 2.69 against 2.90 ms):
# one wave of tiles with its epilogue exposed, two tensor maps encoded per launch and the kernel's set-up cost more
# than the rotary kernel and the launch they save, so the default stays with the library. (A loop of Python-driven
# launches shows the opposite, 21 against 34 us, because there the library path pays two interpreter round trips.)
_TC_MODE = os.environ.get("TOKENMILL_TC_GEMM", "0")
if _TC_MODE == "auto":
    _TC_MODE = "qkv"
if _TC_MODE not in ("qkv", "0", "1"):
    _TC_MODE = "0"
TC_QKV_MIN_TOKENS = 384            # fused q/k/v projection: tokens from which it beats library product + rotary kernel
TC_NARROW_MIN_TOKENS = 1024        # plain narrow product: tokens from which it beats the library product
_tc_error: dict[torch.device, torch.Tensor] = {}
_sm_count: dict[int, int] = {}


def tc_gemm_enabled() -> bool:
    """Whether EVERY prompt-step product goes to the tcgen05 kernels (TOKENMILL_TC_GEMM=1)."""
    return _TC_MODE == "1"


def _sms(device: torch.device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _sm_count:
        _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _sm_count[idx]


def tc_one_wave(T: int, N: int, device: torch.device) -> bool:
    """Whether the tcgen05 kernel takes the product in tiles of 128 columns that fill the chip in one wave (it does
    so while tiles of 256 columns would leave SMs without a tile)."""
    return -(-T // 128) * -(-N // 256) < _sms(device)


def _tc_flag(device: torch.device) -> torch.Tensor:
    if device not in _tc_error:
        _tc_error[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_error[device]


tc_error_word = _tc_flag


_tc_host: dict[torch.device, torch.Tensor] = {}


def tc_post(device: torch.device) -> None:
    """Send the error word on its way to pinned host memory behind the work launched so far, without waiting;
    ``tc_poll`` looks at the copy."""
    flag = _tc_error.get(device)
    if flag is not None:
        if device not in _tc_host:
            _tc_host[device] = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        _tc_host[device].copy_(flag, non_blocking=True)


def tc_poll(device: torch.device) -> None:
    """Raise if the last copy ``tc_post`` made that has arrived holds an error (no synchronisation: a failure
    shows once the stream has been synchronised, at the latest one step later)."""
    host = _tc_host.get(device)
    if host is not None and int(host[0]):
        with torch.inference_mode():         # (the word may have been made inside a step: an inference tensor)
            host.zero_()
        tc_check(device)


def tc_check(device: torch.device) -> None:
    """Raise if a kernel reported through the device error word since the last check: a tcgen05 block that gave
    up on a bounded wait, or a position outside the rotary tables (reads one int back, which waits for the
    device)."""
    flag = _tc_error.get(device)
    if flag is not None:
        code = int(flag.item())
        if code:
            with torch.inference_mode():     # (the word may have been made inside a step: an inference tensor)
                flag.zero_()
            if code == 32:
                raise lib.KernelError("decode attention met a request with more rows than a tile holds, keys beyond "
                                      "max_splits * split_keys or a unit of more stages than it takes; its output is "
                                      "incomplete")
            if code in (33, 34):
                raise lib.KernelError(f"decode attention gave up waiting for {'a stage of keys' if code == 33 else 'a free stage'}"
                                      f" (code {code}); its output is incomplete")
            if code == 41:
                raise lib.KernelError("sampling: a block of a row's cluster gave up waiting for the others; the "
                                      "step's tokens are incomplete")
            if code == 31:
                raise lib.KernelError("a token's position lies outside the position tables (the rotation was not "
                                      "applied as asked; the step's results are wrong)")
            raise lib.KernelError(f"a tcgen05 block gave up waiting (code {code}: matrix product 1 loader, 2/3 issuer, "
                                  f"4 epilogue; attention 11/13 second product, 12 scores, 14 merge; 21 output matrix stream); "
                                  f"its results are incomplete")


def _tc_operands_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2
            and x.shape[0] >= TC_MIN_TOKENS and x.shape[1] % 8 == 0 and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.is_contiguous() and w.data_ptr() % 16 == 0)


def tc_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether a wide prompt product (gate/up, down) goes to the tcgen05 kernels: only with TOKENMILL_TC_GEMM=1."""
    return _TC_MODE == "1" and _tc_operands_ok(x, w)


def tc_qkv_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the q/k/v projection of a prompt step runs as ONE tcgen05 kernel with bias, rotation and cache write
    in its epilogue (else: library product, then the rotary kernel)."""
    if _TC_MODE == "0" or not _tc_operands_ok(x, w):
        return False
    return _TC_MODE == "1" or (x.shape[0] >= TC_QKV_MIN_TOKENS and tc_one_wave(x.shape[0], w.shape[0], x.device))


def tc_narrow_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether a plain narrow prompt product (o_proj) runs on the tcgen05 kernel."""
    if _TC_MODE == "0" or not _tc_operands_ok(x, w):
        return False
    return _TC_MODE == "1" or (x.shape[0] >= TC_NARROW_MIN_TOKENS and tc_one_wave(x.shape[0], w.shape[0], x.device))


def tc_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """x [T, K] . w [N, K]^T -> [T, N] bfloat16 on tcgen05 (N a multiple of 8)."""
    T, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((T, N), dtype=torch.bfloat16, device=x.device)
    lib.call("tm_tc_linear", x.data_ptr(), x.stride(0), w.data_ptr(), _req(out, "out", torch.bfloat16), out.stride(0),
             T, N, K, _tc_flag(x.device).data_ptr(), _stream())
    return out


_TC_ADD = os.environ.get("TOKENMILL_TC_DECODE", "1") != "0"
_TC_ADD_ALL = os.environ.get("TOKENMILL_TC_DECODE", "1") == "all"
TC_ADD_MIN_TOKENS, TC_ADD_MAX_TOKENS = 1, 128
TC_ADD_MIN_K = 2048     # shorter rows: the library's kernel is as fast (o_proj of 896: 4.9 us against 6 us here). Rows of
                        # 3,584 (the 7B sizes' output projection) win inside the step (3.45 against 3.54 ms at batch 8)
                        # although the library's kernel is ahead when both are timed alone (9 against 12 us).


def tc_add_ok(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor | None) -> bool:
    """Whether ``tc_linear_add`` takes this projection: a step of up to 128 tokens (the callers ask the
    weight-streaming kernels first, which take small matrices at up to 16 tokens; above 128 tokens the library
    product is one pass over the weights at full tiles anyway), rows long enough
    that cutting them pays (the down projection: 7.9 us against the library's 9.5 at 64 x 4864 -> 896), bfloat16
    operands, a 32-bit residual stream of the product's shape. TOKENMILL_TC_DECODE=0 switches it off; =all takes
    short rows too."""
    return (_TC_ADD and resid is not None and x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.dim() == 2 and TC_ADD_MIN_TOKENS <= x.shape[0] <= TC_ADD_MAX_TOKENS and x.shape[1] % 8 == 0
            and (x.shape[1] >= TC_ADD_MIN_K or _TC_ADD_ALL)
            and x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.is_contiguous()
            and w.data_ptr() % 16 == 0 and w.shape[0] % 4 == 0 and resid.dtype == torch.float32
            and resid.shape == (x.shape[0], w.shape[0]) and resid.stride(1) == 1 and resid.stride(0) % 4 == 0
            and resid.data_ptr() % 16 == 0)


def tc_swiglu_decode_ok(x: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    """Whether a step of up to 128 tokens takes its gate/up projection with the activation in the epilogue on
    tcgen05 (tiles of 32 gate and 32 up rows, one for every multiprocessor) instead of the library product and
    the activation kernel. Only with TOKENMILL_TC_DECODE=all: measured at 64 tokens, 896 -> 2 x 4864, the fused
    kernel takes about 16 us against the library's 7.0 + 2.8 us (every tile reads all of x again, 14 blocks of K
    one after the other), so a step of 64 requests takes 1.37 ms with it and 1.21 without."""
    return (_TC_ADD_ALL and x.is_cuda and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16 and x.dim() == 2
            and TC_ADD_MIN_TOKENS <= x.shape[0] <= TC_ADD_MAX_TOKENS and x.shape[1] % 8 == 0 and x.stride(1) == 1
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w_gate_up.is_contiguous()
            and w_gate_up.data_ptr() % 16 == 0 and (w_gate_up.shape[0] // 2) % 8 == 0)


def tc_linear_add(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor) -> None:
    """resid [T, N] float32 += x [T, K] . w [N, K]^T on tcgen05, the K range cut over the chip (atomic adds)."""
    T, K = x.shape
    lib.call("tm_tc_linear_add_f32", x.data_ptr(), x.stride(0), w.data_ptr(), _req(resid, "resid", torch.float32),
             resid.stride(0), T, w.shape[0], K, _tc_flag(x.device).data_ptr(), _stream())


def tc_gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out [T, I] = silu(x . gate^T) * (x . up^T) on tcgen05; the [T, 2I] product stays in tensor memory."""
    T, K = x.shape
    lib.call("tm_tc_gate_up_swiglu", x.data_ptr(), x.stride(0), _req(w_gate_up, "w_gate_up", torch.bfloat16),
             _req(out, "out", torch.bfloat16), out.stride(0), T, K, w_gate_up.shape[0] // 2,
             _tc_flag(x.device).data_ptr(), _stream())
    return out


def tc_qkv_rope_write(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor,
                      cos: torch.Tensor, sin: torch.Tensor, slot_map: torch.Tensor | None, q_out: torch.Tensor,
                      kcache: torch.Tensor | None, vcache: torch.Tensor | None, nh: int, nkv: int, D: int) -> None:
    """The fused q/k/v projection of a prompt step on tcgen05, epilogue as skinny_qkv_rope_write."""
    T, K = x.shape
    bf = torch.bfloat16
    lib.call("tm_tc_qkv_rope_write", x.data_ptr(), x.stride(0), _req(w, "w", bf), _opt(bias, "bias", torch.float32),
             _req(positions, "positions", torch.int32), _req(cos, "cos", torch.float32),
             _req(sin, "sin", torch.float32), _opt(slot_map, "slot_map", torch.int32), _req(q_out, "q_out", bf),
             _opt(kcache, "kcache", bf), _opt(vcache, "vcache", bf), T, K, nh, nkv, D, cos.shape[0],
             _tc_flag(x.device).data_ptr(), _stream())
