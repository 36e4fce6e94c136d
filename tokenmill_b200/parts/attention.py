"""Grouped-query attention mixer over the paged cache.

Order of operations (src/infer/model/layers.py:127-150, src/infer/kv/context.py:63-80): fused
q/k/v projection with bias; position encoding of q and k; the step's k and v are written to their
cache slots BEFORE attention, so a prompt portion reads its own keys back from the cache; causal
attention of every query over its own request's keys; output projection without bias. The projection
weights are stored fused, rows [q; k; v], from the checkpoint's q_proj / k_proj / v_proj tensors
(src/infer/model/loader.py:45,68-70,111-113).

Every size and constant is a constructor parameter: head counts, head size, whether q/k/v carry a
bias, the softmax scale, an optional window, and the position encoding (itself a part, looked up by
kind). A window of w keys means a query at position p reads keys p-w+1..p. The position encoding may
give rotate-half tables (applied inside the projection's epilogue), bring a kernel of its own
(``apply(q, k, positions)``, run between the bias and the cache write), or be absent.

What the attention kernels need per step beyond the engine's own arrays (row tiles, work units cut into
key chunks, the key split of short-query steps) is planned in ``step_metadata`` (parts/attention_plan.py)
and reaches the device in the step's one copy; scratch for partial results comes from the step's
workspace.
"""

from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from ..registry import get_part, register_mixer
from .attention_plan import choose_chunk, decode_parts_cap, decode_units, decode_units_pay, packed_units, tiles_for
from .base import (LayerCache, PartMeta, PrefillUnits, StepInputs, StepMetadata, StepShape, part_limit_positions,
                   part_max_positions)
from .spec import PagedKVNeed, PartSpec, StateNeed, WeightSpec

SPLIT_KEYS = 128     # decode attention cuts each request's keys at absolute multiples of this (batch 64 at contexts near 600: 1.27 ms a step against 1.31 with 256 and 1.38 with 64)
MAX_SPLIT_KEYS = 512  # (the kernel with one block per split)
SPLIT_UNITS = 256    # ... or of a larger power-of-two multiple while the step still has this many (request, kv head, split) units


def choose_split(kv_lens: np.ndarray, kv_heads: int) -> int:
    """Keys per split of the decode attention for a step whose requests hold ``kv_lens`` keys: the base size, doubled
    while enough units are left to fill the chip. Every split costs a partial result written and merged, so long
    contexts in large batches want few, long splits (27 requests of 4,400 keys over 4 kv heads of 128: 140 us a layer
    with 128 keys a split, 95 us with 512); short ones want many (what a block takes in per second is limited)."""
    split = SPLIT_KEYS
    while split < MAX_SPLIT_KEYS and int(np.sum(-(-kv_lens // (2 * split)))) * kv_heads >= SPLIT_UNITS:
        split *= 2
    return split


class GroupedQueryAttention:
    def __init__(self, *, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, qkv_bias: bool,
                 position: PartSpec | None, window: int | None = None, scale: float | None = None,
                 dtype: torch.dtype, device: torch.device):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads ({num_heads}) must be a multiple of num_kv_heads ({num_kv_heads})")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim must be a multiple of 16 up to 256, got {head_dim}")
        self.hidden_size, self.nh, self.nkv, self.D = hidden_size, num_heads, num_kv_heads, head_dim
        self.qkv_bias = bool(qkv_bias)
        self.window = int(window) if window else 0
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.dtype, self.device = dtype, device
        self.q_size, self.kv_size = num_heads * head_dim, num_kv_heads * head_dim
        self.position = None
        if position is not None:
            self.position = get_part("position", position.kind)(**position.params)
        self.w_qkv: torch.Tensor | None = None
        self.b_qkv: torch.Tensor | None = None
        self.w_o: torch.Tensor | None = None
        self.cos: torch.Tensor | None = None      # rotate-half tables, when the position encoding has them
        self.sin: torch.Tensor | None = None
        # The tensor-core kernels take bfloat16 heads of 64 or 128; everything else runs the shape-generic kernel.
        self.fast = dtype == torch.bfloat16 and head_dim in (64, 128)
        # Rows of a prompt-attention work unit: 128 for the tcgen05 kernel, 64 for the mma.sync kernel.
        self.prefill_tile = 128 if (self.fast and ops.tc_attention_enabled()) else 64
        self.prefill_chunk = 0          # keys of a work unit; 0: chosen per step (attention_plan.choose_chunk)

    # --- declarations ---------------------------------------------------------------------------

    def weight_specs(self) -> list[WeightSpec]:
        H = self.hidden_size
        specs = []
        for name, rows in (("q_proj", self.q_size), ("k_proj", self.kv_size), ("v_proj", self.kv_size)):
            specs.append(WeightSpec(f"{name}.weight", (rows, H)))
            if self.qkv_bias:
                specs.append(WeightSpec(f"{name}.bias", (rows,), dtype="float32"))
        specs.append(WeightSpec("o_proj.weight", (H, self.q_size)))
        return specs

    def cache_need(self) -> PagedKVNeed:
        return PagedKVNeed(self.nkv, self.D, self.window or None)

    def state_need(self) -> StateNeed | None:
        return None

    def max_positions(self) -> int | None:
        """How far the position encoding reaches (None: it has no limit, or there is none)."""
        return part_max_positions(self.position) if self.position is not None else None

    def limit_positions(self, n: int) -> None:
        """No position >= n will be asked for: the encoding may size its tables so (before ``bind``)."""
        if self.position is not None:
            part_limit_positions(self.position, n)

    def activation_bytes(self, n_tokens: int) -> int:
        """q/k/v product, q, head outputs and the branch output of one step."""
        elt = 4 if self.dtype == torch.float32 else 2
        return n_tokens * (3 * self.q_size + 2 * self.kv_size + self.hidden_size) * elt

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]],
                               dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]],
                                   dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        tables = self.position.tables(self.device) if callable(getattr(self.position, "tables", None)) else None
        if tables is not None:
            self.cos, self.sin = tables
        elif self.position is not None and not callable(getattr(self.position, "apply", None)):
            raise TypeError(f"position encoding {type(self.position).__name__} has neither tables nor apply()")

    # --- what the kernels need per step ---------------------------------------------------------

    def metadata_key(self):
        """Mixers with the same head grouping and kernels share one plan per step."""
        return ("gqa_attention", self.nh // self.nkv, self.nkv, self.prefill_tile, self.fast)

    def step_metadata(self, shape: StepShape) -> StepMetadata:
        """The step's attention work as integer arrays. ``path`` names the kernel the step's shape takes:
        "decode" (tensor cores, every request brings at most 16 query rows per kv head: keys cut at absolute
        multiples of ``split_keys`` across blocks), "prefill_tc" / "prefill" (tensor cores, tcgen05 or
        mma.sync: ``units`` are row tiles cut into key chunks, heaviest first) or "generic" (any head size and
        dtype: tiles of 32 rows, keys split when the queries are few)."""
        G = self.nh // self.nkv
        q_lens, starts = shape.q_lens, shape.starts
        max_q = int(q_lens.max()) if q_lens.size else 0
        # (a captured graph serves every context up to the limit with the launch grid it was captured with: base size)
        split = SPLIT_KEYS if shape.for_graph or not self.fast else choose_split(starts.astype(np.int64) + q_lens, self.nkv)
        host = {"split_keys": split, "max_splits": max(1, -(-int(shape.max_kv_len) // split))}
        arrays: dict[str, np.ndarray] = {}
        constant = True                           # (a graph replays q_lens of 1: nothing else depends on starts)
        if self.fast and max_q * G <= 16:
            host["path"] = "decode"
            if ops.decode_units_ok(shape.page_size, self.D) and decode_units_pay(int(q_lens.size), self.nkv, self.D,
                                                                                    int(shape.max_kv_len), shape.for_graph):
                # The persistent kernel's list of units, made anew for every step (a captured graph has room for
                # the most units its requests can have, and is told at each replay how many there are).
                S = int(q_lens.size)
                cap = decode_parts_cap(shape.max_kv_len)
                slots = ops.decode_units_slots(self.D, self.device)
                records, n_units, max_parts = decode_units(q_lens, starts, self.window, kv_heads=self.nkv, slots=slots,
                                                           cap=cap, head_dim=self.D, rows=S * cap if shape.for_graph else None)
                arrays["decode_units"] = records
                arrays["decode_n_work"] = np.array([n_units * self.nkv], dtype=np.int32)
                host.update(max_parts=cap if shape.for_graph else max_parts,
                            decode_grid=min(slots, records.shape[0] * self.nkv))
                constant = False
        elif self.fast:
            chunk = self.prefill_chunk or choose_chunk(q_lens, starts, G, self.nkv, tile=self.prefill_tile)
            records, n_tiles, n_slots = packed_units(q_lens, starts, G, tile=self.prefill_tile, chunk=chunk)
            arrays["units"] = records
            host.update(path="prefill_tc" if self.prefill_tile == 128 else "prefill", n_units=records.shape[0],
                        n_tiles=n_tiles, n_slots=n_slots, chunk_keys=chunk, tile_rows=self.prefill_tile)
        else:
            tile_seq, tile_row0 = tiles_for(q_lens, G)
            arrays["tile_seq"], arrays["tile_row0"] = tile_seq, tile_row0
            host.update(path="generic", n_tiles32=int(tile_seq.size))
        return StepMetadata(arrays, host, constant_in_graph=constant)

    def _meta(self, step: StepInputs) -> PartMeta:
        return step.meta[self.metadata_key()]

    def attention_path(self, step: StepInputs) -> str:
        return self._meta(step).host["path"]

    @staticmethod
    def _units(meta: PartMeta) -> PrefillUnits:
        h = meta.host
        return PrefillUnits(meta.arrays["units"], h["n_units"], h["n_tiles"], h["n_slots"], h["chunk_keys"], h["tile_rows"])

    # --- run ------------------------------------------------------------------------------------

    adds_to_residual = True      # forward(..., residual=stream) may add its output into the stream and return None

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache,
                residual: torch.Tensor | None = None) -> torch.Tensor | None:
        T = x.shape[0]
        q = torch.empty((T, self.nh, self.D), dtype=self.dtype, device=x.device)
        slot_map = step.slot_maps[cache.group] if cache.writes else None
        kc, vc = (cache.k, cache.v) if cache.writes else (None, None)
        rotary = self.cos is not None
        if rotary and ops.skinny_ok(x, self.w_qkv):
            # decode step: one kernel streams the fused weight and finishes bias, rotation and cache write
            ops.skinny_qkv_rope_write(x, self.w_qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, q,
                                      kc, vc, self.nh, self.nkv, self.D)
        elif rotary and self.D in (64, 128, 256) and ops.tc_qkv_ok(x, self.w_qkv):
            # prompt step: the tcgen05 kernel keeps the product in tensor memory and finishes it the same way
            ops.tc_qkv_rope_write(x, self.w_qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, q,
                                  kc, vc, self.nh, self.nkv, self.D)
        elif rotary and cache.writes and self._decode_by_units(step) and ops.decode_rope_fused_ok():
            # decoding by units: the attention kernel finishes the projection itself (bias, rotation, cache write)
            qkv = ops.linear(x, self.w_qkv)
            self._attend_units(None, step, cache, q, raw=(qkv, slot_map))     # (q is the output buffer here)
            return self._project_out(q, T, residual)
        elif rotary or self.position is None:
            # library (or 32-bit) product, then bias + rotation (none without an encoding) + cache write
            qkv = ops.linear(x, self.w_qkv)
            ops.qkv_rope_write(qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, q, kc, vc,
                               self.nh, self.nkv, self.D)
        else:
            # an encoding with a kernel of its own: bias and split into dense q, k, v; the encoding; the cache write
            qkv = ops.linear(x, self.w_qkv)
            k = torch.empty((T, self.nkv, self.D), dtype=self.dtype, device=x.device)
            v = torch.empty_like(k)
            ops.qkv_rope_write(qkv, self.b_qkv, step.positions, None, None, None, q, k, v, self.nh, self.nkv, self.D)
            self.position.apply(q, k, step.positions)
            if cache.writes:
                ops.kv_cache_write(k, v, slot_map, cache.k, cache.v)
        out = torch.empty_like(q)
        self.attend(q, step, cache, out)
        return self._project_out(out, T, residual)

    def _project_out(self, out: torch.Tensor, T: int, residual: torch.Tensor | None) -> torch.Tensor | None:
        flat = out.view(T, self.q_size)
        if ops.skinny_ok(flat, self.w_o, allow_split=True):
            return ops.skinny_linear(flat, self.w_o, k_splits=ops.skinny_k_splits(T, self.q_size))
        if ops.tc_narrow_ok(flat, self.w_o):
            return ops.tc_linear(flat, self.w_o)
        if ops.tc_add_ok(flat, self.w_o, residual):
            # a few dozen tokens: the output projection cut along K over the whole chip, added into the stream
            ops.tc_linear_add(flat, self.w_o, residual)
            return None
        return ops.linear(flat, self.w_o)

    def _decode_by_units(self, step: StepInputs) -> bool:
        meta = step.meta.get(self.metadata_key())
        return meta is not None and meta.host.get("path") == "decode" and "decode_units" in meta.arrays

    def _attend_units(self, q: torch.Tensor | None, step: StepInputs, cache: LayerCache, out: torch.Tensor, raw=None) -> None:
        """The unit-driven decode kernel: from finished queries ``q``, or (``raw`` = (qkv, slot_map)) from the raw
        q/k/v product, which it then finishes itself."""
        meta = self._meta(step)
        max_parts = meta.host["max_parts"]
        part_acc, part_ml, done = self._decode_scratch(step.workspace, out.shape[0], step.n_seqs, max_parts, "_units")
        common = dict(scale=self.scale, window=self.window, max_parts=max_parts, grid=meta.host["decode_grid"],
                      part_acc=part_acc, part_ml=part_ml, done=done)
        table, units, n_work = step.block_tables[cache.group], meta.arrays["decode_units"], meta.arrays["decode_n_work"]
        if raw is not None:
            qkv, slot_map = raw
            ops.decode_attention_units_rope_bf16(qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, cache.k,
                                                 cache.v, table, step.cu_q, step.kv_before, units, n_work, out, **common)
        else:
            ops.decode_attention_units_bf16(q, cache.k, cache.v, table, step.cu_q, step.kv_before, units, n_work, out,
                                            **common)

    def emit(self, b, x, cache: LayerCache):
        """The prompt-step launches (library product, bias + rotation + cache write, attention, library
        product) written into a step program (kernels/program.py). ``x`` is a workspace buffer; returns the
        output buffer. The attention kernel is chosen per step as in ``attend``: all candidates are in the
        program, each under a step parameter that says whether it runs."""
        from ..kernels.program import (OP_DECODE_ATTENTION, OP_DECODE_ATTENTION_UNITS, OP_GEMM_BF16, OP_PREFILL_ATTENTION, OP_PREFILL_ATTENTION_TC,
                                       OP_QKV_ROPE_WRITE, OP_TC_LINEAR, OP_TC_QKV_ROPE_WRITE, Float)
        if not self.fast or self.cos is None:
            raise NotImplementedError("step programs are built for bfloat16 rotary attention with heads of 64 or 128")
        T, g, G, nh, nkv, D = b.tokens(), cache.group, self.nh // self.nkv, self.nh, self.nkv, self.D
        code = ops.dtype_code(self.dtype)
        n_qkv = self.q_size + 2 * self.kv_size
        qkv = b.buffer("qkv", n_qkv * 2)
        q = b.buffer("q", self.q_size * 2)
        out = b.buffer("attention_out", self.q_size * 2)
        branch = b.buffer("mixer_out", self.hidden_size * 2)
        positions = b.param("positions", lambda s: s.positions.data_ptr())
        slot_map = b.param(f"slot_map{g}", lambda s: s.slot_maps[g].data_ptr()) if cache.writes else None
        kc, vc = (cache.k, cache.v) if cache.writes else (None, None)
        # The projection: ONE tcgen05 kernel with bias, rotation and cache write in its epilogue where that wins (see
        # ops.tc_qkv_ok: prompts long enough, tiles that fill the chip in one wave), else the library product and
        # the rotary kernel behind it. Both are in the program; a step parameter says which runs.
        H = self.hidden_size
        err = ops.tc_error_word(self.device)
        fused_qkv = (lambda s: int(ops._TC_MODE != "0" and s.n_tokens >= ops.TC_MIN_TOKENS and H % 8 == 0 and
                                   (ops._TC_MODE == "1" or (s.n_tokens >= ops.TC_QKV_MIN_TOKENS and
                                                            ops.tc_one_wave(s.n_tokens, n_qkv, self.device)))))
        use_tc = b.param(f"tc_qkv_{n_qkv}_{H}", fused_qkv)
        use_lib = b.param(f"lib_qkv_{n_qkv}_{H}", lambda s: 1 - fused_qkv(s))
        b.emit(OP_TC_QKV_ROPE_WRITE, [x, H, self.w_qkv, self.b_qkv, positions, self.cos, self.sin, slot_map, q, kc, vc, T,
                                      H, nh, nkv, D, self.cos.shape[0], err], cond=use_tc)
        b.emit(OP_GEMM_BF16, [x, self.w_qkv, qkv, T, n_qkv, H, 0], cond=use_lib)
        b.emit(OP_QKV_ROPE_WRITE, [code, code, qkv, self.b_qkv, positions, self.cos, self.sin, slot_map, q, kc, vc, T,
                                   nh, nkv, D, self.cos.shape[0], err], cond=use_lib)

        mkey = self.metadata_key()
        meta = lambda s: s.meta[mkey]                                   # noqa: E731
        path = lambda s: s.meta[mkey].host["path"]                      # noqa: E731
        b.guard(lambda s: mkey in s.meta and path(s) != "generic")
        key = f"G{G}_D{D}_kv{nkv}"
        table = b.param(f"block_table{g}", lambda s: s.block_tables[g].data_ptr())
        bt_stride = b.param(f"block_table_stride{g}", lambda s: s.block_tables[g].stride(0))
        page, scale, window = cache.k.shape[1], Float(self.scale), self.window
        i32 = torch.int32

        # decode kernel: scratch for T * nh rows of max_splits partial results, n_seqs * nkv arrival counters
        # (buffers named for this head shape: a later launch record's buffer never moves an earlier one's)
        by_units = lambda s: path(s) == "decode" and "decode_units" in meta(s).arrays      # noqa: E731
        by_splits = lambda s: path(s) == "decode" and "decode_units" not in meta(s).arrays  # noqa: E731

        def dec(i, units):
            def fn(s):
                if not (by_units(s) if units else by_splits(s)):
                    return 0
                parts = meta(s).host["max_parts" if units else "max_splits"]
                return self._decode_scratch(s.workspace, s.n_tokens, s.n_seqs, parts,
                                            ("_units_" if units else "_") + key)[i].data_ptr()
            return fn
        cu_q = b.param("cu_q", lambda s: s.cu_q.data_ptr())
        kv_before = b.param("kv_before", lambda s: s.kv_before.data_ptr())
        b.emit(OP_DECODE_ATTENTION_UNITS,
               [q, cache.k, cache.v, cache.k.shape[0], table, bt_stride, cu_q, kv_before,
                b.param(f"decode_units_{key}", lambda s: meta(s).arrays["decode_units"].data_ptr() if by_units(s) else 0),
                b.param(f"decode_n_work_{key}", lambda s: meta(s).arrays["decode_n_work"].data_ptr() if by_units(s) else 0),
                b.param(f"decode_max_work_{key}", lambda s: meta(s).arrays["decode_units"].shape[0] * nkv if by_units(s) else 0),
                b.param(f"decode_grid_{key}", lambda s: meta(s).host["decode_grid"] if by_units(s) else 0),
                b.param(f"decode_units_acc_{key}", dec(0, True)), b.param(f"decode_units_ml_{key}", dec(1, True)),
                out, b.param(f"decode_units_done_{key}", dec(2, True)), nh, nkv, D, page, scale, window,
                b.param(f"decode_max_parts_{key}", lambda s: meta(s).host["max_parts"] if by_units(s) else 0),
                ops.tc_error_word(self.device)],
               cond=b.param(f"attention_decode_units_{key}", lambda s: int(by_units(s))))
        b.emit(OP_DECODE_ATTENTION,
               [q, cache.k, cache.v, table, bt_stride, cu_q, kv_before, b.param("n_seqs", lambda s: s.n_seqs),
                b.param(f"decode_acc_{key}", dec(0, False)), b.param(f"decode_ml_{key}", dec(1, False)),
                out, b.param(f"decode_done_{key}", dec(2, False)), nh, nkv, D, page, scale, window,
                b.param(f"split_keys_{key}", lambda s: meta(s).host["split_keys"]),
                b.param(f"max_splits_{key}", lambda s: meta(s).host["max_splits"]), ops.tc_error_word(self.device)],
               cond=b.param(f"attention_decode_{key}", lambda s: int(by_splits(s))))

        # prompt kernels: the step's work units for this head grouping, scratch for the tiles with several chunks
        def pf(i):
            def fn(s):
                if not path(s).startswith("prefill"):
                    return 0
                t = self._prefill_scratch(s.workspace, self._units(meta(s)), key)[i]
                return t.data_ptr() if t is not None else 0
            return fn
        prefill = lambda s: path(s).startswith("prefill")               # noqa: E731
        units = [b.param(f"units_{key}", lambda s: meta(s).arrays["units"].data_ptr() if prefill(s) else 0),
                 b.param(f"n_units_{key}", lambda s: meta(s).host["n_units"] if prefill(s) else 0),
                 b.param(f"chunk_keys_{key}", lambda s: meta(s).host["chunk_keys"] if prefill(s) else 0)]
        scratch = [b.param(f"prefill_acc_{key}", pf(0)), b.param(f"prefill_ml_{key}", pf(1)),
                   b.param(f"prefill_done_{key}", pf(2)),
                   b.param("prefill_counters", lambda s: s.workspace.get("attn_pf_counters", 2, i32, zeroed=True).data_ptr())]
        common = [q, cache.k, cache.v, table, bt_stride, *units, *scratch, out, nh, nkv, D, page, scale, window]
        b.uses_tc_attention = True
        b.emit(OP_PREFILL_ATTENTION_TC, common + [ops.tc_error_word(self.device)],
               cond=b.param(f"attention_prefill_tc_{key}", lambda s: int(path(s) == "prefill_tc")))
        b.emit(OP_PREFILL_ATTENTION, common,
               cond=b.param(f"attention_prefill_{key}", lambda s: int(path(s) == "prefill")))
        # The output projection: a narrow product, on the tcgen05 kernel where its 128-column tiles fill the chip.
        qs = self.q_size
        tc_o = (lambda s: int(ops._TC_MODE != "0" and s.n_tokens >= ops.TC_MIN_TOKENS and qs % 8 == 0 and H % 8 == 0 and
                              (ops._TC_MODE == "1" or (s.n_tokens >= ops.TC_NARROW_MIN_TOKENS and
                                                       ops.tc_one_wave(s.n_tokens, H, self.device)))))
        b.emit(OP_TC_LINEAR, [out, qs, self.w_o, branch, H, T, H, qs, err], cond=b.param(f"tc_o_{H}_{qs}", tc_o))
        b.emit(OP_GEMM_BF16, [out, self.w_o, branch, T, H, qs, 0], cond=b.param(f"lib_o_{H}_{qs}", lambda s: 1 - tc_o(s)))
        return branch

    def _decode_scratch(self, ws, n_tokens: int, n_seqs: int, max_splits: int, suffix: str = ""):
        """(part_acc, part_ml, done) for split-key attention: n_tokens * heads rows of max_splits partial results,
        and an arrival counter (zero between launches) per (request, kv head)."""
        rows = n_tokens * self.nh * max_splits
        return (ws.get("attn_part_acc" + suffix, rows * self.D, torch.float32),
                ws.get("attn_part_ml" + suffix, rows * 2, torch.float32),
                ws.get("attn_done" + suffix, n_seqs * self.nkv, torch.int32, zeroed=True))

    def _prefill_scratch(self, ws, units: PrefillUnits, suffix: str = ""):
        """(part_acc, part_ml, tile_done) for the prompt kernels' per-(row tile, key chunk) partial results:
        n_slots * kv_heads slots of tile_rows rows, and one arrival counter (zero between launches) for each
        (row tile, kv head) pair. Nothing when no tile of the step has more than one chunk."""
        slots = units.n_slots * self.nkv
        if slots <= 0:
            return None, None, None
        need = slots * units.tile_rows
        sfx = f"_{suffix}" if suffix else ""
        return (ws.get("attn_pf_acc" + sfx, need * self.D, torch.float32),
                ws.get("attn_pf_ml" + sfx, need * 2, torch.float32),
                ws.get("attn_pf_done" + sfx, max(units.n_tiles * self.nkv, 1024), torch.int32, zeroed=True))

    def attend(self, q: torch.Tensor, step: StepInputs, cache: LayerCache, out: torch.Tensor) -> None:
        """Run the attention kernel the step's plan names; the shape-generic kernel has its keys split
        when the queries are few and the contexts long."""
        G = self.nh // self.nkv
        meta = self._meta(step)
        path, ws = meta.host["path"], step.workspace
        split_keys, max_splits = meta.host["split_keys"], meta.host["max_splits"]
        if path == "decode" and "decode_units" in meta.arrays:
            self._attend_units(q, step, cache, out)
            return
        if path == "decode":
            part_acc, part_ml, done = self._decode_scratch(ws, q.shape[0], step.n_seqs, max_splits)
            ops.decode_attention_bf16(q, cache.k, cache.v, step.block_tables[cache.group], step.cu_q,
                                      step.kv_before, step.n_seqs, out, scale=self.scale, window=self.window,
                                      split_keys=split_keys, max_splits=max_splits, part_acc=part_acc,
                                      part_ml=part_ml, done=done)
            return
        if path in ("prefill_tc", "prefill"):
            units = self._units(meta)              # row tiles cut into key chunks, heaviest first
            part_acc, part_ml, tile_done = self._prefill_scratch(ws, units)
            kernel = ops.prefill_attention_tc_bf16 if path == "prefill_tc" else ops.prefill_attention_bf16
            kernel(q, cache.k, cache.v, step.block_tables[cache.group], units,
                   ws.get("attn_pf_counters", 2, torch.int32, zeroed=True), out,
                   scale=self.scale, window=self.window, part_acc=part_acc, part_ml=part_ml, tile_done=tile_done)
            return
        tile_seq, tile_row0, n_tiles = meta.arrays["tile_seq"], meta.arrays["tile_row0"], meta.host["n_tiles32"]
        kw = {}
        if step.max_q_len * G <= 32 and max_splits > 1:
            part_acc, part_ml, _ = self._decode_scratch(ws, q.shape[0], step.n_seqs, max_splits)
            kw = dict(split_keys=split_keys, max_splits=max_splits, part_acc=part_acc, part_ml=part_ml,
                      seq_of_token=step.seq_of_token)
        ops.paged_attention(q, cache.k, cache.v, step.block_tables[cache.group], step.cu_q, step.kv_before,
                            tile_seq, tile_row0, n_tiles, out, scale=self.scale, window=self.window, **kw)


register_mixer("gqa_attention", GroupedQueryAttention)
