"""Grouped-query attention mixer over the paged cache.

Order of operations (src/infer/model/layers.py:127-150, src/infer/kv/context.py:63-80): fused
q/k/v projection with bias; rotate-half position encoding of q and k; the step's k and v are
written to their cache slots BEFORE attention, so a prompt portion reads its own keys back from the
cache; causal attention of every query over its own request's keys; output projection without bias.
The projection weights are stored fused, rows [q; k; v], from the checkpoint's q_proj / k_proj /
v_proj tensors (src/infer/model/loader.py:45,68-70,111-113).

Every size and constant is a constructor parameter: head counts, head size, whether q/k/v carry a
bias, the softmax scale, an optional window, and the position encoding (itself a part, looked up by
kind). A window of w keys means a query at position p reads keys p-w+1..p.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from ..registry import get_part, register_mixer
from .base import LayerCache, StepInputs
from .spec import PagedKVNeed, PartSpec, StateNeed, WeightSpec

SPLIT_KEYS = 128     # decode attention cuts each request's keys at absolute multiples of this (batch 64 at contexts near 600: 1.27 ms a step against 1.31 with 256 and 1.38 with 64)


class AttentionScratch:
    """Scratch for split-key attention partials, sized once for the largest decode step."""

    def __init__(self, device: torch.device):
        self.device = device
        self.part_acc: torch.Tensor | None = None
        self.part_ml: torch.Tensor | None = None
        self.done: torch.Tensor | None = None     # zero between launches; the counters that go with the last get()
        self._graph_done: torch.Tensor | None = None
        self._x_acc: torch.Tensor | None = None   # a second set for steps that outgrow what graphs captured
        self._x_ml: torch.Tensor | None = None
        self._x_done: torch.Tensor | None = None
        self.frozen = False      # set once a graph has captured the pointers
        self._counters: torch.Tensor | None = None
        self._pf_acc: torch.Tensor | None = None
        self._pf_ml: torch.Tensor | None = None
        self._pf_done: torch.Tensor | None = None

    def counters(self) -> torch.Tensor:
        """Two zeroed ints the prompt-attention kernel uses as work ticket and done-counter (it leaves
        them zero again)."""
        if self._counters is None:
            self._counters = torch.zeros(2, dtype=torch.int32, device=self.device)
        return self._counters

    def reserve(self, rows: int, max_splits: int, head_dim: int) -> None:
        """Make the buffers that captured graphs point at large enough (before the first capture)."""
        need_acc, need_ml = rows * max_splits * head_dim, rows * max_splits * 2
        if self.part_acc is None or self.part_acc.numel() < need_acc or self.part_ml.numel() < need_ml:
            if self.frozen:
                raise RuntimeError("attention scratch would have to grow after a graph captured it")
            self.part_acc = torch.empty(need_acc, dtype=torch.float32, device=self.device)
            self.part_ml = torch.empty(need_ml, dtype=torch.float32, device=self.device)
        if self._graph_done is None or self._graph_done.numel() < rows:   # arrival counters, one per (request, kv head) at most
            if self.frozen:
                raise RuntimeError("attention scratch would have to grow after a graph captured it")
            self._graph_done = torch.zeros(rows, dtype=torch.int32, device=self.device)
        self.done = self._graph_done

    def get(self, rows: int, max_splits: int, head_dim: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Buffers for ``rows`` rows of ``max_splits`` partial results; ``self.done`` then holds arrival
        counters for as many rows. Once a graph has captured the first set, a step that needs more (a mixed
        step of many tokens between graph replays) gets a second set of its own, which may grow: the graphs
        keep pointing at the first."""
        need_acc, need_ml = rows * max_splits * head_dim, rows * max_splits * 2
        fits = (self.part_acc is not None and self.part_acc.numel() >= need_acc and self.part_ml.numel() >= need_ml
                and self._graph_done is not None and self._graph_done.numel() >= rows)
        if fits or not self.frozen:
            self.reserve(rows, max_splits, head_dim)
            return self.part_acc, self.part_ml
        if torch.cuda.is_current_stream_capturing():     # a graph must never point at the set that may move
            raise RuntimeError("attention scratch would have to grow after a graph captured it")
        if self._x_acc is None or self._x_acc.numel() < need_acc or self._x_ml.numel() < need_ml:
            self._x_acc = torch.empty(need_acc, dtype=torch.float32, device=self.device)
            self._x_ml = torch.empty(need_ml, dtype=torch.float32, device=self.device)
        if self._x_done is None or self._x_done.numel() < rows:
            self._x_done = torch.zeros(rows, dtype=torch.int32, device=self.device)
        self.done = self._x_done
        return self._x_acc, self._x_ml

    def get_prefill(self, slots: int, head_dim: int, tiles: int, tile_rows: int = 64):
        """Scratch for the prompt kernel's per-(row tile, key chunk) partial results: ``slots`` slots of
        ``tile_rows`` rows, and one arrival counter (zero between launches) for each of ``tiles`` (row tile, kv head)
        pairs. Prompt steps are never captured in a graph, so these may grow at any time."""
        if slots <= 0:
            return None, None, None
        need = slots * tile_rows
        if self._pf_acc is None or self._pf_acc.numel() < need * head_dim:
            self._pf_acc = torch.empty(need * head_dim, dtype=torch.float32, device=self.device)
        if self._pf_ml is None or self._pf_ml.numel() < need * 2:
            self._pf_ml = torch.empty(need * 2, dtype=torch.float32, device=self.device)
        if self._pf_done is None or self._pf_done.numel() < tiles:
            self._pf_done = torch.zeros(max(tiles, 1024), dtype=torch.int32, device=self.device)
        return self._pf_acc, self._pf_ml, self._pf_done


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

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.w_qkv = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]],
                               dim=0).contiguous()
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]],
                                   dim=0).contiguous()
        self.w_o = tensors["o_proj.weight"]
        if self.position is not None:
            self.cos, self.sin = self.position.tables(self.device)

    # --- run ------------------------------------------------------------------------------------

    def forward(self, x: torch.Tensor, step: StepInputs, cache: LayerCache) -> torch.Tensor:
        T = x.shape[0]
        q = torch.empty((T, self.nh, self.D), dtype=self.dtype, device=x.device)
        slot_map = step.slot_maps[cache.group] if cache.writes else None
        kc, vc = (cache.k, cache.v) if cache.writes else (None, None)
        if self.position is None:
            raise NotImplementedError("an attention mixer without position encoding is not built")
        if ops.skinny_ok(x, self.w_qkv):
            # decode step: one kernel streams the fused weight and finishes bias, rotation and cache write
            ops.skinny_qkv_rope_write(x, self.w_qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, q,
                                      kc, vc, self.nh, self.nkv, self.D)
        elif self.D in (64, 128, 256) and ops.tc_ok(x, self.w_qkv):
            # prompt step: the tcgen05 kernel keeps the product in tensor memory and finishes it the same way
            ops.tc_qkv_rope_write(x, self.w_qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, q,
                                  kc, vc, self.nh, self.nkv, self.D)
        else:
            qkv = ops.linear(x, self.w_qkv)
            ops.qkv_rope_write(qkv, self.b_qkv, step.positions, self.cos, self.sin, slot_map, q, kc, vc,
                               self.nh, self.nkv, self.D)
        out = torch.empty_like(q)
        self.attend(q, step, cache, out)
        flat = out.view(T, self.q_size)
        if ops.skinny_ok(flat, self.w_o, allow_split=True):
            return ops.skinny_linear(flat, self.w_o, k_splits=ops.skinny_k_splits(T, self.q_size))
        return ops.linear(flat, self.w_o)

    def attention_path(self, step: StepInputs) -> str:
        """Which attention kernel this step's shape takes: "decode" (tensor cores, every request brings at most
        16 query rows per kv head), "prefill_tc" / "prefill" (tensor cores, tcgen05 or mma.sync, row tiles cut
        into key chunks) or "generic" (any head size and dtype)."""
        G = self.nh // self.nkv
        if self.dtype != torch.bfloat16 or self.D not in (64, 128):
            return "generic"
        if step.split_keys and step.max_q_len * G <= 16:
            return "decode"
        if G in step.prefill:
            return "prefill_tc" if step.prefill[G].tile_rows == 128 else "prefill"
        return "generic"

    def emit(self, b, x, cache: LayerCache):
        """The prompt-step launches (library product, bias + rotation + cache write, attention, library
        product) written into a step program (kernels/program.py). ``x`` is a workspace buffer; returns the
        output buffer. The attention kernel is chosen per step as in ``attend``: all candidates are in the
        program, each under a step parameter that says whether it runs."""
        from ..kernels.program import (OP_DECODE_ATTENTION, OP_GEMM_BF16, OP_PREFILL_ATTENTION, OP_PREFILL_ATTENTION_TC,
                                       OP_QKV_ROPE_WRITE, Float)
        if self.dtype != torch.bfloat16 or self.D not in (64, 128) or self.position is None:
            raise NotImplementedError("step programs are built for bfloat16 attention with heads of 64 or 128")
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
        b.emit(OP_GEMM_BF16, [x, self.w_qkv, qkv, T, n_qkv, self.hidden_size, 0])
        b.emit(OP_QKV_ROPE_WRITE, [code, code, qkv, self.b_qkv, positions, self.cos, self.sin, slot_map, q, kc, vc, T,
                                   nh, nkv, D, self.cos.shape[0]])

        path = self.attention_path
        b.guard(lambda s: path(s) != "generic")
        key = f"G{G}_D{D}_kv{nkv}"
        table = b.param(f"block_table{g}", lambda s: s.block_tables[g].data_ptr())
        bt_stride = b.param(f"block_table_stride{g}", lambda s: s.block_tables[g].stride(0))
        page, scale, window = cache.k.shape[1], Float(self.scale), self.window

        # decode kernel: scratch for T * nh rows of max_splits partial results, n_seqs * nkv arrival counters
        def dec(i):
            return lambda s: s.scratch.get(s.n_tokens * nh, s.max_splits, D)[i].data_ptr() if path(s) == "decode" else 0
        def dec_done(s):
            if path(s) != "decode":
                return 0
            s.scratch.get(s.n_tokens * nh, s.max_splits, D)
            return s.scratch.done.data_ptr()
        b.emit(OP_DECODE_ATTENTION,
               [q, cache.k, cache.v, table, bt_stride, b.param("cu_q", lambda s: s.cu_q.data_ptr()),
                b.param("kv_before", lambda s: s.kv_before.data_ptr()), b.param("n_seqs", lambda s: s.n_seqs),
                b.param(f"decode_acc_{key}", dec(0)), b.param(f"decode_ml_{key}", dec(1)), out,
                b.param(f"decode_done_{key}", dec_done), nh, nkv, D, page, scale, window,
                b.param("split_keys", lambda s: s.split_keys), b.param("max_splits", lambda s: s.max_splits)],
               cond=b.param(f"attention_decode_{key}", lambda s: int(path(s) == "decode")))

        # prompt kernels: the step's work units for this group size, scratch for the tiles with several chunks
        def pf(i):
            def fn(s):
                if not path(s).startswith("prefill"):
                    return 0
                u = s.prefill[G]
                t = s.scratch.get_prefill(u.n_slots * nkv, D, u.n_tiles * nkv, u.tile_rows)[i]
                return t.data_ptr() if t is not None else 0
            return fn
        units = [b.param(f"units_{G}", lambda s: s.prefill[G].records.data_ptr() if G in s.prefill else 0),
                 b.param(f"n_units_{G}", lambda s: s.prefill[G].n_units if G in s.prefill else 0),
                 b.param(f"chunk_keys_{G}", lambda s: s.prefill[G].chunk_keys if G in s.prefill else 0)]
        scratch = [b.param(f"prefill_acc_{key}", pf(0)), b.param(f"prefill_ml_{key}", pf(1)),
                   b.param(f"prefill_done_{key}", pf(2)), b.param("prefill_counters", lambda s: s.scratch.counters().data_ptr())]
        common = [q, cache.k, cache.v, table, bt_stride, *units, *scratch, out, nh, nkv, D, page, scale, window]
        b.uses_tc_attention = True
        b.emit(OP_PREFILL_ATTENTION_TC, common + [ops.tc_error_word(self.device)],
               cond=b.param(f"attention_prefill_tc_{key}", lambda s: int(path(s) == "prefill_tc")))
        b.emit(OP_PREFILL_ATTENTION, common,
               cond=b.param(f"attention_prefill_{key}", lambda s: int(path(s) == "prefill")))
        b.emit(OP_GEMM_BF16, [out, self.w_o, branch, T, self.hidden_size, self.q_size, 0])
        return branch

    def attend(self, q: torch.Tensor, step: StepInputs, cache: LayerCache, out: torch.Tensor) -> None:
        """Run the attention kernel that ``attention_path`` names; the shape-generic kernel has its keys split
        when the queries are few and the contexts long."""
        G = self.nh // self.nkv
        rows = step.max_q_len * G
        path = self.attention_path(step)
        if path == "decode":
            part_acc, part_ml = step.scratch.get(q.shape[0] * self.nh, step.max_splits, self.D)
            ops.decode_attention_bf16(q, cache.k, cache.v, step.block_tables[cache.group], step.cu_q,
                                      step.kv_before, step.n_seqs, out, scale=self.scale, window=self.window,
                                      split_keys=step.split_keys, max_splits=step.max_splits, part_acc=part_acc,
                                      part_ml=part_ml, done=step.scratch.done)
            return
        if path in ("prefill_tc", "prefill"):
            units = step.prefill[G]                # row tiles cut into key chunks, heaviest first
            part_acc, part_ml, tile_done = step.scratch.get_prefill(units.n_slots * self.nkv, self.D,
                                                                    units.n_tiles * self.nkv, units.tile_rows)
            kernel = ops.prefill_attention_tc_bf16 if path == "prefill_tc" else ops.prefill_attention_bf16
            kernel(q, cache.k, cache.v, step.block_tables[cache.group], units, step.scratch.counters(), out,
                   scale=self.scale, window=self.window, part_acc=part_acc, part_ml=part_ml, tile_done=tile_done)
            return
        tile_seq, tile_row0, n_tiles = step.attention_tiles(G)
        kw = {}
        if step.split_keys and rows <= 32 and step.max_splits > 1:
            part_acc, part_ml = step.scratch.get(q.shape[0] * self.nh, step.max_splits, self.D)
            kw = dict(split_keys=step.split_keys, max_splits=step.max_splits, part_acc=part_acc, part_ml=part_ml,
                      seq_of_token=step.seq_of_token)
        ops.paged_attention(q, cache.k, cache.v, step.block_tables[cache.group], step.cu_q, step.kv_before,
                            tile_seq, tile_row0, n_tiles, out, scale=self.scale, window=self.window, **kw)


register_mixer("gqa_attention", GroupedQueryAttention)
