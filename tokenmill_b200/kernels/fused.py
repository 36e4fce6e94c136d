"""The whole-step decode kernel (csrc/decode_fused_bf16.cu) seen from Python.

A ``FusedDecoder`` is built from a ``DecoderModel`` when every layer is the arrangement the kernel
implements (pre-norm block, grouped-query attention with rotary encoding, SwiGLU feed-forward, RMSNorm,
bfloat16, head size 64 or 128, one cache group). It owns the kernel's workspaces and the device table of
per-layer pointers; ``run`` launches one cooperative kernel for a step of at most 16 tokens and returns the
normed hidden rows the output matrix is applied to. Models that do not fit simply get no ``FusedDecoder``
and keep the kernel-per-operation path.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_void_p

import torch

from . import lib
from .ops import _stream as ops_stream

MAX_TOKENS = 16
MAX_LAYERS = 96          # entries of the kernel's layer table in shared memory
# Layers beyond this many bytes of weights are left to the separate kernels: the whole-step kernel is made for
# steps that are bound by latency (0.5B layer sizes, 30 MB a layer: 30 us against 53 us); at the 1.5B sizes (93 MB
# a layer) its two remaining ring stages stream at 0.8 TB/s and the library products are faster (117 vs 86 us).
MAX_LAYER_WEIGHT_BYTES = 48 << 20
SPLIT_KEYS = 64          # granularity of the key split of attention (a block attends a multiple of this)
_ENABLED = os.environ.get("TOKENMILL_FUSED_DECODE", "1") != "0"


class _Layer(ctypes.Structure):
    _fields_ = [(n, c_void_p) for n in ("ln1_w", "w_qkv", "b_qkv", "kcache", "vcache", "w_o", "ln2_w", "w_gu", "w_down")]


class _Args(ctypes.Structure):
    _fields_ = (
        [("layers", c_void_p), ("n_layers", c_int)]
        + [(n, c_int) for n in ("H", "nh", "nkv", "D", "I")]
        + [(n, c_float) for n in ("eps1", "eps2", "eps_f", "scale_log2")]
        + [("window", c_int)]
        + [(n, c_void_p) for n in ("embedding", "final_ln_w", "cos_t", "sin_t")]
        + [("n_pos", c_int)]
        + [(n, c_void_p) for n in ("token_ids", "positions", "slot_map", "block_table")]
        + [("bt_stride", c_int)]
        + [(n, c_void_p) for n in ("cu_q", "kv_before", "want_rows", "token_rows")]
        + [(n, c_int) for n in ("T", "S", "n_want", "page_size", "split_keys", "max_splits")]
        + [(n, c_void_p) for n in ("resid", "q", "part_acc", "part_ml", "attn", "act", "attn_count", "bar",
                                   "error", "hidden_out")]
        + [("smem_bytes", c_int), ("stage_bytes", c_int), ("halves", c_int),
           ("timing", c_void_p)]
    )


def eligible(model) -> bool:
    """Whether every layer of the model is the arrangement the fused kernel implements."""
    from ..parts.attention import GroupedQueryAttention
    from ..parts.block import PreNormBlock
    from ..parts.norm import RMSNorm
    from ..parts.swiglu import SwiGLUFeedForward

    if not _ENABLED or model.dtype != torch.bfloat16 or model.device.type != "cuda":
        return False
    if not model.spec.run_order or len(model.spec.run_order) > MAX_LAYERS or \
            any(e.cache_of is not None for e in model.spec.run_order):
        return False
    first = model.blocks[model.spec.run_order[0].layer].mixer
    if not isinstance(first, GroupedQueryAttention):
        return False
    for e in model.spec.run_order:
        b = model.blocks[e.layer]
        m, f = b.mixer, b.feed_forward
        if type(b) is not PreNormBlock or type(m) is not GroupedQueryAttention or type(f) is not SwiGLUFeedForward:
            return False
        if type(b.mixer_norm) is not RMSNorm or type(b.feed_forward_norm) is not RMSNorm:
            return False
        if (m.nh, m.nkv, m.D, m.window, m.scale, m.hidden_size) != (first.nh, first.nkv, first.D, first.window,
                                                                   first.scale, first.hidden_size):
            return False
        if m.cos is None or first.cos is None or m.cos.data_ptr() != first.cos.data_ptr():
            return False
        if f.intermediate_size != model.blocks[model.spec.run_order[0].layer].feed_forward.intermediate_size:
            return False
        if b.mixer_norm.eps != model.blocks[model.spec.run_order[0].layer].mixer_norm.eps or \
                b.feed_forward_norm.eps != model.blocks[model.spec.run_order[0].layer].feed_forward_norm.eps:
            return False
    H, I = model.spec.hidden_size, model.blocks[0].feed_forward.intermediate_size
    if 2 * (H * (first.q_size + 2 * first.kv_size) + first.q_size * H + 3 * H * I) > MAX_LAYER_WEIGHT_BYTES:
        return False
    return (type(model.final_norm) is RMSNorm and first.D in (64, 128) and H % 8 == 0 and I % 8 == 0
            and first.q_size % 8 == 0 and first.nh // first.nkv <= 16 and len(model.cache_layout().groups) == 1)


def persistent_bytes(model) -> int:
    """Device memory a FusedDecoder for this model keeps for good beyond the model's own weights: the packed
    copy of every layer's four matrices (0 when the model gets no whole-step kernel)."""
    if not eligible(model):
        return 0
    total, seen = 0, set()
    for e in model.spec.run_order:
        if e.layer in seen:
            continue
        seen.add(e.layer)
        b = model.blocks[e.layer]
        total += sum(w.numel() * w.element_size() for w in (b.mixer.w_qkv, b.mixer.w_o, b.feed_forward.w_gate_up,
                                                            b.feed_forward.w_down))
    from . import ops
    if ops.lm_head_ok(1, model.spec.hidden_size) and os.environ.get("TOKENMILL_LM_HEAD", "1") != "0":
        total += model.output_weight.numel() * model.output_weight.element_size()      # the output matrix's packed copy
    return total + (64 << 20)


def dev_index(device: torch.device) -> int:
    return device.index if device.index is not None else torch.cuda.current_device()


def pack_rows(w: torch.Tensor) -> torch.Tensor:
    """The copy of a [N, K] weight matrix the fused kernel streams: [N/8 row groups][K/32 chunks][8 rows]
    [4 pieces][8 elements], padded with zeros, so that the 32 lanes of a warp, lane 4 g + t holding row g and
    columns 8 t .. 8 t + 7 of a chunk, read 512 contiguous bytes."""
    N, K = w.shape
    Np, Kp = -(-N // 8) * 8, -(-K // 32) * 32
    if (Np, Kp) != (N, K):
        padded = torch.zeros((Np, Kp), dtype=w.dtype, device=w.device)
        padded[:N, :K] = w
        w = padded
    return w.view(Np // 8, 8, Kp // 32, 4, 8).permute(0, 2, 1, 3, 4).contiguous()


class FusedDecoder:
    def __init__(self, model, layer_caches, max_model_len: int):
        assert ctypes.sizeof(_Args) == lib.load().tm_decode_fused_args_size(), "FusedArgs layout mismatch"
        assert ctypes.sizeof(_Layer) == lib.load().tm_decode_fused_layer_size(), "FusedLayer layout mismatch"
        self.model, self.device = model, model.device
        dev, bf = self.device, torch.bfloat16
        order = model.spec.run_order
        first = model.blocks[order[0].layer]
        m0, f0 = first.mixer, first.feed_forward
        self.H, self.nh, self.nkv, self.D, self.I = model.spec.hidden_size, m0.nh, m0.nkv, m0.D, f0.intermediate_size
        self.max_splits_cap = -(-max_model_len // SPLIT_KEYS)
        self._split_cache: dict[tuple[int, int], int] = {}
        # Tokens a step may bring at these sizes: wide models leave no room for a ring stage beside the staged
        # activations of many tokens (the fallback is the kernel-per-operation path).
        n_sm = torch.cuda.get_device_properties(dev_index(model.device)).multi_processor_count
        self.max_tokens = int(lib.load().tm_decode_fused_max_tokens(self.H, self.nh, self.nkv, self.D, self.I, n_sm))
        layers = (_Layer * len(order))()
        self._packed: dict[int, tuple[torch.Tensor, ...]] = {}      # by layer: a layer run twice is packed once
        for i, e in enumerate(order):
            b, lc = model.blocks[e.layer], layer_caches[i]
            if e.layer not in self._packed:
                self._packed[e.layer] = tuple(pack_rows(w) for w in (b.mixer.w_qkv, b.mixer.w_o,
                                                                     b.feed_forward.w_gate_up, b.feed_forward.w_down))
            w_qkv, w_o, w_gu, w_down = self._packed[e.layer]
            layers[i] = _Layer(b.mixer_norm.weight.data_ptr(), w_qkv.data_ptr(),
                               b.mixer.b_qkv.data_ptr() if b.mixer.b_qkv is not None else None,
                               lc.k.data_ptr(), lc.v.data_ptr(), w_o.data_ptr(),
                               b.feed_forward_norm.weight.data_ptr(), w_gu.data_ptr(), w_down.data_ptr())
        self._layers_dev = torch.frombuffer(bytearray(bytes(layers)), dtype=torch.uint8).to(dev)
        self._keep = layer_caches           # the table holds raw pointers into these tensors
        T, rows = MAX_TOKENS, MAX_TOKENS * self.nh * self.max_splits_cap
        self.resid = torch.empty((T, self.H), dtype=torch.float32, device=dev)
        self.q = torch.empty((T, self.nh, self.D), dtype=bf, device=dev)
        self.part_acc = torch.empty(rows * self.D, dtype=torch.float32, device=dev)
        self.part_ml = torch.empty(rows * 2, dtype=torch.float32, device=dev)
        self.attn = torch.empty((T, self.nh * self.D), dtype=bf, device=dev)
        self.act = torch.empty((T, self.I), dtype=bf, device=dev)
        self.attn_count = torch.zeros(T * self.nkv, dtype=torch.int32, device=dev)
        self.bar = torch.zeros(1, dtype=torch.int32, device=dev)
        self.error = torch.zeros(1, dtype=torch.int32, device=dev)
        self.hidden = torch.empty((T, self.H), dtype=bf, device=dev)
        self._err_host = torch.zeros(1, dtype=torch.int32, pin_memory=True)
        a = _Args()
        a.layers, a.n_layers = self._layers_dev.data_ptr(), len(order)
        a.H, a.nh, a.nkv, a.D, a.I = self.H, self.nh, self.nkv, self.D, self.I
        a.eps1, a.eps2, a.eps_f = first.mixer_norm.eps, first.feed_forward_norm.eps, model.final_norm.eps
        a.scale_log2 = m0.scale * 1.4426950408889634
        a.window = m0.window
        a.embedding, a.final_ln_w = model.embedding.data_ptr(), model.final_norm.weight.data_ptr()
        a.cos_t, a.sin_t, a.n_pos = m0.cos.data_ptr(), m0.sin.data_ptr(), m0.cos.shape[0]
        a.resid = self.resid.data_ptr()
        a.q, a.part_acc, a.part_ml, a.attn = (self.q.data_ptr(), self.part_acc.data_ptr(), self.part_ml.data_ptr(),
                                              self.attn.data_ptr())
        a.act = self.act.data_ptr()
        a.attn_count, a.bar, a.error = self.attn_count.data_ptr(), self.bar.data_ptr(), self.error.data_ptr()
        a.hidden_out = self.hidden.data_ptr()
        self._args = a
        self.n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        self.max_model_len = max_model_len
        self._arange = __import__("numpy").arange(MAX_TOKENS + 1, dtype="int32")
        self.h2d_bytes = 0
        self.launches = 0
        self.timing: torch.Tensor | None = None

    def enable_timing(self) -> torch.Tensor:
        """Profiling aid: block 0 stamps the nanosecond timer at every phase boundary into the returned
        int64 tensor [n_layers * 16 + 1] (slots per layer: 0 start, 1 norm done, 2 QKV done, 3 barrier passed,
        4 attention done, 5 barrier passed, 6 o_proj done, 7 second norm done, 8 gate/up done, 9 down done;
        inside block 0's first attention unit: 10 copies issued, 11 copies landed, 12 keys done, 13 all warps
        done, 14 states merged)."""
        self.timing = torch.zeros(self._args.n_layers * 16 + 1, dtype=torch.int64, device=self.device)
        self._args.timing = self.timing.data_ptr()
        return self.timing

    def split_for(self, n_seqs: int, max_kv_len: int) -> int:
        """Keys per attention unit (a multiple of SPLIT_KEYS). A unit is (request, kv head, split); its eight warps
        take an eighth of its keys each, 16 at a time, and the block that finishes a (request, kv head) last
        merges the splits. Measured at the 0.5B sizes (heads of 64): 1.6 us for every 16 keys a warp takes, 0.13 us
        for every split merged; units beyond one per block wait for a second round; heads of 128 are taken to cost
        twice as much a key (at the 7B sizes the step's time did not depend on the figure). The cheapest count
        under that model (one request of 4,000 keys: 128 or 256 keys a unit, 0.86 ms a step; 64 keys, which fill
        the grid but leave 67 splits to merge, 0.96 ms)."""
        blocks = -(-max(1, max_kv_len) // SPLIT_KEYS)
        key = (n_seqs, blocks)
        best = self._split_cache.get(key)
        if best is None:
            pairs, cost = n_seqs * self.nkv, None
            unit_us = 1.6 * self.D / 64
            for per_unit in range(1, min(blocks, 256) + 1):
                splits = -(-blocks // per_unit)
                rounds = -(-pairs * splits // self.n_sm)
                c = rounds * unit_us * -(-per_unit * SPLIT_KEYS // (8 * 16)) + 0.13 * splits
                if cost is None or c < cost - 1e-9:
                    best, cost = per_unit, c
            self._split_cache[key] = best
        return best * SPLIT_KEYS

    def takes(self, step) -> bool:
        G = self.nh // self.nkv
        return (step.n_tokens <= self.max_tokens and step.max_q_len * G <= 16 and step.n_want > 0
                and step.n_want <= self.max_tokens and len(step.block_tables) == 1)

    # --- plain decode steps: metadata written straight into a pinned ring, no intermediate objects --------

    _RING = 4

    def _decode_ring(self, page_size: int):
        if getattr(self, "_ring", None) is None:
            width = -(-self.max_model_len // page_size)
            n = 7 * 16 + 4 + MAX_TOKENS * width          # seven sections of 16 (cu_q: 20) and the block table
            # per slot: pinned buffer, device buffer, "copy has run" and "the kernel that read it has run" events
            self._ring = [(torch.zeros(n, dtype=torch.int32, pin_memory=True),
                           torch.zeros(n, dtype=torch.int32, device=self.device), torch.cuda.Event(), torch.cuda.Event())
                          for _ in range(self._RING)]
            self._ring_np = [h.numpy() for h, _, _, _ in self._ring]
            self._ring_at = 0
            # The step's integers travel on a stream of their own, so that the copy runs beside the step before
            # it instead of between two kernels; the error word goes back the same way behind the kernel.
            self._copy_stream = torch.cuda.Stream(device=self.device)
            self._launched = torch.cuda.Event()
        return self._ring

    def run_decode(self, entries, page_size: int, token_src: torch.Tensor | None = None,
                   token_rows: list[int] | None = None) -> torch.Tensor:
        """One new token for each of at most 16 requests, logits wanted for every one of them. The step's
        integers (token, position, cache slot, request offsets, block table) go into one of a few pinned
        buffers and from there to the device in one copy; ``h2d_bytes`` says how many. With ``token_src`` (an
        int32 device tensor, e.g. what the previous step's sampling wrote) entry i's token is
        token_src[token_rows[i]] and the entries' own token ids are ignored: the step can be launched before
        the host knows the tokens."""
        ring = self._decode_ring(page_size)
        k = self._ring_at
        self._ring_at = (k + 1) % self._RING
        host, dev, copied, consumed = ring[k]
        copied.synchronize()                              # the copy that last read this pinned buffer is done
        buf = self._ring_np[k]
        S = len(entries)
        max_kv = max(e.start for e in entries) + 1
        width = -(-max_kv // page_size)
        o_tok, o_pos, o_slot, o_cu, o_before, o_want, o_rows, o_tab = 0, 16, 32, 48, 68, 84, 100, 116
        tab = buf[o_tab:o_tab + S * width].reshape(S, width)
        toks, poss, slots = [0] * S, [0] * S, [0] * S
        for i, e in enumerate(entries):
            pos = e.start
            pages = e.handle.tables[0]
            at = pos // page_size
            if len(pages) <= at:
                raise RuntimeError(f"entry {i} holds {len(pages)} pages, its {pos + 1} tokens need {at + 1}")
            page = pages[at]
            if page < 0:
                raise RuntimeError(f"entry {i} writes into a page it has already given back")
            toks[i], poss[i], slots[i] = e.tokens[0], pos, page * page_size + pos % page_size
            n = min(len(pages), width)
            tab[i, :n] = pages[:n]
            if n < width:
                tab[i, n:] = 0
        buf[o_tok:o_tok + S] = toks
        buf[o_pos:o_pos + S] = poss
        buf[o_slot:o_slot + S] = slots
        buf[o_before:o_before + S] = poss
        buf[o_cu:o_cu + S + 1] = self._arange[:S + 1]
        buf[o_want:o_want + S] = self._arange[:S]
        if token_src is not None:
            buf[o_rows:o_rows + S] = token_rows
        used = o_tab + S * width
        main, side = torch.cuda.current_stream(self.device), self._copy_stream
        side.wait_event(consumed)                         # (the kernel that read this slot four steps ago is through)
        with torch.cuda.stream(side):
            dev[:used].copy_(host[:used], non_blocking=True)
            copied.record(side)
        main.wait_event(copied)
        self.h2d_bytes = used * 4
        a, base = self._args, dev.data_ptr()
        a.token_ids, a.positions, a.slot_map = base + 4 * o_tok, base + 4 * o_pos, base + 4 * o_slot
        if token_src is not None:
            if token_src.dtype != torch.int32 or not token_src.is_cuda or len(token_rows) != S:
                raise lib.KernelError("run_decode: token_src must be int32 on the device, one row index per entry")
            a.token_ids, a.token_rows = token_src.data_ptr(), base + 4 * o_rows
        else:
            a.token_rows = None
        a.cu_q, a.kv_before, a.want_rows = base + 4 * o_cu, base + 4 * o_before, base + 4 * o_want
        a.block_table, a.bt_stride = base + 4 * o_tab, width
        a.T, a.S, a.n_want, a.page_size = S, S, S, page_size
        a.split_keys = self.split_for(S, max_kv)
        a.max_splits = -(-max_kv // a.split_keys)
        lib.call("tm_decode_fused", ctypes.addressof(a), ops_stream())
        consumed.record(main)
        side.wait_event(consumed)
        with torch.cuda.stream(side):
            self._err_host.copy_(self.error, non_blocking=True)
        self.launches += 1
        return self.hidden[:S]

    def run(self, step, page_size: int) -> torch.Tensor:
        """Normed hidden rows [n_want, H] (bfloat16) of the step's wanted places."""
        a = self._args
        a.token_ids, a.positions = step.token_ids.data_ptr(), step.positions.data_ptr()
        a.slot_map, a.block_table = step.slot_maps[0].data_ptr(), step.block_tables[0].data_ptr()
        a.bt_stride = step.block_tables[0].stride(0)
        a.cu_q, a.kv_before, a.want_rows = step.cu_q.data_ptr(), step.kv_before.data_ptr(), step.want_rows.data_ptr()
        a.token_rows = None
        a.T, a.S, a.n_want, a.page_size = step.n_tokens, step.n_seqs, step.n_want, page_size
        a.split_keys = self.split_for(step.n_seqs, step.max_kv_len)
        a.max_splits = -(-step.max_kv_len // a.split_keys)
        lib.call("tm_decode_fused", ctypes.addressof(a), ops_stream())
        self._err_host.copy_(self.error, non_blocking=True)     # looked at by check() after the step's own sync
        self.launches += 1
        return self.hidden[:step.n_want]

    def check(self) -> None:
        """Raise if a block of the fused kernel gave up at a barrier in an earlier step. The error word
        travels to pinned host memory behind every launch; this reads the host copy (no synchronisation),
        so it reports a failure once the stream has been synchronised, at the latest one step later."""
        code = int(self._err_host[0])
        if code:
            with torch.inference_mode():     # (whichever mode the caller is in: the words may be inference tensors)
                self._err_host.zero_()
                self.error.zero_()
                self.bar.zero_()
                self.attn_count.zero_()
            what = "the output matrix kernel gave up waiting for its weights" if code == 21 else \
                "a token's position lies outside the position tables" if code == 31 else \
                f"the fused decode kernel gave up at a bounded wait (code {code}: 100 + n grid barrier n, 1000 / 2000 " \
                f"weight ring, 3000 + n readiness counter n)"
            raise lib.KernelError(f"{what}; the step's results are incomplete")
