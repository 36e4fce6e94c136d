"""The step function: run exactly the tokens a step brings, as one batch, from the cache earlier
steps left, and return the logits at the wanted places.

Counterpart of the reference's ModelRunner.prepare / execute (src/infer/engine/model_runner.py:40-97)
with two differences: the result is logits (any wanted row, not only each request's last), sampling
being a separate stage; and prompt portions and decoded tokens are the same kind of entry, so the
attention kernel sees one list of requests instead of three code paths (src/infer/kv/context.py:63-80).

Decode-only steps may replay a captured CUDA graph per batch-size bucket
(src/infer/engine/cuda_graphs.py:45-158). Unlike the reference there are no context-length buckets:
the attention kernel reads each request's true length from device memory, so one graph per batch
size serves every context. Padded rows decode token 0 at position 0 into a sink page the manager
never hands out.
"""

from __future__ import annotations

import bisect
import gc
import os

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pool import CachePools
from ..kernels import fused, lib, ops
from ..kernels import program as program_mod
from ..parts.base import StepInputs, StepShape
from ..parts.model import DecoderModel
from . import batch as batch_mod
from .batch import (Layout, StepEntry, build_step_inputs, collect_metadata, device_meta, extra_sizes,
                    metadata_providers, write_extra)
from .workspace import Workspace

GRAPH_BATCH_SIZES = [1, 2, 4, 8, 16, 32, 64, 128, 256]
FUSED_DECODE_LIMIT_BESIDE_GRAPHS = 10
FUSED_DECODE_MAX_KEYS_BESIDE_GRAPHS = 72_000


class ModelRunner:
    def __init__(self, model: DecoderModel, cache: CacheManager, pools: CachePools, *, max_model_len: int,
                 cuda_graphs: bool = False, cuda_graph_max_batch: int = 64, max_num_seqs: int = 128):
        if model.device.type != "cuda":
            raise RuntimeError(f"the engine runs on a CUDA device only, not on {model.device}")
        self.model, self.cache, self.pools = model, cache, pools
        self.device = model.device
        limit = model.max_positions()
        if max_model_len > limit:
            raise ValueError(f"max_model_len is {max_model_len}, but the model serves {limit} positions (its position "
                             f"tables end there): tokens beyond them would be encoded wrongly")
        self.max_model_len = max_model_len
        self.layout = model.cache_layout()
        self.layer_caches = pools.layer_caches(len(model.spec.run_order))
        # Parts that want arrays of their own in every step's input buffer (by their metadata key), and the
        # scratch buffers parts ask for while they run.
        self.providers = metadata_providers(model.parts())
        self.workspace = Workspace(self.device)
        # Steps of more than 16 tokens run as a step program (one native call walks the launches) where every
        # part of the model can write its launches down; TOKENMILL_STEP_PROGRAM=0 keeps the per-launch path.
        self._program = None
        self._no_program = os.environ.get("TOKENMILL_STEP_PROGRAM", "1") == "0"
        # Steps of every size: what the whole-step kernel and the decode graphs do not take is still cheaper as
        # one native walk over library products than as 200 launches from Python with the weight-streaming
        # kernels (a 16-token prompt at the 0.5B sizes: 1.8 against 2.5 ms). Those kernels serve the captured
        # decode graphs and models without a program.
        self._program_min_tokens = 1
        self.graph_max_batch = min(cuda_graph_max_batch, max_num_seqs) if cuda_graphs else 0
        self._graphs: dict[int, "_DecodeGraph"] = {}
        self._graph_pool = None
        self.kernels_per_graph: dict[int, int] = {}
        self.stats = {"steps": 0, "graph_steps": 0, "fused_steps": 0, "program_steps": 0, "tokens": 0, "h2d_bytes": 0}   # h2d: last step
        # One kernel per decode step when the model is the arrangement that kernel implements.
        self.fused = None
        if fused.eligible(model) and len(self.layout.groups) == 1:
            self.fused = fused.FusedDecoder(model, self.layer_caches, max_model_len)
            if self.fused.max_tokens == 0:          # not even one token fits beside a ring stage at these sizes
                self.fused = None
        # Decode steps of up to this many requests take the whole-step kernel. Beside decode graphs the graph wins
        # from 11 requests on (0.5B sizes: 9 / 10 / 12 / 16 requests 0.88 / 0.95 / 0.97 / 1.00 ms a step in the
        # kernel, which takes 9 to 16 tokens in two passes, against 0.95 to 0.96 ms for any of them in the graph).
        self._fused_decode_limit = 0
        if self.fused is not None:
            self._fused_decode_limit = min(self.fused.max_tokens, FUSED_DECODE_LIMIT_BESIDE_GRAPHS) \
                if self.graph_max_batch >= self.fused.max_tokens else self.fused.max_tokens
        # The output matrix of those steps goes through this library's own streaming kernel, from a packed copy of
        # the matrix (as much memory again; hidden sizes up to 1024). It runs at the memory's read rate like the
        # library's kernel (52 against 50 us for 272 MB), and it finds the arg-max of greedy rows in its epilogue,
        # which saves writing and re-reading the logits and two launches (15 to 20 us a step). TOKENMILL_LM_HEAD=0
        # keeps the library product and saves the copy.
        self._packed_output = None
        if self.fused is not None and ops.lm_head_ok(1, model.spec.hidden_size) and \
                os.environ.get("TOKENMILL_LM_HEAD", "1") != "0":
            self._packed_output = fused.pack_rows(model.output_weight)
        if self.graph_max_batch:
            if any(s < 0 for s in pools.sink) or (pools.state and pools.state_sink < 0):
                raise RuntimeError("decode graphs need pools built with a sink page (and a sink state slot)")

    # --- the step -------------------------------------------------------------------------------

    @torch.inference_mode()
    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        """Logits [n_wanted, vocab] float32, in the order of the entries and of each entry's want."""
        for e in entries:
            if e.handle.fresh_state:
                self.pools.zero_state(e.handle.state_slot)
                e.handle.fresh_state = False
            if e.start + len(e.tokens) > self.max_model_len:
                raise ValueError(f"a request would reach {e.start + len(e.tokens)} tokens; max_model_len is "
                                 f"{self.max_model_len}")
        self.stats["steps"] += 1
        self.stats["tokens"] += sum(len(e.tokens) for e in entries)
        ops.tc_poll(self.device)
        if self.fused is not None:
            self.fused.check()
            decoding = all(len(e.tokens) == 1 and e.want == [0] for e in entries)
            if decoding and self._fused_takes_decode(entries):
                self.stats["fused_steps"] += 1
                hidden = self.fused.run_decode(entries, self.cache.page_size)
                self.stats["h2d_bytes"] = self.fused.h2d_bytes
                return self._decode_logits(hidden)
            if sum(len(e.tokens) for e in entries) <= self.fused.max_tokens and \
                    not (decoding and len(entries) <= self.graph_max_batch):
                # A short prompt has more rows per kv head than an attention unit of the kernel holds: it goes in
                # as several pieces of a few tokens each (same pages, consecutive starts). All keys and values of
                # a layer are in the cache before its attention begins, so a piece sees the pieces before it.
                step = self._inputs(self._pieces_for_fused(entries) or entries)
                if self.fused.takes(step):
                    self.stats["fused_steps"] += 1
                    hidden = self.fused.run(step, self.cache.page_size)
                    return self._decode_logits(hidden)
                return self._general_step(entries, step=step)      # a short prompt: too many rows per kv head
        if self.graph_max_batch and len(entries) <= self.graph_max_batch and \
                all(len(e.tokens) == 1 and e.want == [0] for e in entries):
            return self._graph_step(entries)
        return self._general_step(entries)

    def _pieces_for_fused(self, entries: list[StepEntry]) -> list[StepEntry] | None:
        """The entries with every run of tokens cut to what one attention unit of the whole-step kernel takes
        (16 rows of (token, head in group) per kv head), or None where that cannot be done (wanted places out
        of order, more than 16 pieces)."""
        rows = 16 // (self.fused.nh // self.fused.nkv)
        if rows < 1 or all(len(e.tokens) <= rows for e in entries):
            return None
        pieces = []
        for e in entries:
            if list(e.want) != sorted(e.want):
                return None
            for a in range(0, len(e.tokens), rows):
                b = min(a + rows, len(e.tokens))
                pieces.append(StepEntry(e.handle, e.tokens[a:b], e.start + a, [w - a for w in e.want if a <= w < b]))
        return pieces if len(pieces) <= fused.MAX_TOKENS else None

    def _inputs(self, entries: list[StepEntry]) -> StepInputs:
        """The step's batch on the device (one packed buffer, one copy)."""
        step = build_step_inputs(entries, self.cache, self.device, self.providers, workspace=self.workspace)
        self.stats["h2d_bytes"] = batch_mod.last_h2d_bytes
        return step

    def _general_step(self, entries: list[StepEntry], token_src: torch.Tensor | None = None,
                      token_rows: list[int] | None = None, step: StepInputs | None = None) -> torch.Tensor:
        """Any step, through the step program where the model has one, else through the parts' forward
        methods. With ``token_src`` (int32, on the device) the entries bring one token each and entry i's is
        token_src[token_rows[i]], gathered into the step's input buffer behind its copy."""
        if step is None:
            step = self._inputs(entries)
        if token_src is not None:
            rows = torch.as_tensor(token_rows, dtype=torch.int64).pin_memory().to(self.device, non_blocking=True)
            torch.index_select(token_src, 0, rows, out=step.token_ids)
        prog = self._step_program(step.n_tokens)
        if prog is not None and prog.takes(step, self._program_min_tokens):
            self.stats["program_steps"] += 1
            step.logits_out = torch.empty((step.n_want, self.model.spec.vocab_size), dtype=torch.float32,
                                          device=self.device)
            prog.run(step)
            logits = step.logits_out
        else:
            logits = self.model.forward(step, self.layer_caches)
        # A tcgen05 block that gave up on a wait must not pass silently: after steps with prompt portions (the
        # only ones that launch such kernels) the error word travels to the host behind the step, and the next
        # step (or whoever has synchronised: trace replay, drain) looks at it. Nothing waits here: a prompt cut
        # into portions keeps the host one step ahead of the GPU.
        if self.model.dtype == torch.bfloat16 and (step.max_q_len > 1 or ops.tc_gemm_enabled()):
            ops.tc_post(self.device)
        return logits

    def _decode_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        """Logits of a whole-step decode: hidden [T <= 16, H] times the output matrix."""
        if self._packed_output is not None and ops.lm_head_ok(hidden.shape[0], hidden.shape[1]):
            return ops.lm_head(hidden, self._packed_output, self.model.spec.vocab_size, error=self.fused.error)
        return ops.linear(hidden, self.model.output_weight, out_dtype=torch.float32)

    def _fused_takes_decode(self, entries: list[StepEntry]) -> bool:
        """Whether a decode step of these requests goes to the whole-step kernel. Beside decode graphs it does not
        where four or more requests hold very long contexts: the kernel's attention phase copies keys with
        16-byte loads by a unit's own warps (2.2 TB/s at best), the graph's attention kernel with tensor-map
        copies (8 requests of 16,000 keys, 0.5B sizes: 1.52 ms a step in the kernel, 1.34 in the graph; they
        meet at 8 x 8,000 keys; one to two requests stay faster in the kernel up to 32,000 keys and beyond)."""
        n = len(entries)
        if self.fused is None or not 0 < n <= self._fused_decode_limit:
            return False
        if self.graph_max_batch >= n >= 4 and self._fused_decode_limit < self.fused.max_tokens:
            return sum(e.start + 1 for e in entries) <= FUSED_DECODE_MAX_KEYS_BESIDE_GRAPHS
        return True

    def takes_greedy_steps(self, n_entries: int, entries: list[StepEntry] | None = None) -> bool:
        """Whether ``step_greedy`` takes a decode step of this many requests (of these requests, when given)."""
        if not (self.fused is not None and self._packed_output is not None and 0 < n_entries <= self._fused_decode_limit
                and ops.lm_head_ok(n_entries, self.model.spec.hidden_size)):
            return False
        return entries is None or self._fused_takes_decode(entries)

    @torch.inference_mode()
    def step_greedy(self, entries: list[StepEntry], out: torch.Tensor, token_src: torch.Tensor | None = None,
                    token_rows: list[int] | None = None) -> None:
        """A decode step (one token per entry) of which only each entry's most likely next token is wanted:
        out[:n] (int32, on the device) receives the arg-max of entry i's logits, the lowest index on ties, and no
        logits are written. With ``token_src`` the entries' tokens come from the device as in ``step_fed``. For
        steps the whole-step kernel takes (``takes_greedy_steps``)."""
        n = len(entries)
        if not self.takes_greedy_steps(n, entries) or any(len(e.tokens) != 1 for e in entries):
            raise RuntimeError("this step cannot have its arg-max taken in the output matrix's epilogue")
        for e in entries:
            if e.start + 1 > self.max_model_len:
                raise ValueError(f"a request would reach {e.start + 1} tokens; max_model_len is {self.max_model_len}")
        self.stats["steps"] += 1
        self.stats["tokens"] += n
        self.stats["fused_steps"] += 1
        ops.tc_poll(self.device)
        self.fused.check()
        hidden = self.fused.run_decode(entries, self.cache.page_size, token_src=token_src, token_rows=token_rows)
        self.stats["h2d_bytes"] = self.fused.h2d_bytes
        ops.lm_head_argmax(hidden, self._packed_output, self.model.spec.vocab_size, out, error=self.fused.error)

    def _step_program(self, n_tokens: int):
        """The model's step program with room for ``n_tokens`` (built on first need, rebuilt with a larger
        workspace when a step outgrows it), or None where there is none."""
        if self._no_program or n_tokens < self._program_min_tokens or ops.tc_gemm_enabled():
            return None      # (with every prompt product on the tcgen05 kernels the parts' forward methods run)
        if self._program is None or self._program.capacity < n_tokens:
            capacity = max(256, 1 << (n_tokens - 1).bit_length())
            self._program = self.model.program(self.layer_caches, capacity)
            if self._program is None:
                self._no_program = True
        return self._program

    @property
    def feeds_tokens_on_device(self) -> bool:
        """Whether some decode steps can take their token ids from the device (``step_fed``)."""
        return self.fused is not None or self.graph_max_batch > 0 or self._step_program(program_mod.MIN_TOKENS) is not None

    def can_feed_tokens_on_device(self, n_entries: int) -> bool:
        """Whether ``step_fed`` takes a decode step of this many requests: the whole-step kernel reads the ids
        itself, a captured graph has them gathered into its static input buffer."""
        if self.fused is not None and 0 < n_entries <= self._fused_decode_limit:
            return True
        if 0 < n_entries <= self.graph_max_batch:
            return True
        return n_entries >= self._program_min_tokens and self._step_program(n_entries) is not None

    @torch.inference_mode()
    def step_fed(self, entries: list[StepEntry], token_src: torch.Tensor, token_rows: list[int]) -> torch.Tensor:
        """A decode step (one token per entry, logits wanted for each) whose token ids are not known on the
        host yet: entry i continues with token_src[token_rows[i]], an int32 device tensor the previous step's
        sampling wrote. Everything else (positions, pages) comes from the entries as usual."""
        if not self.can_feed_tokens_on_device(len(entries)):
            raise RuntimeError("this step cannot take its tokens from the device")
        for e in entries:
            if e.start + 1 > self.max_model_len:
                raise ValueError(f"a request would reach {e.start + 1} tokens; max_model_len is {self.max_model_len}")
        self.stats["steps"] += 1
        self.stats["tokens"] += len(entries)
        if not self._fused_takes_decode(entries):
            if len(entries) <= self.graph_max_batch:
                return self._graph_step(entries, token_src, token_rows)
            return self._general_step(entries, token_src, token_rows)
        self.fused.check()
        self.stats["fused_steps"] += 1
        hidden = self.fused.run_decode(entries, self.cache.page_size, token_src=token_src, token_rows=token_rows)
        self.stats["h2d_bytes"] = self.fused.h2d_bytes
        return self._decode_logits(hidden)

    # --- decode graphs --------------------------------------------------------------------------

    def _graph_sizes(self) -> list[int]:
        """The batch sizes decode graphs are captured for."""
        if self.fused is not None:
            return [self.graph_max_batch]
        return [b for b in GRAPH_BATCH_SIZES if b < self.graph_max_batch] + [self.graph_max_batch]

    @torch.inference_mode()
    def capture_decode_graphs(self) -> int:
        """Capture every decode graph now instead of at the first step that needs it (a capture takes tens of
        milliseconds, which a serving loop would otherwise pay in the middle of its requests; the reference captures
        at start-up too, src/infer/engine/cuda_graphs.py:45-80). Returns how many graphs there are."""
        if not self.graph_max_batch:
            return 0
        for bucket in sorted(self._graph_sizes(), reverse=True):        # the largest first: the others share its buffers
            if self.fused is not None and bucket <= self._fused_decode_limit:
                continue
            if bucket not in self._graphs:
                self._graphs[bucket] = _DecodeGraph(self, bucket)
        return len(self._graphs)

    def _graph_step(self, entries: list[StepEntry], token_src: torch.Tensor | None = None,
                    token_rows: list[int] | None = None) -> torch.Tensor:
        n = len(entries)
        if self.fused is not None:
            # Steps of up to 16 tokens take the whole-step kernel, so graphs serve 17 and more requests: ONE graph of
            # the largest batch for all of them. Padding costs little at these sizes, and a second captured graph
            # costs more: once a process has captured library products twice, the kernels of every captured
            # graph stop overlapping with the library kernels in front of them (measured on B200, CUDA 12.9: the
            # same graph of 64 rows replays in 1.18 ms before and 1.29 ms after a graph of 32 rows is captured,
            # which is its time with programmatic dependent launch switched off; an eager step, or a captured
            # graph without library products, does not do that). With the one graph 17 / 32 / 64 requests take
            # 1.18 / 1.22 / 1.26 ms a step; with graphs of 32 and 64 rows they took 1.33 / 1.36 / 1.37.
            sizes = [self.graph_max_batch]
        else:
            sizes = [b for b in GRAPH_BATCH_SIZES if b < self.graph_max_batch] + [self.graph_max_batch]
        bucket = sizes[bisect.bisect_left(sizes, n)]
        if not self._graphs and bucket != sizes[-1]:
            # The largest batch is captured first: its warm-up makes every scratch buffer as large as any
            # graph will need, so the smaller graphs share those buffers instead of getting sets of their own.
            self._graphs[sizes[-1]] = _DecodeGraph(self, sizes[-1])
        g = self._graphs.get(bucket)
        if g is None:
            g = _DecodeGraph(self, bucket)
            self._graphs[bucket] = g
        self.stats["graph_steps"] += 1
        self.stats["h2d_bytes"] = g.lay.total * 4
        return g.run(entries, token_src, token_rows)


class _DecodeGraph:
    """One captured decode step for ``bucket`` requests with static metadata buffers."""

    def __init__(self, runner: ModelRunner, bucket: int):
        self.r, self.bucket = runner, bucket
        self._copied: torch.cuda.Event | None = None
        self._rows_host: torch.Tensor | None = None
        self._rows_dev: torch.Tensor | None = None
        cache, dev = runner.cache, runner.device
        ps = cache.page_size
        self.width = -(-runner.max_model_len // ps)
        B = bucket
        # The parts' own arrays, as they are for B single tokens at any context up to the limit. Those that
        # depend on where the requests stand are written again at every replay (same sizes, or it is an error).
        self.shape = StepShape(np.ones(B, dtype=np.int32), np.zeros(B, dtype=np.int32), ps, runner.max_model_len,
                               for_graph=True)
        metadata = collect_metadata(runner.providers, self.shape)
        self.refill = {k: p for k, p in runner.providers.items() if not metadata[k].constant_in_graph}
        self.host_meta = {k: dict(md.host) for k, md in metadata.items()}
        self.lay = Layout(B, B, B, [self.width] * cache.num_groups, extra_sizes(metadata))
        self.dev = torch.zeros(self.lay.total, dtype=torch.int32, device=dev)
        self.host = torch.zeros(self.lay.total, dtype=torch.int32, pin_memory=True)
        write_extra(self.host.numpy(), self.lay, metadata)
        self._fill([], first=True)
        self.dev.copy_(self.host)
        lay, d = self.lay, self.dev
        self.inputs = StepInputs(
            n_tokens=B, n_seqs=B, token_ids=d[lay.token_ids], positions=d[lay.positions],
            seq_of_token=d[lay.seq_of_token], cu_q=d[lay.cu_q], kv_before=d[lay.kv_before],
            state_slots=d[lay.state_slots],
            block_tables=[d[lay.block_tables[g]].view(B, self.width) for g in range(cache.num_groups)],
            slot_maps=[d[lay.slot_maps[g]] for g in range(cache.num_groups)],
            want_rows=d[lay.want_rows], n_want=B, max_q_len=1, max_kv_len=runner.max_model_len,
            meta=device_meta(d, lay, metadata), workspace=runner.workspace)
        # Warm up outside capture (library handles and workspaces), then capture.
        torch.cuda.synchronize(dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                runner.model.forward(self.inputs, runner.layer_caches)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        launched_before = lib.launch_count
        # No garbage collection while the stream is capturing: collecting an older engine's graphs (a process
        # that has built several engines) destroys CUDA objects, which is not permitted during a capture and
        # invalidates it.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph, pool=runner._graph_pool):
                self.logits = runner.model.forward(self.inputs, runner.layer_caches)
        finally:
            if gc_was_on:
                gc.enable()
        runner.kernels_per_graph[bucket] = lib.launch_count - launched_before   # this library's kernels per replay
        if runner._graph_pool is None:
            runner._graph_pool = self.graph.pool()
        runner.workspace.freeze()

    def _fill(self, entries: list[StepEntry], first: bool = False) -> None:
        lay, buf, B = self.lay, self.host.numpy(), self.bucket
        cache = self.r.cache
        ps, n = cache.page_size, len(entries)
        if first:
            buf[lay.seq_of_token] = np.arange(B, dtype=np.int32)
            buf[lay.cu_q] = np.arange(B + 1, dtype=np.int32)
            buf[lay.want_rows] = np.arange(B, dtype=np.int32)
        tok, pos, slot_state = buf[lay.token_ids], buf[lay.positions], buf[lay.state_slots]
        before = buf[lay.kv_before]
        tok[:] = 0
        pos[:] = 0
        before[:] = 0
        # Padded rows update the sink state slot, never a live request's.
        slot_state[:] = max(self.r.pools.state_sink, 0)
        for i, e in enumerate(entries):
            tok[i], pos[i], before[i] = e.tokens[0], e.start, e.start
            if e.handle.state_slot >= 0:
                slot_state[i] = e.handle.state_slot
        for g in range(cache.num_groups):
            sink = self.r.pools.sink[g]
            table = buf[lay.block_tables[g]].reshape(B, self.width)
            slots = buf[lay.slot_maps[g]]
            table[n:, :] = sink
            slots[n:] = sink * ps
            for i, e in enumerate(entries):
                row = e.handle.tables[g]
                k = min(len(row), self.width)
                table[i, :k] = row[:k]
                page = row[e.start // ps]
                if page < 0:
                    raise RuntimeError("a decoded token would be written into a page already given back")
                slots[i] = page * ps + e.start % ps
        if self.refill and not first:
            self.shape.starts[:] = 0
            self.shape.starts[:n] = [e.start for e in entries]
            metadata = collect_metadata(self.refill, self.shape)
            for key, md in metadata.items():
                if md.host != self.host_meta[key]:
                    raise RuntimeError(f"step metadata {key!r}: the numbers a graph captured ({self.host_meta[key]}) "
                                       f"differ at replay ({md.host})")
            write_extra(buf, lay, metadata)

    def run(self, entries: list[StepEntry], token_src: torch.Tensor | None = None,
            token_rows: list[int] | None = None) -> torch.Tensor:
        """Replay the step. With ``token_src`` (int32, on the device) entry i's token is
        token_src[token_rows[i]], gathered into the static input buffer behind the metadata copy: the host
        need not know the ids yet."""
        if self._copied is not None:
            self._copied.synchronize()       # the pinned buffers are about to be rewritten
        self._fill(entries)
        self.dev.copy_(self.host, non_blocking=True)
        if token_src is not None:
            n = len(entries)
            if self._rows_host is None:
                self._rows_host = torch.zeros(self.bucket, dtype=torch.int64, pin_memory=True)
                self._rows_dev = torch.zeros(self.bucket, dtype=torch.int64, device=self.dev.device)
            self._rows_host[:n] = torch.as_tensor(token_rows, dtype=torch.int64)
            self._rows_dev.copy_(self._rows_host, non_blocking=True)
            torch.index_select(token_src, 0, self._rows_dev[:n], out=self.dev[self.lay.token_ids][:n])
        if self._copied is None:
            self._copied = torch.cuda.Event()
        self._copied.record()
        self.graph.replay()
        return self.logits[:len(entries)]
