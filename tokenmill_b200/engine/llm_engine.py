"""The engine's Python entry point: ``LLMEngine(cfg).generate(prompts, params)``.

Same shape as the reference's LLMEngine (src/infer/engine/engine.py:87-281): synchronous
``add_request`` / ``abort_request`` / ``step`` / ``generate`` / ``has_unfinished``; every step
re-plans the batch, so new requests join at the next step and finished ones leave at once. One step
(engine.py:167-204): plan -> requests that can never fit finish with an error -> run the batch ->
count computed tokens and publish full pages -> append the sampled tokens -> stop checks -> outputs.
Prompts and outputs are token ids; the text side of the reference (tokenizer, HTTP) is not part of
this engine.

Decode steps the whole-step kernel takes are pipelined (``EngineConfig.async_decode``): the next step is
planned and launched, its token ids taken on the device from what the previous step's sampling wrote,
BEFORE the host reads the previous step's tokens; the host's own work per step (planning, metadata,
bookkeeping) then runs while the GPU is busy instead of between two launches. ``step()`` returns the
outputs of the step that was in flight, so a request's tokens arrive one call later than they were
computed; a request that turns out to have ended (end-of-sequence token) has one surplus token computed
and thrown away. Ends the engine can foresee (``max_tokens``, ``max_model_len``) cost nothing. Tokens,
stop reasons and the order of outputs are the same as in the synchronous loop.
"""

from __future__ import annotations

import logging
import random
import time

import torch

from ..cache.manager import CacheManager
from ..cache.pool import CachePools
from ..config.engine_config import EngineConfig
from ..kernels import ops
from ..parts.model import DecoderModel
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from ..weights.loader import load_model, resolve_dtype
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import PLACEHOLDER, RequestOutput, Sequence, Status

log = logging.getLogger("tokenmill_b200.engine")


class RequestRejected(ValueError):
    """The request can never be served (empty prompt, prompt too long, duplicate id)."""


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def kv_budget_bytes(cfg: EngineConfig, model: DecoderModel) -> int:
    """Bytes for the cache pool: ``kv_cache_mb`` if given, else what is left of
    ``gpu_memory_utilization`` x device memory after what is already allocated (the weights), what the
    runner will allocate for good (the whole-step kernel's packed copy of the layer matrices), and an
    allowance for the largest step's activations and logits (src/infer/engine/engine.py:44-61; the reference
    measures the activation peak with a dummy forward, here the parts are asked: ``activation_bytes``)."""
    if cfg.kv_cache_mb is not None:
        return int(cfg.kv_cache_mb * 2 ** 20)
    from ..kernels import fused

    dev = model.device
    total = torch.cuda.get_device_properties(dev).total_memory
    used = torch.cuda.memory_allocated(dev)
    act = 2 * model.activation_bytes(cfg.max_num_batched_tokens)          # twice: temporaries of the library products
    logits = 3 * min(cfg.max_num_seqs, cfg.max_num_batched_tokens) * model.spec.vocab_size * 4
    runner = fused.persistent_bytes(model)
    budget = int(total * cfg.gpu_memory_utilization) - used - runner - act - logits - (512 << 20)
    if budget <= 0:
        raise RuntimeError("no memory left for the cache; lower --max-batched-tokens or raise "
                           "--gpu-memory-utilization")
    return budget


class _InFlight:
    """A decode step that has been launched and whose tokens the host has not read."""

    __slots__ = ("seqs", "index", "pending", "row_of", "void", "plan", "t0")

    def __init__(self, seqs, index, pending, plan, t0):
        self.seqs, self.index, self.pending, self.plan, self.t0 = seqs, index, pending, plan, t0
        self.row_of = {id(s): i for i, s in enumerate(seqs)}
        self.void: set[int] = set()        # rows whose request ended with the step before: token thrown away


class LLMEngine:
    def __init__(self, cfg: EngineConfig, model: DecoderModel | None = None):
        self.cfg = cfg
        if model is None:
            if not cfg.model:
                raise ValueError("EngineConfig.model must name a model folder")
            model = load_model(cfg.model, resolve_dtype(cfg.dtype), torch.device(cfg.device),
                               max_positions=cfg.max_model_len)
        self.model = model
        self.device, self.dtype = model.device, model.dtype
        if cfg.max_model_len > model.max_positions():
            raise ValueError(f"max_model_len is {cfg.max_model_len}, but the model serves {model.max_positions()} "
                             f"positions (max_position_embeddings): lower --max-model-len")
        self.eos_ids = set(model.spec.eos_token_ids)
        layout = model.cache_layout()
        per_token = layout.bytes_per_token(_element_size(self.dtype))
        if per_token > 0:
            num_pages = kv_budget_bytes(cfg, model) // (per_token * cfg.block_size)
            num_pages = min(num_pages, cfg.max_num_seqs * -(-cfg.max_model_len // cfg.block_size))
        else:
            num_pages = cfg.max_num_seqs
        if num_pages < 2:
            raise RuntimeError("cache budget too small for the paged pool")
        n_groups = len(layout.groups)
        n_state = cfg.max_num_seqs if layout.entry_state else 0
        self.cache = CacheManager([num_pages] * n_groups, cfg.block_size, layout.windows, cfg.watermark,
                                  cfg.enable_prefix_caching, num_state_slots=n_state)
        self.pools = CachePools(layout, [num_pages] * n_groups, cfg.block_size, self.dtype, self.device,
                                num_state_slots=n_state, sink_page=cfg.cuda_graphs,
                                run_order_cache_of=[e.cache_of for e in model.spec.run_order])
        self.runner = ModelRunner(model, self.cache, self.pools, max_model_len=cfg.max_model_len,
                                  cuda_graphs=cfg.cuda_graphs, cuda_graph_max_batch=cfg.cuda_graph_max_batch,
                                  max_num_seqs=cfg.max_num_seqs)
        self.scheduler = Scheduler(cfg, self.cache)
        self.sampler = Sampler(self.device)
        self.seqs: dict[str, Sequence] = {}
        self._inflight: _InFlight | None = None
        self._rng = random.Random(cfg.seed)
        self._offline_counter = 0
        self.stats = {"steps": 0, "peak_running": 0, "prefill_steps": 0, "decode_steps": 0,
                      "generated_tokens": 0, "busy_time": 0.0}
        log.info("engine ready: %d pages of %d tokens in %d group(s) (%.0f MiB), dtype %s, device %s", num_pages,
                 cfg.block_size, n_groups, self.pools.nbytes / 2 ** 20, self.dtype, self.device)

    # --- requests -------------------------------------------------------------------------------

    def add_request(self, request_id: str, prompt_ids: list[int], params: SamplingParams,
                    arrival_time: float | None = None) -> Sequence:
        if not prompt_ids:
            raise RequestRejected("prompt is empty")
        if len(prompt_ids) >= self.cfg.max_model_len:
            raise RequestRejected(f"prompt has {len(prompt_ids)} tokens; max_model_len is {self.cfg.max_model_len}")
        if request_id in self.seqs:
            raise RequestRejected(f"duplicate request id {request_id}")
        vocab = self.model.spec.vocab_size
        if any(not (0 <= t < vocab) for t in prompt_ids):
            raise RequestRejected(f"a prompt token id lies outside the vocabulary of {vocab}")
        seq = Sequence(request_id, list(prompt_ids), params, self.cache.new_handle(),
                       arrival_time=time.monotonic() if arrival_time is None else arrival_time)
        if not params.greedy:
            seq.sample_seed = params.seed if params.seed is not None else self._rng.getrandbits(62)
        self.seqs[request_id] = seq
        self.scheduler.add(seq)
        return seq

    def abort_request(self, request_id: str, reason: str = "abort") -> RequestOutput | None:
        seq = self.seqs.pop(request_id, None)
        if seq is None:
            return None
        while seq.output_ids and seq.output_ids[-1] == PLACEHOLDER:      # tokens of steps still in flight
            seq.output_ids.pop()
        seq.finishing = False
        self.scheduler.finish(seq, reason)
        seq.finish_time = time.monotonic()
        return self._output(seq, [])

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    def _pipelining(self) -> bool:
        """Decode steps may stay in flight: the runner can take token ids from the device (the whole-step
        kernel reads them, a captured graph has them gathered), and nothing in the configuration needs a
        step's token ids on the host at once. With chunked prompts a plan that holds a prompt portion is simply
        not launched ahead: it runs once the step in flight has been read. With prefix caching a page is
        published when the step that filled it has been read (its ids are known then), and a preempted request
        whose last token is still on the device waits for it before it is admitted again."""
        return self.cfg.async_decode and self.runner.feeds_tokens_on_device

    # --- one step -------------------------------------------------------------------------------

    def step(self) -> list[RequestOutput]:
        if self._inflight is not None:
            return self._step_behind()
        outputs: list[RequestOutput] = []
        t0 = time.perf_counter()
        plan = self.scheduler.schedule()
        outputs += self._drop_ignored(plan)
        if plan.empty:
            return outputs
        if self._pipelining() and self._is_plain_decode(plan):
            self._inflight = self._launch(plan, None, t0)      # its outputs come with the next call
            return outputs
        return outputs + self._run(plan, t0)

    def _drop_ignored(self, plan) -> list[RequestOutput]:
        outputs = []
        for seq in plan.ignored:
            self.seqs.pop(seq.id, None)
            self.scheduler.finish(seq, "length")
            seq.finish_time = time.monotonic()
            outputs.append(self._output(seq, [], error=None if seq.output_ids else
                                        "prompt does not fit in the KV cache"))
        return outputs

    # --- decode steps in flight -----------------------------------------------------------------

    def _is_plain_decode(self, plan) -> bool:
        return (not plan.prefill_items and self.runner.can_feed_tokens_on_device(len(plan.items))
                and all(it.samples and it.num_tokens == 1 for it in plan.items))

    def _launch(self, plan, prev: _InFlight | None, t0: float) -> _InFlight:
        """Launch the plan's decode step without waiting for anything. With ``prev`` (the step still in
        flight) a request's token is what that step's sampling left on the device."""
        seqs = [it.seq for it in plan.items]
        entries, rows = [], []
        for it in plan.items:
            seq = it.seq
            if prev is None:
                entries.append(StepEntry(seq.cache, [seq.all_token_ids[it.start]], it.start, [0]))
            else:
                entries.append(StepEntry(seq.cache, [0], it.start, [0]))
                rows.append(prev.row_of[id(seq)])
        if prev is None:
            logits = self.runner.step(entries)
        else:
            logits = self.runner.step_fed(entries, prev.pending.dev, rows)
        pending = self.sampler.launch(logits, [s.params for s in seqs], [s.sample_seed for s in seqs],
                                      [s.num_draws for s in seqs])
        index = []
        for it in plan.items:
            seq = it.seq
            seq.num_computed_tokens = it.start + 1
            self.cache.release_behind_window(seq.cache, seq.num_computed_tokens)
            if not seq.params.greedy:
                seq.num_draws += 1
            index.append(len(seq.output_ids))
            seq.output_ids.append(PLACEHOLDER)
        return _InFlight(seqs, index, pending, plan, t0)

    def _step_behind(self) -> list[RequestOutput]:
        """One call while a decode step is in flight: plan and launch the step after it if nothing stands
        in the way, then read the tokens of the step in flight and do its bookkeeping."""
        cur = self._inflight
        outputs: list[RequestOutput] = []
        nxt, leftover = None, None
        t0 = time.perf_counter()
        if self._pipelining():
            for seq, at in zip(cur.seqs, cur.index):
                # Ends the host can foresee: the step in flight brings the request's last token.
                if not seq.is_finished and (at + 1 >= seq.params.max_tokens or
                                            seq.num_prompt_tokens + at + 1 >= self.cfg.max_model_len):
                    seq.finishing = True
            plan = self.scheduler.schedule()
            outputs += self._drop_ignored(plan)
            if not plan.empty:
                if self._is_plain_decode(plan) and all(id(it.seq) in cur.row_of for it in plan.items):
                    nxt = self._launch(plan, cur, t0)
                else:
                    leftover = plan                # planned (pages grown) but not launched: run it below
        outputs += self._collect(cur, nxt)
        self._inflight = nxt
        if leftover is not None:
            outputs += self._run(leftover, t0)
        return outputs

    def _collect(self, cur: _InFlight, nxt: _InFlight | None) -> list[RequestOutput]:
        tokens = self.sampler.collect(cur.pending)
        now = time.monotonic()
        outputs = []
        n_new = 0
        for row, (seq, at) in enumerate(zip(cur.seqs, cur.index)):
            if row in cur.void or seq.is_finished:        # ended a step earlier, or aborted meanwhile
                continue
            tok = tokens[row]
            seq.output_ids[at] = tok
            n_new += 1
            if seq.status == Status.RUNNING:              # (a preempted request holds no pages to publish)
                self.cache.register_computed(seq.cache, seq.prompt_ids + seq.output_ids[:at + 1],
                                             seq.num_prompt_tokens + at)
            if seq.first_token_time is None:
                seq.first_token_time = now
            n_out = at + 1
            reason = None
            if tok in self.eos_ids and not seq.params.ignore_eos:
                reason = "stop"
            elif n_out >= seq.params.max_tokens or seq.num_prompt_tokens + n_out >= self.cfg.max_model_len:
                reason = "length"
            if reason:
                del seq.output_ids[n_out:]                # the place kept for the step after this one
                if nxt is not None and id(seq) in nxt.row_of:
                    nxt.void.add(nxt.row_of[id(seq)])
                seq.finishing = False
                self.scheduler.finish(seq, reason)
                seq.finish_time = now
                self.seqs.pop(seq.id, None)
            outputs.append(self._output(seq, [tok], num_output_tokens=n_out))
        self._record_step(cur.plan, time.perf_counter() - cur.t0, n_new)
        return outputs

    def drain(self) -> list[RequestOutput]:
        """Read the step in flight, if any, without launching another (e.g. before the engine is dropped)."""
        if self._inflight is None:
            ops.tc_check(self.runner.device)     # (errors of prompt steps that nobody has looked at yet)
            return []
        cur, self._inflight = self._inflight, None
        outputs = self._collect(cur, None)
        ops.tc_check(self.runner.device)
        return outputs

    # --- one step, start to end -----------------------------------------------------------------

    def _run(self, plan, t0: float) -> list[RequestOutput]:
        outputs: list[RequestOutput] = []
        entries, sampled = [], []
        items = [it for it in plan.items if not it.seq.is_finished]    # (ended since the plan was made)
        if not items:
            return outputs
        for item in items:
            seq = item.seq
            tokens = seq.all_token_ids[item.start:item.start + item.num_tokens]
            want = [item.num_tokens - 1] if item.samples else []
            entries.append(StepEntry(seq.cache, tokens, item.start, want))
            if item.samples:
                sampled.append(seq)
        logits = self.runner.step(entries)
        tokens = self.sampler.sample(logits, [s.params for s in sampled], [s.sample_seed for s in sampled],
                                     [s.num_draws for s in sampled]) if sampled else []
        now = time.monotonic()
        for item in items:
            seq = item.seq
            seq.num_computed_tokens = item.start + item.num_tokens
            self.cache.register_computed(seq.cache, seq.all_token_ids, seq.num_computed_tokens)
            self.cache.release_behind_window(seq.cache, seq.num_computed_tokens)
        for seq, tok in zip(sampled, tokens):
            seq.output_ids.append(tok)
            if not seq.params.greedy:
                seq.num_draws += 1
            if seq.first_token_time is None:
                seq.first_token_time = now
            reason = self._stop_reason(seq, tok)
            if reason:
                self.scheduler.finish(seq, reason)
                seq.finish_time = now
                self.seqs.pop(seq.id, None)
            outputs.append(self._output(seq, [tok]))
        self._record_step(plan, time.perf_counter() - t0, len(sampled))
        return outputs

    def _stop_reason(self, seq: Sequence, tok: int) -> str | None:
        if tok in self.eos_ids and not seq.params.ignore_eos:
            return "stop"
        if seq.num_output_tokens >= seq.params.max_tokens or seq.length >= self.cfg.max_model_len:
            return "length"
        return None

    def _output(self, seq: Sequence, new_tokens: list[int], error: str | None = None,
                num_output_tokens: int | None = None) -> RequestOutput:
        n_out = seq.num_output_tokens if num_output_tokens is None else num_output_tokens
        return RequestOutput(seq.id, new_tokens, seq.is_finished, seq.finish_reason, seq.num_prompt_tokens,
                             n_out, seq.arrival_time, seq.first_token_time, seq.finish_time,
                             seq.num_preemptions, error)

    def _record_step(self, plan, step_time: float, n_generated: int) -> None:
        s = self.stats
        s["steps"] += 1
        s["busy_time"] += step_time
        s["prefill_steps" if plan.prefill_items else "decode_steps"] += 1
        s["generated_tokens"] += n_generated
        s["peak_running"] = max(s["peak_running"], len(self.scheduler.running))
        if self.cfg.debug_steps:
            log.info("step=%d batch=%d prefill_tokens=%d decode_tokens=%d step_ms=%.2f kv_usage=%.3f waiting=%d "
                     "running=%d preempted=%d", s["steps"], len(plan.items), plan.num_prefill_tokens,
                     len(plan.decode_items), step_time * 1e3, self.cache.usage(), len(self.scheduler.waiting),
                     len(self.scheduler.running), len(plan.preempted))

    # --- offline helper -------------------------------------------------------------------------

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams]) -> list[list[int]]:
        """Run every prompt to completion through the step loop; output token ids in prompt order."""
        plist = params if isinstance(params, list) else [params] * len(prompts)
        seqs = []
        for p, sp in zip(prompts, plist):
            self._offline_counter += 1
            seqs.append(self.add_request(f"offline-{self._offline_counter}", p, sp))
        while self.has_unfinished():
            self.step()
        ops.tc_check(self.runner.device)         # a prompt step's kernel that gave up must not pass silently
        return [s.output_ids for s in seqs]
