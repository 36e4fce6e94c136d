"""Plans every step: which requests run how many tokens, who is admitted, who gives pages back. Host only.

The policy is the reference scheduler's (src/infer/engine/scheduler.py:56-242), restated:

* first come, first served, no skipping: only the head of the queue is ever considered for admission;
* a step's tokens stay under ``max_num_batched_tokens`` (a prompt longer than the whole budget runs
  alone) and the running requests under ``max_num_seqs``;
* admission asks the cache manager OK / LATER / NEVER: LATER ends admission for this step, NEVER takes
  the request out with an error (``StepPlan.rejected``);
* without chunked prefill a step either admits whole prompts or decodes (``prefill_first``: admit
  whenever the head fits; ``decode_first``: decode while anything runs, admit after
  ``max_waiting_steps`` decode steps);
* with chunked prefill a step is mixed: every running request that is through its prompt decodes, then
  prompts in progress and after them new prompts get portions of what is left of the budget;
* when a decoding request needs a page and none is free, the request admitted LAST gives way (pages
  released, nothing cached any more, FRONT of the queue, recomputed from prompt and outputs when it is
  admitted again), repeated until the page is there; the request that asks is the last to go.

Here the plan is one flat list of (request, first token, count) items, prompt portions before single
decoded tokens, which is the layout of the step's batch; both modes are built from the same three
passes (decode, continue, admit). A request whose newest token is still on the device (a decode step in
flight) is not admitted until the host knows it, and one the engine already knows to end with the step in
flight is planned no further.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import AllocStatus, CacheManager
from ..config.engine_config import EngineConfig
from .request import Phase, Request


@dataclass
class PlanItem:
    req: Request
    start: int            # first position this step computes (= tokens the cache already holds)
    count: int
    decode: bool

    @property
    def samples(self) -> bool:
        """The item reaches the request's last known token: the step samples the next one."""
        return self.start + self.count == self.req.n_tokens


@dataclass
class StepPlan:
    items: list[PlanItem] = field(default_factory=list)
    evicted: list[Request] = field(default_factory=list)
    rejected: list[Request] = field(default_factory=list)        # would not fit an empty pool

    @property
    def empty(self) -> bool:
        return not self.items

    @property
    def prompt_items(self) -> list[PlanItem]:
        return [i for i in self.items if not i.decode]

    @property
    def decode_items(self) -> list[PlanItem]:
        return [i for i in self.items if i.decode]

    @property
    def n_tokens(self) -> int:
        return sum(i.count for i in self.items)

    @property
    def n_prompt_tokens(self) -> int:
        return sum(i.count for i in self.items if not i.decode)


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache: CacheManager):
        self.cfg, self.cache = cfg, cache
        self.queue: deque[Request] = deque()      # arrival order; evicted requests re-enter at the front
        self.running: list[Request] = []
        self.evictions = 0
        self._next_seat = 0
        self._decodes_since_admission = 0         # decode_first: decode steps taken while the queue waited

    # --- requests come and go -------------------------------------------------------------------

    def submit(self, req: Request) -> None:
        req.phase = Phase.QUEUED
        self.queue.append(req)

    @property
    def busy(self) -> bool:
        return bool(self.queue) or bool(self.running)

    def retire(self, req: Request, reason: str) -> None:
        """The request is over (wherever it stands): what it holds goes back to the cache manager."""
        if req.done:
            return
        if req.phase is Phase.RUNNING:
            self.running.remove(req)
            self.cache.free(req.cache)
        elif req in self.queue:
            self.queue.remove(req)
        req.phase, req.finish_reason = Phase.DONE, reason

    # --- the plan -------------------------------------------------------------------------------

    def plan_step(self) -> StepPlan:
        plan = StepPlan()
        budget = self.cfg.max_num_batched_tokens
        if self.cfg.enable_chunked_prefill:
            decodes, midway = self._decode_pass(plan)
            budget -= len(decodes)
            portions = self._continue_pass(midway, budget)
            budget -= sum(p.count for p in portions)
            portions += self._admit_pass(plan, budget, whole_prompts=False)
            plan.items = portions + decodes
            return plan
        if self._admission_turn():
            plan.items = self._admit_pass(plan, budget, whole_prompts=True)
            if plan.items:
                self._decodes_since_admission = 0
                return plan
        plan.items, _ = self._decode_pass(plan)
        if self.queue:
            self._decodes_since_admission += 1
        return plan

    def _admission_turn(self) -> bool:
        """Whole-prompt mode: is this step one that admits?"""
        if not self.queue:
            return False
        if self.cfg.policy == "prefill_first" or not self.running:
            return True
        return self._decodes_since_admission >= self.cfg.max_waiting_steps

    # --- the three passes -----------------------------------------------------------------------

    def _decode_pass(self, plan: StepPlan) -> tuple[list[PlanItem], list[Request]]:
        """Running requests in admission order. One that is through its prompt decodes one token, after its
        page is secured; one still inside its prompt is set aside for the continue pass. Returns both."""
        order = deque(sorted((r for r in self.running if not r.closing), key=lambda r: r.seat))
        decodes: list[PlanItem] = []
        midway: list[Request] = []
        while order:
            req = order.popleft()
            if req.backlog > 1:
                midway.append(req)
            elif self._secure_page(req, order, plan):
                decodes.append(PlanItem(req, req.n_tokens - 1, 1, True))
        return decodes, midway

    def _secure_page(self, req: Request, younger: deque[Request], plan: StepPlan) -> bool:
        """Room for ``req``'s next token. While there is none, the youngest request this step has not
        looked at yet is evicted (it may be a prompt in progress; never one older than ``req``), and when
        no such request is left, ``req`` itself. False when ``req`` had to go."""
        while not self.cache.can_grow(req.cache, req.n_tokens):
            victim = younger.pop() if younger else req
            self._evict(victim, plan)
            if victim is req:
                return False
        self.cache.grow(req.cache, req.n_tokens)
        return True

    @staticmethod
    def _continue_pass(midway: list[Request], budget: int) -> list[PlanItem]:
        """Prompts in progress, oldest first, take what the budget still holds."""
        portions = []
        for req in midway:
            if budget <= 0:
                break
            n = min(req.backlog, budget)
            portions.append(PlanItem(req, req.cached_tokens, n, False))
            budget -= n
        return portions

    def _admit_pass(self, plan: StepPlan, budget: int, *, whole_prompts: bool) -> list[PlanItem]:
        """Admit from the head of the queue while the budget lasts. ``whole_prompts``: a prompt is never cut,
        one that does not fit what is left waits for the next step, and one longer than a whole step's budget
        gets a step to itself. Otherwise the last one admitted takes a portion. Pages for all of a request's
        tokens are taken at admission either way."""
        items: list[PlanItem] = []
        while budget > 0:
            req = self._admissible_head(plan)
            if req is None or (whole_prompts and items and req.n_tokens > budget):
                break
            self.queue.popleft()
            self._seat(req)
            n = req.backlog if whole_prompts else min(req.backlog, budget)
            items.append(PlanItem(req, req.cached_tokens, n, False))
            budget -= n
        return items

    def _admissible_head(self, plan: StepPlan) -> Request | None:
        """The head of the queue if it can be admitted now. Heads that can never fit are rejected on the way."""
        while self.queue and len(self.running) < self.cfg.max_num_seqs:
            head = self.queue[0]
            if head.awaits_token:          # evicted with a step in flight: its newest id is not on the host yet
                return None
            verdict = self.cache.admission_status(head.cache, head.tokens)
            if verdict is AllocStatus.OK:
                return head
            if verdict is AllocStatus.LATER:
                return None
            plan.rejected.append(self.queue.popleft())
        return None

    # --- state changes --------------------------------------------------------------------------

    def _seat(self, req: Request) -> None:
        req.cached_tokens = self.cache.allocate(req.cache, req.tokens)      # > 0 after a prefix hit
        req.phase, req.seat = Phase.RUNNING, self._next_seat
        self._next_seat += 1
        self.running.append(req)

    def _evict(self, req: Request, plan: StepPlan) -> None:
        self.running.remove(req)
        self.cache.free(req.cache)
        req.cached_tokens = 0
        req.phase = Phase.EVICTED
        req.evictions += 1
        self.evictions += 1
        self.queue.appendleft(req)
        plan.evicted.append(req)
