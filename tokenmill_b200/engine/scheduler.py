"""Decides, every step, which requests run how many tokens, and who is preempted. Host only.

The decisions are the reference scheduler's (src/infer/engine/scheduler.py:56-242):

* first come, first served, no skipping: only the head of the waiting queue is considered;
* a step's tokens stay under ``max_num_batched_tokens`` (a prompt longer than the whole budget runs
  alone) and its requests under ``max_num_seqs``;
* admission asks the cache manager OK / LATER / NEVER: LATER stops admission for this step, NEVER
  takes the request out with an error ("ignored");
* without chunked prefill a step is either a prefill step or a decode step (``prefill_first``:
  prefill whenever something can be admitted; ``decode_first``: decode while anything runs, prefill
  after ``max_waiting_steps`` decode steps);
* with chunked prefill a step is mixed: every running request decodes, then prompts already in
  progress and then new prompts get portions from what is left of the budget;
* when a decoding request needs a page and none is free, the request admitted LAST is preempted
  (its pages are released, its computed count reset, and it goes to the FRONT of the waiting queue to
  be recomputed: prompt and generated tokens), repeated until the page is there; the request asking
  is the last to go.

The plan is a flat list of (request, first token, number of tokens) items, prompt portions first and
single decoded tokens after them, which is the layout of the step's batch.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import AllocStatus, CacheManager
from ..config.engine_config import EngineConfig
from .sequence import Sequence, Status


@dataclass
class PlanItem:
    seq: Sequence
    start: int            # first position this step computes (= tokens already in the cache)
    num_tokens: int
    is_decode: bool

    @property
    def samples(self) -> bool:
        """True when the item reaches the request's last known token, so a token is sampled."""
        return self.start + self.num_tokens == self.seq.length


@dataclass
class StepPlan:
    items: list[PlanItem] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)
    ignored: list[Sequence] = field(default_factory=list)       # can never fit in the pool

    @property
    def empty(self) -> bool:
        return not self.items

    @property
    def prefill_items(self) -> list[PlanItem]:
        return [i for i in self.items if not i.is_decode]

    @property
    def decode_items(self) -> list[PlanItem]:
        return [i for i in self.items if i.is_decode]

    @property
    def num_batched_tokens(self) -> int:
        return sum(i.num_tokens for i in self.items)

    @property
    def num_prefill_tokens(self) -> int:
        return sum(i.num_tokens for i in self.items if not i.is_decode)


class Scheduler:
    def __init__(self, cfg: EngineConfig, cache: CacheManager):
        self.cfg = cfg
        self.cache = cache
        self.waiting: deque[Sequence] = deque()      # FCFS; preempted requests return to the front
        self.running: list[Sequence] = []            # admission order, oldest first
        self.num_preemptions = 0
        self._admit_counter = 0
        self._decode_steps_since_prefill = 0

    # --- queues ---------------------------------------------------------------------------------

    def add(self, seq: Sequence) -> None:
        seq.status = Status.WAITING
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def finish(self, seq: Sequence, reason: str) -> None:
        """Release everything the request holds. Safe for a request in any queue."""
        if seq.status == Status.FINISHED:
            return
        if seq in self.running:
            self.running.remove(seq)
            self.cache.free(seq.cache)
        else:
            try:
                self.waiting.remove(seq)
            except ValueError:
                pass
        seq.status = Status.FINISHED
        seq.finish_reason = reason

    # --- one step's plan ------------------------------------------------------------------------

    def schedule(self) -> StepPlan:
        plan = StepPlan()
        if self.cfg.enable_chunked_prefill:
            self._schedule_mixed(plan)
            return plan
        if self._should_prefill():
            self._schedule_prefills(plan)
            if plan.items:
                self._decode_steps_since_prefill = 0
                return plan
        self._schedule_decodes(plan, self._oldest_first())
        if self.waiting:
            self._decode_steps_since_prefill += 1
        return plan

    def _should_prefill(self) -> bool:
        if not self.waiting:
            return False
        if self.cfg.policy == "prefill_first" or not self.running:
            return True
        return self._decode_steps_since_prefill >= self.cfg.max_waiting_steps

    def _oldest_first(self) -> list[Sequence]:
        """Running requests, oldest admission first; without those the engine already knows to end with a
        step that is still in flight."""
        return sorted((s for s in self.running if not s.finishing), key=lambda s: s.admit_order)

    def _admit(self, seq: Sequence) -> None:
        tokens = seq.all_token_ids
        seq.num_computed_tokens = self.cache.allocate(seq.cache, tokens)
        seq.status = Status.RUNNING
        seq.admit_order = self._admit_counter
        self._admit_counter += 1
        self.running.append(seq)

    def _head_status(self, plan: StepPlan) -> Sequence | None:
        """The head of the waiting queue if it can be admitted now; drops heads that never fit."""
        while self.waiting and len(self.running) < self.cfg.max_num_seqs:
            seq = self.waiting[0]
            if seq.awaits_token:          # preempted with a step in flight: its last id is not on the host yet
                return None
            status = self.cache.admission_status(seq.cache, seq.all_token_ids)
            if status == AllocStatus.NEVER:
                self.waiting.popleft()
                plan.ignored.append(seq)
                continue
            return seq if status == AllocStatus.OK else None
        return None

    def _schedule_prefills(self, plan: StepPlan) -> None:
        budget = self.cfg.max_num_batched_tokens
        while True:
            seq = self._head_status(plan)
            if seq is None:
                break
            # A prompt that does not fit the budget waits, except that one larger than the whole
            # budget runs alone.
            if seq.length > budget and plan.items:
                break
            self.waiting.popleft()
            self._admit(seq)
            n = seq.num_new_tokens
            plan.items.append(PlanItem(seq, seq.num_computed_tokens, n, False))
            budget -= n
            if budget <= 0:
                break

    def _schedule_decodes(self, plan: StepPlan, queue: list[Sequence]) -> list[PlanItem]:
        """Every request of ``queue`` (oldest first) that is ready decodes one token; growth that
        finds no free page preempts from the newest end. Returns the decode items in order."""
        items: list[PlanItem] = []
        queue = list(queue)
        while queue:
            seq = queue.pop(0)
            preempted_self = False
            while not self.cache.can_grow(seq.cache, seq.length):
                victim = queue.pop() if queue else seq
                self._preempt(victim, plan)
                if victim is seq:
                    preempted_self = True
                    break
            if preempted_self:
                continue
            self.cache.grow(seq.cache, seq.length)
            items.append(PlanItem(seq, seq.length - 1, 1, True))
        plan.items += items
        return items

    def _schedule_mixed(self, plan: StepPlan) -> None:
        budget = self.cfg.max_num_batched_tokens
        # 1. Running requests, oldest first: ready ones decode, ones still inside their prompt wait
        #    for step 2. A victim comes from the newest end of what has not been visited yet, so it
        #    may be a prompt in progress, never one older than the request that needs the page.
        queue = self._oldest_first()
        partial: list[Sequence] = []
        decodes: list[PlanItem] = []
        while queue:
            seq = queue.pop(0)
            if seq.num_new_tokens > 1:
                partial.append(seq)
                continue
            preempted_self = False
            while not self.cache.can_grow(seq.cache, seq.length):
                victim = queue.pop() if queue else seq
                self._preempt(victim, plan)
                if victim is seq:
                    preempted_self = True
                    break
            if preempted_self:
                continue
            self.cache.grow(seq.cache, seq.length)
            decodes.append(PlanItem(seq, seq.length - 1, 1, True))
        budget -= len(decodes)
        # 2. Prompts already in progress, oldest first. 3. New prompts, first come first served.
        prefills: list[PlanItem] = []
        for seq in partial:
            if budget <= 0:
                break
            n = min(seq.num_new_tokens, budget)
            prefills.append(PlanItem(seq, seq.num_computed_tokens, n, False))
            budget -= n
        while budget > 0:
            seq = self._head_status(plan)
            if seq is None:
                break
            self.waiting.popleft()
            self._admit(seq)                               # pages for the whole prompt up front
            n = min(seq.num_new_tokens, budget)
            prefills.append(PlanItem(seq, seq.num_computed_tokens, n, False))
            budget -= n
        plan.items = prefills + decodes

    def _preempt(self, seq: Sequence, plan: StepPlan) -> None:
        self.running.remove(seq)
        self.cache.free(seq.cache)
        seq.num_computed_tokens = 0              # recompute prompt + generated tokens on resume
        seq.status = Status.PREEMPTED
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)             # front of the queue
        plan.preempted.append(seq)
