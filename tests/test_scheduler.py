"""The scheduler's decisions, with requests of made-up tokens and no model: a fake step marks the
planned tokens computed and appends token 7 to every request that sampled (CPU)."""

from __future__ import annotations

from tokenmill_b200.cache import CacheManager
from tokenmill_b200.config import EngineConfig
from tokenmill_b200.engine.scheduler import Scheduler
from tokenmill_b200.engine.request import Phase, Request
from tokenmill_b200.sampling import SamplingParams


def make(num_pages=16, page=4, **kw):
    base = dict(model="x", block_size=page, max_model_len=256, max_num_seqs=32, max_num_batched_tokens=512,
                watermark=0.0)
    base.update(kw)
    cfg = EngineConfig(**base)
    cache = CacheManager(num_pages, page, watermark=cfg.watermark, enable_prefix_caching=cfg.enable_prefix_caching)
    return Scheduler(cfg, cache), cache


def seq(sched, cache, name, n_prompt, first=0):
    s = Request(name, list(range(first, first + n_prompt)), SamplingParams(max_tokens=64), cache.new_handle())
    sched.submit(s)
    return s


def run_step(sched, cache, plan, max_tokens=None):
    for item in plan.items:
        s = item.req
        s.cached_tokens = item.start + item.count
        cache.register_computed(s.cache, s.tokens, s.cached_tokens)
    for item in plan.items:
        if item.samples:
            item.req.output_ids.append(7)
            if max_tokens and item.req.n_output >= max_tokens:
                sched.retire(item.req, "length")


def test_prefill_then_decode():
    sched, cache = make()
    a = seq(sched, cache, "a", 5)
    plan = sched.plan_step()
    assert [(i.req.id, i.start, i.count, i.decode, i.samples) for i in plan.items] == [("a", 0, 5, False, True)]
    assert a.phase == Phase.RUNNING and len(a.cache.tables[0]) == 2
    run_step(sched, cache, plan)
    plan = sched.plan_step()
    assert [(i.start, i.count, i.decode) for i in plan.items] == [(5, 1, True)]


def test_watermark_holds_pages_back():
    sched, cache = make(num_pages=10, watermark=0.2)
    seq(sched, cache, "a", 24)              # 6 pages, leaves 4 >= 2
    b = seq(sched, cache, "b", 12)          # 3 pages would leave 1 < 2
    plan = sched.plan_step()
    assert [i.req.id for i in plan.items] == ["a"] and b.phase == Phase.QUEUED


def test_fcfs_never_skips_the_head():
    sched, cache = make(num_pages=6)
    seq(sched, cache, "big", 20)            # 5 pages
    seq(sched, cache, "big2", 20)           # does not fit next to it
    small = seq(sched, cache, "small", 2)   # would fit, but waits behind big2
    assert [i.req.id for i in sched.plan_step().items] == ["big"]
    assert small.phase == Phase.QUEUED


def test_token_budget_and_oversized_prompt_runs_alone():
    sched, cache = make(num_pages=64, max_num_batched_tokens=16)
    seq(sched, cache, "a", 10)
    seq(sched, cache, "b", 10)              # 10 > 6 left: next step
    plan = sched.plan_step()
    assert [i.req.id for i in plan.items] == ["a"]
    run_step(sched, cache, plan)
    assert [i.req.id for i in sched.plan_step().items] == ["b"]      # prefill first
    sched2, cache2 = make(num_pages=64, max_num_batched_tokens=16)
    seq(sched2, cache2, "huge", 40)
    seq(sched2, cache2, "next", 3)
    assert [(i.req.id, i.count) for i in sched2.plan_step().items] == [("huge", 40)]


def test_max_num_seqs():
    sched, cache = make(num_pages=64, max_num_seqs=2)
    for n in "abc":
        seq(sched, cache, n, 3)
    assert [i.req.id for i in sched.plan_step().items] == ["a", "b"]


def test_never_fits_is_ignored_and_the_queue_moves_on():
    sched, cache = make(num_pages=4)
    never = seq(sched, cache, "never", 100)
    seq(sched, cache, "ok", 4)
    plan = sched.plan_step()
    assert plan.rejected == [never] and [i.req.id for i in plan.items] == ["ok"]


def test_growth_at_a_page_edge():
    sched, cache = make()
    a = seq(sched, cache, "a", 4)
    run_step(sched, cache, sched.plan_step())
    assert len(a.cache.tables[0]) == 1
    plan = sched.plan_step()                  # length 5 needs a second page
    assert len(a.cache.tables[0]) == 2 and plan.items[0].decode


def test_pages_run_out_newest_is_preempted_and_requeued_at_the_front():
    sched, cache = make(num_pages=4)
    a, b = seq(sched, cache, "a", 8), seq(sched, cache, "b", 8)
    run_step(sched, cache, sched.plan_step())
    assert cache.num_free_pages == 0
    later = seq(sched, cache, "later", 2)
    plan = sched.plan_step()                  # both need a page; b (newest) gives way to a
    assert plan.evicted == [b] and [i.req.id for i in plan.items] == ["a"]
    assert b.phase == Phase.EVICTED and b.cached_tokens == 0 and not b.cache.holds_pages
    assert list(sched.queue) == [b, later] and b.evictions == 1 and sched.evictions == 1
    run_step(sched, cache, plan)
    sched.retire(a, "stop")
    plan = sched.plan_step()                  # b resumes: recomputes prompt + its generated token
    assert [(i.req.id, i.start, i.count, i.samples) for i in plan.items][0] == ("b", 0, 9, True)


def test_a_lone_request_that_cannot_grow_preempts_itself():
    sched, cache = make(num_pages=2)
    a = seq(sched, cache, "a", 8)
    run_step(sched, cache, sched.plan_step())
    plan = sched.plan_step()
    assert plan.evicted == [a] and plan.empty and list(sched.queue) == [a]
    # with its 9 tokens it can never fit in 2 pages any more: the next plan ignores it
    assert sched.plan_step().rejected == [a]


def test_finish_frees_everything():
    sched, cache = make()
    a = seq(sched, cache, "a", 9)
    run_step(sched, cache, sched.plan_step())
    sched.retire(a, "stop")
    assert cache.all_free and not sched.busy and a.finish_reason == "stop"
    w = seq(sched, cache, "w", 3)
    sched.retire(w, "abort")                 # still waiting: nothing to free
    assert not sched.busy


def test_decode_first_waits_then_prefills():
    sched, cache = make(policy="decode_first", max_waiting_steps=2)
    seq(sched, cache, "a", 3)
    run_step(sched, cache, sched.plan_step())         # nothing running yet: prefill
    seq(sched, cache, "b", 3)
    kinds = []
    for _ in range(4):
        plan = sched.plan_step()
        kinds.append([(i.req.id, i.decode) for i in plan.items])
        run_step(sched, cache, plan)
    assert kinds[0] == [("a", True)] and kinds[1] == [("a", True)] and kinds[2] == [("b", False)]
    assert kinds[3] == [("a", True), ("b", True)]


def test_chunked_prefill_splits_a_prompt_beside_a_decode():
    sched, cache = make(num_pages=64, enable_chunked_prefill=True, max_num_batched_tokens=8)
    a = seq(sched, cache, "a", 3)
    run_step(sched, cache, sched.plan_step())
    b = seq(sched, cache, "b", 20)
    chunks = []
    while b.cached_tokens < 20:
        plan = sched.plan_step()
        chunks.append([(i.req.id, i.count, i.samples) for i in plan.items])
        run_step(sched, cache, plan)
    # the decode of a takes one token of every step's budget; b gets 7, 7, 6; portions come first
    assert chunks == [[("b", 7, False), ("a", 1, True)], [("b", 7, False), ("a", 1, True)],
                      [("b", 6, True), ("a", 1, True)]]
    assert len(b.cache.tables[0]) == 5               # pages for the whole prompt at admission
    plan = sched.plan_step()
    assert sorted((i.req.id, i.decode) for i in plan.items) == [("a", True), ("b", True)]


def test_chunked_budget_is_shared_first_come_first_served():
    sched, cache = make(num_pages=64, enable_chunked_prefill=True, max_num_batched_tokens=10)
    seq(sched, cache, "a", 6)
    seq(sched, cache, "b", 6)
    plan = sched.plan_step()
    assert [(i.req.id, i.count) for i in plan.items] == [("a", 6), ("b", 4)]
    run_step(sched, cache, plan)
    plan = sched.plan_step()
    assert [(i.req.id, i.start, i.count, i.decode) for i in plan.items] == [("b", 4, 2, False), ("a", 6, 1, True)]


def test_chunked_preemption_takes_the_newest_even_mid_prompt():
    sched, cache = make(num_pages=6, enable_chunked_prefill=True, max_num_batched_tokens=6)
    a = seq(sched, cache, "a", 8)                     # 2 pages
    run_step(sched, cache, sched.plan_step())          # 6 of 8
    run_step(sched, cache, sched.plan_step())          # 2 more, samples
    b = seq(sched, cache, "b", 16)                    # 4 pages: pool full
    plan = sched.plan_step()                           # a decodes at position 8: needs a page -> b? not admitted yet
    run_step(sched, cache, plan)
    assert b.phase == Phase.QUEUED or b.phase == Phase.RUNNING
    # drive to completion: nothing is lost whatever the order of preemptions
    for _ in range(200):
        if not sched.busy:
            break
        plan = sched.plan_step()
        for s in plan.rejected:
            sched.retire(s, "length")
        run_step(sched, cache, plan, max_tokens=6)
    assert not sched.busy and cache.all_free
    cache.check_invariants()


def test_prefix_sharing_skips_computed_tokens():
    sched, cache = make(num_pages=32, enable_prefix_caching=True)
    a = seq(sched, cache, "a", 12)
    run_step(sched, cache, sched.plan_step())
    b = seq(sched, cache, "b", 12)                    # same 12 tokens: 8 reusable ((12-1)//4 pages)
    plan = sched.plan_step()
    assert [(i.req.id, i.start, i.count) for i in plan.items] == [("b", 8, 4)]
    assert b.cache.tables[0][:2] == a.cache.tables[0][:2]


def test_random_workloads_always_drain_and_return_every_page():
    import random

    for seed in range(25):
        rng = random.Random(seed)
        chunked = rng.random() < 0.5
        sched, cache = make(num_pages=rng.randrange(6, 20), enable_chunked_prefill=chunked,
                            max_num_batched_tokens=rng.choice([6, 16, 64]), max_num_seqs=rng.choice([2, 4, 16]),
                            enable_prefix_caching=rng.random() < 0.5)
        seqs = [seq(sched, cache, f"s{i}", rng.randrange(1, 30), first=rng.choice([0, 0, 100])) for i in range(12)]
        for _ in range(3000):
            if not sched.busy:
                break
            plan = sched.plan_step()
            for s in plan.rejected:
                sched.retire(s, "length")
            run_step(sched, cache, plan, max_tokens=rng.choice([1, 5, 9]))
            cache.check_invariants()
        assert not sched.busy, f"seed {seed} did not drain"
        assert cache.all_free and all(s.done for s in seqs)


def test_a_request_whose_last_token_is_still_on_the_device_is_not_admitted():
    """Preempted while a decode step was in flight: its output list ends in a placeholder. Until the engine
    has read that token the request stays at the head of the queue (nothing behind it jumps ahead), and it is
    admitted as soon as the id is known."""
    from tokenmill_b200.engine.request import TOKEN_IN_FLIGHT as PLACEHOLDER
    for chunked in (False, True):
        sched, cache = make(enable_chunked_prefill=chunked, enable_prefix_caching=True)
        a = seq(sched, cache, "a", 6)
        b = seq(sched, cache, "b", 3, first=50)
        a.output_ids += [9, PLACEHOLDER]
        assert a.awaits_token and not b.awaits_token
        plan = sched.plan_step()
        assert plan.empty and a.phase == Phase.QUEUED and b.phase == Phase.QUEUED
        assert not a.cache.page_hashes                     # nothing was hashed over an unknown id
        a.output_ids[-1] = 11
        plan = sched.plan_step()
        assert [i.req.id for i in plan.items][0] == "a" and a.phase == Phase.RUNNING


def test_a_requests_random_numbers_depend_on_its_seed_and_draw_count_only():
    """The sampler's per-request stream: the array form the engine uses gives, bit for bit, the numbers of the
    one-at-a-time form, whichever other requests share the call; numbers lie in [0, 1) and are exact in float32."""
    import random
    import numpy as np
    from tokenmill_b200.sampling.sampler import uniform_for, uniforms_for
    r = random.Random(3)
    seeds = [r.getrandbits(62) for _ in range(500)] + [0, 1, (1 << 64) - 1, (1 << 70) + 5]
    draws = [r.randrange(0, 100000) for _ in range(500)] + [0, 1, 2, 3]
    one = np.array([uniform_for(s, d) for s, d in zip(seeds, draws)], dtype=np.float64)
    many = uniforms_for(seeds, draws)
    assert many.dtype == np.float32 and (many.astype(np.float64) == one).all()
    assert (many >= 0).all() and (many < 1).all()
    assert (uniforms_for(seeds[5:9], draws[5:9]) == many[5:9]).all()
    assert len(set(one.tolist())) > 490                              # (not one number over and over)
