"""The scheduler's decisions, on a CPU cache manager with a stand-in for the model
(next token = a fixed function of the request), no GPU."""
import pytest
import torch

from arle_b200.cache import CacheManager
from arle_b200.engine.scheduler import Scheduler, SchedulerConfig
from arle_b200.parts import CacheNeed
from arle_b200.sampling import SamplingParams


def make(pages=32, page_size=4, slots=4, max_tokens=512, stop=(), **cfg):
    cache = CacheManager([CacheNeed(1, 4)], [], page_size, pages, slots, max_tokens, torch.float32, "cpu")
    return Scheduler(cache, SchedulerConfig(**cfg), stop, default_max_new_tokens=8), cache


def run_tick(s, cache, token_of=lambda r: 100 + len(r.output)):
    """Executes the plans of one tick the way the engine does; returns them."""
    plans = s.schedule()
    for plan in plans:
        cache.append([(e.request.rid, e.count) for e in plan.entries])
        s.on_step_done(plan, [token_of(e.request) for e in plan.entries if e.samples])
        cache.check()
    return plans


def drain(s, cache, limit=2000, **kw):
    ticks = 0
    while s.has_work():
        run_tick(s, cache, **kw)
        ticks += 1
        assert ticks < limit, "scheduler does not drain"
    return ticks


def test_prompt_is_cut_into_portions_under_the_budget():
    s, cache = make(max_num_batched_tokens=10, chunked_prefill_size=6)
    r = s.add_request("a", list(range(20)), SamplingParams(max_new_tokens=3))
    sizes = []
    while r.finish_reason is None:
        plans = run_tick(s, cache)
        sizes.append([e.count for e in plans[0].entries])
    assert sizes[:4] == [[6], [6], [6], [2]] and sizes[4:] == [[1], [1]]
    assert r.output == [100, 101, 102] and r.finish_reason == "length"
    assert cache.free_pages() == [32] and cache.num_free_slots == 4


def test_decode_rows_come_first_and_portions_share_the_rest():
    s, cache = make(max_num_batched_tokens=8, chunked_prefill_size=16)
    a = s.add_request("a", [1, 2, 3], SamplingParams(max_new_tokens=50))
    run_tick(s, cache)
    b = s.add_request("b", list(range(30)), SamplingParams(max_new_tokens=5))
    plan = run_tick(s, cache)[0]
    assert [(e.request.rid, e.count) for e in plan.entries] == [("a", 1), ("b", 7)]    # 8 - 1 decode row
    assert not plan.entries[1].samples and plan.entries[0].samples


def test_split_policy_runs_portions_then_decode_rows():
    s, cache = make(max_num_batched_tokens=64, scheduler_mixed_policy="split")
    s.add_request("a", [1, 2], SamplingParams(max_new_tokens=9))
    run_tick(s, cache)
    s.add_request("b", list(range(9)), SamplingParams(max_new_tokens=9))
    plans = run_tick(s, cache)
    assert len(plans) == 2
    assert [e.request.rid for e in plans[0].entries] == ["b"] and [e.request.rid for e in plans[1].entries] == ["a"]


def test_max_prefill_tokens_and_prefill_max_requests():
    s, cache = make(pages=64, max_num_batched_tokens=100, chunked_prefill_size=50, max_prefill_tokens=12,
                    prefill_max_requests=2)
    for i in range(3):
        s.add_request(i, list(range(10)), SamplingParams(max_new_tokens=2))
    plan = s.schedule()[0]
    assert [(e.request.rid, e.count) for e in plan.entries] == [(0, 10), (1, 2)]


def test_admission_is_fcfs_and_waits_for_slot_and_pages():
    s, cache = make(pages=8, slots=2)          # 32 tokens of cache
    s.add_request("big", list(range(20)), SamplingParams(max_new_tokens=4))
    s.add_request("mid", list(range(14)), SamplingParams(max_new_tokens=4))     # 20+1 and 14+1 do not both fit
    s.add_request("small", [1], SamplingParams(max_new_tokens=4))                # would fit, but is behind mid
    run_tick(s, cache)
    assert [r.rid for r in s.running] == ["big"] and [r.rid for r in s.waiting] == ["mid", "small"]
    drain(s, cache)
    assert [r.rid for r in s.finished] == ["big", "mid", "small"]


def test_finish_reasons_stop_token_is_not_emitted():
    s, cache = make(stop=(7,))
    a = s.add_request("a", [1, 2], SamplingParams(max_new_tokens=5))
    b = s.add_request("b", [1, 2], SamplingParams(max_new_tokens=5, ignore_eos=True))
    c = s.add_request("c", [1, 2], SamplingParams(max_new_tokens=5, stop_token_ids=(9,)))
    z = s.add_request("z", [1, 2], SamplingParams(max_new_tokens=0))
    drain(s, cache, token_of=lambda r: {"a": [5, 7, 5], "b": [7] * 9, "c": [5, 6, 9]}[r.rid][len(r.output)])
    assert (a.output, a.finish_reason) == ([5], "stop")
    assert (b.output, b.finish_reason) == ([7] * 5, "length")
    assert (c.output, c.finish_reason) == ([5, 6], "stop")
    assert (z.output, z.finish_reason) == ([], "length")


def test_intake_limits():
    s, cache = make(pages=4, page_size=4)           # 16 tokens at all
    with pytest.raises(ValueError, match="does not fit"):
        s.add_request("x", list(range(16)))
    with pytest.raises(ValueError, match="empty"):
        s.add_request("y", [])
    r = s.add_request("ok", list(range(10)), SamplingParams(max_new_tokens=100))
    assert r.max_new_tokens == 6                    # clamped to what a request may hold
    drain(s, cache)
    assert r.finish_reason == "length" and len(r.output) == 6


def test_pages_run_out_youngest_is_preempted_and_keeps_its_tokens():
    s, cache = make(pages=6, page_size=4, slots=4)          # 24 tokens of cache
    old = s.add_request("old", list(range(6)), SamplingParams(max_new_tokens=14))
    run_tick(s, cache)
    run_tick(s, cache)                                      # old has generated 2
    young = s.add_request("young", list(range(5)), SamplingParams(max_new_tokens=14))
    seen_preempt = False
    outputs_before = None
    for _ in range(200):
        if not s.has_work():
            break
        run_tick(s, cache)
        if young.preemptions and not seen_preempt:
            seen_preempt = True
            outputs_before = list(young.output)
            assert young.num_computed == 0 and not cache.has_request("young")
            assert s.waiting and s.waiting[0] is young       # back at the front of the queue
    assert seen_preempt and old.preemptions == 0              # fewest generated tokens gives way
    assert old.output == [100 + i for i in range(14)]
    assert young.output == [100 + i for i in range(14)] and young.output[:len(outputs_before)] == outputs_before
    assert cache.free_pages() == [6]


def test_victim_order_fewest_generated_then_longest_prompt():
    s, cache = make(pages=64)
    a = s.add_request("a", [1] * 4)
    b = s.add_request("b", [1] * 9)
    c = s.add_request("c", [1] * 2)
    run_tick(s, cache)
    a.output, b.output, c.output = [1, 2], [1], [1]
    assert s._victim() is b                                   # b and c tie on 1 generated; b's prompt is longer
    c.output = []
    assert s._victim() is c


def test_lone_request_that_cannot_grow_ends_with_length():
    s, cache = make(pages=2, page_size=4, max_tokens=512)    # 8 tokens of cache
    r = s.add_request("a", [1, 2, 3], SamplingParams(max_new_tokens=100))
    assert r.max_new_tokens == 5
    drain(s, cache)
    assert r.finish_reason == "length" and len(r.tokens) == 8 and cache.free_pages() == [2]


@pytest.mark.parametrize("seed", range(4))
def test_saturated_cache_drains(seed):
    import random
    rng = random.Random(seed)
    s, cache = make(pages=12, page_size=4, slots=3, max_num_batched_tokens=16, chunked_prefill_size=8)
    reqs = [s.add_request(i, [1] * rng.randint(1, 30), SamplingParams(max_new_tokens=rng.randint(1, 15)))
            for i in range(12)]
    drain(s, cache)
    assert all(r.finish_reason == "length" and len(r.output) == r.max_new_tokens for r in reqs)
    assert cache.free_pages() == [12] and cache.num_free_slots == 3
