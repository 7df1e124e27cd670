"""The generation loop around the kernels, on the CPU (kernels replaced by their torch
statements): steps are launched before the previous step's tokens are read, so this
checks the placeholder bookkeeping, stop tokens seen one step late, preemption with
tokens still on their way, and the sampler's streams."""
import random

import pytest
import torch

import plain_qwen3 as plain
from arle_b200 import Engine, SamplingParams
from tiny_models import assert_varied, make_varied_model_dir


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = make_varied_model_dir("A", seed=21, root=str(tmp_path_factory.mktemp("gencpu")))
    cfg, w = plain.read_config(d), plain.read_weights(d)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(6, 256, (n,), generator=g).tolist() for n in (1, 5, 11, 23)]
    assert_varied([plain.generate_greedy(w, cfg, p, 12) for p in prompts])
    return d, cfg, w, prompts


def late_stop(ref, least=3):
    """A token of the reference continuation whose first occurrence is at index >= least."""
    for i in range(least, len(ref)):
        if ref[i] not in ref[:i]:
            return ref[i], i
    raise AssertionError(f"no token of {ref} first appears at index {least} or later")


def engine(d, **kw):
    args = dict(dtype="float32", device="cpu", page_size=4, num_pages=48, num_slots=4, chunked_prefill_size=7,
                max_num_batched_tokens=16, cuda_graph=False)
    args.update(kw)
    return Engine(d, **args)


@pytest.mark.parametrize("pages,policy", [(48, "mixed"), (48, "split"), (12, "mixed"), (10, "mixed")])
def test_pipelined_generation_equals_plain_greedy(tiny, cpu_kernels, pages, policy):
    d, cfg, w, prompts = tiny
    eng = engine(d, num_pages=pages, scheduler_mixed_policy=policy)
    seen = {}
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True),
                        on_token=lambda rid, t: seen.setdefault(rid, []).append(t))
    for p, o in zip(prompts, outs):
        assert o.token_ids == plain.generate_greedy(w, cfg, p, 12) and o.finish_reason == "length"
        assert seen[o.request_id] == o.token_ids and -1 not in o.token_ids
    if pages <= 12:
        assert sum(o.preemptions for o in outs) > 0
    eng.runner.cache.check()
    assert eng.runner.cache.free_pages() == eng.runner.cache.total_pages() and not eng._inflight


def test_stop_token_is_seen_one_step_late_and_nothing_after_it_is_emitted(tiny, cpu_kernels):
    d, cfg, w, prompts = tiny
    ref = plain.generate_greedy(w, cfg, prompts[2], 12)
    stop, at = late_stop(ref)
    o = engine(d).generate([prompts[2]], SamplingParams(max_new_tokens=12, stop_token_ids=(stop,)))[0]
    assert o.finish_reason == "stop" and o.token_ids == ref[:at] and len(o.token_ids) >= 3
    # several requests finishing at different times, the first one on its very first token
    refs = [plain.generate_greedy(w, cfg, p, 12) for p in prompts]
    stops = [(refs[0][0], 0)] + [late_stop(r, k) for r, k in zip(refs[1:], (3, 5, 7))]
    outs = engine(d).generate(prompts, [SamplingParams(max_new_tokens=12, stop_token_ids=(t,)) for t, _ in stops])
    for r, (t, at), o in zip(refs, stops, outs):
        assert o.finish_reason == "stop" and o.token_ids == r[:at]


@pytest.mark.parametrize("pages,least", [(12, (7, 4, 6, 5)), (11, (9, 9, 9, 9)), (10, (10, 8, 9, 7))])
def test_stop_tokens_under_page_pressure(tiny, cpu_kernels, pages, least):
    """Requests are preempted and recomputed while others stop: the recomputed request must
    still stop at the same place, and a stopped request's pages must be given back."""
    d, cfg, w, prompts = tiny
    refs = [plain.generate_greedy(w, cfg, p, 12) for p in prompts]
    stops = [late_stop(r, k) for r, k in zip(refs, least)]
    eng = engine(d, num_pages=pages)
    outs = eng.generate(prompts, [SamplingParams(max_new_tokens=12, stop_token_ids=(t,)) for t, _ in stops])
    assert sum(o.preemptions for o in outs) > 0
    for r, (t, at), o in zip(refs, stops, outs):
        assert o.finish_reason == "stop" and o.token_ids == r[:at]
    eng.runner.cache.check()
    assert eng.runner.cache.free_pages() == eng.runner.cache.total_pages() and not eng._inflight


def test_many_outstanding_sample_handles_keep_their_own_tokens(cpu_kernels):
    """A tick of the split policy launches two sampling steps and the next tick launches
    again before either is read: every handle must still return its own tokens."""
    from arle_b200.sampling import Sampler

    s = Sampler(50, "cpu")
    rows = [torch.full((3, 50), -1.0) for _ in range(5)]
    for k, r in enumerate(rows):
        for i in range(3):
            r[i, 10 * k + i] = 1.0
    handles = [s.sample_async(r, [SamplingParams()] * 3, [None] * 3) for r in rows]
    assert [h.result() for h in handles] == [[10 * k + i for i in range(3)] for k in range(5)]
    assert [h.result() for h in reversed(handles)] == [[10 * k + i for i in range(3)] for k in reversed(range(5))]
    assert len(s._free_token_hosts) == 5


def test_split_policy_with_chunked_prompts_returns_each_requests_own_tokens(cpu_kernels, tmp_path):
    d = make_varied_model_dir("B", seed=21, root=str(tmp_path))
    cfg, w = plain.read_config(d), plain.read_weights(d)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(6, cfg["vocab_size"], (n,), generator=g).tolist() for n in (2, 17, 40)]
    refs = [plain.generate_greedy(w, cfg, p, 10) for p in prompts]
    assert_varied(refs)
    eng = engine(d, page_size=8, num_pages=64, chunked_prefill_size=5, max_num_batched_tokens=12,
                 scheduler_mixed_policy="split")
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10, ignore_eos=True))
    assert [o.token_ids for o in outs] == refs


def test_temperature_streams_do_not_depend_on_the_batch(tiny, cpu_kernels):
    d, cfg, w, prompts = tiny
    sp = [SamplingParams(temperature=0.8, seed=50 + i, max_new_tokens=8, ignore_eos=True) for i in range(4)]
    together = engine(d).generate(prompts, sp)
    alone = [engine(d).generate([p], [s])[0] for p, s in zip(prompts, sp)]
    assert [o.token_ids for o in together] == [o.token_ids for o in alone]
    for p, s, o in zip(prompts, sp, together):
        rng, toks = random.Random(s.seed), list(p)
        for t in o.token_ids:
            assert t == plain.sample_from(plain.sampling_distribution(plain.forward(w, cfg, toks)[-1], 0.8), rng.random())
            toks.append(t)


def test_max_new_tokens_one_and_second_round_on_the_same_engine(tiny, cpu_kernels):
    d, cfg, w, prompts = tiny
    eng = engine(d)
    a = eng.generate(prompts[:2], SamplingParams(max_new_tokens=1, ignore_eos=True))
    assert [o.token_ids for o in a] == [plain.generate_greedy(w, cfg, p, 1) for p in prompts[:2]]
    b = eng.generate(prompts[2:], SamplingParams(max_new_tokens=5, ignore_eos=True))
    assert [o.token_ids for o in b] == [plain.generate_greedy(w, cfg, p, 5) for p in prompts[2:]]
