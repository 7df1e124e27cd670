"""The generation loop around the kernels, on the CPU (kernels replaced by their torch
statements): steps are launched before the previous step's tokens are read, so this
checks the placeholder bookkeeping, stop tokens seen one step late, preemption with
tokens still on their way, and the sampler's streams."""
import random

import pytest
import torch

import plain_qwen3 as plain
from arle_b200 import Engine, SamplingParams
from tiny_models import make_model_dir


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    d = make_model_dir("A", seed=4, root=str(tmp_path_factory.mktemp("gencpu")))
    cfg, w = plain.read_config(d), plain.read_weights(d)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(6, 256, (n,), generator=g).tolist() for n in (1, 5, 11, 23)]
    return d, cfg, w, prompts


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
    stop = ref[5]
    o = engine(d).generate([prompts[2]], SamplingParams(max_new_tokens=12, stop_token_ids=(stop,)))[0]
    assert o.finish_reason == "stop" and o.token_ids == ref[:ref.index(stop)]
    # the model's own stop id, and several requests finishing at different times
    outs = engine(d).generate(prompts, [SamplingParams(max_new_tokens=12, stop_token_ids=(plain.generate_greedy(w, cfg, p, 12)[i],))
                                        for i, p in zip((0, 3, 7, 11), prompts)])
    for i, p, o in zip((0, 3, 7, 11), prompts, outs):
        r = plain.generate_greedy(w, cfg, p, 12)
        assert o.finish_reason == "stop" and o.token_ids == r[:r.index(r[i])]


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
