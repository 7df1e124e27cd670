"""The engine against the plain model under every way of cutting the work: each
request alone and whole; most of it in one step and the last 32 tokens one by one;
portions of changing size down to two tokens; and mixed batches of up to four live
requests on so few pages that they are used again.  Run on the GPU in float32 and
bfloat16, and (the same scenarios, with the kernels replaced by their plain torch
statements) on the CPU, where they test everything around the kernels."""
import pytest
import torch

import plain_qwen3 as plain
import traces
from arle_b200.engine import ModelRunner, load_model
from tiny_models import CONFIGS, PAGE_SIZES, make_model_dir

LENGTHS = {"A": [1, 5, 11, 23, 70, 130], "B": [2, 17, 40, 96, 67, 33], "C": [3, 50, 90, 120, 64, 35],
           "D": [2, 65, 190, 128, 77, 40], "E": [1, 70, 129, 64, 300, 18], "F": [3, 66, 150, 64, 40, 97]}
CUTS = ["whole", "tail_decode", "portions", "mixed"]
# absolute tolerance on logits of magnitude ~1.5: float32 rounding through a few
# layers; bfloat16 rounding of activations (8 mantissa bits) through the same.
ATOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}
MEAN = {torch.float32: 2e-6, torch.bfloat16: 6e-3}

_cache = {}


def model_and_oracle(name, tmp_path_factory):
    if name not in _cache:
        d = make_model_dir(name, seed=11, root=str(tmp_path_factory.mktemp(f"tiny{name}")))
        cfg, w = plain.read_config(d), plain.read_weights(d)
        reqs = traces.make_requests(cfg["vocab_size"], LENGTHS[name], seed=5)
        oracle = {r: plain.forward(w, cfg, t) for r, t in reqs.items()}
        _cache[name] = (d, reqs, oracle)
    return _cache[name]


def build_steps(cut, reqs):
    if cut == "mixed":
        return traces.mixed(reqs, seed=3)
    return getattr(traces, cut)(reqs)


def check(name, dtype, cut, device, tmp_path_factory, page_size=None, kernel_set="fast"):
    d, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = build_steps(cut, reqs)
    ps = page_size or PAGE_SIZES[name]
    # requests hold multiples of 64 tokens at the peak; a page size that does not divide 64 needs a page more each
    pages = traces.peak_tokens(steps) // ps if 64 % ps == 0 or ps % 64 == 0 else -(-traces.peak_tokens(steps) // ps) + 4
    model = load_model(d, dtype, device)
    runner = ModelRunner(model, ps, pages, 4, device=device, kernel_set=kernel_set)
    got = traces.run_trace(runner, steps)
    runner.cache.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups), "pages not given back"
    for r, want in oracle.items():
        err = (got[r].double() - want).abs()
        assert got[r].shape == want.shape
        first_bad = (err.max(dim=1).values > ATOL[dtype]).nonzero()
        assert err.max().item() <= ATOL[dtype], (
            f"{name} {cut} {dtype}: request {r} first wrong position {int(first_bad[0])} of {len(reqs[r])}, "
            f"max error {err.max().item():.3g}")
        assert err.mean().item() <= MEAN[dtype]


@pytest.mark.gpu
@pytest.mark.parametrize("cut", CUTS)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
def test_cuttings_gpu(name, dtype, cut, tmp_path_factory):
    check(name, dtype, cut, "cuda", tmp_path_factory)


@pytest.mark.gpu
@pytest.mark.parametrize("cut", ["tail_decode", "mixed"])
@pytest.mark.parametrize("name,page_size", [("D", 32), ("E", 64), ("E", 48)])
def test_cuttings_gpu_larger_pages(name, page_size, cut, tmp_path_factory):
    """The TMA-fed attention kernels fetch keys in boxes of 16: pages of 32, 48 and 64 slots."""
    check(name, torch.bfloat16, cut, "cuda", tmp_path_factory, page_size=page_size)


@pytest.mark.gpu
@pytest.mark.parametrize("cut", ["tail_decode", "mixed"])
@pytest.mark.parametrize("name", ["D", "E", "F"])
def test_cuttings_gpu_plain_kernel_set(name, cut, tmp_path_factory, monkeypatch):
    """The same traces in bfloat16 on the general kernels only (plain FFMA products, general
    attention, separate gate): none of the fast kernels may be launched, and the logits meet
    the same bounds."""
    from arle_b200 import ops
    lib = ops.library()
    called = []
    for fast in ("arle_gemm_skinny", "arle_gemm_skinny_gated", "arle_gemm_tcgen05", "arle_paged_attention_decode_stream",
                 "arle_paged_attention_decode", "arle_paged_attention_prefill", "arle_paged_attention_prefill_tc"):
        real = getattr(lib, fast)
        monkeypatch.setattr(lib, fast, lambda *a, _n=fast, _f=real: (called.append(_n), _f(*a))[1], raising=False)
    mm = torch.mm
    monkeypatch.setattr(torch, "mm", lambda *a, **k: (called.append("torch.mm"), mm(*a, **k))[1])
    check(name, torch.bfloat16, cut, "cuda", tmp_path_factory, kernel_set="plain")
    assert not called, f"the plain kernel set launched {sorted(set(called))}"


@pytest.mark.parametrize("cut", CUTS)
@pytest.mark.parametrize("name,dtype", [("A", torch.float32), ("B", torch.bfloat16), ("C", torch.float32)],
                         ids=["A-f32", "B-bf16", "C-f32"])
def test_cuttings_around_the_kernels_cpu(name, dtype, cut, tmp_path_factory, cpu_kernels):
    check(name, dtype, cut, "cpu", tmp_path_factory)


def check_preempted(name, dtype, device, tmp_path_factory):
    d, reqs, oracle = model_and_oracle(name, tmp_path_factory)
    steps = traces.preempted(reqs)
    victim = max(reqs, key=lambda r: len(reqs[r]))
    ps = PAGE_SIZES[name]
    model = load_model(d, dtype, device)
    runner = ModelRunner(model, ps, traces.peak_tokens(steps) // ps, 4, device=device)
    rows = traces.run_trace_by_position(runner, steps)
    runner.cache.check()
    assert all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups), "pages not given back"
    seen = {}
    for r, pos, row in rows:
        err = (row.double() - oracle[r][pos]).abs().max().item()
        assert err <= ATOL[dtype], f"{name} {dtype}: request {r} position {pos} (time {seen.get((r, pos), 0) + 1}): error {err:.3g}"
        seen[(r, pos)] = seen.get((r, pos), 0) + 1
    assert all(seen.get((r, p), 0) >= 1 for r, t in reqs.items() for p in range(len(t)))
    assert seen[(victim, 0)] == 2 and seen[(victim, len(reqs[victim]) - 1)] == 1      # computed again from its first token


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("name", ["B", "C", "D", "E", "F"])
def test_an_ended_request_starts_again_gpu(name, dtype, tmp_path_factory):
    """A request is ended half-way, others take its pages, and it is prefilled again from its first
    token under the same name (preemption by recomputation as a trace)."""
    check_preempted(name, dtype, "cuda", tmp_path_factory)


@pytest.mark.parametrize("name", ["A", "C"])
def test_an_ended_request_starts_again_cpu(name, tmp_path_factory, cpu_kernels):
    check_preempted(name, torch.float32, "cpu", tmp_path_factory)


def test_preempted_trace_shape():
    reqs = traces.make_requests(100, LENGTHS["B"], seed=5)
    steps = traces.preempted(reqs)
    victim = max(reqs, key=lambda r: len(reqs[r]))
    ends = [s["step"] for s in steps if victim in s["end"]]
    starts = [s["step"] for s in steps for e in s["entries"] if e["id"] == victim and e["tokens"][:2] == reqs[victim][:2]]
    assert len(ends) == 2 and len(starts) == 2 and starts[1] > ends[0]
    assert traces.peak_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())


def test_mixed_trace_reuses_pages():
    reqs = traces.make_requests(100, LENGTHS["A"], seed=5)
    steps = traces.mixed(reqs, seed=3)
    assert traces.peak_tokens(steps) < sum(-(-len(t) // 64) * 64 for t in reqs.values())
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len(e["tokens"]) == 1 for s in steps for e in s["entries"]) and \
        any(len(e["tokens"]) == 2 for s in steps for e in s["entries"])


def test_graph_table_width_never_exceeds_the_host_table(tmp_path_factory, cpu_kernels):
    """A captured decode step fixes its block-table width at a power of two; the host tables
    have ceil(limit / page) columns, which need not be one.  The width must be cut to them."""
    from arle_b200.engine import StepContext, StepEntry, Workspace

    d, reqs, oracle = model_and_oracle("A", tmp_path_factory)
    model = load_model(d, torch.float32, "cpu")
    runner = ModelRunner(model, 4, 64, 2, max_tokens_per_request=40, device="cpu")       # 10 columns
    runner._graphs, runner._max_graph_rows = {}, 8                                       # as enable_graphs() leaves them
    toks = reqs["r4"][:34]
    runner.step([StepEntry("x", toks[:33], ())])
    entries = [StepEntry("x", toks[33:34], (0,))]
    key = runner._graph_key(entries, [33])               # 9 pages: the next power of two is 16
    assert key == (1, 10)
    runner.cache.append([("x", 1)])
    ctx = StepContext(runner.cache, Workspace("cpu")).build(entries, [33], key[1])
    assert tuple(ctx.groups[0].block_table.shape) == (1, 10)
    logits = model.forward(ctx)
    assert (logits[0].double() - oracle["r4"][33]).abs().max().item() <= ATOL[torch.float32]
    # fewer columns than the narrowest graph is wide
    small = ModelRunner(model, 4, 64, 2, max_tokens_per_request=20, device="cpu")        # 5 columns
    small._graphs, small._max_graph_rows = {}, 8
    assert small._graph_key([StepEntry("y", [3], (0,))], [2]) == (1, 5)


def test_a_step_starts_with_an_empty_memo(tmp_path_factory, cpu_kernels):
    """What parts keep in ``ctx.memo`` (tables derived from a step's positions or lengths) belongs to one pass over
    one step: building the next step empties it, and so does every pass that the runner starts."""
    from arle_b200.engine import StepContext, StepEntry, Workspace
    from arle_b200.engine.runner import _forward

    d, reqs, oracle = model_and_oracle("A", tmp_path_factory)
    model = load_model(d, torch.float32, "cpu")
    runner = ModelRunner(model, 4, 64, 2, device="cpu")
    toks = reqs["r3"]
    runner.cache.add_request("x")
    runner.cache.append([("x", 5)])
    ctx = StepContext(runner.cache, Workspace("cpu")).build([StepEntry("x", toks[:5], (4,))], [0])
    ctx.memo["left over"] = 1
    logits = _forward(model, ctx)
    assert "left over" not in ctx.memo
    assert (logits[0].double() - oracle["r3"][4]).abs().max().item() <= ATOL[torch.float32]
    ctx.memo["left over"] = 2
    runner.cache.append([("x", 1)])
    ctx.build([StepEntry("x", toks[5:6], (0,))], [5])
    assert ctx.memo == {}


def test_token_ids_outside_the_vocabulary_are_refused_before_anything_changes(tmp_path_factory, cpu_kernels):
    from arle_b200 import Engine
    from arle_b200.engine import StepEntry

    d, reqs, oracle = model_and_oracle("A", tmp_path_factory)
    vocab = CONFIGS["A"]["vocab_size"]
    model = load_model(d, torch.float32, "cpu")
    runner = ModelRunner(model, 4, 16, 2, device="cpu")
    for bad in ([3, vocab, 5], [3, -1, 5], [vocab + 7]):
        with pytest.raises(ValueError, match="outside the vocabulary"):
            runner.step([StepEntry("x", bad, ())])
        assert runner.cache.num_tokens("x") == 0 and all(g.pool.num_free == g.pool.num_pages for g in runner.cache.groups)
    eng = Engine(d, dtype="float32", device="cpu", page_size=4, num_pages=16, num_slots=2)
    with pytest.raises(ValueError, match=f"token id {vocab} is outside the vocabulary"):
        eng.add_request([1, 2, vocab])
    with pytest.raises(ValueError, match="token id -4 is outside the vocabulary"):
        eng.add_request([1, -4])
