#!/usr/bin/env python3
"""Decode and prefill throughput of the engine at Qwen3-8B layer sizes, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

Prints ONE JSON line.  ``value`` is decoded tokens per second at batch 8 with every
request at a 2,048-token context (device time of K decode steps, CUDA events);
``points`` holds batch 1 and 64; ``prefill`` one 2,048-token prompt (``ms``: a single
step after a pause, as a request meets a waiting GPU; ``ms_in_a_row``: steps that follow
the decode runs and one another, when the 1 kW power cap has the clocks down); ``roofline``
the bytes the decode step must read (each weight once + the live requests' cache)
over its time against the measured copy bandwidth; ``e2e`` the same decode metric
through ``Engine.generate`` with token ids going in from and coming back to the
host.  Weights are seeded random, token ids uniform random, the cache of the
device-timed runs is filled with random values (synthetic data).  The engine is a
single-GPU one: for --gpus above 1 it says so and exits with 2.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=36, hidden_size=4096, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936, rope_theta=1e6,
                rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=40960, hidden_act="silu")
# two more sizes of the same architecture (Qwen3-0.6B and Qwen3-32B), for runs beside the default one
QWEN3_0_6B = dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                  intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)
SIZES = {"8b": QWEN3_8B, "0.6b": QWEN3_0_6B, "32b": QWEN3_32B}
CONTEXT = 2048
PREFILL_TOKENS = 2048
PREFILL_PAUSE_S = 0.25            # idle time before each single prefill step that is timed (0.1 s and 1.5 s give the same figure)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(p):
        try:
            with open(p) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d.get("bf16_tflops", 1590.0)),
                    "bf16_tflops_sustained": d.get("bf16_tflops_sustained"), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region is timed."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc, self.lines = None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True).start()
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def gemm_table(args, sizes, torch, ops) -> int:
    """The four projections of a layer at --prefill-tokens rows: cuBLAS (torch.mm) against the package's one-SM
    and two-SM tcgen05 kernels, CUDA events over --steps back-to-back launches on rotating weights (more
    than L2 holds).  One JSON line."""
    dev, rows = "cuda:0", args.prefill_tokens
    H, I = sizes["hidden_size"], sizes["intermediate_size"]
    dq = sizes["num_attention_heads"] * sizes["head_dim"]
    dkv = sizes["num_key_value_heads"] * sizes["head_dim"]
    shapes = {"qkv": (dq + 2 * dkv, H), "o": (H, dq), "gate_up": (2 * I, H), "down": (H, I)}
    steps = max(3, min(args.steps, 40))

    def timed(fn):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        time.sleep(0.25)            # every kernel starts from a GPU at rest: in a row, the later ones would run under the power cap
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        return round(e0.elapsed_time(e1) / steps * 1000.0, 1)

    table = {}
    for name, (N, K) in shapes.items():
        if args.gemm_product not in ("all", name):
            continue
        copies = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        xs = [torch.randn(rows, K, device=dev, dtype=torch.bfloat16) for _ in range(4)]
        out = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)
        row = {"N": N, "K": K,
               "cublas_us": timed(lambda i: torch.mm(xs[i % 4], ws[i % copies].t(), out=out)),
               "one_sm_us": timed(lambda i: ops.gemm_tcgen05(xs[i % 4], ws[i % copies], out)),
               "two_sm_us": timed(lambda i: ops.gemm_tcgen05_pair(xs[i % 4], ws[i % copies], out))}
        if name == "gate_up":
            act = torch.empty(rows, N // 2, device=dev, dtype=torch.bfloat16)
            row["gate_kernel_us"] = timed(lambda i: ops.silu_mul(out, act))
            row["two_sm_gated_us"] = timed(lambda i: ops.gemm_tcgen05_pair(xs[i % 4], ws[i % copies], act, gated=True))
        row["tflops_two_sm"] = round(2.0 * rows * N * K / row["two_sm_us"] / 1e6, 1)
        table[name] = row
        del ws, xs, out
    ops.check_errors(dev)
    print(json.dumps({"only": "gemm", "rows": rows, "steps": steps, "products": table}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than Qwen3-8B's 36 (named in config)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--more-points", action="store_true",
                    help="also decode at Qwen3-0.6B and Qwen3-32B layer sizes and at 8,192 / 32,768-token contexts (points_more)")
    ap.add_argument("--sizes", choices=sorted(SIZES), default="8b", help="layer sizes (default: Qwen3-8B, the contract's)")
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill", "gemm"],
                    help="profiling aid: run only the decode steps at --batch, only the prefill, or (gemm) the four "
                         "projections of a layer at --prefill-tokens rows on cuBLAS and on the package's tcgen05 kernels")
    ap.add_argument("--gemm-product", default="all", choices=["all", "qkv", "o", "gate_up", "down"],
                    help="with --only gemm: one product only (for a profiler capture)")
    ap.add_argument("--context", type=int, default=CONTEXT, help="with --only decode: tokens each request holds")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS, help="with --only prefill: tokens of the prompt")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--timeline", action="store_true",
                    help="with --only decode: also the kernels of one graph-replayed step in order, with the device time "
                         "of each (from torch's profiler: shares of the step, not a benchmark figure)")
    ap.add_argument("--pdl", type=int, nargs="?", const=1, default=0,
                    help="programmatic dependent launch: 1 every kernel, 2 the weight-streaming products only")
    ap.add_argument("--tcgen05-gemm", action="store_true", help="products of 128 rows and more through the package's tcgen05 kernel instead of cuBLAS")
    ap.add_argument("--gated-min-rows", type=int, default=None, help="rows from which the gated product runs on the two-SM tcgen05 kernel (default: the package's)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "cklxx/arle's engine is a Rust workspace (no cargo/rustc in this image); the one offline pip "
                          "install of the reference yields only its tooling metadata (arle-pytools), no engine"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    if args.only == "all" and (args.context != CONTEXT or args.prefill_tokens != PREFILL_TOKENS):
        print("bench.py: --context and --prefill-tokens go with --only decode / --only prefill; the full run keeps the contract's sizes")
        return 2
    globals()["CONTEXT"], globals()["PREFILL_TOKENS"] = args.context, args.prefill_tokens

    import torch

    from arle_b200 import ops
    from arle_b200.engine import ModelRunner, StepEntry, random_model
    from arle_b200.engine.engine import Engine, EngineOptions
    from arle_b200.sampling import Sampler, SamplingParams

    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    if args.pdl:
        ops.set_programmatic_launch(args.pdl)
    if args.tcgen05_gemm:
        ops.set_tcgen05_min_rows(128)
    if args.gated_min_rows is not None:
        ops.set_gated_tcgen05_min_rows(args.gated_min_rows)
    pk = peaks()
    sizes = SIZES[args.sizes]
    if args.only == "gemm":
        return gemm_table(args, sizes, torch, ops)
    layers = args.layers or sizes["num_hidden_layers"]
    model = random_model(sizes, seed=0, dtype="bfloat16", device=dev, num_layers=layers)
    spec = model.spec
    vocab = spec.vocab_size
    page = 16
    max_batch = max(64, args.batch) if args.only == "all" else (args.batch if args.only == "decode" else 1)
    per_req = max(CONTEXT + args.steps + args.warmup + 64, PREFILL_TOKENS + 64 if args.only != "decode" else 0)
    def make_runner(model, max_batch, per_req):
        pages = max_batch * -(-per_req // page) + 64
        r = ModelRunner(model, page, pages, max_batch, per_req + 1024, dev)
        if not args.no_cuda_graph:
            r.enable_graphs()
        for g in r.cache.groups:
            for a in g.arrays:
                a.normal_(0.0, 0.5)                              # synthetic cache contents
        return r

    runner = main_runner = make_runner(model, max_batch, per_req)
    sampler = main_sampler = Sampler(vocab, dev)
    gen = torch.Generator().manual_seed(1)
    weight_bytes = model.weight_bytes_per_step()
    kv_bytes_per_token = runner.cache.bytes_per_token()

    def decode_run(batch, steps, warmup, clocks=None, runner=None, sampler=None, context=None, stats=None):
        runner = runner or main_runner
        sampler = sampler or main_sampler
        context = context or CONTEXT
        rids = [f"b{batch}-{i}" for i in range(batch)]
        for r in rids:
            runner.add_request(r)
        runner.cache.append([(r, context - 1) for r in rids])      # contexts of context - 1 tokens; the first step completes them
        toks = torch.randint(0, vocab, (batch,), generator=gen).tolist()
        greedy = [SamplingParams()] * batch
        first = runner.step([StepEntry(r, [t], (0,)) for r, t in zip(rids, toks)])
        pending = [sampler.sample_async(first, greedy, [None] * batch, runner.last_ctx.want_slots, runner.last_token)]

        def one():
            # the step takes each request's last token from the device (placeholder id -1);
            # the tokens of the step before are read while this one runs
            logits = runner.step([StepEntry(r, [-1], (0,)) for r in rids])
            pending.append(sampler.sample_async(logits, greedy, [None] * batch, runner.last_ctx.want_slots, runner.last_token))
            pending.pop(0).result()

        for _ in range(warmup):
            one()
        torch.cuda.synchronize()
        if clocks:
            clocks.start()
        l0 = ops.launch_count()
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        marks[0].record()
        for i in range(steps):
            one()
            marks[i + 1].record()
        torch.cuda.synchronize()
        pending.pop(0).result()
        ms = marks[0].elapsed_time(marks[-1]) / steps           # the K steps as one interval: the contract's figure
        per_step = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
        if stats is not None:
            stats["median_ms"] = per_step[steps // 2]
        launches = ops.launch_count() - l0
        ctx_mid = context + 1 + warmup + steps // 2
        for r in rids:
            runner.end_request(r)
        return ms, launches, ctx_mid

    if args.only == "decode":
        ms, launches, _ = decode_run(args.batch, args.steps, args.warmup)
        rec = {"only": "decode", "batch": args.batch, "layers": layers, "ms_per_step": round(ms, 4), "gpu_launches": int(launches)}
        if args.timeline:
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                decode_run(args.batch, 3, 3)
            evs = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                          if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda t: t[0])
            last = max(i for i, k in enumerate(evs) if "embedding" in k[2])          # the last step starts with the embedding
            step = evs[last:]
            rec["timeline_span_us"] = round(step[-1][1] - step[0][0], 1)
            rec["timeline"] = [[k[2].replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:48],
                                round(k[1] - k[0], 2)] for k in step]
        print(json.dumps(rec))
        return 0
    clocks = ClockSampler()
    stats = {}
    ms, launches, ctx_mid = (0.0, 0, CONTEXT) if args.only == "prefill" else decode_run(args.batch, args.steps, args.warmup, clocks,
                                                                                        stats=stats)
    clk = clocks.stop()
    value = args.batch * 1000.0 / ms if ms else 0.0
    step_bytes = weight_bytes + args.batch * ctx_mid * kv_bytes_per_token
    achieved = step_bytes / (ms * 1e-3) / 1e9 if ms else 0.0
    points = {}
    for b in (() if args.only == "prefill" else (1, 64)):
        m, _, _ = decode_run(b, max(8, args.steps // 2), args.warmup)
        points[f"decode_b{b}"] = round(b * 1000.0 / m, 1)

    # prefill of one 2,048-token prompt, one step
    def prefill_once(tag):
        rid = f"p-{tag}"
        ids = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=gen).tolist()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        runner.step([StepEntry(rid, ids, (PREFILL_TOKENS - 1,))])
        e1.record()
        torch.cuda.synchronize()
        runner.end_request(rid)
        return e0.elapsed_time(e1)

    for i in range(1 if args.only == "prefill" else 3):
        prefill_once(f"w{i}")
    pf_loop_ms = sorted(prefill_once(f"t{i}") for i in range(1 if args.only == "prefill" else 5))[0 if args.only == "prefill" else 2]
    # The same step on its own, as a request that arrives at a waiting GPU meets it: the steps above follow the decode
    # runs and one another without a pause, so the power cap (1 kW) has already taken the clocks down when they start.
    pf_ms = pf_loop_ms
    if args.only != "prefill":
        apart = []
        for i in range(5):
            torch.cuda.synchronize()
            time.sleep(PREFILL_PAUSE_S)
            apart.append(prefill_once(f"a{i}"))
        pf_ms = sorted(apart)[2]
    if args.only == "prefill":
        rec = {"only": "prefill", "layers": layers, "ms": round(pf_ms, 3)}
        if args.timeline:
            from torch.profiler import ProfilerActivity, profile
            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                prefill_once("prof")
            evs = sorted(((e.time_range.start, e.time_range.end, e.name) for e in prof.events()
                          if e.device_type == torch.autograd.DeviceType.CUDA), key=lambda t: t[0])
            rec["timeline_span_us"] = round(evs[-1][1] - evs[0][0], 1)
            rec["timeline"] = [[k[2].replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:48],
                                round(k[1] - k[0], 2)] for k in evs]
        print(json.dumps(rec))
        return 0
    c = model.config
    mm_params = layers * (c.hidden_size * (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
                          + c.num_attention_heads * c.head_dim * c.hidden_size + 3 * c.hidden_size * c.intermediate_size)
    T = PREFILL_TOKENS
    flops = 2.0 * T * mm_params + 2.0 * vocab * c.hidden_size \
        + layers * 4.0 * c.num_attention_heads * c.head_dim * (T * (T + 1) / 2)
    pf_tflops = flops / (pf_ms * 1e-3) / 1e12
    prefill = {"value": round(T * 1000.0 / pf_ms, 1), "tokens": T, "ms": round(pf_ms, 3),
               "frac": round(pf_tflops / pk["bf16_tflops"], 4), "tflops": round(pf_tflops, 1),
               "timed": f"median of 5 single steps, each after {PREFILL_PAUSE_S} s without work; ms_in_a_row: median of 5 steps "
                        "that follow the decode runs and one another without a pause"}
    # in a row, the steps run under the power cap: that figure stands beside the measured sustained peak
    prefill["ms_in_a_row"] = round(pf_loop_ms, 3)
    if pk.get("bf16_tflops_sustained"):
        prefill["frac_of_sustained_in_a_row"] = round(flops / (pf_loop_ms * 1e-3) / 1e12 / float(pk["bf16_tflops_sustained"]), 4)

    # end to end through the public entry point: host token ids in, host token ids out
    e2e = None
    if not args.no_e2e:
        del runner
        main_runner = None
        torch.cuda.empty_cache()
        n_new = args.steps + 1
        eng = Engine(model=model, options=EngineOptions(
            dtype="bfloat16", device="cuda:0", page_size=page, num_pages=args.batch * -(-(CONTEXT + n_new + 16) // page) + 8,
            num_slots=args.batch, max_seq_len=CONTEXT * 2 + 1024, chunked_prefill_size=CONTEXT,
            max_prefill_tokens=args.batch * CONTEXT, max_num_batched_tokens=args.batch * CONTEXT + 64,
            cuda_graph=not args.no_cuda_graph))
        prompts = [torch.randint(0, vocab, (CONTEXT,), generator=gen).tolist() for _ in range(args.batch)]
        stamps = []

        def on_token(rid, tok):
            stamps.append(time.perf_counter())

        eng.generate(prompts, SamplingParams(max_new_tokens=max(4, args.warmup), ignore_eos=True))   # warm-up: captures the decode graph
        eng.generate(prompts, SamplingParams(max_new_tokens=n_new, ignore_eos=True), on_token=on_token)
        torch.cuda.synchronize()
        # all prompts are prefilled in the first tick, which yields each request's first token;
        # the decode steps after it are what is timed
        first_done = stamps[args.batch - 1]
        decoded = len(stamps) - args.batch
        dt = stamps[-1] - first_done
        e2e = {"value": round(decoded / dt, 1), "unit": "tokens/s", "h2d_bytes_per_step": int(eng.runner.last_ctx.h2d_bytes),
               "d2h_bytes_per_step": 4 * args.batch, "decoded_tokens": decoded}

    # further sizes and contexts, off by default: Qwen3-0.6B and Qwen3-32B layer sizes at their own contexts, and
    # the 8B sizes at longer contexts; tokens per second, device-timed like ``points``
    more = {}
    if args.more_points:
        import gc
        steps_m = max(8, args.steps // 4)
        if "eng" in locals():
            del eng
        main_runner = runner = None
        gc.collect()
        torch.cuda.empty_cache()
        for ctx_len in (8192, 32768):
            r = make_runner(model, 8, ctx_len + steps_m + args.warmup + 64)
            m, _, _ = decode_run(8, steps_m, args.warmup, runner=r, sampler=main_sampler, context=ctx_len)
            more[f"8b_decode_b8_ctx{ctx_len}"] = round(8 * 1000.0 / m, 1)
            del r
            gc.collect()
            torch.cuda.empty_cache()
        del model
        gc.collect()
        torch.cuda.empty_cache()
        for name, ctx_len in (("0.6b", 1152), ("32b", 2048)):
            mdl = random_model(SIZES[name], seed=0, dtype="bfloat16", device=dev)
            r = make_runner(mdl, 64, ctx_len + steps_m + args.warmup + 64)
            smp = Sampler(mdl.spec.vocab_size, dev)
            for b in (1, 8, 64):
                m, _, _ = decode_run(b, steps_m, args.warmup, runner=r, sampler=smp, context=ctx_len)
                more[f"{name}_decode_b{b}_ctx{ctx_len}"] = round(b * 1000.0 / m, 1)
            if name == "32b":
                # a 2,048-token prompt as four portions of 512 beside eight requests that decode at a 2,048-token
                # context: four mixed steps, the median of five such prompts
                rids = [f"mix-{i}" for i in range(8)]
                for q in rids:
                    r.add_request(q)
                r.cache.append([(q, ctx_len) for q in rids])
                times = []
                for rep in range(8):
                    ids = torch.randint(0, mdl.spec.vocab_size, (PREFILL_TOKENS,), generator=gen).tolist()
                    r.add_request(f"mixp-{rep}")
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for part in range(4):
                        toks = ids[part * 512:(part + 1) * 512]
                        r.step([StepEntry(q, [7], (0,)) for q in rids] + [StepEntry(f"mixp-{rep}", toks, (511,) if part == 3 else ())])
                    e1.record()
                    torch.cuda.synchronize()
                    r.end_request(f"mixp-{rep}")
                    if rep >= 3:
                        times.append(e0.elapsed_time(e1))
                for q in rids:
                    r.end_request(q)
                t_mixed = sorted(times)[len(times) // 2]
                more["32b_prefill_4x512_beside_8_decodes_tok_s"] = round(PREFILL_TOKENS * 1000.0 / t_mixed, 1)
                more["32b_mixed_step_ms"] = round(t_mixed / 4, 3)
            del r, smp, mdl
            gc.collect()
            torch.cuda.empty_cache()

    out = {
        "metric": f"decode tokens/s at batch {args.batch}, 2048-token context (Qwen3-{args.sizes.upper()} sizes, bf16, one B200)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_median": round(stats.get("median_ms", ms), 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded random weights, uniform random token ids, random cache contents)",
        "impl": "ours",
        "config": {"model": f"Qwen3-{args.sizes.upper()} sizes, random weights", "layers": layers,
                   "layers_of_config": sizes["num_hidden_layers"],
                   "hidden_size": c.hidden_size, "num_attention_heads": c.num_attention_heads,
                   "num_key_value_heads": c.num_key_value_heads, "head_dim": c.head_dim,
                   "intermediate_size": c.intermediate_size, "vocab_size": vocab, "global_batch": args.batch,
                   "seq_len": CONTEXT, "page_size": page, "parallelism": "single-gpu",
                   "cuda_graph": not args.no_cuda_graph, "l2": "inputs larger than L2 (weights read once per step)",
                   "peaks": pk["source"]},
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk["source"], "bytes_per_step": int(step_bytes)},
        "points": points,
        "e2e": e2e,
        **({"points_more": more} if more else {}),
        "gpu_launches": int(launches),
        "clocks": clk,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
