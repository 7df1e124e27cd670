"""Command line in the manner of cklxx/arle's ``arle`` and ``infer`` binaries.

    python -m arle_b200 --model-path DIR [--max-tokens N] [--temperature T] [--no-cuda-graph] \\
        run (--prompt "1 2 3" | --stdin) [--json]
    python -m arle_b200 random-model --config CONFIG.json --seed S --out DIR

Top-level ``--model-path``, ``--max-tokens``, ``--temperature`` and
``--no-cuda-graph`` and the ``run`` sub-command with ``--prompt`` / ``--stdin`` /
``--json`` are the reference's (crates/cli/src/args.rs:187-303); the engine knobs
carry the names of its server (infer/src/main.rs:27-237).  There is no tokenizer
here: a prompt is a list of token ids separated by spaces or commas.
"""
from __future__ import annotations

import argparse
import json
import re
import sys


def _ids(text: str):
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    if not parts:
        raise SystemExit("empty prompt: give token ids separated by spaces or commas")
    try:
        return [int(p) for p in parts]
    except ValueError:
        raise SystemExit("a prompt is a list of token ids (this engine has no tokenizer)")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="arle_b200", description="Qwen3 dense inference engine for one B200")
    ap.add_argument("--model-path", help="model folder with config.json and model.safetensors")
    ap.add_argument("--max-tokens", type=int, default=256, help="most tokens to generate per prompt")
    ap.add_argument("--temperature", type=float, default=0.0, help="sampling temperature (0.0 = greedy)")
    ap.add_argument("--top-k", type=int, default=-1)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--no-cuda-graph", action="store_true", help="disable CUDA graphs for decode steps")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--num-slots", type=int, default=64, help="most requests running at a time")
    ap.add_argument("--max-seq-len", type=int, default=None, help="most tokens a request may hold")
    ap.add_argument("--chunked-prefill-size", type=int, default=16384)
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--max-prefill-tokens", type=int, default=None)
    ap.add_argument("--prefill-max-requests", type=int, default=None)
    ap.add_argument("--scheduler-mixed-policy", default="mixed", choices=["mixed", "split"])
    ap.add_argument("--mem-fraction-static", type=float, default=0.85)
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--num-pages", type=int, default=None)
    ap.add_argument("--kernel-set", default="fast", choices=["fast", "plain"],
                    help="plain: run the general kernels only (to bisect a discrepancy)")
    sub = ap.add_subparsers(dest="command")
    run = sub.add_parser("run", help="run prompts and exit")
    g = run.add_mutually_exclusive_group(required=True)
    g.add_argument("--prompt", action="append", help="token ids of one prompt; may be given several times")
    g.add_argument("--stdin", action="store_true", help="read prompts from stdin, one per line")
    run.add_argument("--json", action="store_true", help="one machine-readable JSON document on stdout")
    rm = sub.add_parser("random-model", help="write a model folder with seeded random weights")
    rm.add_argument("--config", required=True, help="a config.json to build the model from")
    rm.add_argument("--seed", type=int, default=0)
    rm.add_argument("--sigma", type=float, default=0.02)
    rm.add_argument("--gain-jitter", type=float, default=0.1)
    rm.add_argument("--out", required=True)
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if args.command == "random-model":
        from .weights import write_random_model

        with open(args.config) as f:
            cfg = json.load(f)
        print(write_random_model(args.out, cfg, args.seed, args.sigma, args.gain_jitter))
        return 0
    if args.command != "run":
        ap.print_help()
        return 2
    if not args.model_path:
        ap.error("--model-path is required")
    prompts = [_ids(p) for p in args.prompt] if args.prompt else [_ids(l) for l in sys.stdin if l.strip()]
    from .engine.engine import Engine, EngineOptions
    from .sampling import SamplingParams

    eng = Engine(args.model_path, options=EngineOptions(
        dtype=args.dtype, page_size=args.page_size, num_pages=args.num_pages,
        mem_fraction_static=args.mem_fraction_static, num_slots=args.num_slots, max_seq_len=args.max_seq_len,
        max_num_batched_tokens=args.max_num_batched_tokens, chunked_prefill_size=args.chunked_prefill_size,
        max_prefill_tokens=args.max_prefill_tokens, prefill_max_requests=args.prefill_max_requests,
        scheduler_mixed_policy=args.scheduler_mixed_policy, max_tokens=args.max_tokens, seed=args.seed,
        cuda_graph=not args.no_cuda_graph, kernel_set=args.kernel_set))
    sp = SamplingParams(temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p,
                        ignore_eos=args.ignore_eos, max_new_tokens=args.max_tokens)
    outs = eng.generate(prompts, sp)
    if args.json:
        print(json.dumps({"model": args.model_path, "backend": "cuda-sm100a", "dtype": args.dtype,
                          "outputs": [{"prompt_token_ids": o.prompt_token_ids, "token_ids": o.token_ids,
                                       "finish_reason": o.finish_reason,
                                       "usage": {"prompt_tokens": len(o.prompt_token_ids),
                                                 "completion_tokens": len(o.token_ids)}} for o in outs],
                          "stats": eng.stats()}))
    else:
        for o in outs:
            print(" ".join(str(t) for t in o.token_ids))
    return 0


if __name__ == "__main__":
    sys.exit(main())
