"""Trace replay: feeds given token ids through the model step by step and writes
the logits at the wanted places.  It samples nothing and has no forward pass,
cache or loader of its own: it drives ``load_model`` and ``ModelRunner.step``,
the same objects generation uses.

Input, one JSON object per line on standard input::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which something is wanted, ``<out>/<step>.f32`` gets the logits as
little-endian float32 [wanted, vocab], in the order of the entries and of their
``want`` lists.  After every step a line ``done <step>`` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each request rounded up to 64); sizes the cache")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (must divide 64)")
    ap.add_argument("--max-live", type=int, default=8, help="most requests live at a time")
    ap.add_argument("--kernels", default="fast", choices=["fast", "plain"],
                    help="fast: the kernels serving uses (shapes decide); plain: the general kernels only")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0 or args.page_size <= 0 or 64 % args.page_size:
        ap.error("--max-tokens must be positive and --page-size must divide 64")

    print("[trace_run] loading torch and the CUDA kernels ...", file=sys.stderr, flush=True)
    import torch

    from .. import ops
    from .batch import StepEntry
    from .loading import load_model
    from .runner import ModelRunner

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; this engine has no CPU path", file=sys.stderr)
        return 2
    ops.library()                       # builds the kernels at the first call, with progress lines
    os.makedirs(args.out, exist_ok=True)
    model = load_model(args.model, args.dtype, args.device)
    pages = -(-args.max_tokens // args.page_size)
    runner = ModelRunner(model, args.page_size, pages, args.max_live, device=args.device, kernel_set=args.kernels)
    print(f"[trace_run] model loaded ({args.dtype}); cache: {pages} pages of {args.page_size} tokens",
          file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        logits = runner.step(entries) if entries else None
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
            arr.tofile(os.path.join(args.out, f"{step}.f32"))
        else:
            torch.cuda.synchronize()
        for rid in rec.get("end", ()):
            runner.end_request(rid)
        print(f"done {step}", flush=True)
    ops.check_errors(args.device)
    return 0


if __name__ == "__main__":
    sys.exit(main())
