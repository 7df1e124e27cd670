"""bin/trace_run as a user runs it: a subprocess fed JSON steps on standard input,
writing <step>.f32 files; the same requests whole, with the last 32 tokens decoded
one by one, in portions of changing size, and mixed with other requests on so few
pages that they are used again, in float32 and bfloat16, against the plain model."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import traces
from tiny_models import make_model_dir

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LENGTHS = {"B": [40, 96, 67, 33, 120, 51], "C": [50, 90, 140, 64, 35], "D": [70, 200, 45, 133, 64]}
ATOL = {"float32": 2e-5, "bfloat16": 4e-2}


@pytest.fixture(scope="module")
def setups(tmp_path_factory):
    out = {}
    for name in LENGTHS:
        d = make_model_dir(name, seed=31, root=str(tmp_path_factory.mktemp(f"replay{name}")))
        cfg, w = plain.read_config(d), plain.read_weights(d)
        reqs = traces.make_requests(cfg["vocab_size"], LENGTHS[name], seed=9)
        out[name] = (d, cfg, reqs, {r: plain.forward(w, cfg, t) for r, t in reqs.items()})
    return out


def replay(model_dir, dtype, steps, out_dir, max_tokens, extra=()):
    """Feeds the steps one at a time, each only after the previous 'done' line."""
    p = subprocess.Popen([os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype, "--out", out_dir,
                          "--max-tokens", str(max_tokens), *extra], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True,
                         cwd=ROOT)
    try:
        for s in steps:
            p.stdin.write(json.dumps(s) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {s['step']}", f"expected 'done {s['step']}', got {line!r}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()


def gather(steps, out_dir, vocab):
    got = {}
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        path = os.path.join(out_dir, f"{s['step']}.f32")
        if n == 0:
            assert not os.path.exists(path)
            continue
        arr = np.fromfile(path, dtype="<f4")
        assert arr.size == n * vocab
        arr = arr.reshape(n, vocab)
        at = 0
        for e in s["entries"]:
            for k, w in enumerate(e["want"]):
                got.setdefault(e["id"], {}).setdefault(e["_pos0"] + w, []).append(arr[at + k])
            at += len(e["want"])
    return got


def with_positions(steps):
    seen = {}
    for s in steps:
        for e in s["entries"]:
            e["_pos0"] = seen.get(e["id"], 0)
            seen[e["id"]] = e["_pos0"] + len(e["tokens"])
        for r in s["end"]:
            seen.pop(r, None)                     # a request that starts again starts at position 0
    return steps


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed", "preempted"])
@pytest.mark.parametrize("name", ["B", "C", "D"])
def test_replay_matches_plain_model(setups, tmp_path, name, cut, dtype):
    d, cfg, reqs, oracle = setups[name]
    steps = traces.mixed(reqs, seed=4) if cut == "mixed" else getattr(traces, cut)(reqs)
    if cut == "portions":
        for s in steps[::3]:                      # some steps want nothing, some only their last place
            s["entries"][0]["want"] = []
        for s in steps[1::3]:
            s["entries"][0]["want"] = [len(s["entries"][0]["tokens"]) - 1]
    steps = with_positions(steps)
    clean = [{"step": s["step"], "entries": [{k: v for k, v in e.items() if k != "_pos0"} for e in s["entries"]],
              "end": s["end"]} for s in steps]
    out_dir = str(tmp_path / "out")
    replay(d, dtype, clean, out_dir, traces.peak_tokens(steps))
    got = gather(steps, out_dir, cfg["vocab_size"])
    checked = 0
    for r, rows in got.items():
        for pos, times in rows.items():
            for row in times:                     # more than one only where a request was started again
                err = np.abs(row.astype(np.float64) - oracle[r][pos].numpy()).max()
                assert err <= ATOL[dtype], f"{name} {cut} {dtype}: request {r} position {pos}: error {err:.3g}"
                checked += 1
    assert checked > 50
    if cut == "preempted":
        assert any(len(times) == 2 for rows in got.values() for times in rows.values())


def test_replay_on_the_plain_kernel_set(setups, tmp_path):
    """--kernels plain: the same trace on the general kernels; both runs meet the bound, and they
    are not bit-equal in bfloat16 (the fast kernels did run in the default one)."""
    d, cfg, reqs, oracle = setups["D"]
    steps = with_positions(traces.mixed(reqs, seed=4))
    clean = [{"step": s["step"], "entries": [{k: v for k, v in e.items() if k != "_pos0"} for e in s["entries"]],
              "end": s["end"]} for s in steps]
    outs = {}
    for kernels in ("fast", "plain"):
        out_dir = str(tmp_path / kernels)
        replay(d, "bfloat16", clean, out_dir, traces.peak_tokens(steps), extra=("--kernels", kernels))
        outs[kernels] = gather(steps, out_dir, cfg["vocab_size"])
        for r, rows in outs[kernels].items():
            for pos, times in rows.items():
                assert np.abs(times[0].astype(np.float64) - oracle[r][pos].numpy()).max() <= ATOL["bfloat16"]
    differ = sum(not np.array_equal(outs["fast"][r][p][0], outs["plain"][r][p][0]) for r in outs["fast"] for p in outs["fast"][r])
    assert differ > 0
