"""Ways of cutting the same requests into steps, in the replay tool's step format
``{"step": n, "entries": [{"id", "tokens", "want"}], "end": [...]}``, and helpers
to run such a trace and gather each request's logits by position."""
from __future__ import annotations

import random
from typing import Dict, List

import torch

from arle_b200.engine import StepEntry


def make_requests(vocab: int, lengths, seed: int = 0) -> Dict[str, List[int]]:
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def _step(n, entries, end=()):
    return {"step": n, "entries": entries, "end": list(end)}


def _entry(rid, toks):
    return {"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}


def whole(requests) -> list:
    """Each request alone, its whole sequence in one step."""
    return [_step(i, [_entry(r, t)], [r]) for i, (r, t) in enumerate(requests.items())]


def tail_decode(requests, tail: int = 32) -> list:
    """Most of the sequence in one step, the last ``tail`` tokens one by one."""
    steps = []
    for r, t in requests.items():
        cut = max(1, len(t) - tail)
        steps.append(_step(len(steps), [_entry(r, t[:cut])]))
        for i in range(cut, len(t)):
            steps.append(_step(len(steps), [_entry(r, t[i:i + 1])], [r] if i == len(t) - 1 else []))
        if cut == len(t):
            steps[-1]["end"] = [r]
    return steps


def portions(requests, sizes=(7, 2, 13, 2, 5, 3, 17, 2, 64, 9)) -> list:
    """Portions of changing size, down to two tokens."""
    steps = []
    for r, t in requests.items():
        at, k = 0, 0
        while at < len(t):
            n = min(sizes[k % len(sizes)], len(t) - at)
            at += n
            k += 1
            steps.append(_step(len(steps), [_entry(r, t[at - n:at])], [r] if at == len(t) else []))
    return steps


def mixed(requests, seed: int = 0, max_live: int = 4, tail: int = 8) -> list:
    """Up to ``max_live`` requests at a time; each step takes a random subset of the
    live ones and gives a portion (2..19 tokens) to those still in their prompt and
    one token to those in their last ``tail`` tokens.  Finished requests end, and
    the next ones start on the pages they gave back."""
    rng = random.Random(seed)
    todo = list(requests)
    live, done_upto = [], {}
    steps = []
    while todo or live:
        while todo and len(live) < max_live:
            r = todo.pop(0)
            live.append(r)
            done_upto[r] = 0
        chosen = [r for r in live if rng.random() < 0.75] or [rng.choice(live)]
        entries, end = [], []
        for r in chosen:
            t, at = requests[r], done_upto[r]
            left = len(t) - at
            n = 1 if left <= tail else min(left - tail, rng.choice([2, 2, 3, 5, 8, 13, 19]))
            if left > tail and left - tail - n == 1:
                n += 1                       # never leave a one-token prompt portion
            entries.append(_entry(r, t[at:at + n]))
            done_upto[r] = at + n
            if at + n == len(t):
                end.append(r)
        steps.append(_step(len(steps), entries, end))
        live = [r for r in live if r not in end]
    return steps


def preempted(requests, victim: str = None, tail: int = 6) -> list:
    """Every request runs as a portion and then token by token, up to three at a time; the
    ``victim`` (the longest request by default) is ended half-way through, its pages go to the
    others, and later it starts again from its first token under the same name, as a scheduler
    that preempts by recomputation would have it.  Logits are wanted everywhere, so the victim's
    early positions come out twice."""
    names = list(requests)
    victim = victim or max(names, key=lambda r: len(requests[r]))
    steps = []

    def run(rids, stop_victim_at=None):
        upto = {r: 0 for r in rids}
        live = list(rids)
        while live:
            entries, end = [], []
            for r in list(live):
                t, at = requests[r], upto[r]
                left = len(t) - at
                n = 1 if left <= tail or at > 0 and left <= tail + 3 else max(2, min(left - tail, 11 if at else left - tail))
                entries.append(_entry(r, t[at:at + n]))
                upto[r] = at + n
                if upto[r] == len(t) or (r == victim and stop_victim_at is not None and upto[r] >= stop_victim_at):
                    end.append(r)
                    live.remove(r)
            steps.append(_step(len(steps), entries, end))

    first = [r for r in names if r != victim][:2]
    run([victim] + first, stop_victim_at=max(2, len(requests[victim]) // 2))
    rest = [r for r in names if r != victim and r not in first]
    run(rest[:1] + [victim] + rest[1:2])
    run(rest[2:])
    return steps


def peak_tokens(steps, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count
    rounded up to a multiple of ``round_to`` (the replay tool's --max-tokens)."""
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for r in s["end"]:
            held.pop(r, None)
    return peak


def run_trace(runner, steps) -> Dict[str, torch.Tensor]:
    """Feeds the steps to a ModelRunner; returns per request the logits of every
    wanted place, in position order."""
    got: Dict[str, list] = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = runner.step(entries)
        at = 0
        for e in s["entries"]:
            n = len(e["want"])
            if n:
                got.setdefault(e["id"], []).append(logits[at:at + n].detach().float().cpu().clone())
            at += n
        for r in s["end"]:
            runner.end_request(r)
    return {r: torch.cat(v) for r, v in got.items()}


def run_trace_by_position(runner, steps) -> list:
    """Like ``run_trace`` for traces in which a request may start again after it ended:
    returns (request, position, logits row) for every wanted place, in the order they came."""
    out, held = [], {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]
        logits = runner.step(entries)
        at = 0
        for e in s["entries"]:
            base = held.get(e["id"], 0)
            for k, w in enumerate(e["want"]):
                out.append((e["id"], base + w, logits[at + k].detach().float().cpu().clone()))
            at += len(e["want"])
            held[e["id"]] = base + len(e["tokens"])
        for r in s["end"]:
            runner.end_request(r)
            held.pop(r, None)
    return out
