"""Continuous-batching scheduler: admits requests, cuts prompts into portions under
a token budget, decodes, finishes and frees.  Pure host logic over the cache
manager's bookkeeping; it never touches a tensor, so its decisions are tested
without a GPU.

Policies, and where cklxx/arle has the same:

* Every request is a token list (prompt + generated) of which ``num_computed`` are
  in the cache; a step gives it its next tokens.  A request with exactly one token
  left is a *decode row*; all decode rows run every step
  (infer/src/scheduler/cuda/decode.rs:29-50).
* Token budget: a step runs at most ``max_num_batched_tokens`` tokens; what the
  decode rows leave, capped by ``max_prefill_tokens``, goes to prompt portions in
  arrival order, each at most ``chunked_prefill_size``
  (infer/src/scheduler/cuda/budget.rs:242-254; execution.rs:265-317).  A portion
  that does not fit the rest of the budget is cut to fit (the reference skips it).
* Admission, first come first served: a waiting request is admitted when a slot
  is free and every cache group has pages for its tokens + 1 beyond what the
  already admitted prompts still need (scheduler_loop.rs:229-313).
* ``scheduler_mixed_policy``: "mixed" runs decode rows and portions in one step;
  "split" (the reference's default, scheduler/types.rs:204) runs the portions,
  then the decode rows, as two steps of the same tick.
* Pages run out: before decode rows are planned, while the pages they need exceed
  the free ones, the request with the fewest generated tokens (ties: the longest
  prompt) is preempted: its pages and slot are freed and it goes back to the
  FRONT of the waiting queue (decode.rs:82-116, :145-184).  Unlike the reference,
  which restarts from the prompt and samples again, the preempted request keeps
  its generated tokens and recomputes them as part of its prompt, so its output
  is unchanged.  A lone request that cannot grow is finished with reason
  "length".
* A step may be launched before the tokens of the step before it are known on the host:
  ``on_launch`` appends a placeholder (-1) for every token that step will sample, so the
  next ``schedule`` can plan the following decode rows (whose token the device hands over
  itself), and ``on_step_done`` fills the placeholders in when the tokens arrive.  cklxx/arle
  overlaps launch and readback the same way (scheduler/cuda/execution.rs:677-709).  A stop
  token is therefore seen one step late: the extra step's token is dropped.
* Finish: a sampled stop token (the model's and the request's, unless
  ``ignore_eos``) ends the request with "stop" and is not emitted
  (decode.rs:785-791); ``max_new_tokens`` generated, or the most tokens a request
  may hold, ends it with "length" (prefill.rs:550-619).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..sampling.params import SamplingParams


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 16384
    chunked_prefill_size: int = 16384
    max_prefill_tokens: Optional[int] = None          # None: chunked_prefill_size
    prefill_max_requests: Optional[int] = None        # None: the token budget alone decides
    scheduler_mixed_policy: str = "mixed"             # "mixed" | "split"
    max_waiting_requests: int = 256

    def validate(self) -> None:
        if self.max_num_batched_tokens <= 0 or self.chunked_prefill_size <= 0:
            raise ValueError("max_num_batched_tokens and chunked_prefill_size must be positive")
        if self.max_prefill_tokens is not None and self.max_prefill_tokens <= 0:
            raise ValueError("max_prefill_tokens must be positive")
        if self.scheduler_mixed_policy not in ("mixed", "split"):
            raise ValueError("scheduler_mixed_policy must be 'mixed' or 'split'")


@dataclass
class Request:
    rid: object
    prompt: List[int]
    params: SamplingParams
    max_new_tokens: int
    number: int = 0
    tokens: List[int] = field(default_factory=list)    # prompt + generated
    output: List[int] = field(default_factory=list)
    num_computed: int = 0
    finish_reason: Optional[str] = None
    preemptions: int = 0
    unresolved: Deque[int] = field(default_factory=deque)   # places in ``tokens`` whose sampled token is still on its way
    closed: bool = False                                     # its last token has been launched; it is not scheduled again

    @property
    def remaining(self) -> int:
        return len(self.tokens) - self.num_computed


@dataclass
class PlannedEntry:
    request: Request
    start: int
    count: int
    samples: bool = False      # the portion reaches the request's last known token: a token is sampled

    def __post_init__(self):
        self.samples = self.start + self.count == len(self.request.tokens)

    @property
    def tokens(self) -> List[int]:
        return self.request.tokens[self.start:self.start + self.count]


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    launched: bool = False

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


class Scheduler:
    def __init__(self, cache, config: SchedulerConfig, stop_token_ids: Sequence[int] = (),
                 default_max_new_tokens: int = 256):
        config.validate()
        self.cache = cache
        self.cfg = config
        self.stop_ids = frozenset(int(t) for t in stop_token_ids)
        self.default_max_new_tokens = default_max_new_tokens
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.finished: List[Request] = []
        self._count = 0
        self.stats = {"steps": 0, "preemptions": 0, "admitted": 0, "finished": 0, "prefill_tokens": 0,
                      "decode_tokens": 0}

    # ----------------------------------------------------------------- intake
    def max_request_tokens(self) -> int:
        """Most tokens one request may hold: the cache manager's per-request limit
        and what the smallest cache group can hold at all."""
        pool = min(self.cache.total_pages()) * self.cache.page_size
        return min(self.cache.max_tokens_per_request, pool)

    def add_request(self, rid, prompt: Sequence[int], params: SamplingParams = None) -> Request:
        params = params or SamplingParams()
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        limit = self.max_request_tokens()
        if len(prompt) >= limit:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit: a request may hold {limit} tokens "
                             f"(context length and cache size)")
        if len(self.waiting) >= self.cfg.max_waiting_requests:
            raise RuntimeError(f"waiting queue is full ({self.cfg.max_waiting_requests})")
        want = params.max_new_tokens if params.max_new_tokens is not None else self.default_max_new_tokens
        req = Request(rid, prompt, params, max(0, min(want, limit - len(prompt))), self._count, list(prompt))
        self._count += 1
        if req.max_new_tokens == 0:
            req.finish_reason = "length"
            self.finished.append(req)
            self.stats["finished"] += 1
        else:
            self.waiting.append(req)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # --------------------------------------------------------------- planning
    def _free(self) -> List[int]:
        return list(self.cache.free_pages())

    def _victim(self, exclude=()) -> Optional[Request]:
        cands = [r for r in self.running if r not in exclude]
        if not cands:
            return None
        return min(cands, key=lambda r: (len(r.output), -len(r.prompt), -r.number))

    def _preempt(self, req: Request) -> None:
        self.cache.free_request(req.rid)
        self.running.remove(req)
        req.num_computed = 0
        req.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(req)

    def _finish(self, req: Request, reason: str) -> None:
        if req.finish_reason is not None:
            return
        req.finish_reason = reason
        if self.cache.has_request(req.rid):
            self.cache.free_request(req.rid)
        if req in self.running:
            self.running.remove(req)
        if req in self.waiting:
            self.waiting.remove(req)
        self.finished.append(req)
        self.stats["finished"] += 1

    def _admit(self, reserved: List[int]) -> None:
        """Move waiting requests to running while a slot is free and their tokens + 1
        fit beyond ``reserved`` (pages already promised per group)."""
        while self.waiting and self.cache.num_free_slots > 0:
            req = self.waiting[0]
            need = self.cache.pages_for_new_request(len(req.tokens) + 1)
            free = self._free()
            if any(n + r > f for n, r, f in zip(need, reserved, free)):
                break
            self.waiting.popleft()
            self.cache.add_request(req.rid)
            self.running.append(req)
            self.stats["admitted"] += 1
            for g, n in enumerate(need):
                reserved[g] += n

    def _fit_tokens(self, req: Request, want: int, avail: List[int]) -> int:
        """Largest n <= want whose pages fit ``avail`` (free minus promised)."""
        def fits(n):
            return all(p <= a for p, a in zip(self.cache.pages_needed(req.rid, n), avail))

        if want <= 0 or fits(want):
            return max(want, 0)
        lo, hi = 0, want                      # fits(lo), not fits(hi); pages needed grow with n
        while hi - lo > 1:
            mid = (lo + hi) // 2
            lo, hi = (mid, hi) if fits(mid) else (lo, mid)
        return lo

    def schedule(self) -> List[StepPlan]:
        """Plans of this tick: one mixed step, or (policy "split") a step of prompt
        portions followed by a step of decode rows.  Empty when nothing can run."""
        ngroups = len(self.cache.free_pages())
        # 1. decode rows, making room by preemption
        while True:
            decode = [r for r in self.running if r.remaining == 1]
            need = [0] * ngroups
            for r in decode:
                for g, p in enumerate(self.cache.pages_needed(r.rid, 1)):
                    need[g] += p
            if all(n <= f for n, f in zip(need, self._free())):
                break
            victim = self._victim()
            if len(self.running) == 1:
                self._finish(victim, "length")      # alone and still no room: the cache is too small
            else:
                self._preempt(victim)
        promised = list(need)
        # 2. admitted prompts still to run keep their pages promised; then admit more
        prefill = [r for r in self.running if r.remaining > 1]
        reserved = list(promised)
        for r in prefill:
            for g, p in enumerate(self.cache.pages_needed(r.rid, r.remaining + 1)):
                reserved[g] += p
        before = len(self.running)
        self._admit(reserved)
        prefill += [r for r in self.running[before:] if r.remaining > 1]
        decode += [r for r in self.running[before:] if r.remaining == 1]
        if len(self.running) > before:
            for r in self.running[before:]:
                if r.remaining == 1:
                    for g, p in enumerate(self.cache.pages_needed(r.rid, 1)):
                        promised[g] += p
        # 3. portions under the token budget
        budget = self.cfg.max_num_batched_tokens - len(decode)
        budget = min(budget, self.cfg.max_prefill_tokens or self.cfg.chunked_prefill_size)
        avail = [f - p for f, p in zip(self._free(), promised)]
        portions: List[PlannedEntry] = []
        for r in prefill:
            if budget <= 0:
                break
            if self.cfg.prefill_max_requests is not None and len(portions) >= self.cfg.prefill_max_requests:
                break
            n = self._fit_tokens(r, min(r.remaining, self.cfg.chunked_prefill_size, budget), avail)
            if n <= 0:
                continue
            for g, p in enumerate(self.cache.pages_needed(r.rid, n)):
                avail[g] -= p
            portions.append(PlannedEntry(r, r.num_computed, n))
            budget -= n
        rows = [PlannedEntry(r, r.num_computed, 1) for r in decode]
        if not rows and not portions:
            if not self.running:
                return []
            # admitted prompts that cannot get a single page: the youngest gives way
            if len(self.running) > 1:
                self._preempt(self._victim())
            else:
                self._finish(self.running[0], "length")
            return self.schedule()
        if self.cfg.scheduler_mixed_policy == "split" and rows and portions:
            return [StepPlan(portions), StepPlan(rows)]
        return [StepPlan(rows + portions)]

    # ---------------------------------------------------------------- results
    def on_launch(self, plan: StepPlan) -> None:
        """The plan's step has been handed to the device.  Its tokens count as computed,
        and every token it will sample is entered as a placeholder (-1) to be filled in by
        ``on_step_done``.  A request whose last token this is (``max_new_tokens``, or the
        most tokens a request may hold) leaves the running set and gives its cache back
        now: whatever is launched later runs after this step on the device."""
        plan.launched = True
        self.stats["steps"] += 1
        limit = self.max_request_tokens()
        for e in plan.entries:
            r = e.request
            r.num_computed += e.count
            if e.count == 1 and r.output:
                self.stats["decode_tokens"] += 1
            else:
                self.stats["prefill_tokens"] += e.count
            if not e.samples:
                continue
            r.unresolved.append(len(r.tokens))
            r.tokens.append(-1)
            r.output.append(-1)
            if len(r.output) >= r.max_new_tokens or len(r.tokens) >= limit:
                r.closed = True
                if r in self.running:
                    self.running.remove(r)
                if self.cache.has_request(r.rid):
                    self.cache.free_request(r.rid)

    def on_step_done(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        """``sampled``: one token per entry of the plan that ``samples``, in order.
        Returns the requests that finished."""
        if not plan.launched:
            self.on_launch(plan)
        done = []
        it = iter(sampled)
        for e in plan.entries:
            if not e.samples:
                continue
            tok = int(next(it))
            r = e.request
            if r.finish_reason == "stop" or not r.unresolved:
                continue                                    # a token sampled past a stop token: dropped
            at = r.unresolved.popleft()
            stops = self.stop_ids | set(r.params.stop_token_ids)
            if not r.params.ignore_eos and tok in stops:
                del r.tokens[at:]                           # the stop token is not emitted, nor anything after it
                del r.output[at - len(r.prompt):]
                r.unresolved.clear()
                self._finish(r, "stop")
                done.append(r)
                continue
            r.tokens[at] = tok
            r.output[at - len(r.prompt)] = tok
            if r.closed and not r.unresolved:
                was_open = r.finish_reason is None
                self._finish(r, "length")
                if was_open:
                    done.append(r)
        return done
