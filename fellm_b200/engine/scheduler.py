"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

FeLLM's scheduler (crates/fellm-runtime/src/scheduler.rs) keeps waiting and running deques
(156-166,238-246), admits FIFO while pages are free (728-786), plans every iteration as all
decodes first, then prompt portions in order of age, `count = min(remaining, budget left,
n_ubatch)` under `n_batch` tokens (88-152; 415-469), samples, emits Token / Done / Error events
(381-492), and finishes on a stop token, `max_tokens` or the end of the context (706-724).  A
hybrid model's portion is clamped to one token there (423-427); here portions of any length run.

When pages run out (FeLLM: every sequence of the batch gets an Error event, 644-665):
  1. at admission a request waits (FIFO, the head blocks the rest);
  2. a planned batch that the pool cannot cover is shrunk: prompt portions are shortened or
     dropped, newest request first;
  3. if the decodes alone do not fit, the newest running request is preempted: its pages and slot
     are given back and it returns to the FRONT of the waiting queue with prompt + generated
     tokens as its new prompt (recomputed later; its sampled tokens stay as they are);
  4. a request that could never fit (prompt + max_tokens beyond the context, or more pages than
     the pool has) is refused at enqueue with SchedulerError.
No request fails because another one needed pages.

One step ahead: while the requests that decode together stay the same, the next step is launched
before the tokens of the last one have been read (its inputs are the sampled tokens where they
lie on the device), so the host's work on a step overlaps the device's work on the next.  A
request that ends on a stop token has then run one token too many; that token is dropped and the
request's pages go back as usual (the launch that frees them for another request comes later in
the stream).  Ends that the host can foresee (max_tokens, the end of the context) are not run ahead.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence

from ..config.errors import SchedulerError
from ..sampling.params import GenParams, GenStats
from .step import StepItem


@dataclass
class Event:
    """kind: 'token' (token set), 'done' (stats set, reason in stats.finish_reason), 'error'."""
    kind: str
    req: int
    token: Optional[int] = None
    stats: Optional[GenStats] = None
    message: str = ""


@dataclass(eq=False)                  # a request is itself: `r in running` must not compare prompts
class Request:
    id: int
    prompt: List[int]                 # what has to be in the cache before the next sample
    params: GenParams
    n_prompt_orig: int
    generated: List[int] = field(default_factory=list)
    fed: int = 0                      # tokens of `prompt` already run
    pending: Optional[int] = None     # sampled token not yet run (decode input)
    draws: int = 0
    t_enqueue: float = 0.0
    t_first: Optional[float] = None
    preemptions: int = 0
    seq: int = 0                      # admission order (age)

    @property
    def prefilling(self) -> bool:
        return self.fed < len(self.prompt)


@dataclass
class PlanItem:
    req: Request
    n_tokens: int
    decode: bool


@dataclass
class InFlight:
    """A launched step whose tokens have not been read yet."""
    handle: object
    plan: List[PlanItem]
    samplers: List[Request]
    dropped: set = field(default_factory=set)     # ids of requests that ended while this step ran ahead


def plan_batch(running: Sequence[Request], n_batch: int, n_ubatch: int) -> List[PlanItem]:
    """Decode-first, then prompt portions by priority and age, under n_batch tokens
    (scheduler.rs:88-152)."""
    order = sorted(running, key=lambda r: (-r.params.priority, r.seq))
    plan: List[PlanItem] = []
    budget = n_batch
    for r in order:
        if not r.prefilling and r.pending is not None and budget > 0:
            plan.append(PlanItem(r, 1, True))
            budget -= 1
    for r in order:
        if r.prefilling and budget > 0:
            n = min(len(r.prompt) - r.fed, budget, n_ubatch)
            plan.append(PlanItem(r, n, False))
            budget -= n
    return plan


class Scheduler:
    """`backend` provides: .cache (CacheManager), .n_ctx, .start_request(slot, prompt, params) and
    .run(items, sample_rows) -> host token list for the rows that asked for a sample; or, to run
    one step ahead, .launch(items, sample_rows, chain) -> handle and .collect(handle) -> host token
    list (chain: the items' tokens are the last launch's samples, in order, still on the device)."""

    def __init__(self, backend, n_batch: int, n_ubatch: int, lookahead: bool = True):
        self.backend, self.cache = backend, backend.cache
        self.n_batch, self.n_ubatch = int(n_batch), int(n_ubatch)
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []
        self.events: Deque[Event] = deque()
        self.lookahead = bool(lookahead) and hasattr(backend, "launch")
        self.inflight: Optional[InFlight] = None
        self._next_id, self._next_seq = 0, 0
        self.counters = {"requests": 0, "admitted": 0, "preempted": 0, "finished": 0, "steps": 0,
                         "shrunk": 0, "tokens_run": 0, "admission_waits": 0, "ran_ahead": 0, "dropped": 0,
                         "mixed_steps": 0}

    # ---- enqueue / cancel
    def enqueue_ids(self, ids: Sequence[int], params: Optional[GenParams] = None) -> int:
        params = params or GenParams()
        ids = [int(t) for t in ids]
        if not ids:
            raise SchedulerError("a request needs at least one prompt token")
        total = len(ids) + max(params.max_tokens, 0)
        if len(ids) + 1 > self.backend.n_ctx:
            raise SchedulerError(f"a prompt of {len(ids)} tokens does not fit the context of {self.backend.n_ctx}")
        pages_alone = -(-min(total, self.backend.n_ctx) // self.cache.page_tokens)
        if self.cache.paged and pages_alone > self.cache.n_pages:
            raise SchedulerError(f"the request needs {pages_alone} cache pages by itself; the pool has "
                                 f"{self.cache.n_pages}")
        rid = self._next_id
        self._next_id += 1
        self.waiting.append(Request(rid, ids, params, len(ids), t_enqueue=time.perf_counter()))
        self.counters["requests"] += 1
        return rid

    def cancel(self, rid: int) -> bool:
        for r in list(self.waiting):
            if r.id == rid:
                self.waiting.remove(r)
                return True
        for r in self.running:
            if r.id == rid:
                self._finish(r, "cancelled")
                if self.inflight is not None:
                    self.inflight.dropped.add(rid)
                return True
        return False

    def idle(self) -> bool:
        return not self.waiting and not self.running and self.inflight is None

    # ---- admission
    def _admit(self):
        while self.waiting:
            r = self.waiting[0]
            if not self.cache.can_admit():
                self.counters["admission_waits"] += 1
                return
            # FeLLM admits on room for one token (scheduler.rs:728-786) and fails the batch when pages run out
            # mid-run; here a request that does not fit is preempted and recomputed, so one is admitted beside
            # running requests only when its whole prompt (which for a preempted request includes what it had
            # generated) and one token more fit the free pages: admitted on less it is cut page by page, dropped
            # and preempted again, each time with its prompt to run anew (measured on a pool of 45 pages under 40
            # slots: 1,624 preemptions and 31% more tokens run than the requests hold with the one-token rule, 1,150 and
            # 26% with this one)
            need = -(-(len(r.prompt) + 1) // self.cache.page_tokens) if self.cache.paged else 0
            if need > self.cache.free_pages() and self.running:
                self.counters["admission_waits"] += 1
                return                                  # waits; the head of the queue blocks the rest
            self.waiting.popleft()
            slot = self.cache.add_request(r.id)
            r.seq = self._next_seq
            self._next_seq += 1
            self.backend.start_request(slot, r.prompt, r.params)
            self.running.append(r)
            self.counters["admitted"] += 1

    # ---- making the batch fit
    def _fit(self, plan: List[PlanItem]) -> List[PlanItem]:
        while plan:
            if self.cache.can_reserve([(p.req.id, p.n_tokens) for p in plan]):
                return plan
            prefills = [p for p in plan if not p.decode]
            if prefills:
                victim = max(prefills, key=lambda p: p.req.seq)          # newest first
                self.counters["shrunk"] += 1
                others = [(p.req.id, p.n_tokens) for p in plan if p is not victim]
                n, pt, have = victim.n_tokens, self.cache.page_tokens, self.cache.length(victim.req.id)
                while n > 0 and not self.cache.can_reserve(others + [(victim.req.id, n)]):
                    n = max(((have + n - 1) // pt) * pt - have, 0)      # one page fewer
                if n > 0:
                    victim.n_tokens = n
                    return plan
                plan.remove(victim)
                continue
            victim = max(self.running, key=lambda r: r.seq)
            self._preempt(victim)
            plan = [p for p in plan if p.req is not victim]
        return plan

    def _preempt(self, r: Request):
        self.cache.release(r.id)
        self.running.remove(r)
        # the last generated token is the pending decode input: it becomes the new prompt's end,
        # and the sample after it is the request's next token
        r.prompt = r.prompt[:r.n_prompt_orig] + r.generated
        r.fed, r.pending = 0, None
        r.preemptions += 1
        self.waiting.appendleft(r)
        self.counters["preempted"] += 1

    # ---- one iteration
    def step(self) -> List[Event]:
        """Runs one batch (if anything can run); returns, and removes from the queue, every event
        queued so far."""
        self._iterate()
        out = list(self.events)
        self.events.clear()
        return out

    def _iterate(self):
        cur = self.inflight
        self.inflight = None
        if cur is None:
            cur = self._launch()
            if cur is None:
                return
        if self.lookahead:
            self.inflight = self._launch_ahead(cur)
        self._collect(cur)

    def _launch(self) -> Optional[InFlight]:
        """Plans a batch from what the host knows and launches it."""
        self._admit()
        plan = self._fit(plan_batch(self.running, self.n_batch, self.n_ubatch))
        if not plan:
            if self.waiting and not self.running:
                # nothing runs and the head cannot be admitted: it can never fit
                r = self.waiting.popleft()
                self.events.append(Event("error", r.id, message="request cannot be placed in the cache"))
            return None
        items, sample_rows, samplers = [], [], []
        for p in plan:
            r = p.req
            if p.decode:
                toks = [r.pending]
                wants = True
            else:
                toks = r.prompt[r.fed:r.fed + p.n_tokens]
                wants = r.fed + p.n_tokens == len(r.prompt)
            items.append(StepItem(r.id, toks, [len(toks) - 1] if wants else []))
            if wants:
                sample_rows.append((self.cache.slot(r.id), r.params, r.draws))
                samplers.append(r)
        try:
            if self.lookahead:
                handle = self.backend.launch(items, sample_rows, False)
            else:
                handle = self.backend.run(items, sample_rows)
        except Exception as e:                          # a failed launch ends the batch's requests
            for p in plan:
                self._finish(p.req, "error", error=str(e))
            raise
        self.counters["steps"] += 1
        self.counters["tokens_run"] += sum(p.n_tokens for p in plan)
        if any(p.decode for p in plan) and not all(p.decode for p in plan):
            self.counters["mixed_steps"] += 1             # prompt portions beside decode tokens
        for p in plan:
            if p.decode:
                p.req.pending = None
            else:
                p.req.fed += p.n_tokens
        return InFlight(handle, plan, samplers)

    def _launch_ahead(self, cur: InFlight) -> Optional[InFlight]:
        """The step after `cur`, launched before cur's tokens are read: only when it is the same
        requests decoding one more token each, none of which the host can see ending, with nobody
        waiting for admission and a page for everyone who needs one."""
        if self.waiting or cur.dropped or len(cur.samplers) != len(cur.plan) or len(cur.plan) != len(self.running):
            return None
        n_ctx = self.backend.n_ctx
        for r in cur.samplers:
            if r.prefilling or r.pending is not None:
                return None
            # after cur: len(generated) + 1 tokens; the request goes on only if that is not its end
            if len(r.generated) + 1 >= r.params.max_tokens or self.cache.length(r.id) + 1 >= n_ctx:
                return None
        if not self.cache.can_reserve([(r.id, 1) for r in cur.samplers]):
            return None
        items = [StepItem(r.id, [0], [0]) for r in cur.samplers]          # the tokens are on the device
        sample_rows = [(self.cache.slot(r.id), r.params, r.draws + 1) for r in cur.samplers]
        try:
            handle = self.backend.launch(items, sample_rows, True)
        except Exception:                                # decided again, with the tokens known, after the collect
            return None
        self.counters["steps"] += 1
        self.counters["ran_ahead"] += 1
        self.counters["tokens_run"] += len(items)
        return InFlight(handle, [PlanItem(r, 1, True) for r in cur.samplers], list(cur.samplers))

    def _collect(self, cur: InFlight):
        """Reads a launched step's tokens and does the bookkeeping that follows from them."""
        try:
            tokens = self.backend.collect(cur.handle) if self.lookahead else cur.handle
        except Exception as e:
            ahead, self.inflight = self.inflight, None
            for p in cur.plan:
                if p.req in self.running:
                    self._finish(p.req, "error", error=str(e))
            if ahead is not None:
                try:
                    self.backend.collect(ahead.handle)
                except Exception:
                    pass
            raise
        ahead = self.inflight
        now = time.perf_counter()
        for r, tok in zip(cur.samplers, tokens):
            if r.id in cur.dropped:                      # ended on a stop token while this step ran ahead
                self.counters["dropped"] += 1
                continue
            tok = int(tok)
            r.draws += 1
            if r.t_first is None:
                r.t_first = now
            r.generated.append(tok)
            self.events.append(Event("token", r.id, token=tok))
            length = self.cache.length(r.id) - (1 if ahead is not None else 0)      # as it was after this step
            if tok in r.params.stop_token_ids:
                self._finish(r, "stop")
            elif len(r.generated) >= r.params.max_tokens:
                self._finish(r, "length")
            elif length + 1 >= self.backend.n_ctx:          # scheduler.rs:706-724: position+1 >= n_ctx
                self._finish(r, "length")
            elif ahead is None:
                r.pending = tok
            # else: the token is already being run by the step ahead
            if ahead is not None and r not in self.running:
                ahead.dropped.add(r.id)

    def _finish(self, r: Request, reason: str, error: str = ""):
        if r in self.running:
            self.running.remove(r)
            if self.cache.has(r.id):
                self.cache.release(r.id)
        now = time.perf_counter()
        t_first = r.t_first if r.t_first is not None else now
        stats = GenStats(prompt_tokens=r.n_prompt_orig, predicted_tokens=len(r.generated),
                         prompt_ms=(t_first - r.t_enqueue) * 1e3, total_ms=(now - r.t_enqueue) * 1e3,
                         time_to_first_token_ms=(t_first - r.t_enqueue) * 1e3, finish_reason=reason)
        self.counters["finished"] += 1
        if reason == "error":
            self.events.append(Event("error", r.id, stats=stats, message=error))
        else:
            self.events.append(Event("done", r.id, stats=stats))

    def poll_event(self, reqs=None) -> Optional[Event]:
        """The next event, running iterations until there is one; None when all work is done.

        reqs: a request id or a collection of ids: the next event of THOSE requests; events of
        other requests stay queued, in order, for whoever asks for them (two token streams, or a
        stream beside generate_batch, each read their own and lose nothing)."""
        if reqs is None:
            while not self.events:
                if self.idle():
                    return None
                self._iterate()
            return self.events.popleft()
        mine = {reqs} if isinstance(reqs, int) else set(reqs)
        scanned = 0
        while True:
            for i in range(scanned, len(self.events)):
                if self.events[i].req in mine:
                    ev = self.events[i]
                    del self.events[i]
                    return ev
            scanned = len(self.events)
            if self.idle():
                return None
            self._iterate()
