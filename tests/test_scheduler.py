"""The scheduler's decisions, without a GPU: a fake backend stands in for the model (it returns
a token that is a function of the request's whole history, so a recomputed request must reproduce
its tokens) over the real cache manager on CPU tensors."""
import pytest
import torch

from fellm_b200.cache import CacheManager
from fellm_b200.config import SchedulerError
from fellm_b200.engine.scheduler import Request, Scheduler, plan_batch
from fellm_b200.parts.base import FixedState, PagedKV
from fellm_b200.sampling import GenParams


class FakeBackend:
    def __init__(self, page_tokens=4, max_tokens=64, max_requests=4, n_ctx=64):
        self.cache = CacheManager([FixedState((2, 4)), PagedKV(1, 16, None)], page_tokens=page_tokens,
                                  max_tokens=max_tokens, max_requests=max_requests, n_ctx=n_ctx,
                                  dtype=torch.float32, device="cpu")
        self.n_ctx = n_ctx
        self.history = {}          # request -> every token run so far
        self.batches = []

    def start_request(self, slot, prompt, params):
        pass

    def run(self, items, sample_rows):
        self.batches.append([(it.req, len(it.tokens), bool(it.want)) for it in items])
        out = []
        for it in items:
            if self.cache.length(it.req) == 0:
                self.history[it.req] = []
            self.cache.reserve(it.req, len(it.tokens))
            self.cache.advance(it.req, len(it.tokens))
            self.history[it.req] += list(it.tokens)
            if it.want:
                h = self.history[it.req]
                out.append((sum(h) * 31 + len(h) * 7) % 97 + 3)
        self.cache.audit()
        assert len(out) == len(sample_rows)
        return out


def run_all(sched, limit=10_000):
    toks, done = {}, {}
    for _ in range(limit):
        ev = sched.poll_event()
        if ev is None:
            break
        if ev.kind == "token":
            toks.setdefault(ev.req, []).append(ev.token)
        elif ev.kind == "done":
            done[ev.req] = ev.stats
        else:
            raise AssertionError(ev)
    return toks, done


def G(n, **kw):
    return GenParams.greedy(n, **kw)


def test_plan_decode_first_then_prefill_by_age_under_budget():
    # scheduler.rs:930-1004: decode-first, then chunked prefill, never above the budget
    def req(i, prompt, fed, pending=None, prio=0):
        r = Request(i, list(range(prompt)), G(8, priority=prio), prompt, fed=fed, pending=pending)
        r.seq = i
        return r
    running = [req(0, 40, 0), req(1, 10, 10, pending=5), req(2, 30, 8), req(3, 6, 6, pending=9)]
    plan = plan_batch(running, n_batch=24, n_ubatch=16)
    assert [(p.req.id, p.n_tokens, p.decode) for p in plan] == [(1, 1, True), (3, 1, True), (0, 16, False), (2, 6, False)]
    assert sum(p.n_tokens for p in plan) == 24
    plan = plan_batch(running, n_batch=1, n_ubatch=16)
    assert [(p.req.id, p.decode) for p in plan] == [(1, True)]
    running[2].params.priority = 5
    plan = plan_batch(running, n_batch=24, n_ubatch=16)
    assert [p.req.id for p in plan] == [1, 3, 2, 0]


def test_portions_and_mixed_batches():
    b = FakeBackend()
    s = Scheduler(b, n_batch=12, n_ubatch=8)
    r0 = s.enqueue_ids(list(range(1, 20)), G(3))
    evs = s.step()
    assert b.batches[-1] == [(r0, 8, False)]
    r1 = s.enqueue_ids([5, 6, 7], G(2))
    evs += s.step()
    assert b.batches[-1] == [(r0, 8, False), (r1, 3, True)]         # budget 12: 8 + 3
    evs += s.step()
    assert b.batches[-1] == [(r1, 1, True), (r0, 3, True)]          # decode first, then the last portion
    toks, done = run_all(s)
    done.update({e.req: e.stats for e in evs if e.kind == "done"})
    assert set(done) == {r0, r1} and done[r0].finish_reason == "length"
    assert done[r0].prompt_tokens == 19 and done[r0].predicted_tokens == 3
    assert b.cache.free_pages() == b.cache.n_pages and b.cache.slots.free_count == 4


def test_finish_reasons_and_release():
    b = FakeBackend(n_ctx=16)
    s = Scheduler(b, 64, 64)
    a = s.enqueue_ids([1, 2, 3], G(50))                    # runs into the end of the context
    toks, done = run_all(s)
    assert done[a].finish_reason == "length" and 3 + len(toks[a]) == 16
    first = (sum([1, 2, 3]) * 31 + 3 * 7) % 97 + 3
    c = s.enqueue_ids([1, 2, 3], G(50, stop_token_ids=(first,)))
    toks, done = run_all(s)
    assert done[c].finish_reason == "stop" and toks[c] == [first]
    assert b.cache.free_pages() == b.cache.n_pages


def test_refused_at_enqueue():
    b = FakeBackend(page_tokens=4, max_tokens=16, n_ctx=64)
    s = Scheduler(b, 64, 64)
    with pytest.raises(SchedulerError, match="cache pages by itself"):
        s.enqueue_ids(list(range(10)), G(20))
    with pytest.raises(SchedulerError, match="does not fit the context"):
        s.enqueue_ids(list(range(64)), G(1))
    with pytest.raises(SchedulerError, match="at least one"):
        s.enqueue_ids([], G(1))


def test_waits_for_a_slot_fifo():
    b = FakeBackend(max_requests=2)
    s = Scheduler(b, 64, 64)
    ids = [s.enqueue_ids([1 + i, 2, 3], G(4)) for i in range(4)]
    s.step()
    assert [r.id for r in s.running] == ids[:2] and [r.id for r in s.waiting] == ids[2:]
    toks, done = run_all(s)
    assert set(done) == set(ids) and s.counters["admission_waits"] > 0


def test_shrinks_portions_then_preempts_newest_and_tokens_do_not_change():
    prompts = [[3 + i, 9, 4, 7, 1, 8] for i in range(3)]
    alone = {}
    for i, p in enumerate(prompts):                         # each request by itself, roomy pool
        s = Scheduler(FakeBackend(max_tokens=64), 64, 64)
        rid = s.enqueue_ids(p, G(14))
        alone[i] = run_all(s)[0][rid]
    b = FakeBackend(page_tokens=4, max_tokens=40, max_requests=4)   # 10 pages: 3 x 20 tokens do not fit
    s = Scheduler(b, 64, 64)
    ids = [s.enqueue_ids(p, G(14)) for p in prompts]
    toks, done = run_all(s)
    assert s.counters["preempted"] > 0
    for i, rid in enumerate(ids):
        assert toks[rid] == alone[i], f"request {i} changed under preemption"
        assert done[rid].predicted_tokens == 14
    assert b.cache.free_pages() == b.cache.n_pages


def test_a_prompt_that_does_not_fit_the_free_pages_waits():
    """Beside running requests one is admitted only when its whole prompt and one token more fit the free pages."""
    b = FakeBackend(page_tokens=4, max_tokens=24, max_requests=4)   # 6 pages
    s = Scheduler(b, 64, 64)
    r0 = s.enqueue_ids(list(range(1, 15)), G(2))            # 14 tokens -> 4 pages
    evs = s.step()
    r1 = s.enqueue_ids(list(range(1, 13)), G(2))            # 12 tokens + 1 want 4 pages, 2 are free
    evs += s.step()
    assert b.batches[-1] == [(r0, 1, True)] and s.counters["admission_waits"] >= 1 and s.counters["shrunk"] == 0
    assert [r.id for r in s.waiting] == [r1]
    toks, done = run_all(s)
    done.update({e.req: e.stats for e in evs if e.kind == "done"})
    assert set(done) == {r0, r1} and done[r1].predicted_tokens == 2 and s.counters["preempted"] == 0
    assert b.cache.free_pages() == b.cache.n_pages


def test_prefill_portion_shrinks_to_the_pages_left():
    """A request is admitted when its prompt fits, but its prompt runs in portions, and meanwhile a decoding request
    may take a page: the portion that no longer fits is cut to the pages left (or left out of the step)."""
    alone = {}
    prompts = [[5, 1, 4, 2, 6, 3, 9], list(range(1, 12))]
    for i, p in enumerate(prompts):
        s = Scheduler(FakeBackend(max_tokens=64), 64, 64)
        rid = s.enqueue_ids(p, G(6 if i else 12))
        alone[i] = run_all(s)[0][rid]
    b = FakeBackend(page_tokens=4, max_tokens=20, max_requests=4)   # 5 pages
    s = Scheduler(b, 64, 4)                                 # portions of up to 4 tokens
    r0 = s.enqueue_ids(prompts[0], G(12))                   # 7 tokens: 2 pages, growing to 5
    s.step(); s.step()
    r1 = s.enqueue_ids(prompts[1], G(6))                    # 11 tokens + 1: 3 pages, 3 are free: admitted
    toks, done = run_all(s)
    assert s.counters["shrunk"] >= 1
    assert toks[r0][-len(alone[0]):] == alone[0][-len(toks[r0]):] and toks[r1] == alone[1]
    assert set(done) >= {r1} and b.cache.free_pages() == b.cache.n_pages


def test_cancel():
    b = FakeBackend()
    s = Scheduler(b, 64, 64)
    a = s.enqueue_ids([1, 2, 3], G(30))
    w = s.enqueue_ids([4, 5], G(30))
    s.step()
    assert s.cancel(a) and s.cancel(w) and not s.cancel(99)
    toks, done = run_all(s)
    assert done[a].finish_reason == "cancelled" and b.cache.free_pages() == b.cache.n_pages


class AheadBackend(FakeBackend):
    """The same fake with launch / collect: a launched step's tokens can be taken later, and a
    chained launch reads its items' tokens from the launch before it."""

    def __init__(self, **kw):
        super().__init__(**kw)
        self.launched, self.last_out, self.open_handles = {}, [], 0

    def launch(self, items, sample_rows, chain=False):
        if chain:
            assert len(items) == len(self.last_out) and all(len(it.tokens) == 1 for it in items)
            items = [type(it)(it.req, [tok], it.want) for it, tok in zip(items, self.last_out)]
        out = FakeBackend.run(self, items, sample_rows)
        self.last_out = out
        h = len(self.launched)
        self.launched[h] = out
        self.open_handles += 1
        assert self.open_handles <= 2                      # one step ahead, never more
        return h

    def collect(self, handle):
        self.open_handles -= 1
        return self.launched[handle]


def _scenario(backend_cls, lookahead, **bk):
    import random
    b = backend_cls(**bk)
    s = Scheduler(b, n_batch=16, n_ubatch=8, lookahead=lookahead) if backend_cls is AheadBackend else Scheduler(b, 16, 8)
    rng = random.Random(3)
    ids, early = [], []
    for i in range(9):
        prompt = [rng.randrange(1, 90) for _ in range(rng.randrange(1, 14))]
        stops = tuple(rng.sample(range(3, 100), 12)) if i % 2 else ()
        ids.append(s.enqueue_ids(prompt, G(rng.randrange(1, 12), stop_token_ids=stops)))
        if i % 3 == 2:
            for _ in range(rng.randrange(1, 5)):
                early += s.step()
    toks, done = {}, {}
    for _ in range(10_000):
        evs = early + s.step()
        early = []
        for ev in evs:
            if ev.kind == "token":
                toks.setdefault(ev.req, []).append(ev.token)
            elif ev.kind == "done":
                done[ev.req] = ev.stats
            else:
                raise AssertionError(ev)
        if s.idle():
            break
    b.cache.audit()
    assert b.cache.free_pages() == b.cache.n_pages and b.cache.slots.free_count == bk.get("max_requests", 4)
    return s, toks, {r: (d.finish_reason, d.predicted_tokens) for r, d in done.items()}


def test_one_step_ahead_gives_the_same_tokens_and_reasons():
    _, want_toks, want_done = _scenario(FakeBackend, False, page_tokens=4, max_tokens=64, max_requests=4, n_ctx=64)
    s, toks, done = _scenario(AheadBackend, True, page_tokens=4, max_tokens=64, max_requests=4, n_ctx=64)
    assert toks == want_toks and done == want_done
    assert s.counters["ran_ahead"] > 0
    s2, toks2, done2 = _scenario(AheadBackend, False, page_tokens=4, max_tokens=64, max_requests=4, n_ctx=64)
    assert toks2 == want_toks and done2 == want_done and s2.counters["ran_ahead"] == 0


def test_one_step_ahead_drops_the_token_after_a_stop_and_is_not_taken_before_a_foreseen_end():
    b = AheadBackend()
    s = Scheduler(b, 64, 64)
    first = (sum([1, 2, 3]) * 31 + 3 * 7) % 97 + 3
    second = ((sum([1, 2, 3]) + first) * 31 + 4 * 7) % 97 + 3
    a = s.enqueue_ids([1, 2, 3], G(50, stop_token_ids=(second,)))
    toks, done = run_all(s)
    assert toks[a] == [first, second] and done[a].finish_reason == "stop"
    assert s.counters["dropped"] == 1 and s.counters["ran_ahead"] == 2       # the step after `second` ran and was dropped
    assert b.cache.free_pages() == b.cache.n_pages and s.idle()
    # max_tokens is seen coming: the last step is not followed by one ahead
    b = AheadBackend()
    s = Scheduler(b, 64, 64)
    a = s.enqueue_ids([4, 5], G(4))
    toks, done = run_all(s)
    assert len(toks[a]) == 4 and done[a].finish_reason == "length"
    assert s.counters["steps"] == 4 and s.counters["dropped"] == 0 and s.counters["ran_ahead"] == 3


def test_one_step_ahead_under_page_pressure_matches_the_plain_order():
    kw = dict(page_tokens=4, max_tokens=24, max_requests=3, n_ctx=40)
    _, want_toks, want_done = _scenario(FakeBackend, False, **kw)
    s, toks, done = _scenario(AheadBackend, True, **kw)
    assert toks == want_toks and done == want_done


def test_two_readers_each_get_their_own_events():
    """Two requests read one after the other, each through poll_event(its id): the first reader
    runs the iterations that also produce the second's tokens, and those must still be there when
    the second reader comes (an engine with two live token streams reads them this way)."""
    want_toks, want_done = run_all(_two(Scheduler(FakeBackend(), 64, 64))[0])
    s, a, b = _two(Scheduler(FakeBackend(), 64, 64))
    got = {a: [], b: []}
    stats = {}
    for rid in (a, b):
        while True:
            ev = s.poll_event(rid)
            if ev is None:
                break
            assert ev.req == rid
            if ev.kind == "token":
                got[rid].append(ev.token)
            else:
                stats[rid] = ev.stats
                break
    assert got == want_toks and len(got[b]) == 9
    assert {r: st.finish_reason for r, st in stats.items()} == {r: st.finish_reason for r, st in want_done.items()}
    assert s.poll_event() is None and s.idle()
    # a set of ids: events of both, in the order they were made; a third request's stay behind
    s, a, b = _two(Scheduler(FakeBackend(), 64, 64))
    c = s.enqueue_ids([9, 9], G(2))
    seen = []
    while True:
        ev = s.poll_event({a, b})
        if ev is None:
            break
        seen.append(ev.req)
    assert set(seen) == {a, b} and c not in seen
    rest = []
    while (ev := s.poll_event()) is not None:
        rest.append((ev.req, ev.kind))
    assert rest == [(c, "token"), (c, "token"), (c, "done")]


def _two(s):
    a = s.enqueue_ids([1, 2, 3, 4, 5], G(6))
    b = s.enqueue_ids([7, 8], G(9))
    return s, a, b
