"""Many requests arriving and finishing at random through the scheduler, on a pool so small that requests are
preempted again and again: with CUDA graphs (decode steps captured at every count up to 16 and at every eighth count
above, rows of nobody filling them up, graphs evicted and captured again) the greedy tokens are those of the same
engine without graphs, and the cache's books are in order all the way."""
import numpy as np
import pytest

import tiny
from fellm_b200.engine import GenParams

pytestmark = pytest.mark.gpu


def run(graphs, seed, n_req, max_live, pool_tokens):
    rng = np.random.default_rng(seed)
    eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=graphs, max_requests=max_live,
                           max_tokens=pool_tokens, n_batch=512, n_ubatch=128)
    sched = eng.scheduler()
    pending = [(tiny.tokens("C", int(rng.integers(1, 150)), 5000 + i), int(rng.integers(1, 120))) for i in range(n_req)]
    out, rids, steps = {}, [], 0
    while pending or not sched.idle():
        for _ in range(int(rng.integers(0, 4))):            # a few arrivals now and then
            if pending:
                p, b = pending.pop()
                r = sched.enqueue_ids(p, GenParams.greedy(b))
                rids.append(r)
                out[r] = []
        for ev in sched.step():
            assert ev.kind != "error", ev.message
            if ev.kind == "token":
                out[ev.req].append(ev.token)
        steps += 1
        if steps % 50 == 0:
            eng.cache.audit()
    eng.check_status()
    eng.cache.audit()
    assert eng.cache.free_pages() == eng.cache.n_pages
    return [out[r] for r in rids], dict(sched.counters), eng


def test_random_arrivals_on_a_small_pool_with_and_without_graphs():
    with_graphs, counters, eng = run(True, 1, 200, 40, 40 * 72)
    assert counters["preempted"] > 50 and counters["mixed_steps"] > 50
    assert any(k[0] in (24, 32, 40) for k in eng.stepper.graphs if k[0] != "rows")      # padded decode steps took part
    directly, counters2, _ = run(False, 1, 200, 40, 40 * 72)
    assert counters2["preempted"] == counters["preempted"]
    assert with_graphs == directly
