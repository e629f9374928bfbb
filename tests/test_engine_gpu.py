"""The engine in process: long decoding, the first tokens of a sequence, greedy generation
through the entry point, and the scheduler with a pool so small that it must preempt."""
import pytest
import torch

import plain_lfm2
import tiny
from fellm_b200.engine import GenParams, StepItem

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding(name, dtype):
    n = 330                                               # many pages of 16, far keys, every page edge
    eng = tiny.make_engine(name, dtype)
    toks, want = tiny.tokens(name, n, 40), tiny.plain_logits(name, n, 40)
    eng.add_request("d")
    rows = [eng.step([StepItem("d", toks[:10], list(range(10)))])]
    for t in range(10, n):
        rows.append(eng.step([StepItem("d", [toks[t]], [0])]))
    eng.check_status()
    ok, err, tol = tiny.close(torch.cat(rows), want, dtype)
    assert ok, (err, tol)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_first_tokens(name, dtype):
    """Positions 0, 1, 2 ...: shorter than the conv history, one key only."""
    eng = tiny.make_engine(name, dtype)
    toks, want = tiny.tokens(name, 6, 41), tiny.plain_logits(name, 6, 41)
    eng.add_request("one")                                # one by one from the first token
    rows = [eng.step([StepItem("one", [t], [0])]) for t in toks]
    ok, err, tol = tiny.close(torch.cat(rows), want, dtype)
    assert ok, (err, tol)
    eng.add_request("single")                             # a prompt of one token, alone
    lg = eng.step([StepItem("single", toks[:1], [0])])
    ok, err, tol = tiny.close(lg, want[:1], dtype)
    assert ok, (err, tol)
    eng.check_status()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(name, dtype):
    cfg, w = tiny.plain_model(name)
    eng = tiny.make_engine(name, dtype, n_ubatch=8, n_batch=16)
    for length, seed in ((7, 50), (16, 51), (33, 52)):
        prompt = tiny.tokens(name, length, seed)
        want = plain_lfm2.greedy(cfg, w, prompt, 8)
        stream = eng.generate(prompt, GenParams.greedy(8))
        got = list(stream)
        if dtype == "bfloat16" and got != want:
            # a near-tie may flip under bfloat16: the first difference must be one
            i = next(k for k in range(8) if got[k] != want[k])
            lg = plain_lfm2.forward(cfg, w, prompt + want[:i])[-1]
            assert abs(float(lg[got[i]] - lg[want[i]])) < 0.05 * float(lg.abs().max()), (got, want)
        else:
            assert got == want
        st = stream.finish_stats()
        assert st.prompt_tokens == length and st.predicted_tokens == 8 and st.finish_reason == "length"
    assert eng.cache.free_pages() == eng.cache.n_pages


@pytest.mark.parametrize("graphs", [False, True])
def test_scheduler_one_step_ahead_gives_the_same_tokens_and_drops_what_follows_a_stop(graphs):
    """Batched generation with the scheduler running one step ahead (tokens fed back on the device)
    against the same with every step read before the next is launched: same tokens, same reasons;
    a stop token ends its request although the step after it has already run."""
    from fellm_b200.engine.scheduler import Scheduler
    name = "B"
    prompts = [tiny.tokens(name, n, 80 + i) for i, n in enumerate((9, 21, 14))]
    eng = tiny.make_engine(name, "float32", cuda_graphs=graphs)
    plain_sched = Scheduler(eng, eng.options.n_batch, eng.options.n_ubatch, lookahead=False)
    eng._scheduler = plain_sched
    want, _ = eng.generate_batch(prompts, GenParams.greedy(20))
    assert plain_sched.counters["ran_ahead"] == 0
    eng._scheduler = Scheduler(eng, eng.options.n_batch, eng.options.n_ubatch, lookahead=True)
    got, stats = eng.generate_batch(prompts, GenParams.greedy(20))
    assert got == want and eng._scheduler.counters["ran_ahead"] > 10
    # stop at each request's 6th token
    stops = [GenParams.greedy(20, stop_token_ids=(w[5],)) for w in want]
    got2, stats2 = eng.generate_batch(prompts, stops)
    for g, w, st in zip(got2, want, stats2):
        cut = w.index(w[5]) + 1
        assert g == w[:cut] and st.finish_reason == "stop" and st.predicted_tokens == cut
    assert eng._scheduler.counters["dropped"] >= 1
    eng.cache.audit()
    assert eng.cache.free_pages() == eng.cache.n_pages


def test_scheduler_preempts_on_a_small_pool_and_tokens_stay():
    name = "B"
    prompts = [tiny.tokens(name, n, 60 + i) for i, n in enumerate((40, 33, 25, 47))]
    roomy = tiny.make_engine(name, "float32", n_ubatch=16, n_batch=48)
    alone = [roomy.generate_batch([p], GenParams.greedy(24))[0][0] for p in prompts]
    small = tiny.make_engine(name, "float32", max_tokens=160, n_ubatch=16, n_batch=48)     # 10 pages of 16
    got, stats = small.generate_batch(prompts, GenParams.greedy(24))
    sched = small.scheduler()
    assert sched.counters["preempted"] > 0 or sched.counters["shrunk"] > 0
    assert got == alone
    cfg, w = tiny.plain_model(name)
    assert got[0] == plain_lfm2.greedy(cfg, w, prompts[0], 24)       # and both are the plain implementation's tokens
    assert got[3][:6] == plain_lfm2.greedy(cfg, w, prompts[3], 6)
    assert all(s.finish_reason == "length" and s.predicted_tokens == 24 for s in stats)
    small.cache.audit()
    assert small.cache.free_pages() == small.cache.n_pages


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_name_that_comes_again_in_another_slot(dtype):
    """Requests a, b, c decode together, are released, and the same names come again in other slots
    (the slot list is last in, first out): the decode step must follow the slots, not the names."""
    name = "A"
    eng = tiny.make_engine(name, dtype)
    lens = {"a": 5, "b": 19, "c": 11}
    for round_ in range(2):
        order = ["a", "b", "c"] if round_ == 0 else ["c", "a", "b"]
        for r in order:
            eng.add_request(r)
        slots = {r: eng.cache.slot(r) for r in lens}
        toks = {r: tiny.tokens(name, n + 4, 30 + i + 10 * round_) for i, (r, n) in enumerate(lens.items())}
        for r, n in lens.items():
            eng.step([StepItem(r, toks[r][:n], [])])
        for t in range(4):
            got = eng.step([StepItem(r, [toks[r][lens[r] + t]], [0]) for r in ("a", "b", "c")])
            for i, (r, n) in enumerate(lens.items()):
                want = tiny.plain_logits(name, n + 4, 30 + i + 10 * round_)[n + t]
                ok, err, tol = tiny.close(got[i], want, dtype)
                assert ok, (round_, r, t, err, tol)
        eng.check_status()
        if round_ == 0:
            first_slots = slots
        else:
            assert slots != first_slots                   # the names did move
        for r in ("a", "b", "c"):
            eng.release(r)


def test_step_refuses_what_it_cannot_place():
    from fellm_b200.config import CacheError, FellmError
    eng = tiny.make_engine("A", "float32", max_tokens=32)
    eng.add_request("a")
    with pytest.raises(CacheError, match="unknown request"):
        eng.step([StepItem("nobody", [1], [0])])
    with pytest.raises(FellmError, match="outside the vocabulary"):
        eng.step([StepItem("a", [256], [0])])
    with pytest.raises(CacheError, match="out of cache pages"):
        eng.step([StepItem("a", tiny.tokens("A", 40, 1), [])])
    assert eng.cache.length("a") == 0 and eng.cache.free_pages() == 2
    eng.cache.audit()


@pytest.mark.parametrize("graphs", [False, True])
def test_decode_at_model_width_against_the_plain_implementation(graphs):
    """A model of width 1024 with heads of 64 and pages of 64 tokens, bfloat16: the decode step then
    runs the single-shot products, the convolution inside the input product and the TMA attention.
    Several requests of different lengths decode together across a page's edge, directly and
    replayed from a CUDA graph, against the plain implementation."""
    lens = [3, 50, 61]
    n_dec = 24
    toks = [tiny.tokens("C", n + n_dec, 70 + i) for i, n in enumerate(lens)]
    eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=graphs)
    for i, n in enumerate(lens):
        eng.add_request(i)
        eng.step([StepItem(i, toks[i][:n], [])])
    rows = []
    for t in range(n_dec):
        rows.append(eng.step([StepItem(i, [toks[i][lens[i] + t]], [0]) for i in range(len(lens))]).clone())
    eng.check_status()
    got = torch.stack(rows)                                 # [n_dec, requests, vocab]
    if graphs:
        assert len(eng.stepper.graphs) >= 1
    for i, n in enumerate(lens):
        want = tiny.plain_logits("C", n + n_dec, 70 + i)[n:]
        ok, err, tol = tiny.close(got[:, i], want, "bfloat16")
        assert ok, (i, err, tol)
    # the same tokens fed as whole prompts give the same logits beyond rounding
    eng2 = tiny.make_engine("C", "bfloat16", page_tokens=64)
    for i, n in enumerate(lens):
        eng2.add_request(i)
        whole = eng2.step([StepItem(i, toks[i], list(range(n, n + n_dec)))])
        ok, err, tol = tiny.close(got[:, i], whole, "bfloat16")
        assert ok, (i, err, tol)


@pytest.mark.parametrize("name,dtype", [("B", "bfloat16"), ("A", "float32"), ("C", "bfloat16")])
def test_prompt_portions_of_a_shape_that_comes_again_are_replayed_from_a_graph(name, dtype):
    """The same shape of step (one portion of 37 tokens, then one of 12 behind it, then both kinds
    mixed with a decoding request) for several requests: the first goes directly, the second is
    captured, the rest are replayed; every one against the plain implementation."""
    pt = 64 if name == "C" else 16
    eng = tiny.make_engine(name, dtype, cuda_graphs=True, page_tokens=pt)
    n1, n2 = 37, 12
    for i in range(5):
        toks = tiny.tokens(name, n1 + n2, 40 + i)
        want = tiny.plain_logits(name, n1 + n2, 40 + i)
        eng.add_request(i)
        a = eng.step([StepItem(i, toks[:n1], [0, n1 - 1])]).clone()
        b = eng.step([StepItem(i, toks[n1:], list(range(n2)))]).clone()
        eng.check_status()
        for got, exp in ((a, want[[0, n1 - 1]]), (b, want[n1:])):
            ok, err, tol = tiny.close(got, exp, dtype)
            assert ok, (i, err, tol)
        eng.release(i)
    keys = [k for k in eng.stepper.graphs if k[0] == "rows"]
    assert len(keys) == 2, keys
    # both kinds beside a decoding request: each mixed shape four times (direct, captured, replayed twice)
    dec_toks, dec_want = tiny.tokens(name, 30, 77), tiny.plain_logits(name, 30, 77)
    eng.add_request("dec")
    eng.step([StepItem("dec", dec_toks[:20], [])])
    for j in range(4):
        toks, want = tiny.tokens(name, n1 + n2, 60 + j), tiny.plain_logits(name, n1 + n2, 60 + j)
        eng.add_request(f"m{j}")
        a = eng.step([StepItem("dec", [dec_toks[20 + 2 * j]], [0]), StepItem(f"m{j}", toks[:n1], [n1 - 1])])
        b = eng.step([StepItem(f"m{j}", toks[n1:], [n2 - 1]), StepItem("dec", [dec_toks[21 + 2 * j]], [0])])
        eng.check_status()
        for got, exp in ((a[0:1], dec_want[[20 + 2 * j]]), (a[1:2], want[[n1 - 1]]), (b[0:1], want[[n1 + n2 - 1]]),
                         (b[1:2], dec_want[[21 + 2 * j]])):
            ok, err, tol = tiny.close(got, exp, dtype)
            assert ok, (j, err, tol)
        eng.release(f"m{j}")
    eng.release("dec")
    assert len([k for k in eng.stepper.graphs if k[0] == "rows"]) == 4
    # more shapes than graphs are kept: the oldest are dropped, nothing breaks
    from fellm_b200.engine import step as step_mod
    for n in range(20, 20 + step_mod.MAX_ROW_GRAPHS + 3):
        for rep in range(2):
            toks = tiny.tokens(name, n, 90 + n)
            eng.add_request("x")
            got = eng.step([StepItem("x", toks, [n - 1])]).clone()
            ok, err, tol = tiny.close(got, tiny.plain_logits(name, n, 90 + n)[[n - 1]], dtype)
            assert ok, (n, rep, err, tol)
            eng.release("x")
    assert len([k for k in eng.stepper.graphs if k[0] == "rows"]) <= step_mod.MAX_ROW_GRAPHS
    eng.cache.audit()


def test_command_line_run_prints_tokens_and_timing_lines():
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    prompt = tiny.tokens("A", 9, 80)
    cfg, w = tiny.plain_model("A")
    want = plain_lfm2.greedy(cfg, w, prompt, 5)
    p = subprocess.run([sys.executable, str(root / "bin" / "fellm"), "run", tiny.model_folder("A"), "--prompt",
                        ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--repetition-penalty", "1.0",
                        "--dtype", "float32", "--ctx-size", "0", "--page-tokens", "16"],
                       capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == want
    for line in ("prompt eval: 9 tok in", "eval: 5 tok in", "TTFT:", "total:"):       # crates/fellm-cli/src/main.rs:953-967
        assert line in p.stderr, p.stderr[-1000:]
