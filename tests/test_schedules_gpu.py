"""Logits of the schedules that the benchmark times, against the plain implementation: decode
steps of 17 to 97 requests (other kernels than small steps: the tcgen05 product of few rows with the
norm handed on and, up to 64 rows, the convolution in its epilogue; decode attention beyond one wave), the real layer
sizes of the 350M / 700M / 1.2B shapes in two-layer cuts, and mixed steps replayed from CUDA graphs
whose layout differs from the one they were captured with."""
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_lfm2
import tiny
from fellm_b200.config.options import EngineOptions
from fellm_b200.engine import Engine, StepItem
from fellm_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu
_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_schedules_")


def check(tag, got, want, dtype):
    ok, err, tol = tiny.close(got, want, dtype)
    assert ok, f"{tag}: error {err:.3e} > {tol:.3e}"


@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("n_req", [20, 33, 64, 97])
def test_many_requests_decode_together(n_req, graphs):
    """Width 1024, heads of 64, pages of 64 tokens, bfloat16: 20, 33 (under graphs: filled up to 24 and 40 rows) and 64 requests with prompts of
    different lengths decode 8 steps together, and 97 (104 rows: beyond 64 the few-rows tcgen05 product has TMEM and
    partial tiles of 128 columns) (some cross a page's edge), directly and from a CUDA
    graph; every row of every step against the plain implementation."""
    n_dec = 8
    rng = np.random.default_rng(n_req)
    lens = [int(x) for x in rng.integers(1, 130, n_req)]
    lens[0], lens[1], lens[2] = 60, 63, 64                   # a page's edge inside the decoded steps
    toks = [tiny.tokens("C", n + n_dec, 300 + i) for i, n in enumerate(lens)]
    eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=graphs, max_requests=max(64, n_req), max_tokens=64 * 256)
    for i, n in enumerate(lens):
        eng.add_request(i)
        eng.step([StepItem(i, toks[i][:n], [])])
    rows = []
    for t in range(n_dec):
        rows.append(eng.step([StepItem(i, [toks[i][lens[i] + t]], [0]) for i in range(n_req)]).clone())
    eng.check_status()
    got = torch.stack(rows)                                  # [n_dec, requests, vocab]
    if graphs:
        assert len(eng.stepper.graphs) >= 1
    for i, n in enumerate(lens):
        want = tiny.plain_logits("C", n + n_dec, 300 + i)[n:]
        check(f"request {i} of {n_req} (prompt {n})", got[:, i], want, "bfloat16")


SHAPES = {   # the layer sizes of the benchmark shapes; two layers (one convolution, one attention) keep the plain side at seconds
    "350m": dict(hidden_size=1024, num_attention_heads=16, block_ff_dim=6656),
    "700m": dict(hidden_size=1536, num_attention_heads=24, block_ff_dim=10752),
    "1.2b": dict(hidden_size=2048, num_attention_heads=32, block_ff_dim=12288),
}


def shape_config(name):
    cfg = dict(architectures=["Lfm2ForCausalLM"], vocab_size=65536, num_hidden_layers=2, num_key_value_heads=8,
               head_dim=64, layer_types=["conv", "full_attention"], block_auto_adjust_ff_dim=True,
               block_ffn_dim_multiplier=1.0, block_multiple_of=256, rope_theta=1000000.0, rope_pairing="split_half",
               conv_L_cache=3, conv_bias=False, norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=128000)
    cfg.update(SHAPES[name])
    return cfg


@pytest.mark.parametrize("name", list(SHAPES))
def test_the_benchmark_shapes_in_two_layer_cuts(name):
    """Real widths, feed-forward sizes, head counts and the vocabulary of 65,536: a prompt of 70 tokens
    whole, then in portions, then 6 decode steps (alone, and beside 8 and 39 other requests, which
    moves the products to other kernels), in float32 and bfloat16."""
    cfg = shape_config(name)
    folder = write_model_folder(Path(_tmp.name) / name, cfg, 11)
    pcfg, w = plain_lfm2.load_folder(str(folder))
    assert plain_lfm2.ff_dim(pcfg) == {"350m": 4608, "700m": 7168, "1.2b": 8192}[name]
    rng = np.random.default_rng(5)
    n, n_dec = 70, 6
    toks = [int(t) for t in rng.integers(0, 65536, n + n_dec)]
    want = plain_lfm2.forward(pcfg, w, toks)
    del w
    others = [[int(t) for t in rng.integers(0, 65536, 3 + n_dec)] for _ in range(39)]
    for dtype in ("float32", "bfloat16"):
        eng = Engine.open(str(folder), EngineOptions(dtype=dtype, n_ctx=4096, max_requests=48, cuda_graphs=False,
                                                     max_tokens=48 * 128, page_tokens=64, n_batch=4096))
        eng.add_request("w")
        check(f"{name} {dtype}: whole", eng.step([StepItem("w", toks[:n], list(range(n)))]), want[:n], dtype)
        for t in range(n, n + n_dec):
            check(f"{name} {dtype}: decode at {t}", eng.step([StepItem("w", [toks[t]], [0])]), want[t:t + 1], dtype)
        eng.release("w")
        eng.add_request("p")
        at = 0
        for s in (33, 2, 35):
            check(f"{name} {dtype}: portion {at}+{s}", eng.step([StepItem("p", toks[at:at + s], list(range(s)))]),
                  want[at:at + s], dtype)
            at += s
        if dtype == "bfloat16":
            # the same decode steps beside 8, then 39 other requests: 9 and 40 rows a step
            for k, o in enumerate(others):
                eng.add_request(k)
                eng.step([StepItem(k, o[:3], [])])
            for j, t in enumerate(range(n, n + n_dec)):
                beside = 8 if j < 3 else 39
                items = [StepItem(k, [others[k][3 + j]], []) for k in range(beside)]
                items.insert(4, StepItem("p", [toks[t]], [0]))
                check(f"{name} {dtype}: decode at {t} beside {beside}", eng.step(items), want[t:t + 1], dtype)
        eng.check_status()
        del eng
        torch.cuda.empty_cache()


@pytest.mark.parametrize("name,dtype,far", [("B", "float32", 900), ("B", "bfloat16", 900), ("C", "bfloat16", 400)])
def test_a_replayed_graph_of_a_mixed_step_takes_another_layout(name, dtype, far):
    """A step that is not pure decode is replayed from a graph keyed by its counts (rows, items, wanted
    rows, the longest item): the same counts come again with the items in another order, with other
    slots and pages, and at a cached prefix of hundreds of tokens instead of none."""
    pt = 64 if name == "C" else 16
    eng = tiny.make_engine(name, dtype, cuda_graphs=True, page_tokens=pt, max_tokens=4096, max_requests=12)
    n1, n2 = 37, 12
    serial = 0

    def fresh(prefix):
        nonlocal serial
        serial += 1
        rid = f"r{serial}"
        eng.add_request(rid)
        toks = tiny.tokens(name, prefix + n1, 500 + serial)
        if prefix:
            eng.step([StepItem(rid, toks[:prefix], [])])
        return rid, toks, tiny.plain_logits(name, prefix + n1, 500 + serial), prefix

    def mixed(first_long, prefixes):
        """Two items, 37 and 12 tokens (in this or the other order), wanted: the last row of each."""
        a, b = fresh(prefixes[0]), fresh(prefixes[1])
        la, lb = (n1, n2) if first_long else (n2, n1)
        items = [StepItem(a[0], a[1][a[3]:a[3] + la], [la - 1]), StepItem(b[0], b[1][b[3]:b[3] + lb], [lb - 1])]
        got = eng.step(items)
        check(f"{first_long} {prefixes}: first item", got[0:1], a[2][[a[3] + la - 1]], dtype)
        check(f"{first_long} {prefixes}: second item", got[1:2], b[2][[b[3] + lb - 1]], dtype)
        return a[0], b[0]

    held = []
    held += mixed(True, (0, 0))               # runs directly
    held += mixed(True, (0, 0))               # captured
    n_graphs = len([k for k in eng.stepper.graphs if k[0] == "rows"])
    held += mixed(False, (0, 0))              # replayed: the short item first
    eng.release(held.pop(0)), eng.release(held.pop(0))
    held += mixed(True, (far, 3))             # replayed: a long cached prefix, other slots and pages
    held += mixed(False, (5, far))
    assert len([k for k in eng.stepper.graphs if k[0] == "rows"]) >= n_graphs >= 1
    eng.check_status()
    for r in held:
        eng.release(r)
    eng.cache.audit()


@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_steps_that_skip_the_logits_give_the_plain_tokens(graphs):
    """Width 1024 (the head's product then runs on the single-shot kernel): a greedy decode step asks for
    the tokens themselves and the head picks them without storing the logits.  The tokens must be those
    of the plain implementation (a near-tie may flip under bfloat16: then the two logits must be close),
    and the same as the engine's own logits give."""
    from fellm_b200 import ops
    from fellm_b200.engine import GenParams
    cfg, w = tiny.plain_model("C")
    eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=graphs)
    assert ops.head_argmax_scratch(3, 384, 1024, True) > 0
    prompts = [tiny.tokens("C", n, 700 + i) for i, n in enumerate((5, 40, 23))]
    before = ops.launch_count()
    got, stats = eng.generate_batch(prompts, GenParams.greedy(12))
    assert all(s.predicted_tokens == 12 for s in stats)
    for p, g in zip(prompts, got):
        want = plain_lfm2.greedy(cfg, w, p, 12)
        if g != want:
            i = next(k for k in range(12) if g[k] != want[k])
            lg = plain_lfm2.forward(cfg, w, p + want[:i])[-1]
            assert abs(float(lg[g[i]] - lg[want[i]])) < 0.05 * float(lg.abs().max()), (g, want)
    # the same requests through logits and the sampler's own argmax: the same tokens
    eng2 = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=False)
    for i, p in enumerate(prompts):
        eng2.add_request(i)
        seq = list(p)
        lg = eng2.step([StepItem(i, seq, [len(seq) - 1])])
        for t in range(12):
            tok = int(torch.argmax(lg[0]))
            assert tok == got[i][t], (i, t)
            lg = eng2.step([StepItem(i, [tok], [0])])
    eng.check_status()


@pytest.mark.parametrize("n_req", [3, 12])
def test_decode_steps_hand_the_norms_on(n_req, monkeypatch):
    """Width 1024, decode steps of 3 and of 12 rows (one and two token tiles of the products): every product that adds into the residual rows leaves them weighted
    for the norm that reads them next (all but the first norm of a step, which follows the embedding), and the
    logits stay those of the plain implementation; with the hand-over switched off, too."""
    from fellm_b200 import ops
    taken = []
    real = ops._announce_row_scale
    monkeypatch.setattr(ops, "_announce_row_scale", lambda *a, **k: (taken.append(a[1:4]), real(*a, **k))[1])
    lens = (7, 64, 30, 1, 63, 12, 100, 5, 33, 65, 2, 90)[:n_req]
    prompts = [tiny.tokens("C", n + 6, 810 + i) for i, n in enumerate(lens)]
    logits = {}
    for on in (True, False):
        monkeypatch.setattr(ops, "NORM_HANDOFF", on)
        eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=False, max_requests=16, max_tokens=16 * 256)
        for i, n in enumerate(lens):
            eng.add_request(i)
            eng.step([StepItem(i, prompts[i][:n], [])])
        taken.clear()
        rows = [eng.step([StepItem(i, [prompts[i][lens[i] + t]], [0]) for i in range(n_req)]).clone() for t in range(6)]
        eng.check_status()
        logits[on] = torch.stack(rows)
        n_layers = len(tiny.CONFIGS["C"][0]["layer_types"])
        assert len(taken) == (6 * 2 * n_layers if on else 0), (on, len(taken))
        for i, n in enumerate(lens):
            want = tiny.plain_logits("C", n + 6, 810 + i)[n:]
            check(f"hand-over {on}: request {i}", logits[on][:, i], want, "bfloat16")


@pytest.mark.parametrize("graphs", [False, True])
def test_every_row_count_from_1_to_40_with_and_without_the_handed_on_norm(graphs, monkeypatch):
    """Width 1024: decode steps of 1, 2, ... 40 requests (each count picks its own kernels, tile counts and shared
    memory sizes), run by an engine that hands the norms on and by one that does not, on the same tokens: the
    logits agree within twice the tolerance each has against the plain implementation, and the last step of
    some requests is compared with that directly.  Under CUDA graphs the counts above 16 are filled up to 24, 32
    and 40 rows with rows of nobody: three graphs for 24 counts, the same logits for the real rows, and the
    cache's books in order."""
    from fellm_b200 import ops
    n_max, n_dec = 40, 41
    lens = [1 + (7 * i) % 23 for i in range(n_max)]
    toks = [tiny.tokens("C", lens[i] + n_dec, 900 + i) for i in range(n_max)]
    engines = {}
    for on in (True, False):
        monkeypatch.setattr(ops, "NORM_HANDOFF", on)
        eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=graphs, max_requests=n_max, max_tokens=n_max * 128)
        for i in range(n_max):
            eng.add_request(i)
            eng.step([StepItem(i, toks[i][:lens[i]], [])])
        engines[on] = eng
    done = [0] * n_max
    last = {}
    for n in range(1, n_max + 1):
        items = [StepItem(i, [toks[i][lens[i] + done[i]]], [0]) for i in range(n)]
        out = {}
        for on in (True, False):
            monkeypatch.setattr(ops, "NORM_HANDOFF", on)
            out[on] = engines[on].step(items).clone()
        for i in range(n):
            done[i] += 1
        scale = float(out[False].abs().max())
        err = float((out[True] - out[False]).abs().max())
        assert err <= 2 * 2.5e-2 * scale, (n, err, scale)
        last[n] = out[True]
    for on in (True, False):
        engines[on].check_status()
        engines[on].cache.audit()
        if graphs:
            decode_keys = [k for k in engines[on].stepper.graphs if k[0] != "rows" and k[1] > 0]      # (a prompt of one token is such a step too, with no row wanted)
            assert sorted(k[0] for k in decode_keys) == list(range(1, 17)) + [24, 32, 40], decode_keys
    # request i took part in the steps n = i + 1 .. 40: its row of the last step against the plain implementation
    for i in (0, 7, 15, 16, 31, 39):
        want = tiny.plain_logits("C", lens[i] + done[i], 900 + i)[-1:]
        check(f"request {i} after {done[i]} steps", last[n_max][i:i + 1], want, "bfloat16")


@pytest.mark.parametrize("temperature", [0.0, 0.7])
def test_twenty_one_requests_through_the_scheduler_under_graphs(temperature):
    """21 prompts of different lengths and token budgets through generate_batch with CUDA graphs on: the decode
    steps carry 21, 20, ... requests as they finish, filled up to 24 and 16.. rows (rows of nobody beside the real
    ones, the greedy head writing tokens for them too); greedy tokens against the plain implementation (a near-tie
    may flip under bfloat16), and with a temperature the same tokens as the engine gives without graphs."""
    from fellm_b200.engine import GenParams
    cfg, w = tiny.plain_model("C")
    prompts = [tiny.tokens("C", 3 + (5 * i) % 40, 1200 + i) for i in range(21)]
    budgets = [4 + (i % 9) for i in range(21)]
    def run(graphs):
        eng = tiny.make_engine("C", "bfloat16", page_tokens=64, cuda_graphs=graphs, max_requests=24, max_tokens=24 * 128)
        sched = eng.scheduler()
        rids = []
        for p, b in zip(prompts, budgets):
            params = GenParams.greedy(b) if temperature == 0 else GenParams(max_tokens=b, temperature=temperature, top_k=20, seed=5)
            rids.append(sched.enqueue_ids(p, params))
        out = {r: [] for r in rids}
        while not sched.idle():
            for ev in sched.step():
                if ev.kind == "token":
                    out[ev.req].append(ev.token)
                assert ev.kind != "error", ev.message
        eng.check_status()
        eng.cache.audit()
        assert eng.cache.free_pages() == eng.cache.n_pages
        return [out[r] for r in rids], eng
    got, eng = run(True)
    assert any(k[0] == 24 for k in eng.stepper.graphs if k[0] != "rows"), list(eng.stepper.graphs)
    assert [len(g) for g in got] == budgets
    if temperature == 0:
        for p, g, b in zip(prompts[::4], got[::4], budgets[::4]):
            want = plain_lfm2.greedy(cfg, w, p, b)
            if g != want:
                i = next(k for k in range(b) if g[k] != want[k])
                lg = plain_lfm2.forward(cfg, w, p + want[:i])[-1]
                assert abs(float(lg[g[i]] - lg[want[i]])) < 0.05 * float(lg.abs().max()), (g, want)
    else:
        direct, _ = run(False)
        same = sum(a == b for a, b in zip(got, direct))
        assert same >= 19, (same, got, direct)        # (a draw that sits on a rounding boundary may differ between the two)
