"""Trace replay against the plain implementation: each request whole; most of it in one step and
the last 32 tokens one by one; in portions of changing size down to two tokens; and mixed, up to
four live requests with so few pages that they are used again - in float32 and bfloat16, for both
tiny configurations."""
import pytest
import torch

import tiny
from replay import collect, run_trace

pytestmark = pytest.mark.gpu

DTYPES = ["float32", "bfloat16"]
LENGTHS = {"A": [7, 16, 33, 70], "B": [1, 5, 29, 64, 93]}


def check(name, dtype, steps, results, seeds):
    """Every wanted row equals the plain implementation's logits of that request at that place."""
    got = collect(steps, results)
    worst = 0.0
    for rid, rows in got.items():
        length, seed = seeds[rid]
        want = tiny.plain_logits(name, length, seed)
        for p, row in rows.items():
            ok, err, tol = tiny.close(row, want[p], dtype)
            worst = max(worst, err / tol)
            assert ok, f"{name} {dtype} request {rid} position {p}: error {err:.3e} > {tol:.3e}"
    return worst


def vocab(name):
    return tiny.CONFIGS[name][0]["vocab_size"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_whole(name, dtype):
    steps, seeds = [], {}
    for i, n in enumerate(LENGTHS[name]):
        rid = f"r{i}"
        seeds[rid] = (n, i)
        steps.append({"entries": [{"id": rid, "tokens": tiny.tokens(name, n, i), "want": list(range(n))}],
                      "end": [rid]})
    res = run_trace(tiny.model_folder(name), dtype, 128, steps, vocab(name))
    check(name, dtype, steps, res, seeds)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_last_32_one_by_one(name, dtype):
    n = 90
    toks = tiny.tokens(name, n, 7)
    steps = [{"entries": [{"id": "x", "tokens": toks[:n - 32], "want": [0, n - 33]}]}]
    steps += [{"entries": [{"id": "x", "tokens": [toks[t]], "want": [0]}]} for t in range(n - 32, n)]
    steps[-1]["end"] = ["x"]
    res = run_trace(tiny.model_folder(name), dtype, 128, steps, vocab(name), page_tokens=16)
    check(name, dtype, steps, res, {"x": (n, 7)})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_of_changing_size(name, dtype):
    n = 101
    toks = tiny.tokens(name, n, 11)
    sizes = [13, 2, 8, 5, 3, 2, 2, 17, 1, 2, 21, 2, 3, 16, 4]
    assert sum(sizes) == n
    steps, at = [], 0
    for s in sizes:
        steps.append({"entries": [{"id": "p", "tokens": toks[at:at + s], "want": list(range(s))}]})
        at += s
    steps[-1]["end"] = ["p"]
    res = run_trace(tiny.model_folder(name), dtype, 128, steps, vocab(name), page_tokens=16)
    check(name, dtype, steps, res, {"p": (n, 11)})


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B"])
def test_mixed_with_pages_used_again(name, dtype):
    """Six requests, at most four live, 64 tokens each at most: the pool (256 tokens) is full when
    four are live, so every later request gets pages and a state slot that an earlier one used."""
    lens = [64, 37, 50, 64, 29, 58]
    toks = {f"m{i}": tiny.tokens(name, n, 20 + i) for i, n in enumerate(lens)}
    seeds = {f"m{i}": (n, 20 + i) for i, n in enumerate(lens)}
    portion = {"m0": 9, "m1": 5, "m2": 2, "m3": 11, "m4": 3, "m5": 7}
    prefill_until = {k: len(v) - 12 for k, v in toks.items()}       # then decode the rest one by one
    at = {k: 0 for k in toks}
    waiting = list(toks)
    live, steps = [], []
    while waiting or live:
        while waiting and len(live) < 4:
            live.append(waiting.pop(0))
        entries, ended = [], []
        for k in list(live):
            if len(steps) % 5 == 3 and k == live[0] and len(live) > 1:
                continue                                  # a request may be left out of a step
            if at[k] < prefill_until[k]:
                n = min(portion[k], prefill_until[k] - at[k])
                portion[k] = max(2, (portion[k] * 3) % 13)      # sizes keep changing, never below two
                want = [n - 1] if n > 1 else [0]
            else:
                n, want = 1, [0]
            entries.append({"id": k, "tokens": toks[k][at[k]:at[k] + n], "want": want})
            at[k] += n
            if at[k] == len(toks[k]):
                ended.append(k)
                live.remove(k)
        steps.append({"entries": entries, "end": ended})
    assert max(len(s["entries"]) for s in steps) == 4
    assert any(len(e["tokens"]) > 1 for s in steps for e in s["entries"] if any(len(f["tokens"]) == 1 for f in s["entries"]))
    res = run_trace(tiny.model_folder(name), dtype, 256, steps, vocab(name))
    check(name, dtype, steps, res, seeds)


@pytest.mark.parametrize("name", ["A", "B"])
def test_float32_does_not_depend_on_the_cut(name):
    """The same request whole, and cut into portions beside another request, in float32: the
    logits are bit-equal (every sum runs in an order that depends on the position only)."""
    n = 75
    toks, other = tiny.tokens(name, n, 31), tiny.tokens(name, 40, 32)
    whole = [{"entries": [{"id": "w", "tokens": toks, "want": list(range(n))}], "end": ["w"]}]
    a = collect(whole, run_trace(tiny.model_folder(name), "float32", 128, whole, vocab(name), page_tokens=16))["w"]
    steps, at, sizes = [], 0, [6, 2, 19, 1, 1, 30, 3, 13]
    steps.append({"entries": [{"id": "o", "tokens": other[:17], "want": []}]})      # takes the first pages
    for i, s in enumerate(sizes):
        e = [{"id": "w", "tokens": toks[at:at + s], "want": list(range(s))}]
        if i % 2 == 0:
            e.insert(0, {"id": "o", "tokens": other[17 + i:18 + i], "want": [0]})
        steps.append({"entries": e})
        at += s
    assert at == n
    b = collect(steps, run_trace(tiny.model_folder(name), "float32", 192, steps, vocab(name), page_tokens=16))["w"]
    for p in range(n):
        assert torch.equal(a[p], b[p]), f"position {p} differs by {(a[p] - b[p]).abs().max().item():.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_request_longer_than_max_position_embeddings_in_one_step(dtype):
    """Replay holds a request as long as the pool lets it (configuration A says 512 positions), and a
    step takes a whole prompt of more tokens than a scheduler iteration would."""
    name, n = "A", 4400
    toks = tiny.tokens(name, n, 21)
    cut = n - 3
    places = [0, 63, 64, 511, 512, 513, 2047, 2048, 4095, 4096, cut - 1]
    steps = [{"entries": [{"id": "long", "tokens": toks[:cut], "want": places}]}]
    steps += [{"entries": [{"id": "long", "tokens": [toks[t]], "want": [0]}]} for t in range(cut, n)]
    steps[-1]["end"] = ["long"]
    res = run_trace(tiny.model_folder(name), dtype, 4416, steps, vocab(name))
    check(name, dtype, steps, res, {"long": (n, 21)})
