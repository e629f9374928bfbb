"""Random configurations of the architecture (sizes that are no power of two, every head size in
steps of 16, any number of heads and groups, 2..5 taps, biases, both pairings, tied or not) through
the engine against the plain implementation, in float32 and bfloat16: each request whole; most of
it in one step and the last 32 tokens one by one; portions of changing size; and up to four live
requests, portions of some beside decoded tokens of others, on a pool so small that pages and state
slots are used again."""
import tempfile
from pathlib import Path

import numpy as np
import pytest

import plain_lfm2
import tiny

pytestmark = pytest.mark.gpu

_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_random_")


def random_config(rng):
    hd = int(rng.choice([16, 32, 48, 64, 80, 96, 128]))
    groups = int(rng.choice([1, 2, 3, 4, 8]))
    heads = groups * int(rng.choice([1, 2, 3, 4, 5, 8]))
    n_layers = int(rng.integers(2, 6))
    kinds = [str(rng.choice(["conv", "full_attention"])) for _ in range(n_layers)]
    if rng.random() < 0.8:
        if "conv" not in kinds:
            kinds[0] = "conv"
        if "full_attention" not in kinds:
            kinds[-1] = "full_attention"
    auto = bool(rng.random() < 0.4)
    cfg = dict(architectures=["Lfm2ForCausalLM"], vocab_size=int(rng.integers(90, 2500)),
               hidden_size=int(rng.choice([32, 48, 72, 96, 104, 136, 200, 264, 320, 520, 768, 1024, 1280])),
               num_hidden_layers=n_layers, num_attention_heads=heads, num_key_value_heads=groups, head_dim=hd,
               layer_types=kinds, block_ff_dim=int(rng.choice([64, 96, 176, 200, 344, 512, 1000, 2048, 4608])),
               block_auto_adjust_ff_dim=auto, rope_theta=float(rng.choice([10000.0, 1000000.0, 50000.0])),
               rope_pairing=str(rng.choice(["adjacent", "split_half"])), conv_L_cache=int(rng.integers(2, 6)),
               conv_bias=bool(rng.random() < 0.5), norm_eps=float(rng.choice([1e-5, 1e-6, 3e-5])),
               tie_word_embeddings=bool(rng.random() < 0.5), max_position_embeddings=2048)
    if auto:
        cfg["block_ffn_dim_multiplier"] = float(rng.choice([1.0, 0.75, 1.3]))
        cfg["block_multiple_of"] = int(rng.choice([16, 32, 64, 256]))
    return cfg


def check(tag, got, want, dtype):
    ok, err, tol = tiny.close(got, want, dtype)
    assert ok, f"{tag}: error {err:.3e} > {tol:.3e}"


def mixed_phase(eng, rng, tag, toks, lens, want, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, a request left out
    of a step now and then; eight requests through a pool that holds far fewer, so that pages and
    state slots are used again."""
    from fellm_b200.engine import StepItem
    queue, live, serial = list(range(5)) + [0, 1, 2], {}, 0   # mixed, pages and slots used again
    while queue or live:
        while queue and len(live) < 4:
            idx = queue.pop(0)
            name = f"m{serial}"
            serial += 1
            eng.add_request(name)
            live[name] = [idx, 0]
        items, refs = [], []
        for name, (idx, at) in list(live.items()):
            if rng.random() < 0.2 and len(live) > 1:
                continue                                     # left out of this step
            n = lens[idx]
            s = 1 if at >= n - 32 else int(min(n - 32 - at, rng.choice([2, 3, 7, 16, 30, 64, 100])))
            s = max(1, min(s, n - at))
            items.append(StepItem(name, toks[idx][at:at + s], list(range(s))))
            refs.append((idx, at, s))
            live[name][1] = at + s
        if not items:
            continue
        lg = eng.step(items)
        row = 0
        for idx, at, s in refs:
            check(f"{tag}: mixed request {idx} at {at}+{s}", lg[row:row + s], want[idx][at:at + s], dtype)
            row += s
        for name in [k for k, v in live.items() if v[1] >= lens[v[0]]]:
            eng.release(name)
            del live[name]


@pytest.mark.parametrize("trial", range(10))
def test_a_random_configuration_under_every_cut(trial):
    from fellm_b200.config.options import EngineOptions
    from fellm_b200.engine import Engine, StepItem
    from fellm_b200.weights import write_model_folder
    rng = np.random.default_rng(7000 + trial)
    cfg = random_config(rng)
    folder = Path(_tmp.name) / f"m{trial}"
    write_model_folder(folder, cfg, trial)
    pcfg, w = plain_lfm2.load_folder(str(folder))
    lens = [int(rng.integers(40, 230)) for _ in range(5)]
    if trial % 3 == 0:
        lens[0], lens[3] = int(rng.integers(300, 700)), int(rng.integers(300, 600))
    toks = [[int(t) for t in rng.integers(0, cfg["vocab_size"], n)] for n in lens]
    want = [plain_lfm2.forward(pcfg, w, t) for t in toks]
    pool = 2 * 1024 + 512 if trial % 3 == 0 else 4 * 256
    for dtype in ("float32", "bfloat16"):
        eng = Engine.open(str(folder), EngineOptions(dtype=dtype, n_ctx=0, max_requests=8, cuda_graphs=False,
                                                     max_tokens=pool, n_batch=4096))
        tag = f"trial {trial} {dtype} {cfg}"
        for i in range(2):                                       # whole
            eng.add_request(f"w{i}")
            check(f"{tag}: whole {i}", eng.step([StepItem(f"w{i}", toks[i], list(range(lens[i])))]), want[i], dtype)
            eng.release(f"w{i}")
        i, n = 2, lens[2]                                        # the last 32 one by one
        eng.add_request("d")
        check(f"{tag}: head", eng.step([StepItem("d", toks[i][:n - 32], [0, n - 33])]), want[i][[0, n - 33]], dtype)
        for t in range(n - 32, n):
            check(f"{tag}: decode at {t}", eng.step([StepItem("d", [toks[i][t]], [0])]), want[i][t:t + 1], dtype)
        eng.release("d")
        i, n, at = 3, lens[3], 0                                 # portions of changing size
        eng.add_request("p")
        while at < n:
            s = int(min(n - at, rng.choice([1, 2, 2, 3, 5, 8, 13, 17, 21, 40, 64, 65])))
            check(f"{tag}: portion {at}+{s}", eng.step([StepItem("p", toks[i][at:at + s], list(range(s)))]),
                  want[i][at:at + s], dtype)
            at += s
        eng.release("p")
        mixed_phase(eng, np.random.default_rng(trial), tag, toks, lens, want, dtype)
        eng.check_status()
        del eng
        if dtype == "bfloat16" or trial % 2:
            # the same mixed schedule three times with steps replayed from CUDA graphs where their counts
            # come again: the first pass runs directly, the second captures, the third replays, each on
            # the slots and pages that the pass before left free
            eng = Engine.open(str(folder), EngineOptions(dtype=dtype, n_ctx=0, max_requests=8, cuda_graphs=True,
                                                         max_tokens=pool, n_batch=4096))
            for rep in range(3):
                mixed_phase(eng, np.random.default_rng(trial), f"{tag} graphs pass {rep}", toks, lens, want, dtype)
            assert any(k[0] == "rows" for k in eng.stepper.graphs)
            eng.check_status()
            eng.cache.audit()
            del eng
