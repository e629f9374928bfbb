#!/usr/bin/env python3
"""Decode and prefill throughput of fellm_b200 at the LFM2-350M shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout.  `value`: decoded tokens a second at batch 8 over K decode steps in the MIDDLE
of the contexts' growth from the 2,048-token prompts to 4,096 (3,072 is the mean context of that
growth): K = 2048 times the whole growth, a small K the steps that end at 3,072, the steps before
them running untimed; `metric` and `config` name the contexts the timed steps covered.  Timed on the device with
CUDA events around K decode steps that include greedy sampling and feed the sampled tokens back on
the device.
`e2e`: the same through the Python entry point's scheduler (host tokens in from pinned memory and
out every step).  `prefill`: one 2,048-token prompt in one step.  `roofline`: bytes the decode step
has to read (every weight once, the live requests' cache and conv state) / its time, against the
measured copy bandwidth.  `points`: decode at batch 1 and 64.  The engine works on one GPU:
--gpus N > 1 prints a line that says so and exits with 2.

    python bench.py --shape 700m --workload mixed        # prompts of 128..4096 ids in portions of 512 beside decode tokens
    python bench.py --shape 1.2b --workload concurrent   # 64 requests x 2,048-id prompts x 512 steps at temperature 0.8

print one line each for the two other workloads of the benchmark (through the scheduler, host
tokens in and out); the default run adds both to the headline line under "workloads"
(`--no-workloads` leaves them out).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

LFM2_350M = dict(   # the 350M shape of the benchmark: 16 layers, attention at 2,5,8,10,12,14
    architectures=["Lfm2ForCausalLM"], vocab_size=65536, hidden_size=1024, num_hidden_layers=16,
    num_attention_heads=16, num_key_value_heads=8, head_dim=64, full_attn_idxs=[2, 5, 8, 10, 12, 14],
    block_ff_dim=6656, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256,
    rope_theta=1000000.0, rope_pairing="split_half", conv_L_cache=3, conv_bias=False, norm_eps=1e-5,
    tie_word_embeddings=True, max_position_embeddings=128000)
SEED = 2
PROMPT, CONTEXT_END, PREFILL_TOKENS = 2048, 4096, 2048
# the other shapes of the benchmark: same layers and vocabulary, (hidden, heads, block_ff_dim, seed)
SHAPES = {"350m": (1024, 16, 6656, 2), "700m": (1536, 24, 10752, 3), "1.2b": (2048, 32, 12288, 4)}


def shape_config(name):
    hidden, heads, ff, seed = SHAPES[name]
    cfg = dict(LFM2_350M)
    cfg.update(hidden_size=hidden, num_attention_heads=heads, block_ff_dim=ff)
    return cfg, seed


def untimed_steps(steps, warmup, prompt=PROMPT, context_end=CONTEXT_END):
    """Decode steps to run before the timed ones: the timed window ends at the middle of the growth from
    `prompt` to `context_end` (a window longer than half the growth is centred on it).  A window of a few
    steps then lies inside one 1,024-bucket of contexts: no step of it is the first of a new CUDA graph."""
    half = (context_end - prompt) // 2
    return max(warmup, half - steps if steps <= half else (context_end - prompt - steps) // 2)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    return 6650.0, 1590.0, 1400.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc:
            self.proc.terminate()
        sm = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 2 + i and r[2 + i] == "Active" for r in self.rows)]
        mx = max((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), default=0)
        # the median of the upper half: samples between the timed regions are idle
        busy = sm[len(sm) // 2:] if sm else []
        return {"sm_mhz": busy[len(busy) // 2] if busy else 0, "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


def model_bytes(engine):
    """Bytes a decode step reads of the weights: every matrix and vector once; the embedding
    table is the head when tied, so it counts once; the embedding gather itself reads B rows."""
    seen, total = set(), 0
    for part in engine.model.all_parts():
        for t in part.w.values():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
    return total


def flops_per_token(cfg, n_layers_attn, context):
    d, F, V = cfg.hidden_size, cfg.ff_dim, cfg.vocab_size
    H, G, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    n_conv = cfg.num_hidden_layers - n_layers_attn
    mm = n_conv * (3 * d * d + d * d) + n_layers_attn * ((H + 2 * G) * hd * d + H * hd * d) + cfg.num_hidden_layers * 3 * d * F
    return 2 * mm, 2 * V * d, 4 * H * hd * n_layers_attn        # matmul flops/token, head flops/row, attention flops per (token, key)


def run_decode(engine, batch, steps, warmup, rng, prompt=PROMPT, context_end=CONTEXT_END):
    """Prefills `batch` requests of `prompt` random ids, decodes untimed up to the `steps` steps in the
    middle of the growth from `prompt` to `context_end` (at least `warmup` steps), then times those on the device.
    Returns (tokens/s, ms/step, launches in the timed region, mean context, first and last context)."""
    import torch
    from fellm_b200.engine import GenParams, StepItem
    vocab = engine.spec.vocab_size
    reqs = [f"b{batch}_{i}" for i in range(batch)]
    params = GenParams.greedy()
    rows = []
    first = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    for i, r in enumerate(reqs):
        slot = engine.add_request(r)
        ids = rng.integers(0, vocab, prompt).tolist()
        for lo in range(0, prompt, PROMPT):                     # portions of at most PROMPT tokens (--context: longer prompts)
            part = ids[lo:lo + PROMPT]
            logits = engine.step([StepItem(r, part, [len(part) - 1] if lo + PROMPT >= prompt else [])])
        rows.append((slot, params, 0))
        first[i:i + 1] = engine.sampler.sample(logits, [rows[-1]])
    engine.check_status()
    tokens = first.clone()
    items = [StepItem(r, [0], [0]) for r in reqs]
    step = engine.stepper.step                      # the step function itself: its logits are read by the sampler at once
    sampler_launches = 0
    def one():
        # greedy rows: the step may hand back the tokens themselves (the head picks them without storing
        # the logits); else the sampler's two argmax kernels run on the logits
        nonlocal tokens, sampler_launches
        logits = step(items, device_tokens=tokens, greedy_tokens=engine.sampler.out_tokens)
        if logits is None:
            tokens = engine.sampler.out_tokens[:batch]
        else:
            tokens = engine.sampler.sample(logits, rows)
            sampler_launches += 2
    for _ in range(untimed_steps(steps, warmup, prompt, context_end)):
        one()
    torch.cuda.synchronize()
    l0 = engine.stepper.launches
    sampler_launches = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = engine.cache.length(reqs[0])
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    engine.check_status()
    launches = engine.stepper.launches - l0 + sampler_launches
    mean_ctx = ctx0 + (steps + 1) / 2                # a step at cache length c reads c + 1 positions
    for r in reqs:
        engine.release(r)
    return batch * steps / (ms / 1e3), ms / steps, launches, mean_ctx, ctx0 + 1, ctx0 + steps


def run_timeline(engine, batch, context, out_path):
    """One decode step's kernel timeline (FELLM_B200_TRACE=1): `batch` requests with `context` tokens
    of random cache each (pages reserved, no prefill), a few steps so that the step's CUDA graph
    exists, then one traced replay.  Writes a table of every launch and sums by kernel."""
    import torch
    from fellm_b200.engine import StepItem
    from fellm_b200.engine.timeline import Timeline
    reqs = [f"t{i}" for i in range(batch)]
    for r in reqs:
        engine.add_request(r)
        engine.cache.reserve(r, context)
        engine.cache.advance(r, context)
    engine.cache.flush()
    for g in engine.cache.paged:
        g.pool.normal_(0, 1)
    items = [StepItem(r, [5], [0]) for r in reqs]
    for _ in range(4):
        engine.step(items)
    torch.cuda.synchronize()
    graph = list(engine.stepper.graphs.values())[-1][0]
    tl = Timeline()
    for _ in range(3):
        graph.replay()
    tl.reset()
    graph.replay()
    launches = tl.launches(detail=True)
    tl.close()
    total = write_timeline(out_path, f"batch {batch}, context {context}", launches)
    for r in reqs:
        engine.release(r)
    return len(launches), total


def run_prefill_timeline(engine, tokens, out_path, rng):
    """The kernel timeline of one prefill step of `tokens` ids of one request (FELLM_B200_TRACE=1): three steps
    first (the shape's CUDA graph exists from the second), then one traced step."""
    import torch
    from fellm_b200.engine import StepItem
    from fellm_b200.engine.timeline import Timeline
    vocab = engine.spec.vocab_size

    def one(tag):
        engine.add_request(tag)
        engine.step([StepItem(tag, rng.integers(0, vocab, tokens).tolist(), [tokens - 1])])
        torch.cuda.synchronize()
        engine.release(tag)
    for i in range(3):
        one(f"pw{i}")
    tl = Timeline()
    one("px")
    tl.reset()
    one("pt")
    launches = tl.launches(detail=True)
    tl.close()
    return len(launches), write_timeline(out_path, f"prefill of {tokens} tokens", launches)


def write_timeline(out_path, title, launches):
    from fellm_b200.engine.timeline import Timeline
    total = launches[-1].end_us - launches[0].begin_us
    agg, prev_end = {}, None
    for l in launches:
        a = agg.setdefault((l.name, l.blocks), [0, 0.0, 0.0, 0.0])
        a[0] += 1
        a[1] += l.end_us - l.waited_us
        a[2] += l.waited_us - l.begin_us
        if prev_end is not None:
            a[3] += l.begin_us - prev_end
        prev_end = l.end_us
    lines = [f"{title}: {len(launches)} launches, {total:.1f} us from the first entry to the last exit",
             "", "| kernel | CTAs | launches | run us (mean) | before its wait us (mean) | gap to the kernel before us (mean) | sum us |",
             "|---|---|---|---|---|---|---|"]
    for (name, blocks), a in sorted(agg.items(), key=lambda kv: -(kv[1][1] + kv[1][2] + kv[1][3])):
        lines.append(f"| {name} | {blocks} | {a[0]} | {a[1] / a[0]:.2f} | {a[2] / a[0]:.2f} | {a[3] / a[0]:.2f} | {a[1] + a[2] + a[3]:.1f} |")
    lines += ["", "Per CTA, between its own wait and its exit, cut at the kernel's marks:", "", Timeline.phases(launches)]
    lines += ["", Timeline.table(launches), ""]
    with open(out_path, "w") as f:
        f.write("\n".join(lines))
    return total


def run_e2e(engine, batch, steps, warmup, rng):
    """The scheduler loop a user drives: host token ids in (pinned staging, one copy a step), the
    sampled ids back on the host every step.  Timed by the wall clock around synchronised steps."""
    import torch
    from fellm_b200.engine import GenParams
    sched = engine.scheduler()
    vocab = engine.spec.vocab_size
    # the timed steps end just below the middle of the growth: the first token comes with the prompt's last
    # portion, the scheduler launches one step ahead, and a step's graph goes by the length AFTER the step
    # (and the requests whose prompts were run first are as many tokens ahead as the prompts took steps)
    skew = -(-batch * PROMPT // 4096)
    ahead = max(untimed_steps(steps, warmup) - 6 - skew, warmup)
    for _ in range(batch):
        sched.enqueue_ids(rng.integers(0, vocab, PROMPT).tolist(), GenParams.greedy(ahead + steps + 8 + skew))   # none ends inside the window
    while any(r.prefilling for r in list(sched.running) + list(sched.waiting)) or sched.waiting:
        sched.step()
    for _ in range(ahead):
        sched.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 0
    for _ in range(steps):
        n += sum(1 for ev in sched.step() if ev.kind == "token")
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    for r in list(sched.running):
        sched.cancel(r.id)
    sched.step()
    h2d = (7 * batch + 1 + batch) * 4                             # the step's index arrays: tokens, positions, row->item, row->slot,
                                                                  # item starts (+1), item slots, item lengths, wanted rows (greedy rows ship no sampling records)
    d2h = (batch + 1) * 4                                         # sampled ids + status word
    return n / dt, h2d, d2h


def run_prefill(engine, tokens, reps, rng):
    import torch
    from fellm_b200.engine import StepItem
    vocab = engine.spec.vocab_size
    # `reps` prompts of `tokens` ids, each whole in one step, the steps queued one behind the other between two
    # events (as the decode steps are): while the device runs a step the host prepares the next, as it does under
    # the scheduler.  The time of one step alone, host preparation included, is ~0.25 ms longer.
    def steps(n, tag):
        names = [f"pf{tag}{i}" for i in range(n)]
        ids = [rng.integers(0, vocab, tokens).tolist() for _ in names]
        for r in names:
            engine.add_request(r)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for r, t in zip(names, ids):
            engine.step([StepItem(r, t, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        for r in names:
            engine.release(r)
        return e0.elapsed_time(e1) / n
    steps(2, "w")                                                 # the first runs directly, the second captures the graph
    ms = steps(reps, "t")
    engine.check_status()
    return ms


def run_mixed_workload(engine, rng, n_requests, max_new):
    """Prompts of 128..4,096 random ids through the scheduler (n_ubatch 512: prompt portions of up to
    512 tokens beside the decode tokens of the requests already generating), greedy, max_new tokens
    each.  The figures are FeLLM's (crates/fellm-cli/src/main.rs:953-967, crates/fellm-runtime/src/
    engine.rs:230-264): prompt eval = prompt tokens / time to the first token, eval = generated
    tokens / time after it, here as means over the requests, beside the batch's own totals."""
    import torch
    from fellm_b200.engine import GenParams
    sched = engine.scheduler()
    vocab = engine.spec.vocab_size
    lens = [int(n) for n in rng.integers(128, 4097, n_requests)]
    base = dict(sched.counters)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for n in lens:
        sched.enqueue_ids(rng.integers(0, vocab, n).tolist(), GenParams.greedy(max_new))
    stats, n_tok = [], 0
    while not sched.idle():
        for ev in sched.step():
            if ev.kind == "token":
                n_tok += 1
            elif ev.kind == "done":
                stats.append(ev.stats)
            elif ev.kind == "error":
                raise RuntimeError(ev.message)
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    c = {k: sched.counters[k] - base.get(k, 0) for k in sched.counters}
    return {"requests": n_requests, "prompt_tokens": sum(lens), "generated_tokens": n_tok, "wall_s": round(wall, 3),
            "tokens_per_s": round((sum(lens) + n_tok) / wall, 1),
            "prompt_eval_tok_s_mean": round(sum(s.prompt_tok_per_sec() for s in stats) / len(stats), 1),
            "eval_tok_s_mean": round(sum(s.generation_tok_per_sec() for s in stats) / len(stats), 1),
            "steps": c["steps"], "rows_per_step_mean": round(c["tokens_run"] / max(c["steps"], 1), 1),
            "mixed_step_share": round(c["mixed_steps"] / max(c["steps"], 1), 3), "preempted": c["preempted"],
            "n_ubatch": sched.n_ubatch, "n_batch": sched.n_batch}


def run_concurrent_workload(engine, rng, n_requests, prompt, steps, temperature, hbm):
    """n_requests prompts of `prompt` random ids admitted together, `steps` tokens each, sampled at
    `temperature` over the whole vocabulary (no top-k, no penalties) by the sampling kernel inside the
    loop; through the scheduler, host tokens out every step.  Decode figures cover the steps in which
    every request decodes."""
    import torch
    from fellm_b200.engine import GenParams
    sched = engine.scheduler()
    vocab = engine.spec.vocab_size
    params = GenParams(max_tokens=steps, temperature=temperature, top_k=0, top_p=1.0, min_p=0.0, seed=7,
                       repetition_penalty=1.0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_requests):
        sched.enqueue_ids(rng.integers(0, vocab, prompt).tolist(), params)
    n_tok, t_decode, tok_at_decode, ctx_sum, dec_steps = 0, None, 0, 0.0, 0
    t_decode_end, tok_at_end = None, 0
    distinct = set()
    while not sched.idle():
        all_decode = (not sched.waiting and len(sched.running) == n_requests
                      and not any(r.prefilling for r in sched.running))
        if all_decode and t_decode is None:
            torch.cuda.synchronize()
            t_decode, tok_at_decode = time.perf_counter(), n_tok
        if not all_decode and t_decode is not None and t_decode_end is None:
            # the first request is through: what follows (fewer and fewer rows a step, the requests whose prompts
            # ran first being that many tokens ahead) is not part of the decode figures
            torch.cuda.synchronize()
            t_decode_end, tok_at_end = time.perf_counter(), n_tok
        if all_decode:
            ctx_sum += sum(engine.cache.length(r.id) for r in sched.running) / n_requests + 1
            dec_steps += 1
        for ev in sched.step():
            if ev.kind == "token":
                n_tok += 1
                distinct.add(ev.token)
            elif ev.kind == "error":
                raise RuntimeError(ev.message)
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    if t_decode_end is None:
        t_decode_end, tok_at_end = t1, n_tok
    prefill_s, decode_s = t_decode - t0, t_decode_end - t_decode
    mean_ctx = ctx_sum / max(dec_steps, 1)
    wbytes = model_bytes(engine)
    state_bytes = sum(g.bytes_per_request() for g in engine.cache.fixed)
    step_bytes = wbytes + n_requests * (mean_ctx * engine.cache.bytes_per_token() + 2 * state_bytes)
    ms_step = decode_s / max(dec_steps, 1) * 1e3
    return {"requests": n_requests, "prompt_len": prompt, "decode_steps": dec_steps, "temperature": temperature,
            "prompt_eval_tok_s": round(n_requests * prompt / prefill_s, 1),
            "decode_tok_s": round((tok_at_end - tok_at_decode) / decode_s, 1), "ms_per_step": round(ms_step, 4),
            "wall_s": round(t1 - t0, 3),
            "context_mean": round(mean_ctx, 1), "distinct_tokens": len(distinct),
            "roofline_frac": round(step_bytes / (ms_step / 1e3) / 1e9 / hbm, 4), "weights_mb": wbytes // 1000000}


def workload_engine(shape, workload, layers=None):
    from fellm_b200.config import EngineOptions
    from fellm_b200.engine import Engine
    cfg, seed = shape_config(shape)
    if layers and layers < cfg["num_hidden_layers"]:
        cfg["num_hidden_layers"] = layers
        cfg["full_attn_idxs"] = [i for i in cfg["full_attn_idxs"] if i < layers]
    if workload == "mixed":
        opts = EngineOptions(dtype="bfloat16", n_ctx=8192, n_batch=2048, n_ubatch=512, page_tokens=64, max_requests=16,
                             max_tokens=16 * 4480, cuda_graphs=True)
    else:
        opts = EngineOptions(dtype="bfloat16", n_ctx=4096, n_batch=4096, n_ubatch=2048, page_tokens=64, max_requests=64,
                             max_tokens=64 * 2624, cuda_graphs=True)
    return Engine.random(cfg, seed, opts)


def run_workload(shape, workload, hbm, layers=None):
    import numpy as np
    import torch
    engine = workload_engine(shape, workload, layers)
    rng = np.random.default_rng(SHAPES[shape][3])
    c = engine.config
    if workload == "mixed":
        run_mixed_workload(engine, np.random.default_rng(0), 32, 8)         # every kernel of such a run loaded, graphs of the common shapes captured
        out = run_mixed_workload(engine, rng, 32, 128)
    else:
        run_concurrent_workload(engine, np.random.default_rng(0), 64, 128, 8, 0.8, hbm)
        out = run_concurrent_workload(engine, rng, 64, 2048, 512, 0.8, hbm)
    out.update(shape=shape, workload=workload, hidden=c.hidden_size, heads=c.num_attention_heads, ff=c.ff_dim,
               layers=c.num_hidden_layers, dtype="bf16")
    del engine
    torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2048)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="350m")
    ap.add_argument("--workload", choices=["mixed", "concurrent"], default=None,
                    help="run one of the other workloads of the benchmark at --shape and print its line")
    ap.add_argument("--no-workloads", action="store_true",
                    help="skip the two other workloads (700m/mixed, 1.2b/concurrent) that follow the headline measurement "
                         "and are reported under 'workloads'")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print a short line (for profiling a small case; not a bench value)")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="with FELLM_B200_TRACE=1: write the kernel timeline of one decode step (--batch requests, or with --only prefill of one prefill step; "
                         "--context tokens each) to FILE and stop; not a bench value")
    ap.add_argument("--context", type=int, default=PROMPT)
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "orielhaim/FeLLM is a Rust workspace (cargo + the cuda-oxide "
                          "nightly toolchain); no Rust toolchain is installed and pip cannot build it offline"}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"error": "fellm_b200 is a single-GPU engine: run with --gpus 1", "n_gpus": args.gpus}))
        return 2
    import numpy as np
    import torch
    from fellm_b200.config import EngineOptions
    from fellm_b200.engine import Engine

    hbm, tf_burst, tf_sus, src = peaks()
    if args.workload:
        clocks = ClockSampler()
        clocks.start()
        out = run_workload(args.shape, args.workload, hbm, args.layers)
        out["clocks"] = clocks.stop()
        print(json.dumps(out))
        return 0

    warmup = max(args.warmup, 3)
    cfg, seed = shape_config(args.shape)
    full_layers = cfg["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["full_attn_idxs"] = [i for i in cfg["full_attn_idxs"] if i < args.layers]
    steps = args.steps
    ctx_end = max(PROMPT, args.context) + untimed_steps(steps, warmup) + steps + 16
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    opts = EngineOptions(dtype="bfloat16", n_ctx=max(ctx_end, CONTEXT_END + 64), n_batch=4096, n_ubatch=2048, page_tokens=64,
                         max_requests=max_batch, max_tokens=max_batch * (max(ctx_end, CONTEXT_END) + 64), cuda_graphs=True)
    engine = Engine.random(cfg, seed, opts)
    rng = np.random.default_rng(seed)
    clocks = ClockSampler()
    clocks.start()

    if args.timeline and args.only == "prefill":
        n, us = run_prefill_timeline(engine, PREFILL_TOKENS, args.timeline, rng)
        print(json.dumps({"timeline": args.timeline, "prefill_tokens": PREFILL_TOKENS, "launches": n, "us": round(us, 1)}))
        clocks.stop()
        return 0
    if args.timeline:
        n, us = run_timeline(engine, args.batch, args.context, args.timeline)
        print(json.dumps({"timeline": args.timeline, "batch": args.batch, "context": args.context, "launches": n, "us": round(us, 1)}))
        clocks.stop()
        return 0
    if args.only:
        if args.only == "decode":
            v, ms, _, _, c0, c1 = run_decode(engine, args.batch, steps, warmup, rng, prompt=args.context,
                                             context_end=args.context + warmup + steps)
            print(json.dumps({"only": "decode", "batch": args.batch, "layers": cfg["num_hidden_layers"], "tokens_per_s": round(v, 1),
                              "ms_per_step": round(ms, 4), "contexts": [c0, c1]}))
        else:
            ms = run_prefill(engine, PREFILL_TOKENS, max(1, min(steps, 5)), rng)
            print(json.dumps({"only": "prefill", "layers": cfg["num_hidden_layers"], "tokens": PREFILL_TOKENS, "ms": round(ms, 4)}))
        clocks.stop()
        return 0
    value, ms_step, launches, mean_ctx, ctx_first, ctx_last = run_decode(engine, args.batch, steps, warmup, rng)
    prefill_ms = run_prefill(engine, PREFILL_TOKENS, 5, rng)
    e2e, h2d, d2h = run_e2e(engine, args.batch, min(steps, 512), warmup, rng)
    points = {}
    if not args.skip_points:
        points["decode_b1"] = round(run_decode(engine, 1, min(steps, 512), warmup, rng)[0], 1)
        points["decode_b64"] = round(run_decode(engine, 64, min(steps, 256), warmup, rng)[0], 1)
    clk = clocks.stop()

    c = engine.config
    n_attn = len(c.full_attn_idxs)
    wbytes = model_bytes(engine)
    kv_per_token = engine.cache.bytes_per_token()
    state_bytes = sum(g.bytes_per_request() for g in engine.cache.fixed)
    step_bytes = wbytes + args.batch * (mean_ctx * kv_per_token + 2 * state_bytes)
    achieved = step_bytes / (ms_step / 1e3) / 1e9
    mm, head, att = flops_per_token(c, n_attn, PREFILL_TOKENS)
    pf_flops = mm * PREFILL_TOKENS + head * 1 + att * PREFILL_TOKENS * (PREFILL_TOKENS + 1) / 2
    label = {"350m": "LFM2-350M", "700m": "LFM2-700M", "1.2b": "LFM2-1.2B"}[args.shape]
    out = {
        "metric": f"decode tok/s at batch {args.batch} ({label} shape, {PROMPT}-token prompts, timed steps at contexts "
                  f"{ctx_first}..{ctx_last})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": f"synthetic: seeded uniform-random token ids, random weights N(0,0.02) seed {seed}",
        "config": {"model": f"{label} shape", "layers": c.num_hidden_layers, "layers_of_config": full_layers,
                   "attention_layers": n_attn, "hidden": c.hidden_size, "heads": c.num_attention_heads,
                   "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim, "ff": c.ff_dim, "vocab": c.vocab_size,
                   "conv_L_cache": c.conv_L_cache, "global_batch": args.batch, "seq_len": ctx_last,
                   "context_first": ctx_first, "prompt_len": PROMPT, "page_tokens": opts.page_tokens,
                   "parallelism": "single GPU", "l2": "weights (%d MB) exceed L2, no flush" % (wbytes // 1000000),
                   "sampling": "greedy on device"},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 4), "frac": round(pf_flops / (prefill_ms / 1e3) / (tf_burst * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm, "unit": "GB/s",
                     "frac": round(achieved / hbm, 4), "peaks": src, "context_mean": round(mean_ctx, 1)},
        "points": points,
        "clocks": clk,
    }
    if not args.no_workloads and args.shape == "350m" and not args.layers:
        del engine
        torch.cuda.empty_cache()
        out["workloads"] = {}
        for key, shape, workload in (("700m_mixed", "700m", "mixed"), ("1.2b_concurrent", "1.2b", "concurrent")):
            try:
                out["workloads"][key] = run_workload(shape, workload, hbm)
            except Exception as e:                       # the headline line stands by itself
                out["workloads"][key] = {"error": f"{type(e).__name__}: {e}"[:200]}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
