#!/usr/bin/env python3
"""Decode and prefill throughput of fellm_b200 at the LFM2-350M shape with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout.  `value`: decoded tokens a second at batch 8, contexts growing from the
2,048-token prompts (K = 2048 steps reach 4,096), timed on the device with CUDA events around K
decode steps that include greedy sampling and feed the sampled tokens back on the device.
`e2e`: the same through the Python entry point's scheduler (host tokens in from pinned memory and
out every step).  `prefill`: one 2,048-token prompt in one step.  `roofline`: bytes the decode step
has to read (every weight once, the live requests' cache and conv state) / its time, against the
measured copy bandwidth.  `points`: decode at batch 1 and 64.  The engine works on one GPU:
--gpus N > 1 prints a line that says so and exits with 2.
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


def run_decode(engine, batch, steps, warmup, rng, prompt=PROMPT):
    """Prefills `batch` requests of `prompt` random ids, then times `steps` decode steps on the
    device.  Returns (tokens/s, ms/step, launches in the timed region, mean context)."""
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
        logits = engine.step([StepItem(r, ids, [prompt - 1])])
        rows.append((slot, params, 0))
        first[i:i + 1] = engine.sampler.sample(logits, [rows[-1]])
    engine.check_status()
    tokens = first.clone()
    items = [StepItem(r, [0], [0]) for r in reqs]
    def one():
        nonlocal tokens
        logits = engine.step(items, device_tokens=tokens)
        tokens = engine.sampler.sample(logits, rows)
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    l0 = engine.stepper.launches
    s0 = engine.stepper.steps_run
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx0 = engine.cache.length(reqs[0])
    e0.record()
    for _ in range(steps):
        one()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    engine.check_status()
    launches = engine.stepper.launches - l0 + 2 * (engine.stepper.steps_run - s0)   # + the two argmax kernels a step
    mean_ctx = ctx0 + steps / 2
    for r in reqs:
        engine.release(r)
    return batch * steps / (ms / 1e3), ms / steps, launches, mean_ctx


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
    launches = tl.launches()
    tl.close()
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
    lines = [f"batch {batch}, context {context}: {len(launches)} launches, {total:.1f} us from the first entry to the last exit",
             "", "| kernel | CTAs | launches | run us (mean) | before its wait us (mean) | gap to the kernel before us (mean) | sum us |",
             "|---|---|---|---|---|---|---|"]
    for (name, blocks), a in sorted(agg.items(), key=lambda kv: -(kv[1][1] + kv[1][2] + kv[1][3])):
        lines.append(f"| {name} | {blocks} | {a[0]} | {a[1] / a[0]:.2f} | {a[2] / a[0]:.2f} | {a[3] / a[0]:.2f} | {a[1] + a[2] + a[3]:.1f} |")
    lines += ["", Timeline.table(launches), ""]
    with open(out_path, "w") as f:
        f.write("\n".join(lines))
    for r in reqs:
        engine.release(r)
    return len(launches), total


def run_e2e(engine, batch, steps, warmup, rng):
    """The scheduler loop a user drives: host token ids in (pinned staging, one copy a step), the
    sampled ids back on the host every step.  Timed by the wall clock around synchronised steps."""
    import torch
    from fellm_b200.engine import GenParams
    sched = engine.scheduler()
    vocab = engine.spec.vocab_size
    for _ in range(batch):
        sched.enqueue_ids(rng.integers(0, vocab, PROMPT).tolist(), GenParams.greedy(warmup + steps + 8))
    while any(r.prefilling for r in list(sched.running) + list(sched.waiting)) or sched.waiting:
        sched.step()
    for _ in range(warmup):
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
    times = []
    for i in range(reps + 2):
        r = f"pf{i}"
        engine.add_request(r)
        ids = rng.integers(0, vocab, tokens).tolist()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([StepItem(r, ids, [tokens - 1])])
        e1.record()
        torch.cuda.synchronize()
        if i >= 2:
            times.append(e0.elapsed_time(e1))
        engine.release(r)
    engine.check_status()
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2048)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the configuration (named in config)")
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one part only and print a short line (for profiling a small case; not a bench value)")
    ap.add_argument("--timeline", default=None, metavar="FILE",
                    help="with FELLM_B200_TRACE=1: write the kernel timeline of one decode step (--batch requests, "
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

    warmup = max(args.warmup, 3)
    cfg = dict(LFM2_350M)
    full_layers = cfg["num_hidden_layers"]
    if args.layers and args.layers < full_layers:
        cfg["num_hidden_layers"] = args.layers
        cfg["full_attn_idxs"] = [i for i in cfg["full_attn_idxs"] if i < args.layers]
    steps = args.steps
    ctx_end = PROMPT + warmup + steps + 16
    max_batch = args.batch if args.skip_points else max(args.batch, 64)
    opts = EngineOptions(dtype="bfloat16", n_ctx=max(ctx_end, CONTEXT_END + 64), n_batch=4096, n_ubatch=2048, page_tokens=64,
                         max_requests=max_batch, max_tokens=max_batch * (max(ctx_end, CONTEXT_END) + 64), cuda_graphs=True)
    engine = Engine.random(cfg, SEED, opts)
    rng = np.random.default_rng(SEED)
    hbm, tf_burst, tf_sus, src = peaks()
    clocks = ClockSampler()
    clocks.start()

    if args.timeline:
        n, us = run_timeline(engine, args.batch, args.context, args.timeline)
        print(json.dumps({"timeline": args.timeline, "batch": args.batch, "context": args.context, "launches": n, "us": round(us, 1)}))
        clocks.stop()
        return 0
    if args.only:
        if args.only == "decode":
            v, ms, _, _ = run_decode(engine, args.batch, steps, warmup, rng)
            print(json.dumps({"only": "decode", "batch": args.batch, "layers": cfg["num_hidden_layers"], "tokens_per_s": round(v, 1), "ms_per_step": round(ms, 4)}))
        else:
            ms = run_prefill(engine, PREFILL_TOKENS, max(1, min(steps, 5)), rng)
            print(json.dumps({"only": "prefill", "layers": cfg["num_hidden_layers"], "tokens": PREFILL_TOKENS, "ms": round(ms, 4)}))
        clocks.stop()
        return 0
    value, ms_step, launches, mean_ctx = run_decode(engine, args.batch, steps, warmup, rng)
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
    out = {
        "metric": "decode tok/s at batch 8 (LFM2-350M shape, contexts 2048 growing to 4096)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random weights N(0,0.02) seed 2",
        "config": {"model": "LFM2-350M shape", "layers": c.num_hidden_layers, "layers_of_config": full_layers,
                   "attention_layers": n_attn, "hidden": c.hidden_size, "heads": c.num_attention_heads,
                   "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim, "ff": c.ff_dim, "vocab": c.vocab_size,
                   "conv_L_cache": c.conv_L_cache, "global_batch": args.batch, "seq_len": CONTEXT_END,
                   "prompt_len": PROMPT, "page_tokens": opts.page_tokens, "parallelism": "single GPU",
                   "l2": "weights (%d MB) exceed L2, no flush" % (wbytes // 1000000), "sampling": "greedy on device",
                   "peaks": src},
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
        "gpu_launches": int(launches),
        "prefill": {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                    "ms": round(prefill_ms, 4), "frac": round(pf_flops / (prefill_ms / 1e3) / (tf_burst * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm, "unit": "GB/s",
                     "frac": round(achieved / hbm, 4)},
        "points": points,
        "clocks": clk,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
