"""Command line in FeLLM's manner: `fellm run MODEL ...` and `fellm inspect MODEL`
(crates/fellm-cli/src/main.rs:32-40,42-200,357-472,594-975,990-1013).

Options keep FeLLM's names and meanings where it has them (--max-tokens, --temperature, --top-k,
--top-p, --min-p, --frequency-penalty, --presence-penalty, --logit-bias TOKEN_ID=BIAS, --seed,
--repetition-penalty, -c/--ctx-size, -b/--batch-size, --ubatch-size, --kv-device-budget,
--kv-memory-fraction, --echo-prompt, --config, --log); precedence is command line > config file
> default (main.rs:362-366), and the file is FeLLM's fellm.toml with a [run] table whose unknown
keys are errors (crates/fellm-cli/src/config.rs:4-17).  This engine works on token ids: --prompt
takes ids ("5,17,3" or "5 17 3"), --prompt-len N makes N seeded random ids, and the generated ids
are printed to stdout; the four timing lines go to stderr as in main.rs:953-967.  `fellm bench` runs N random prompts
together through the scheduler and prints the same prompt-eval / eval figures for the batch.
--log sets the level of the `fellm_b200` logger (FeLLM: the tracing filter, main.rs:561-577).
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
import time
from pathlib import Path

log = logging.getLogger("fellm_b200")
LOG_LEVELS = {"error": logging.ERROR, "warn": logging.WARNING, "warning": logging.WARNING, "info": logging.INFO,
              "debug": logging.DEBUG, "trace": logging.DEBUG}

RUN_DEFAULTS = dict(  # fellm.toml [run]
    max_tokens=128, temperature=0.2, top_k=80, top_p=1.0, min_p=0.0, seed=0, repetition_penalty=1.05,
    frequency_penalty=0.0, presence_penalty=0.0, ctx_size=8192, batch_size=2048, ubatch_size=512,
    kv_device_budget=0, kv_memory_fraction=0.25, dtype="bfloat16", page_tokens=64, max_requests=64)


def _parser():
    ap = argparse.ArgumentParser(prog="fellm", description="fellm_b200: LFM2 inference on one B200")
    ap.add_argument("--config", help="TOML file with a [run] table (FeLLM's fellm.toml layout)")
    ap.add_argument("--log", default=None, choices=sorted(LOG_LEVELS), help="log level of the fellm_b200 logger (stderr)")
    sub = ap.add_subparsers(dest="cmd", required=True)
    run = sub.add_parser("run", help="generate from a prompt of token ids")
    run.add_argument("model", nargs="?", help="folder with config.json and model.safetensors")
    run.add_argument("--random", metavar="CONFIG_JSON", help="random weights for this config.json instead of a folder")
    run.add_argument("--prompt", help="prompt token ids, separated by commas or spaces")
    run.add_argument("--prompt-len", type=int, help="use this many seeded random token ids as the prompt")
    run.add_argument("--max-tokens", type=int)
    run.add_argument("--temperature", type=float)
    run.add_argument("--top-k", type=int)
    run.add_argument("--top-p", type=float)
    run.add_argument("--min-p", type=float)
    run.add_argument("--frequency-penalty", type=float)
    run.add_argument("--presence-penalty", type=float)
    run.add_argument("--logit-bias", action="append", default=[], metavar="TOKEN_ID=BIAS")
    run.add_argument("--seed", type=int)
    run.add_argument("--repetition-penalty", type=float)
    run.add_argument("--ctx-size", "-c", type=int, help="context size; 0 = the model's maximum")
    run.add_argument("--batch-size", "-b", type=int, help="tokens per scheduler iteration (n_batch)")
    run.add_argument("--ubatch-size", type=int, help="longest prompt portion in one step (n_ubatch)")
    run.add_argument("--kv-device-budget", "--kv-cache-bytes", type=int, dest="kv_device_budget",
                     help="bytes of cache pages (0 = from free memory)")
    run.add_argument("--kv-memory-fraction", type=float)
    run.add_argument("--dtype", choices=["bfloat16", "float32"])
    run.add_argument("--page-tokens", type=int)
    run.add_argument("--echo-prompt", action="store_true")
    bench = sub.add_parser("bench", help="run N random prompts together and print prompt-eval / eval tokens a second")
    bench.add_argument("model", nargs="?")
    bench.add_argument("--random", metavar="CONFIG_JSON")
    bench.add_argument("--requests", type=int, default=8)
    bench.add_argument("--prompt-len", type=int, default=512)
    bench.add_argument("--max-tokens", type=int)
    bench.add_argument("--temperature", type=float)
    bench.add_argument("--seed", type=int)
    for flag, kw in (("--ctx-size", dict(type=int)), ("--batch-size", dict(type=int)), ("--ubatch-size", dict(type=int)),
                     ("--kv-device-budget", dict(type=int)), ("--kv-memory-fraction", dict(type=float)),
                     ("--dtype", dict(choices=["bfloat16", "float32"])), ("--page-tokens", dict(type=int))):
        bench.add_argument(flag, **kw)
    ins = sub.add_parser("inspect", help="print a model folder's configuration and tensors")
    ins.add_argument("--model", required=True)
    return ap


def load_run_config(path):
    """The [run] table of a fellm.toml; unknown keys are errors."""
    import tomllib
    from .config.errors import ConfigError
    data = tomllib.loads(Path(path).read_text())
    run = data.get("run", {})
    for k in run:
        if k not in RUN_DEFAULTS:
            raise ConfigError(f"{path}: unknown key [run].{k}")
    for k in data:
        if k not in ("run", "log"):
            raise ConfigError(f"{path}: unknown table [{k}]")
    return run


def _file_log_level(path):
    """`log = "info"` at the top of the file (the command line's --log wins)."""
    import tomllib
    from .config.errors import ConfigError
    level = tomllib.loads(Path(path).read_text()).get("log")
    if level is not None and level not in LOG_LEVELS:
        raise ConfigError(f"{path}: log must be one of {', '.join(sorted(LOG_LEVELS))}")
    return level


def resolve_run(args) -> dict:
    """Command line > config file > default."""
    out = dict(RUN_DEFAULTS)
    if args.config:
        out.update(load_run_config(args.config))
    for k in RUN_DEFAULTS:
        v = getattr(args, k, None)
        if v is not None:
            out[k] = v
    return out


def parse_logit_bias(items):
    from .config.errors import ConfigError
    out = {}
    for it in items:
        try:
            t, b = it.split("=", 1)
            out[int(t)] = out.get(int(t), 0.0) + float(b)
        except ValueError:
            raise ConfigError(f"--logit-bias wants TOKEN_ID=BIAS, got {it!r}") from None
    return out


def parse_ids(text):
    return [int(t) for t in text.replace(",", " ").split()]


def _open_engine(args, r):
    """The engine of `run` and `bench`: options resolved as command line > file > default."""
    from .config.errors import ConfigError
    from .config.options import EngineOptions
    from .engine import Engine
    opts = EngineOptions(dtype=r["dtype"], n_ctx=r["ctx_size"], n_batch=r["batch_size"], n_ubatch=r["ubatch_size"],
                         page_tokens=r["page_tokens"], max_requests=r["max_requests"],
                         kv_memory_fraction=r["kv_memory_fraction"], kv_device_budget=r["kv_device_budget"])
    t0 = time.perf_counter()
    if args.random:
        cfg = json.loads(Path(args.random).read_text())
        engine = Engine.random(cfg, r["seed"], opts)
    elif args.model:
        engine = Engine.open(args.model, opts)
    else:
        raise ConfigError(f"fellm {args.cmd} needs a model folder or --random CONFIG_JSON")
    log.info("loaded %s in %.0f ms: context %d, cache of %d pages of %d tokens (%d bytes a token), %d request slots",
             engine.spec.architecture, (time.perf_counter() - t0) * 1e3, engine.n_ctx, engine.cache.n_pages,
             engine.cache.page_tokens, engine.cache.bytes_per_token(), engine.options.max_requests)
    print(f"loaded in {(time.perf_counter() - t0) * 1e3:.0f} ms", file=sys.stderr)
    return engine


def cmd_run(args) -> int:
    from .config.errors import ConfigError
    from .engine import GenParams
    r = resolve_run(args)
    engine = _open_engine(args, r)
    if args.prompt is not None:
        ids = parse_ids(args.prompt)
    elif args.prompt_len:
        import numpy as np
        ids = [int(t) for t in np.random.default_rng(r["seed"]).integers(0, engine.spec.vocab_size, args.prompt_len)]
    else:
        raise ConfigError("fellm run needs --prompt IDS or --prompt-len N")
    params = GenParams(max_tokens=r["max_tokens"], temperature=r["temperature"], top_k=r["top_k"], top_p=r["top_p"],
                       min_p=r["min_p"], seed=r["seed"], repetition_penalty=r["repetition_penalty"],
                       frequency_penalty=r["frequency_penalty"], presence_penalty=r["presence_penalty"],
                       logit_bias=parse_logit_bias(args.logit_bias))
    if args.echo_prompt:
        print(" ".join(map(str, ids)), end=" ", flush=True)
    stream = engine.generate(ids, params)
    for tok in stream:
        print(tok, end=" ", flush=True)
    print()
    st = stream.finish_stats()
    print(f"prompt eval: {st.prompt_tokens} tok in {st.prompt_ms:.2f}ms ({st.prompt_tok_per_sec():.2f} tok/s)", file=sys.stderr)
    print(f"eval: {st.predicted_tokens} tok in {max(st.total_ms - st.prompt_ms, 0.0):.2f}ms "
          f"({st.generation_tok_per_sec():.2f} tok/s)", file=sys.stderr)
    print(f"TTFT: {st.time_to_first_token_ms:.2f}ms", file=sys.stderr)
    print(f"total: {st.total_ms:.2f}ms", file=sys.stderr)
    log.debug("scheduler counters: %s", engine.scheduler().counters)
    return 0


def cmd_bench(args) -> int:
    """N seeded random prompts of --prompt-len ids run together through the scheduler; the figures
    are FeLLM's (crates/fellm-runtime/src/engine.rs:230-264): prompt eval = prompt tokens over the
    time to the first token, eval = generated tokens over the time after it, for the whole batch."""
    import numpy as np
    from .engine import GenParams
    r = resolve_run(args)
    r["max_requests"] = max(r["max_requests"], args.requests)
    engine = _open_engine(args, r)
    rng = np.random.default_rng(r["seed"])
    prompts = [[int(t) for t in rng.integers(0, engine.spec.vocab_size, args.prompt_len)] for _ in range(args.requests)]
    params = GenParams(max_tokens=r["max_tokens"], temperature=r["temperature"], top_k=r["top_k"], top_p=r["top_p"],
                       min_p=r["min_p"], seed=r["seed"], repetition_penalty=r["repetition_penalty"])
    engine.generate_batch([p[:8] for p in prompts[:1]], GenParams.greedy(2))          # kernels loaded before the clock starts
    t0 = time.perf_counter()
    _, stats = engine.generate_batch(prompts, params)
    total = time.perf_counter() - t0
    first = max(st.time_to_first_token_ms for st in stats) / 1e3
    n_prompt, n_gen = sum(st.prompt_tokens for st in stats), sum(st.predicted_tokens for st in stats)
    print(f"prompt eval: {n_prompt} tok in {first * 1e3:.2f}ms ({n_prompt / max(first, 1e-9):.2f} tok/s)")
    print(f"eval: {n_gen} tok in {max(total - first, 0.0) * 1e3:.2f}ms ({n_gen / max(total - first, 1e-9):.2f} tok/s)")
    print(f"total: {total * 1e3:.2f}ms for {args.requests} requests")
    log.debug("scheduler counters: %s", engine.scheduler().counters)
    return 0


def cmd_inspect(args) -> int:
    from .config.registry import read_model_config
    from .weights.safetensors_io import SafetensorsFile
    arch, cfg = read_model_config(args.model)
    print(f"architecture: {arch.name}")
    for k, v in (cfg.to_dict() if hasattr(cfg, "to_dict") else vars(cfg)).items():
        print(f"  {k}: {v}")
    if hasattr(cfg, "ff_dim"):
        print(f"  (feed-forward width after auto-adjust: {cfg.ff_dim})")
    f = SafetensorsFile(Path(args.model) / "model.safetensors")
    total = 0
    for name in sorted(f.names()):
        shape = f.shape(name)
        n = 1
        for s in shape:
            n *= s
        total += n
        print(f"{name}\t{str(f.dtype(name)).replace('torch.', '')}\t{list(shape)}")
    print(f"{len(f.names())} tensors, {total} parameters")
    f.close()
    return 0


def main(argv=None) -> int:
    from .config.errors import FellmError
    args = _parser().parse_args(argv)
    level = args.log
    try:
        if level is None and args.config:
            level = _file_log_level(args.config)
        if level is not None:
            logging.basicConfig(stream=sys.stderr, format="%(levelname)s %(name)s: %(message)s")
            log.setLevel(LOG_LEVELS[level])
        return {"run": cmd_run, "bench": cmd_bench, "inspect": cmd_inspect}[args.cmd](args)
    except FellmError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
