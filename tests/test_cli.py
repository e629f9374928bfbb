"""The command line's option handling (no GPU): precedence command line > file > default,
FeLLM's option names, the [run] table, logit bias and prompt parsing."""
import pytest

from fellm_b200 import cli
from fellm_b200.config import ConfigError


def parse(argv):
    return cli._parser().parse_args(argv)


def test_defaults_are_fellms():
    r = cli.resolve_run(parse(["run", "model_dir", "--prompt", "1 2 3"]))
    # fellm.toml [run]: max_tokens 128, temperature 0.2, top_k 80, top_p 1.0, seed 0, repetition_penalty 1.05,
    # ctx_size 8192, batch_size 2048, ubatch_size 512, kv_memory_fraction 0.25
    assert (r["max_tokens"], r["temperature"], r["top_k"], r["top_p"], r["seed"]) == (128, 0.2, 80, 1.0, 0)
    assert (r["repetition_penalty"], r["ctx_size"], r["batch_size"], r["ubatch_size"]) == (1.05, 8192, 2048, 512)
    assert r["kv_memory_fraction"] == 0.25 and r["dtype"] == "bfloat16"


def test_command_line_beats_file_beats_default(tmp_path):
    f = tmp_path / "fellm.toml"
    f.write_text('log = "info"\n[run]\nmax_tokens = 7\ntemperature = 0.9\nctx_size = 0\n')
    r = cli.resolve_run(parse(["--config", str(f), "run", "m", "--prompt", "1", "--temperature", "0.0", "-c", "4096",
                               "-b", "64", "--ubatch-size", "16", "--top-k", "5", "--min-p", "0.1"]))
    assert r["max_tokens"] == 7                     # file over default
    assert r["temperature"] == 0.0 and r["ctx_size"] == 4096            # command line over file
    assert (r["batch_size"], r["ubatch_size"], r["top_k"], r["min_p"]) == (64, 16, 5, 0.1)
    assert r["top_p"] == 1.0                        # default


def test_unknown_keys_in_the_file_are_errors(tmp_path):
    f = tmp_path / "bad.toml"
    f.write_text("[run]\nmax_tokenz = 7\n")
    with pytest.raises(ConfigError, match=r"unknown key \[run\].max_tokenz"):
        cli.load_run_config(f)
    f.write_text("[server]\nport = 1\n")
    with pytest.raises(ConfigError, match=r"unknown table \[server\]"):
        cli.load_run_config(f)


def test_logit_bias_and_prompt_ids():
    assert cli.parse_logit_bias(["5=1.5", "7=-2", "5=0.5"]) == {5: 2.0, 7: -2.0}
    with pytest.raises(ConfigError, match="TOKEN_ID=BIAS"):
        cli.parse_logit_bias(["5:1.5"])
    assert cli.parse_ids("5,17, 3 9") == [5, 17, 3, 9]


def test_errors_become_exit_code_one(tmp_path, capsys):
    assert cli.main(["inspect", "--model", str(tmp_path)]) == 1
    assert "no config.json" in capsys.readouterr().err
    assert cli.main(["run", "--prompt", "1"]) == 1      # neither a folder nor --random


def test_every_parsed_option_reaches_the_engine_options(tmp_path, monkeypatch):
    """An option that is parsed is used: --kv-device-budget becomes EngineOptions.kv_device_budget
    (bytes of cache pages, crates/fellm-cli/src/main.rs:42-200), --log sets the logger's level."""
    import logging
    seen = {}

    class FakeEngine:
        @staticmethod
        def open(folder, opts):
            seen["opts"] = opts
            raise ConfigError("stop here")

    import fellm_b200.engine as engine_mod
    monkeypatch.setattr(engine_mod, "Engine", FakeEngine)
    rc = cli.main(["--log", "debug", "run", "some_folder", "--prompt", "1", "--kv-device-budget", "1048576",
                   "--kv-memory-fraction", "0.5", "-c", "1024", "--page-tokens", "16"])
    assert rc == 1
    o = seen["opts"]
    assert (o.kv_device_budget, o.kv_memory_fraction, o.n_ctx, o.page_tokens) == (1048576, 0.5, 1024, 16)
    assert logging.getLogger("fellm_b200").level == logging.DEBUG
    f = tmp_path / "fellm.toml"
    f.write_text('log = "warn"\n[run]\nkv_device_budget = 4096\n')
    assert cli.main(["--config", str(f), "bench", "some_folder", "--requests", "3"]) == 1
    assert seen["opts"].kv_device_budget == 4096 and logging.getLogger("fellm_b200").level == logging.WARNING


def test_cache_size_from_a_byte_budget():
    """pages = budget / page_bytes (crates/fellm-runtime/src/kv_fabric/fabric.rs:59-61), in whole pages."""
    from fellm_b200.cache import CacheManager
    from fellm_b200.parts.base import FixedState, PagedKV
    needs = [FixedState((2, 64)), PagedKV(2, 16, None), None, PagedKV(2, 16, None), [PagedKV(1, 32, 100), FixedState((4,))]]
    per_token = (2 * 2 * 16 * 2) * 2 + 2 * 1 * 32 * 2          # bfloat16: two layers of 2x16, one of 1x32
    f = CacheManager.tokens_for_budget
    assert f(needs, 2, per_token * 1000, 16, 10 ** 9) == 992    # whole pages of 16
    assert f(needs, 2, per_token * 1000, 16, 640) == 640        # capped
    assert f(needs, 2, 10, 16, 640) == 16                       # never less than one page
    assert f(needs, 4, per_token * 1000, 64, 10 ** 9) == 448    # float32 cache: half the tokens
    assert f([FixedState((3,)), None], 2, 10 ** 6, 64, 10 ** 9) == 64
