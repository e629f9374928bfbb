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
