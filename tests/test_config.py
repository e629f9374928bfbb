"""Configuration and registry (no GPU)."""
import copy
import json

import pytest

import tiny
from fellm_b200.config import (ConfigError, EngineOptions, Lfm2Config, adjusted_ff_dim, architectures,
                               config_from_dict, get_architecture, read_model_config)
from fellm_b200.models import build_model
from fellm_b200.parts.base import FixedState, PagedKV


def test_reads_every_key_of_both_tiny_configs():
    a = Lfm2Config.from_dict(tiny.TINY_A)
    b = Lfm2Config.from_dict(tiny.TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (144, 6, 1, 48)
    assert a.ff_dim == 192 and b.ff_dim == 320
    assert a.full_attn_idxs == (1, 3) and b.full_attn_idxs == (2, 4)
    assert a.rope_pairing == "adjacent" and b.rope_pairing == "split_half"
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert (a.conv_L_cache, a.conv_bias, a.norm_eps) == (3, False, 1e-5)
    assert (b.conv_L_cache, b.conv_bias, b.norm_eps) == (4, True, 1e-6)


def test_ff_auto_adjust():
    assert adjusted_ff_dim(6656, True, 1.0, 256) == 4608
    assert adjusted_ff_dim(10752, True, 1.0, 256) == 7168
    assert adjusted_ff_dim(12288, True, 1.0, 256) == 8192
    assert adjusted_ff_dim(480, True, 1.0, 64) == 320
    assert adjusted_ff_dim(480, False, 1.0, 64) == 480
    assert adjusted_ff_dim(480, True, None, 64) == 320


def test_full_attn_idxs_instead_of_layer_types():
    d = copy.deepcopy(tiny.TINY_A)
    del d["layer_types"]
    d["full_attn_idxs"] = [1, 3]
    assert Lfm2Config.from_dict(d).layer_types == ("conv", "full_attention", "conv", "full_attention")
    d["layer_types"] = ["conv", "conv", "conv", "full_attention"]
    with pytest.raises(ConfigError, match="disagree"):
        Lfm2Config.from_dict(d)


@pytest.mark.parametrize("edit, match", [
    (lambda d: d.pop("hidden_size"), "missing key 'hidden_size'"),
    (lambda d: d.update(num_attention_heads=0), "num_attention_heads must be >= 1"),
    (lambda d: d.update(num_key_value_heads=3), "not a multiple"),
    (lambda d: d.update(layer_types=["conv", "full_attention"]), "2 entries for 4 layers"),
    (lambda d: d.update(layer_types=["conv", "mamba", "conv", "conv"]), "unknown layer type 'mamba'"),
    (lambda d: d.update(conv_L_cache=0), "conv_L_cache is missing or 0"),
    (lambda d: d.update(rope_pairing="both"), "rope_pairing"),
    (lambda d: d.update(norm_eps=0.0), "norm_eps"),
    (lambda d: d.update(architectures=[]), "architectures"),
    (lambda d: d.update(vocab_size="many"), "must be an integer"),
    (lambda d: d.update(head_dim=15), "must be even"),
])
def test_config_errors(edit, match):
    d = copy.deepcopy(tiny.TINY_A)
    edit(d)
    with pytest.raises(ConfigError, match=match):
        Lfm2Config.from_dict(d)


def test_registry():
    assert "Lfm2ForCausalLM" in architectures()
    arch, cfg = config_from_dict(tiny.TINY_B)
    assert arch is get_architecture("Lfm2ForCausalLM") and isinstance(cfg, Lfm2Config)
    d = dict(tiny.TINY_A, architectures=["LlamaForCausalLM"])
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'"):
        config_from_dict(d)


def test_read_model_config_errors(tmp_path):
    with pytest.raises(ConfigError, match="no config.json"):
        read_model_config(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_model_config(tmp_path)
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    assert read_model_config(tmp_path)[1].vocab_size == 256


def test_spec_is_data_and_parts_follow_it():
    arch, cfg = config_from_dict(tiny.TINY_B)
    spec = arch.build_spec(cfg)
    assert [l.mixer.kind for l in spec.layers] == ["shortconv", "shortconv", "attention", "shortconv",
                                                   "attention", "shortconv"]
    assert [r.layer for r in spec.schedule] == list(range(6)) and all(r.cache_of is None for r in spec.schedule)
    m = build_model(spec, "float32")
    needs = m.cache_needs()
    assert needs[0] == FixedState((3, 144)) and needs[2] == PagedKV(1, 48, None)
    names = m.param_table()
    assert "model.layers.2.self_attn.q_layernorm.weight" in names and "lm_head.weight" in names
    assert names["model.layers.0.feed_forward.w1.weight"][1] == "gate.weight"
    assert names["model.layers.0.conv.conv.weight"][2].shape == (144, 4)


def test_engine_options_validate():
    EngineOptions().validate()
    with pytest.raises(ConfigError):
        EngineOptions(dtype="float16").validate()
    with pytest.raises(ConfigError):
        EngineOptions(page_tokens=48).validate()
