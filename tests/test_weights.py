"""Weights: the container, binding by name with one clear error, kept dtypes, the random mode."""
import json
import struct

import pytest
import torch

import tiny
from fellm_b200.config import WeightError, config_from_dict
from fellm_b200.models import build_model
from fellm_b200.weights import (SafetensorsFile, bind_tensors, kept_dtype, load_into, random_tensors,
                                write_model_folder, write_safetensors)


def _model(name="A", dtype="bfloat16"):
    arch, cfg = config_from_dict(tiny.CONFIGS[name][0])
    return build_model(arch.build_spec(cfg), dtype)


def test_safetensors_roundtrip(tmp_path):
    t = {"a": torch.randn(3, 5).bfloat16(), "b": torch.arange(7, dtype=torch.int32), "c": torch.randn(4)}
    write_safetensors(tmp_path / "x.safetensors", t, metadata={"k": "v"})
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.names()) == ["a", "b", "c"]
    for k in t:
        assert torch.equal(f.tensor(k), t[k]) and f.tensor(k).dtype == t[k].dtype
    f.close()
    # the independent reader of the plain implementation agrees
    import plain_lfm2
    r = plain_lfm2.read_safetensors(tmp_path / "x.safetensors")
    assert torch.equal(r["a"], t["a"])


def test_container_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(WeightError, match="header length"):
        SafetensorsFile(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 8]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightError, match="8 bytes for shape"):
        SafetensorsFile(p)
    hdr = json.dumps({"t": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightError, match="outside the file"):
        SafetensorsFile(p)
    hdr = json.dumps({"t": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 2]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)
    with pytest.raises(WeightError, match="unsupported dtype"):
        SafetensorsFile(p)
    with pytest.raises(WeightError, match="no weight file"):
        SafetensorsFile(tmp_path / "none.safetensors")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    m = _model("A")
    t = random_tensors(m, 0)
    del t["model.layers.1.self_attn.q_proj.weight"]
    del t["model.embedding_norm.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(2)
    t["model.layers.0.conv.in_proj.weight"] = torch.zeros(64, 192).bfloat16()
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    write_safetensors(tmp_path / "model.safetensors", t)
    with pytest.raises(WeightError) as e:
        load_into(m, tmp_path, "cpu")
    msg = str(e.value)
    assert "missing tensors (2): model.embedding_norm.weight, model.layers.1.self_attn.q_proj.weight" in msg
    assert "unexpected tensors (1): model.layers.9.extra.weight" in msg
    assert "wrong shapes (1): model.layers.0.conv.in_proj.weight: file has [64, 192], model wants [192, 64]" in msg


def test_kept_dtypes():
    assert kept_dtype("matrix", torch.bfloat16, "bfloat16") == torch.bfloat16
    assert kept_dtype("matrix", torch.float32, "bfloat16") == torch.float32      # stored 32-bit stays
    assert kept_dtype("matrix", torch.float16, "bfloat16") == torch.bfloat16
    assert kept_dtype("matrix", torch.bfloat16, "float32") == torch.float32
    assert kept_dtype("vector", torch.bfloat16, "bfloat16") == torch.float32
    assert kept_dtype("table", torch.int64, "bfloat16") == torch.int32


def test_bind_on_cpu_keeps_and_fuses(tmp_path):
    m = _model("B", "bfloat16")
    t = random_tensors(m, 1)
    t["model.layers.2.self_attn.out_proj.weight"] = t["model.layers.2.self_attn.out_proj.weight"].float()
    t["model.layers.0.conv.conv.weight"] = t["model.layers.0.conv.conv.weight"].reshape(144, 1, 4)
    bind_tensors(m, t, "cpu")
    att = m.blocks[2].mixer
    assert att.w["qkv.weight"].shape == ((6 + 2) * 48, 144) and att.w["qkv.weight"].dtype == torch.bfloat16
    assert att.w["out_proj.weight"].dtype == torch.float32
    assert att.w["q_norm.weight"].dtype == torch.float32
    conv = m.blocks[0].mixer
    assert conv.w["conv.weight"].shape == (144, 4) and conv.w["conv.weight"].dtype == torch.float32
    assert m.blocks[0].ffn.w["gate_up.weight"].shape == (640, 144)
    assert m.head.w["weight"].shape == (515, 144)
    ma = _model("A", "float32")
    bind_tensors(ma, random_tensors(ma, 0), "cpu")
    assert ma.head.w["weight"] is ma.embedding.w["weight"]                       # tied
    assert ma.embedding.w["weight"].dtype == torch.float32


def test_random_mode_is_seeded_and_per_tensor(tmp_path):
    m = _model("A")
    a, b, c = random_tensors(m, 0), random_tensors(m, 0), random_tensors(m, 5)
    name = "model.layers.0.conv.in_proj.weight"
    assert torch.equal(a[name], b[name]) and not torch.equal(a[name], c[name])
    assert a[name].dtype == torch.bfloat16 and abs(float(a[name].float().std()) - 0.02) < 0.003
    assert torch.equal(a["model.layers.0.ffn_norm.weight"].float(), torch.ones(64))
    mb = _model("B")
    tb = random_tensors(mb, 1)
    assert abs(float(tb["model.layers.0.conv.in_proj.bias"].float().std()) - 0.01) < 0.003
    folder = write_model_folder(tmp_path / "m", tiny.TINY_A, 0)
    f = SafetensorsFile(folder / "model.safetensors")
    assert torch.equal(f.tensor(name), a[name])
    f.close()
    assert json.loads((folder / "config.json").read_text())["conv_L_cache"] == 3


def test_a_tied_model_takes_a_file_that_also_stores_the_head(tmp_path):
    """Files written from a state dict often carry lm_head.weight although the embeddings are
    tied: a copy of the embedding matrix is accepted, anything else is refused by name (FeLLM reads
    `output.weight` when it is there and ties otherwise, crates/fellm-model/src/graph.rs:29-34)."""
    m = _model("A", "float32")
    t = random_tensors(m, 0)
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    (tmp_path / "config.json").write_text(json.dumps(tiny.TINY_A))
    write_safetensors(tmp_path / "model.safetensors", t)
    load_into(m, tmp_path, "cpu")
    assert m.head.w["weight"] is m.embedding.w["weight"]
    t["lm_head.weight"] = t["lm_head.weight"] + 1.0
    with pytest.raises(WeightError, match="ties lm_head.weight to model.embed_tokens.weight"):
        bind_tensors(m, t, "cpu")
    t["lm_head.weight"] = torch.zeros(3, 64)
    with pytest.raises(WeightError, match="lm_head.weight: file has \\[3, 64\\], but it is tied"):
        bind_tensors(m, t, "cpu")
