"""Random-weights mode: tensors from a configuration and a seed, and a model folder written from
them (config.json + model.safetensors), so that the loader is the path every model takes.

Matrices, embeddings and conv taps ~ N(0, 0.02), biases ~ N(0, 0.01), norm weights 1.0 (each
part's ParamDecl.init says which).  Every tensor has its own generator, seeded from the seed and
the tensor's name, so a tensor's values do not depend on which other tensors exist.  Values are
rounded to bfloat16 (the dtype the folder stores) before anything uses them.  FeLLM has no such
mode.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Dict

import torch

from ..config.registry import config_from_dict
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensors(model, seed: int, store_dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """{file name: CPU tensor in store_dtype} for every parameter of `model`."""
    out = {}
    for name, (_, _, decl) in model.param_table().items():
        if decl.init[0] == "ones":
            t = torch.ones(decl.shape, dtype=torch.float32)
        elif decl.init[0] == "normal":
            g = torch.Generator(device="cpu")
            g.manual_seed(_tensor_seed(seed, name))
            t = torch.empty(decl.shape, dtype=torch.float32).normal_(0.0, float(decl.init[1]), generator=g)
        else:
            raise ValueError(f"unknown init {decl.init!r} for {name}")
        out[name] = t.to(store_dtype)
    return out


def write_model_folder(folder, config_dict: dict, seed: int, store_dtype=torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config_dict` with random weights."""
    from ..models.model import build_model
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    arch, cfg = config_from_dict(config_dict)
    model = build_model(arch.build_spec(cfg), "float32")
    tensors = random_tensors(model, seed, store_dtype)
    (folder / "config.json").write_text(json.dumps(cfg.to_dict() if hasattr(cfg, "to_dict") else config_dict,
                                                   indent=1))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": seed})
    return folder
