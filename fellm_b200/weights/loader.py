"""Binds a model's parameters to the tensors of a safetensors file by name.

Every tensor a part declares is looked up under the name the architecture gave it; all problems
are gathered and raised as ONE WeightError that lists missing tensors, unexpected tensors and
wrong shapes (FeLLM stops at the first: `missing tensor <name>`,
plugins/dspark/src/checkpoint.rs:150-153; shape checks in
crates/backend-cpu/src/kernels/shortconv.rs:44-68).

What is kept: matrices in bfloat16 under a bfloat16 engine unless the file stores them in 32-bit,
in which case they stay 32-bit; everything float32 under a float32 engine; vectors (norm weights,
conv taps, biases) always float32 (checkpoint.rs:154-169 promotes rank-1 tensors); integer tables
int32.
"""
from __future__ import annotations

from pathlib import Path
from typing import Dict

import numpy as np
import torch

from ..config.errors import WeightError
from .safetensors_io import SafetensorsFile


def kept_dtype(role: str, stored: torch.dtype, engine_dtype: str) -> torch.dtype:
    if role == "table":
        return torch.int32
    if role == "vector" or engine_dtype == "float32":
        return torch.float32
    if stored == torch.float32:
        return torch.float32              # a tensor stored in 32-bit stays so
    return torch.bfloat16


def _convert(t: torch.Tensor, decl, engine_dtype: str, device) -> torch.Tensor:
    want = kept_dtype(decl.role, t.dtype, engine_dtype)
    t = t.reshape(decl.shape)
    return t.to(device=device, dtype=want).contiguous()


def check_and_collect(model, available: Dict[str, tuple]):
    """available: {name: shape}.  Returns the problems as three lists."""
    table = model.param_table()
    aliases = model.tied_aliases()
    missing = [n for n in table if n not in available]
    unexpected = [n for n in available if n not in table and n not in aliases]
    wrong = []
    for alias, owner in aliases.items():
        if alias in available and owner in available and tuple(available[alias]) != tuple(available[owner]):
            wrong.append(f"{alias}: file has {list(available[alias])}, but it is tied to {owner} {list(available[owner])}")
    for name, (_, _, decl) in table.items():
        if name in available:
            shape = tuple(available[name])
            if shape != tuple(decl.shape) and shape not in decl.also:
                wrong.append(f"{name}: file has {list(shape)}, model wants {list(decl.shape)}")
    return missing, unexpected, wrong


def _raise_if_any(where, missing, unexpected, wrong):
    if not (missing or unexpected or wrong):
        return
    parts = [f"{where} does not match the model:"]
    if missing:
        parts.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        parts.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        parts.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(sorted(wrong)))
    raise WeightError("\n".join(parts))


def _check_aliases(where, model, names, get):
    """A tensor the model ties to another one may be in the file too, but only as a copy."""
    for alias, owner in model.tied_aliases().items():
        if alias in names and not torch.equal(get(alias), get(owner)):
            raise WeightError(f"{where}: the model ties {alias} to {owner}, but the file's {alias} holds other "
                              "values; set tie_word_embeddings to false to use it")


def load_into(model, folder, device) -> None:
    """Reads <folder>/model.safetensors and binds every parameter of `model`."""
    path = Path(folder) / "model.safetensors"
    f = SafetensorsFile(path)
    try:
        missing, unexpected, wrong = check_and_collect(model, {n: f.shape(n) for n in f.names()})
        _raise_if_any(str(path), missing, unexpected, wrong)
        _check_aliases(str(path), model, set(f.names()), f.tensor)
        tensors = {}
        for name, (_, _, decl) in model.param_table().items():
            tensors[name] = _convert(f.tensor(name), decl, model.dtype, device)
    finally:
        f.close()
    model.bind(tensors)


def bind_tensors(model, tensors: Dict[str, torch.Tensor], device) -> None:
    """Binds from tensors in memory (the random-weights mode without a file)."""
    missing, unexpected, wrong = check_and_collect(model, {n: tuple(t.shape) for n, t in tensors.items()})
    _raise_if_any("the given tensors", missing, unexpected, wrong)
    _check_aliases("the given tensors", model, set(tensors), tensors.__getitem__)
    table = model.param_table()
    model.bind({n: _convert(tensors[n], table[n][2], model.dtype, device) for n in table})
