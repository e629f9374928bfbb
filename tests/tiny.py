"""The tiny LFM2 configurations the tests run, their model folders (random weights, made in a
temporary folder) and helpers to drive the engine and the plain implementation side by side.
A and B differ in every size and option."""
from __future__ import annotations

import functools
import tempfile
from pathlib import Path

import numpy as np
import torch

TINY_A = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=256, hidden_size=64, num_hidden_layers=4,
    num_attention_heads=4, num_key_value_heads=2, head_dim=16,
    layer_types=["conv", "full_attention", "conv", "full_attention"],
    block_ff_dim=192, block_auto_adjust_ff_dim=False, rope_theta=1000000.0, rope_pairing="adjacent",
    conv_L_cache=3, conv_bias=False, norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=512)
SEED_A = 0

TINY_B = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=515, hidden_size=144, num_hidden_layers=6,
    num_attention_heads=6, num_key_value_heads=1, head_dim=48,
    layer_types=["conv", "conv", "full_attention", "conv", "full_attention", "conv"],
    block_ff_dim=480, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=64,
    rope_theta=10000.0, rope_pairing="split_half", conv_L_cache=4, conv_bias=True, norm_eps=1e-6,
    tie_word_embeddings=False, max_position_embeddings=1024)
SEED_B = 1

# Not tiny in width: the sizes at which the decode step takes its single-shot products, the
# convolution in the input product's epilogue and the TMA decode attention (pages of 64 tokens).
WIDE_C = dict(
    architectures=["Lfm2ForCausalLM"], vocab_size=384, hidden_size=1024, num_hidden_layers=3,
    num_attention_heads=16, num_key_value_heads=8, head_dim=64,
    layer_types=["conv", "full_attention", "conv"],
    block_ff_dim=2048, block_auto_adjust_ff_dim=False, rope_theta=1000000.0, rope_pairing="split_half",
    conv_L_cache=3, conv_bias=False, norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=512)
SEED_C = 2

CONFIGS = {"A": (TINY_A, SEED_A), "B": (TINY_B, SEED_B), "C": (WIDE_C, SEED_C)}
_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_tests_")


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    from fellm_b200.weights import write_model_folder
    cfg, seed = CONFIGS[name]
    folder = Path(_tmp.name) / f"tiny_{name}"
    write_model_folder(folder, cfg, seed)
    return str(folder)


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    import plain_lfm2
    return plain_lfm2.load_folder(model_folder(name))


def tokens(name: str, length: int, seed: int):
    cfg, _ = CONFIGS[name]
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, cfg["vocab_size"], size=length)]


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int) -> torch.Tensor:
    import plain_lfm2
    cfg, w = plain_model(name)
    return plain_lfm2.forward(cfg, w, tokens(name, length, seed))


def make_engine(name: str, dtype: str, **opts):
    from fellm_b200.config.options import EngineOptions
    from fellm_b200.engine import Engine
    o = dict(dtype=dtype, n_ctx=0, max_requests=8, max_tokens=4096, page_tokens=16, cuda_graphs=False)
    o.update(opts)
    return Engine.open(model_folder(name), EngineOptions(**o))


# tolerances: float32 differs from the plain implementation by summation order only; bfloat16
# rounds weights-times-activations products' inputs and the activations between kernels.
def close(got: torch.Tensor, want: torch.Tensor, dtype: str):
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs().max().item()
    scale = want.abs().max().item()
    tol = (2e-5 if dtype == "float32" else 2.5e-2) * max(scale, 1e-6)
    return err <= tol, err, tol
