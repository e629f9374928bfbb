"""Typed configuration of the LFM2 ShortConv hybrid, read from its config.json keys.

FeLLM derives the same quantities from GGUF metadata and tensor names
(crates/fellm-model/src/probe.rs:202-525): block_count, embedding_length, head counts,
key_length, feed_forward_length, layer_norm_rms_epsilon, rope.freq_base, context_length,
vocab_size, shortconv.l_cache, and the per-layer mixer kind.  Here every one of them comes
from config.json; no size stands in code.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional, Tuple

from .errors import ConfigError

LAYER_KINDS = ("conv", "full_attention")
ROPE_PAIRINGS = ("adjacent", "split_half")


def adjusted_ff_dim(block_ff_dim: int, auto_adjust: bool, multiplier: Optional[float],
                    multiple_of: int) -> int:
    """Feed-forward width after the auto-adjust rule: F = floor(2F/3); F = floor(mult*F);
    rounded up to a multiple of `multiple_of` (6656 -> 4608 at 256; 480 -> 320 at 64).
    FeLLM's GGUF path receives the final width (probe.rs:232)."""
    f = int(block_ff_dim)
    if auto_adjust:
        f = int(2 * f / 3)
        if multiplier is not None:
            f = int(multiplier * f)
        f = multiple_of * ((f + multiple_of - 1) // multiple_of)
    return f


@dataclass(frozen=True)
class Lfm2Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    layer_types: Tuple[str, ...]
    block_ff_dim: int
    block_auto_adjust_ff_dim: bool
    block_ffn_dim_multiplier: Optional[float]
    block_multiple_of: int
    norm_eps: float
    rope_theta: float
    rope_pairing: str
    conv_L_cache: int
    conv_bias: bool
    tie_word_embeddings: bool
    max_position_embeddings: int
    extra: dict = field(default_factory=dict, compare=False)

    # ---- derived
    @property
    def ff_dim(self) -> int:
        return adjusted_ff_dim(self.block_ff_dim, self.block_auto_adjust_ff_dim,
                               self.block_ffn_dim_multiplier, self.block_multiple_of)

    @property
    def full_attn_idxs(self) -> Tuple[int, ...]:
        return tuple(i for i, k in enumerate(self.layer_types) if k == "full_attention")

    # ---- reading
    @classmethod
    def from_dict(cls, d: dict) -> "Lfm2Config":
        def need(key):
            if key not in d or d[key] is None:
                raise ConfigError(f"config.json: missing key {key!r}")
            return d[key]

        def as_int(key, value, minimum=1):
            if isinstance(value, bool) or not isinstance(value, int):
                raise ConfigError(f"config.json: {key} must be an integer, got {value!r}")
            if value < minimum:
                raise ConfigError(f"config.json: {key} must be >= {minimum}, got {value}")
            return value

        archs = d.get("architectures") or []
        if not archs:
            raise ConfigError("config.json: missing key 'architectures'")
        n_layers = as_int("num_hidden_layers", need("num_hidden_layers"))
        hidden = as_int("hidden_size", need("hidden_size"))
        heads = as_int("num_attention_heads", need("num_attention_heads"))   # probe.rs:216-219
        kv_heads = as_int("num_key_value_heads", d.get("num_key_value_heads", heads))
        if heads % kv_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads {heads} is not a multiple of "
                              f"num_key_value_heads {kv_heads}")
        hd = d.get("head_dim")
        if hd is None:
            if hidden % heads != 0:
                raise ConfigError(f"config.json: hidden_size {hidden} is not a multiple of "
                                  f"num_attention_heads {heads} and head_dim is not given")
            hd = hidden // heads                                               # probe.rs:225-227
        hd = as_int("head_dim", hd)
        if hd % 2 != 0:
            raise ConfigError(f"config.json: head_dim {hd} must be even (rotary pairs)")

        if d.get("layer_types") is not None:
            kinds = tuple(d["layer_types"])
            if len(kinds) != n_layers:
                raise ConfigError(f"config.json: layer_types has {len(kinds)} entries for "
                                  f"{n_layers} layers")
            if d.get("full_attn_idxs") is not None:
                idx = tuple(i for i, k in enumerate(kinds) if k == "full_attention")
                if tuple(sorted(d["full_attn_idxs"])) != idx:
                    raise ConfigError("config.json: layer_types and full_attn_idxs disagree")
        elif d.get("full_attn_idxs") is not None:
            idx = set()
            for i in d["full_attn_idxs"]:
                i = as_int("full_attn_idxs entry", i, minimum=0)
                if i >= n_layers:
                    raise ConfigError(f"config.json: full_attn_idxs entry {i} >= {n_layers} layers")
                idx.add(i)
            kinds = tuple("full_attention" if i in idx else "conv" for i in range(n_layers))
        else:
            raise ConfigError("config.json: need layer_types or full_attn_idxs")
        for i, k in enumerate(kinds):
            if k not in LAYER_KINDS:                                           # probe.rs:394-403
                raise ConfigError(f"config.json: layer {i} has unknown layer type {k!r} "
                                  f"(known: {', '.join(LAYER_KINDS)})")

        lc = d.get("conv_L_cache")
        if "conv" in kinds:
            if lc is None or lc == 0:                                          # probe.rs:448-452
                raise ConfigError("config.json: conv layers present but conv_L_cache is missing or 0")
            lc = as_int("conv_L_cache", lc, minimum=2)
        else:
            lc = int(lc or 0)

        mult = d.get("block_ffn_dim_multiplier")
        if mult is not None:
            mult = float(mult)
            if not mult > 0:
                raise ConfigError(f"config.json: block_ffn_dim_multiplier must be > 0, got {mult}")
        pairing = d.get("rope_pairing", "split_half")
        if pairing not in ROPE_PAIRINGS:
            raise ConfigError(f"config.json: rope_pairing {pairing!r} not in {ROPE_PAIRINGS}")
        eps = float(d.get("norm_eps", 1e-5))                                   # probe.rs:255-257
        if not eps > 0:
            raise ConfigError(f"config.json: norm_eps must be > 0, got {eps}")
        theta = float(d.get("rope_theta", 10000.0))                            # probe.rs:258
        if not theta > 0:
            raise ConfigError(f"config.json: rope_theta must be > 0, got {theta}")
        tied = d.get("tie_word_embeddings", d.get("tie_embedding", True))      # probe.rs:270
        known = {f for f in cls.__dataclass_fields__} | {"architectures", "full_attn_idxs",
                                                         "tie_embedding"}
        cfg = cls(
            architecture=str(archs[0]),
            vocab_size=as_int("vocab_size", need("vocab_size")),
            hidden_size=hidden,
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=hd,
            layer_types=kinds,
            block_ff_dim=as_int("block_ff_dim", need("block_ff_dim")),
            block_auto_adjust_ff_dim=bool(d.get("block_auto_adjust_ff_dim", False)),
            block_ffn_dim_multiplier=mult,
            block_multiple_of=as_int("block_multiple_of", d.get("block_multiple_of", 256)),
            norm_eps=eps,
            rope_theta=theta,
            rope_pairing=pairing,
            conv_L_cache=lc,
            conv_bias=bool(d.get("conv_bias", False)),
            tie_word_embeddings=bool(tied),
            max_position_embeddings=as_int("max_position_embeddings",
                                           d.get("max_position_embeddings", 4096)),  # probe.rs:262
            extra={k: v for k, v in d.items() if k not in known},
        )
        return cfg

    @classmethod
    def from_file(cls, path) -> "Lfm2Config":
        path = Path(path)
        try:
            d = json.loads(path.read_text())
        except FileNotFoundError:
            raise ConfigError(f"no config.json at {path}") from None
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON: {e}") from None
        if not isinstance(d, dict):
            raise ConfigError(f"{path}: top level must be an object")
        return cls.from_dict(d)

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        return {
            "architectures": [self.architecture],
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "layer_types": list(self.layer_types),
            "full_attn_idxs": list(self.full_attn_idxs),
            "block_ff_dim": self.block_ff_dim,
            "block_auto_adjust_ff_dim": self.block_auto_adjust_ff_dim,
            "block_ffn_dim_multiplier": self.block_ffn_dim_multiplier,
            "block_multiple_of": self.block_multiple_of,
            "norm_eps": self.norm_eps,
            "rope_theta": self.rope_theta,
            "rope_pairing": self.rope_pairing,
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": self.conv_bias,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
        }
