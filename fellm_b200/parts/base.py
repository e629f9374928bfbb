"""Interfaces of the parts a layer is made of, and the registries that map a PartSpec.kind to
the class that builds it.

FeLLM marks the same seams with enums: `MixKind::{Attention, ShortConv, ...}`
(crates/fellm-model/src/probe.rs:36-56), the FFN kind next to it, and, for what a mixer keeps
between steps, `KvGroupKind::{FullAttention, SlidingWindow, Recurrent}`
(crates/fellm-runtime/src/kv_fabric/types.rs:101-111) plus `mutable_state_input_count`
(crates/fellm-runtime/src/compiled.rs:815-823).

No part knows which model it is in: a part gets its sizes and constants as constructor
arguments, its tensors by the local names it declares, and at run time a StepContext (who is in
the batch, at which positions) and a view of its own cache.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

# ----------------------------------------------------------------------------- parameters


@dataclass(frozen=True)
class ParamDecl:
    """A tensor a part owns.  role 'matrix': kept in the engine's dtype (bfloat16, or float32
    when the file stores 32-bit or the engine runs in 32-bit); 'vector': norm weights, conv taps
    and biases, always promoted to float32 (plugins/dspark/src/checkpoint.rs:154-169 promotes
    rank-1 tensors the same way); 'table': integer tables, int32.
    `init`: ('normal', std) | ('ones',) for the random-weights mode.
    `also`: other shapes of the same element count that a file may use."""
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal", 0.02)
    also: Tuple[Tuple[int, ...], ...] = ()


# ----------------------------------------------------------------------------- cache needs


@dataclass(frozen=True)
class PagedKV:
    """Keys and values per token: `kv_heads * head_dim` each.  `window` = how many of the
    latest positions a query reads (None: all of them)."""
    kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request, float32, zero when a request starts."""
    shape: Tuple[int, ...]


# ----------------------------------------------------------------------------- parts


class Part:
    """Base of every part.  Subclasses fill `self.decls` in __init__, get `self.w[local]`
    tensors from bind(), and may repack them in prepare()."""

    def __init__(self):
        self.decls: Dict[str, ParamDecl] = {}
        self.w: Dict[str, torch.Tensor] = {}

    def param_decls(self) -> Dict[str, ParamDecl]:
        return self.decls

    def bind(self, tensors: Dict[str, torch.Tensor]):
        self.w = dict(tensors)
        self.prepare()

    def prepare(self):
        """Called once after bind(): repack or fuse weights for the kernels."""

    def weight_order(self):
        """The part's matrices in the order its forward() reads them (for the engine's chain of weights:
        each product asks the L2 for the matrix of the product after it)."""
        return []

    def reserve(self, device, max_rows: int, n_ctx: int):
        """Called once by the engine, after bind() and before the first step: allocate here what
        the part's kernels need besides inputs and outputs, sized for steps of up to max_rows rows
        and contexts of up to n_ctx (so that nothing grows under a captured CUDA graph)."""

    def kernel_modules(self, dtype: str):
        """[(module name, defines)] of the CUDA modules this part launches in `dtype`, so that
        they can be compiled before the first step."""
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None):
        """x: float32 [T, size] (the residual stream).  Returns [T or len(rows), size] in
        out_dtype; `rows` (int32, device) picks rows of x."""
        raise NotImplementedError

    def expect(self, x: torch.Tensor):
        """A block says, before a part adds into the residual rows x: this norm reads x next.  A norm
        whose work the adding product can do on the way (RMSNorm in a decode step) arranges that here;
        nothing has to happen."""


class PositionEncoding(Part):
    """What an attention mixer needs to place queries and keys: for rotary encodings the
    inverse-frequency table and the pairing; for none, nothing."""
    kind = "none"


class Mixer(Part):
    def cache_need(self):
        """What the mixer keeps between steps: PagedKV, FixedState, None, or a list of those when
        it keeps several things (pages and a state, or two states of different shapes); `cache` in
        forward() is then a list of views in the same order."""
        return None

    def forward(self, xn: torch.Tensor, ctx, cache, out: torch.Tensor, reads_only: bool = False):
        """xn: [T, d] normed input in the engine's dtype; `out`: float32 [T, d] residual stream,
        to which the mixer ADDS its result in place.  `cache` is this run's view of its cache
        group (PagedView / StateView / None; a list of views when cache_need() returned a list).  `reads_only`: the cache belongs to an earlier run;
        read it, write nothing."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, hn: torch.Tensor, ctx, out: torch.Tensor):
        """hn: [T, d] normed input; ADDS its result to the float32 residual stream `out`."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens int32 [T] -> float32 [T, d]."""
        raise NotImplementedError


class Head(Part):
    def forward(self, xf: torch.Tensor) -> torch.Tensor:
        """xf [W, d] normed -> float32 logits [W, vocab]."""
        raise NotImplementedError

    def forward_greedy(self, xf, out_tokens: torch.Tensor) -> bool:
        """Greedy tokens of the rows without their logits: out_tokens[i] (int32, device) = argmax of row i's
        logits, ties to the lower id.  Returns False where the head has no such path for these sizes (the
        caller then takes forward() and the sampler)."""
        return False


# ----------------------------------------------------------------------------- registries

MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
EMBEDDINGS: Dict[str, type] = {}
HEADS: Dict[str, type] = {}

_TABLES = {"mixer": MIXERS, "feed_forward": FEED_FORWARDS, "norm": NORMS,
           "position": POSITION_ENCODINGS, "embedding": EMBEDDINGS, "head": HEADS}


def register_part(category: str, kind: str):
    """Class decorator: `@register_part('mixer', 'attention')`."""
    table = _TABLES[category]

    def deco(cls):
        table[kind] = cls
        cls.kind = kind
        return cls
    return deco


def build_part(category: str, spec, dtype: str):
    from ..config.errors import ConfigError
    table = _TABLES[category]
    if spec.kind not in table:
        raise ConfigError(f"unknown {category} kind {spec.kind!r}; registered: {', '.join(sorted(table))}")
    part = table[spec.kind](dtype=dtype, **spec.kwargs())
    part.spec = spec
    return part
