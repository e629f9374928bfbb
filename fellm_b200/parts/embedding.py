"""Token embedding (no scaling, promoted to float32: crates/fellm-model/src/graph.rs:58-65) and
the output head (final norm is a Norm part; logits = W xf in float32, W = the embedding matrix
when tied: graph.rs:29-39,111-131)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, ParamDecl, register_part
from .linear import linear, linear_modules


@register_part("embedding", "table")
class TableEmbedding(Embedding):
    def __init__(self, *, dtype: str, vocab: int, size: int):
        super().__init__()
        self.vocab, self.size = int(vocab), int(size)
        self.decls = {"weight": ParamDecl((self.vocab, self.size))}

    def forward(self, tokens, status=None):
        out = torch.empty((tokens.numel(), self.size), dtype=torch.float32, device=tokens.device)
        return ops.embed_rows(tokens, self.w["weight"], out, status)

    def kernel_modules(self, dtype):
        return [("elementwise", None)]


@register_part("head", "linear")
class LinearHead(Head):
    """tied=True: owns no tensor; the model hands it the embedding matrix."""

    def __init__(self, *, dtype: str, vocab: int, size: int, tied: bool):
        super().__init__()
        self.vocab, self.size, self.tied = int(vocab), int(size), bool(tied)
        self.decls = {} if self.tied else {"weight": ParamDecl((self.vocab, self.size))}

    takes_lazy_norm = True

    def forward(self, xf):
        return linear(xf, self.w["weight"], out_dtype=torch.float32)

    def weight_order(self):
        return [self.w["weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype)
