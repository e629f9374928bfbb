"""Token embedding (no scaling, promoted to float32: crates/fellm-model/src/graph.rs:58-65) and
the output head (final norm is a Norm part; logits = W xf in float32, W = the embedding matrix
when tied: graph.rs:29-39,111-131)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Embedding, Head, ParamDecl, register_part
from .linear import LazyNorm, linear, linear_modules


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

    def reserve(self, device, max_rows, n_ctx):
        # best (value, index) of every CTA's part of a row, for greedy steps that skip the logits
        self._argmax_keys = torch.zeros(16 * 1024, dtype=torch.int64, device=device)

    def forward_greedy(self, xf, out_tokens):
        w = self.w["weight"]
        keys = getattr(self, "_argmax_keys", None)
        if keys is None or w.dtype != torch.bfloat16 or not ops.FUSED_ARGMAX:
            return False
        rows = xf.shape[0]
        h = xf.handed_on() if isinstance(xf, LazyNorm) else None
        if h is not None and ops.row_scale_takes(rows, w.shape[0], w.shape[1]):
            need = ops.head_argmax_scratch(rows, w.shape[0], w.shape[1], False)
            if need and need <= keys.numel():
                ops.gemm_bf16_argmax(h.xg, w, None, keys, out_tokens, row_scale=(h.ssq, h.parts, xf.norm.eps))
                return True
        fused = isinstance(xf, LazyNorm) and xf.fusable_with(w)
        need = ops.head_argmax_scratch(rows, w.shape[0], w.shape[1], fused)
        if not need or need > keys.numel():
            return False
        if fused:
            ops.gemm_bf16_argmax(xf.x, w, None, keys, out_tokens, norm=(xf.norm.w["weight"], xf.norm.eps))
        else:
            x = xf.tensor() if isinstance(xf, LazyNorm) else xf
            if not ops.fast_gemm_takes(x, w):
                return False
            ops.gemm_bf16_argmax(x, w, None, keys, out_tokens)
        return True

    def weight_order(self):
        return [self.w["weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype)
