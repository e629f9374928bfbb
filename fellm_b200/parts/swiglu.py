"""SwiGLU feed-forward: f = W_down (silu(W_gate h) * (W_up h)), silu(g) = g/(1+exp(-g))
(crates/fellm-model/src/graph.rs:2260-2287; crates/backend-cpu/src/kernels/swiglu.rs:4-16)."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, ParamDecl, register_part
from .linear import LazyNorm, linear, linear_modules


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    def __init__(self, *, dtype: str, size: int, ff: int):
        super().__init__()
        self.size, self.ff = int(size), int(ff)
        self.decls = {"gate.weight": ParamDecl((self.ff, self.size)),
                      "up.weight": ParamDecl((self.ff, self.size)),
                      "down.weight": ParamDecl((self.size, self.ff))}

    def prepare(self):
        """One product for gate and up.  On the tensor-core path the rows are interleaved in blocks
        of 8 gate / 8 up so that the product's epilogue computes SiLU(gate)*up itself; otherwise
        [2F, d] with the gate rows first, and a separate SiLU kernel."""
        g, u = self.w.pop("gate.weight"), self.w.pop("up.weight")
        if g.dtype != u.dtype:
            g, u = g.float(), u.float()
        self.fused = (g.dtype == torch.bfloat16 and g.is_cuda and self.ff % 8 == 0 and self.size % 8 == 0)
        if self.fused:
            self.w["gate_up.weight"] = ops.interleave_gate_up(g, u)
        else:
            self.w["gate_up.weight"] = torch.cat([g, u], dim=0).contiguous()

    takes_lazy_norm = True

    def forward(self, hn, ctx, out):
        if self.fused:
            z = linear(hn, self.w["gate_up.weight"], swiglu=True)
        else:
            z = ops.silu_mul(linear(hn, self.w["gate_up.weight"]))
        linear(z, self.w["down.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["gate_up.weight"], self.w["down.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("elementwise", None)]
