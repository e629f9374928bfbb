"""RMSNorm: y = x * 1/sqrt(mean(x^2) + eps) * w (crates/backend-cpu/src/kernels/norm.rs:6-39)."""
from __future__ import annotations

from .. import ops
from .base import Norm, ParamDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, *, dtype: str, size: int, eps: float):
        super().__init__()
        self.size, self.eps = int(size), float(eps)
        self.decls = {"weight": ParamDecl((self.size,), role="vector", init=("ones",))}

    def forward(self, x, out_dtype, rows=None):
        return ops.rmsnorm(x, self.w["weight"], self.eps, out_dtype, rows=rows)

    def kernel_modules(self, dtype):
        return [("elementwise", None)]
