"""RMSNorm: y = x * 1/sqrt(mean(x^2) + eps) * w (crates/backend-cpu/src/kernels/norm.rs:6-39)."""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, ParamDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    def __init__(self, *, dtype: str, size: int, eps: float):
        super().__init__()
        self.size, self.eps, self.dtype = int(size), float(eps), dtype
        self.decls = {"weight": ParamDecl((self.size,), role="vector", init=("ones",))}

    def forward(self, x, out_dtype, rows=None):
        return ops.rmsnorm(x, self.w["weight"], self.eps, out_dtype, rows=rows)

    def reserve(self, device, max_rows, n_ctx):
        if self.w["weight"].dtype == torch.float32 and self.dtype == "bfloat16":
            ops.reserve_norm_handoff(device, self.size)

    def expect(self, x):
        ops.expect_norm(x, self.w["weight"])

    def kernel_modules(self, dtype):
        return [("elementwise", None)]
