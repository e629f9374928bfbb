"""y = x W^T (+ b): the one place that picks the matrix-product kernel.

bfloat16 x bfloat16 goes to the tensor-core kernels; everything else (the 32-bit engine, and a
matrix a file stores in 32-bit under a bfloat16 engine) to the float32-FMA kernel.  FeLLM's CUDA
plugin has one dense product, bf16_matmul_rows (plugins/cuda_kernels/src/oxide_kernels.rs:3165),
with the residual fused as a third input on the CPU side (crates/backend-cpu/src/backend.rs:923-934).

A block hands a part that says `takes_lazy_norm = True` its input as a LazyNorm: the float32
residual rows and the norm that is to be applied.  linear() then runs the norm inside the product
where the kernel can (decode-sized batches), and as a kernel of its own otherwise.  Where the product
that last added into those rows has already left them weighted for this norm (ops.expect_norm /
ops.norm_handoff), the product reads that instead and only scales its sums.
"""
from __future__ import annotations

import torch

from .. import ops


class LazyNorm:
    """Rows of the residual stream with a norm still to be applied."""

    def __init__(self, x: torch.Tensor, norm, act_dtype: torch.dtype):
        self.x, self.norm, self.act_dtype = x, norm, act_dtype
        self._done = None

    @property
    def shape(self):
        return self.x.shape

    def tensor(self) -> torch.Tensor:
        if self._done is None:
            self._done = self.norm.forward(self.x, self.act_dtype)
        return self._done

    def handed_on(self):
        """What the product that last added into the rows left for this norm (ops.norm_handoff), or None."""
        if self._done is not None or getattr(self.norm, "kind", None) != "rmsnorm":
            return None
        return ops.norm_handoff(self.x, self.norm.w["weight"])

    def fusable_with(self, w) -> bool:
        rms = getattr(self.norm, "kind", None) == "rmsnorm"
        return rms and self._done is None and ops.norm_fusable(self.x, w, self.norm.w["weight"])


def linear(x, w, bias=None, *, out=None, out_dtype=None, accumulate=False, swiglu=False):
    """x [T, K] (a tensor or a LazyNorm), w [N, K] -> [T, N].  accumulate=True adds into the
    float32 `out` (the residual stream) instead of storing; swiglu=True: w is the interleaved
    gate/up matrix and the result is SiLU(gate)*up."""
    if isinstance(x, LazyNorm):
        h = x.handed_on()
        if (h is not None and ops.fast_gemm_takes(h.xg, w) and w.data_ptr() % 16 == 0
                and ops.row_scale_takes(h.rows, w.shape[0], w.shape[1])
                and not (swiglu and out is not None and out.stride(0) % 8)):
            return ops.gemm_bf16(h.xg, w, bias, out=out, out_dtype=out_dtype, accumulate=accumulate, swiglu=swiglu,
                                 row_scale=(h.ssq, h.parts, x.norm.eps))
        if x.fusable_with(w):
            return ops.gemm_bf16(x.x, w, bias, out=out, out_dtype=out_dtype, accumulate=accumulate, swiglu=swiglu,
                                 norm=(x.norm.w["weight"], x.norm.eps))
        x = x.tensor()
    if ops.fast_gemm_takes(x, w):
        return ops.gemm_bf16(x, w, bias, out=out, out_dtype=out_dtype, accumulate=accumulate, swiglu=swiglu)
    assert not swiglu
    return ops.gemm_simt(x, w, bias, out=out, out_dtype=out_dtype, accumulate=accumulate)


def linear_modules(dtype: str):
    mods = [("gemm_simt", None)]
    if dtype == "bfloat16":
        mods += ops.fast_gemm_modules()
    return mods
