"""y = x W^T (+ b): the one place that picks the matrix-product kernel.

bfloat16 x bfloat16 goes to the tensor-core kernels; everything else (the 32-bit engine, and a
matrix a file stores in 32-bit under a bfloat16 engine) to the float32-FMA kernel.  FeLLM's CUDA
plugin has one dense product, bf16_matmul_rows (plugins/cuda_kernels/src/oxide_kernels.rs:3165),
with the residual fused as a third input on the CPU side (crates/backend-cpu/src/backend.rs:923-934).
"""
from __future__ import annotations

import torch

from .. import ops


def linear(x, w, bias=None, *, out=None, out_dtype=None, accumulate=False):
    """x [T, K], w [N, K] -> [T, N].  accumulate=True adds into the float32 `out` (the residual
    stream) instead of storing."""
    if ops.fast_gemm_takes(x, w):
        return ops.gemm_bf16(x, w, bias, out=out, out_dtype=out_dtype, accumulate=accumulate)
    return ops.gemm_simt(x, w, bias, out=out, out_dtype=out_dtype, accumulate=accumulate)


def linear_modules(dtype: str):
    mods = [("gemm_simt", None)]
    if dtype == "bfloat16":
        mods += ops.fast_gemm_modules()
    return mods
