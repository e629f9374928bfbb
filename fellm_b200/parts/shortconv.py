"""ShortConv mixer: [B; C; X] = W_in xn; bx = B*X; y = W_out (C * conv(bx)) with a causal
depthwise convolution of Lc taps whose history lives in a fixed-size state per request
(crates/backend-cpu/src/kernels/shortconv.rs:61-106; crates/fellm-model/src/graph.rs:1780-1820).
FeLLM runs it for one token per request and step (crates/fellm-runtime/src/scheduler.rs:423-427);
here a request may bring a portion of any length, and the state after the portion equals the
state after the same tokens one by one."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import FixedState, Mixer, ParamDecl, register_part
from .linear import LazyNorm, linear, linear_modules


import os

FUSE_DECODE_CONV = os.environ.get("FELLM_B200_FUSE_CONV", "1") != "0"


@register_part("mixer", "shortconv")
class ShortConv(Mixer):
    def __init__(self, *, dtype: str, size: int, taps: int, bias: bool):
        super().__init__()
        self.size, self.taps, self.bias = int(size), int(taps), bool(bias)
        if not 2 <= self.taps <= ops.MAX_CONV_TAPS:
            raise ConfigError(f"shortconv: conv_L_cache {self.taps} is outside 2..{ops.MAX_CONV_TAPS}")
        d = self.size
        self.decls = {"in_proj.weight": ParamDecl((3 * d, d)),
                      "conv.weight": ParamDecl((d, self.taps), role="vector", also=((d, 1, self.taps),)),
                      "out_proj.weight": ParamDecl((d, d))}
        if self.bias:
            self.decls.update({"in_proj.bias": ParamDecl((3 * d,), role="vector", init=("normal", 0.01)),
                               "conv.bias": ParamDecl((d,), role="vector", init=("normal", 0.01)),
                               "out_proj.bias": ParamDecl((d,), role="vector", init=("normal", 0.01))})

    takes_lazy_norm = True
    blocked = False

    def prepare(self):
        """On the tensor-core path the input projection's rows are put in blocks of 16 channels (16
        B rows, 16 C rows, 16 X rows), so that one CTA of a decode step's product holds B, C and X
        of its channels and runs the convolution itself; the convolution kernel of the other steps
        reads the same order."""
        w = self.w["in_proj.weight"]
        self.blocked = w.dtype == torch.bfloat16 and w.is_cuda and self.size % 16 == 0
        if self.blocked:
            self.w["in_proj.weight"] = ops.block_bcx_rows(w)
            if "in_proj.bias" in self.w:
                self.w["in_proj.bias"] = ops.block_bcx_rows(self.w["in_proj.bias"])

    def cache_need(self):
        return FixedState((self.taps - 1, self.size))

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only:
            raise ConfigError("a shortconv layer cannot run on another layer's state")
        w_in, b_in = self.w["in_proj.weight"], self.w.get("in_proj.bias")
        if self.blocked and FUSE_DECODE_CONV and ctx.all_single and ops.conv_product_takes(ctx.n_rows, 3 * self.size, self.size, self.taps):
            # a decode step: product and convolution in one launch
            h = xn.handed_on() if isinstance(xn, LazyNorm) else None
            scale = None
            if h is not None:
                x, norm, scale = h.xg, None, (h.ssq, h.parts, xn.norm.eps)
            elif ctx.n_rows <= 16 and isinstance(xn, LazyNorm) and xn.fusable_with(w_in):
                x, norm = xn.x, (xn.norm.w["weight"], xn.norm.eps)
            else:
                x, norm = (xn.tensor() if isinstance(xn, LazyNorm) else xn), None
            y = ops.gemm_bf16_conv(x, w_in, b_in, self.w["conv.weight"], self.w.get("conv.bias"), cache.states,
                                   cache.item_slot, norm=norm, row_scale=scale)
        else:
            bcx = linear(xn, w_in, b_in)
            y = ops.shortconv(bcx, self.w["conv.weight"], self.w.get("conv.bias"), cache.states, cache.item_slot,
                              ctx.item_start, ctx.row_item, ctx.n_items, ctx.all_single, blocked=self.blocked)
        linear(y, self.w["out_proj.weight"], self.w.get("out_proj.bias"), out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["in_proj.weight"], self.w["out_proj.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("shortconv", None)]
