"""ShortConv mixer: [B; C; X] = W_in xn; bx = B*X; y = W_out (C * conv(bx)) with a causal
depthwise convolution of Lc taps whose history lives in a fixed-size state per request
(crates/backend-cpu/src/kernels/shortconv.rs:61-106; crates/fellm-model/src/graph.rs:1780-1820).
FeLLM runs it for one token per request and step (crates/fellm-runtime/src/scheduler.rs:423-427);
here a request may bring a portion of any length, and the state after the portion equals the
state after the same tokens one by one."""
from __future__ import annotations

from .. import ops
from ..config.errors import ConfigError
from .base import FixedState, Mixer, ParamDecl, register_part
from .linear import linear, linear_modules


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

    def cache_need(self):
        return FixedState((self.taps - 1, self.size))

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only:
            raise ConfigError("a shortconv layer cannot run on another layer's state")
        bcx = linear(xn, self.w["in_proj.weight"], self.w.get("in_proj.bias"))
        y = ops.shortconv(bcx, self.w["conv.weight"], self.w.get("conv.bias"), cache.states,
                          cache.item_slot, ctx.item_start, ctx.row_item, ctx.n_items, ctx.all_single)
        linear(y, self.w["out_proj.weight"], self.w.get("out_proj.bias"), out=out, accumulate=True)
        return out

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("shortconv", None)]
