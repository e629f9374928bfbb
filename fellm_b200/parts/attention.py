"""GQA attention mixer with optional per-head QK RMSNorm and a position encoding, over the
paged cache (crates/fellm-model/src/graph.rs:2014-2246 for one token, 856-1050 for a batch):
q,k,v = W xn; RMSNorm per head on q,k; rotary on q,k; k (normed, rotated) and v written to the
cache; scores scaled by 1/sqrt(hd); kv head g = h // (H/G); causal, optionally windowed; W_o."""
from __future__ import annotations

import math

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import Mixer, PagedKV, ParamDecl, build_part, register_part
from .linear import linear, linear_modules


@register_part("mixer", "attention")
class Attention(Mixer):
    def __init__(self, *, dtype: str, size: int, heads: int, kv_heads: int, head_dim: int, qk_norm: bool,
                 norm_eps: float, position, window=None, shares_cache: bool = False):
        """`position`: a PartSpec of the 'position' category.  `shares_cache`: this layer keeps no
        keys and values (it has no k/v weights) and reads those of the run its schedule entry
        names."""
        super().__init__()
        self.size, self.H, self.G, self.hd = int(size), int(heads), int(kv_heads), int(head_dim)
        if self.H % self.G:
            raise ConfigError(f"attention: {self.H} heads are not a multiple of {self.G} kv heads")
        if self.hd % 16 or not 16 <= self.hd <= 256:
            raise ConfigError(f"attention: head_dim {self.hd} must be a multiple of 16 in 16..256")
        self.qk_norm, self.eps = bool(qk_norm), float(norm_eps)
        self.window = None if window is None else int(window)
        self.shares_cache = bool(shares_cache)
        self.position = build_part("position", position, dtype)
        # what the kernels need of a position part: inv_freq (float32 [rot_dim/2], or None for no
        # rotation), pairing, rot_dim <= head_dim (the rotated leading elements of a head)
        self.rot_dim = self.hd if self.position.inv_freq is None else int(getattr(self.position, "rot_dim", self.hd))
        if self.rot_dim % 2 or not 2 <= self.rot_dim <= self.hd:
            raise ConfigError(f"attention: rotary dimension {self.rot_dim} must be even and within head_dim {self.hd}")
        if self.position.inv_freq is not None and self.position.inv_freq.numel() != self.rot_dim // 2:
            raise ConfigError(f"attention: the position part gives {self.position.inv_freq.numel()} frequencies "
                              f"for a rotary dimension of {self.rot_dim}")
        self.scale = 1.0 / math.sqrt(self.hd)              # fixed in code, graph.rs:2379
        d, H, G, hd = self.size, self.H, self.G, self.hd
        self.decls = {"q_proj.weight": ParamDecl((H * hd, d)), "out_proj.weight": ParamDecl((d, H * hd))}
        if not self.shares_cache:
            self.decls.update({"k_proj.weight": ParamDecl((G * hd, d)), "v_proj.weight": ParamDecl((G * hd, d))})
        if self.qk_norm:
            self.decls["q_norm.weight"] = ParamDecl((hd,), role="vector", init=("ones",))
            if not self.shares_cache:
                self.decls["k_norm.weight"] = ParamDecl((hd,), role="vector", init=("ones",))

    takes_lazy_norm = True

    def cache_need(self):
        return PagedKV(self.G, self.hd, self.window)

    def prepare(self):
        q = self.w.pop("q_proj.weight")
        if self.shares_cache:
            self.w["qkv.weight"] = q.contiguous()
        else:
            k, v = self.w.pop("k_proj.weight"), self.w.pop("v_proj.weight")
            if not (q.dtype == k.dtype == v.dtype):
                q, k, v = q.float(), k.float(), v.float()
            self.w["qkv.weight"] = torch.cat([q, k, v], dim=0).contiguous()      # [(H+2G)*hd, d]
        self.position.to(q.device)

    def reserve(self, device, max_rows, n_ctx):
        if self.w["qkv.weight"].dtype == torch.bfloat16:
            floats, counters = ops.decode_scratch_need(max_rows, self.H, self.G, self.hd, n_ctx)
            ops.reserve_decode_scratch(device, 1, self.H, self.G, self.hd, 1, floats=floats, counters=counters)

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only != self.shares_cache:
            raise ConfigError("attention: a layer built with shares_cache must run with cache_of, and only it")
        G = 0 if self.shares_cache else self.G
        qkv = linear(xn, self.w["qkv.weight"])
        if (ctx.all_single and not self.shares_cache and qkv.dtype == torch.bfloat16 and self.rot_dim == self.hd
                and ops.decode_fuses_rope(self.H, self.G, self.hd, cache.page_tokens, cache.pool)):
            # a decode step: norm, rotation and the cache write happen inside the attention kernel
            a = ops.attention_decode(None, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                                     self.scale, self.window, ctx.max_len,
                                     fuse=(qkv, self.w.get("q_norm.weight"), self.w.get("k_norm.weight"), self.eps,
                                           self.position.inv_freq, self.position.pairing))
            linear(a, self.w["out_proj.weight"], out=out, accumulate=True)
            return out
        q = ops.qk_rope_write(qkv, self.w.get("q_norm.weight"), self.w.get("k_norm.weight"), self.eps,
                              self.position.inv_freq, self.position.pairing, ctx.positions, ctx.row_slot,
                              cache.block_table, cache.pool, cache.layer, cache.page_tokens, self.H, G,
                              self.hd, write_kv=not self.shares_cache, status=ctx.status, rot_dim=self.rot_dim)
        a = ops.paged_attention(q, cache, ctx, self.scale, self.window)
        linear(a, self.w["out_proj.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["qkv.weight"], self.w["out_proj.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("qk_rope_write", None)] + ops.attention_modules(dtype, self.hd)
