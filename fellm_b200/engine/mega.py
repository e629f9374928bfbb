"""The whole-step decode kernel's host side: turns a model's parts into the stage program that
fellm_b200/csrc/decode_mega.cu interprets, and runs it.

A decode step of the bfloat16 engine (every item one token, at most 16 items, logits wanted for
every row) is ~90 dependent kernel launches on the per-kernel path; here it is one cooperative
launch whose stages are separated by grid barriers.  The builder knows these parts: table
embedding, RMSNorm, ShortConv, Attention (QK norm, rotary or none), SwiGLU, linear head.  A model
with any other part (a test's toy mixer, say) keeps the per-kernel path: `MegaDecoder.supported`
is False.  FeLLM replays a captured per-op graph instead (crates/backend-cuda/src/graph.rs:39-160).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import numpy as np
import torch

from .. import ops
from ..cache.manager import PagedView, StateView
from ..config.errors import KernelError
from ..parts.attention import Attention
from ..parts.embedding import LinearHead, TableEmbedding
from ..parts.rmsnorm import RMSNorm
from ..parts.rope import NoPosition, Rotary
from ..parts.shortconv import ShortConv
from ..parts.swiglu import SwiGLU

K_EMBED, K_GEMM, K_ROPE, K_ATTN, K_ARGMAX_PART, K_ARGMAX_FIN = range(6)
E_STORE, E_ACC, E_SWIGLU, E_F32 = range(4)
SLOTS = 40
WARPS = 8
ROUND_K = 2 * 5 * 32            # k a warp keeps in flight: two rounds of five 32-wide chunks
MAX_ROWS = 16


def _f(x: float) -> int:
    return int(np.float64(x).view(np.int64))


def _p(t: Optional[torch.Tensor]) -> int:
    return 0 if t is None else t.data_ptr()


class MegaDecoder:
    def __init__(self, model, cache, device):
        self.model, self.cache, self.device = model, cache, device
        self.n_sm = torch.cuda.get_device_properties(device).multi_processor_count
        self.reason = self._unsupported_reason()
        self.supported = self.reason is None
        self.programs: Dict[tuple, dict] = {}
        self.barrier = torch.zeros(self.n_sm, dtype=torch.int32, device=device) if self.supported else None
        self._fn = None
        self.launches = 0
        self.trace_next = False          # set to True to have the next step record per-stage times (last_trace)
        self.last_trace = None
        self.last_kinds = None

    # ------------------------------------------------------------------ can this model be fused?
    def _unsupported_reason(self) -> Optional[str]:
        m = self.model
        if m.dtype != "bfloat16":
            return "the fused decode step is a bfloat16 kernel"
        if not isinstance(m.embedding, TableEmbedding) or m.embedding.w["weight"].dtype != torch.bfloat16:
            return "embedding part or dtype not known to the builder"
        if not isinstance(m.head, LinearHead) or not isinstance(m.final_norm, RMSNorm):
            return "head or final norm not known to the builder"
        hd = None
        for b in m.blocks:
            if not (isinstance(b.norm1, RMSNorm) and isinstance(b.norm2, RMSNorm) and isinstance(b.ffn, SwiGLU)):
                return "a block's norm or feed-forward is not known to the builder"
            if not b.ffn.fused:
                return "feed-forward width or dtype keeps the SiLU epilogue off"
            mats = [b.ffn.w["gate_up.weight"], b.ffn.w["down.weight"]]
            if isinstance(b.mixer, ShortConv):
                mats += [b.mixer.w["in_proj.weight"], b.mixer.w["out_proj.weight"]]
            elif isinstance(b.mixer, Attention):
                a = b.mixer
                if a.shares_cache or a.window is not None and a.window < 1:
                    return "attention variant not known to the builder"
                if not isinstance(a.position, (Rotary, NoPosition)):
                    return "position encoding not known to the builder"
                if hd is not None and hd != a.hd:
                    return "layers with different head sizes"
                hd = a.hd
                mats += [a.w["qkv.weight"], a.w["out_proj.weight"]]
            else:
                return f"mixer {type(b.mixer).__name__} is not known to the builder"
            for w in mats:
                if w.dtype != torch.bfloat16 or w.shape[1] % 8 or w.stride(0) % 8:
                    return "a matrix is not bfloat16 or its width is not a multiple of 8"
        if m.head.w["weight"].dtype != torch.bfloat16:
            return "head dtype"
        if any(r.cache_of is not None for r in m.schedule):
            return "a layer reads another layer's cache"
        if m.spec.hidden_size % 8:
            return "width is not a multiple of 8"
        self.hd = hd or 64
        return None

    # ------------------------------------------------------------------ stage records
    def _gemm(self, M, W, out, epi, *, x=None, xf=None, norm=None, bias=None, conv=None, upd=None):
        N, K = W.shape
        n_tiles = -(-N // 16)
        slices = 1
        while slices < WARPS and -(-K // slices) > ROUND_K:
            slices *= 2
        if n_tiles * slices > 2 * self.n_sm * WARPS:        # too many items to hold in flight: stream whole-K slabs
            slices = 1
        warps_k = slices
        k_per_warp = -(-(-(-K // warps_k)) // 32) * 32
        k_cta = warps_k * k_per_warp
        xs_stride = k_cta + (32 if k_cta % 64 == 0 else 0)
        warps_n = WARPS // warps_k
        tiles_per_warp = -(-n_tiles // (self.n_sm * warps_n))
        mt = 1 if M <= 8 else 2
        smem = mt * 8 * xs_stride * 2 + (0 if warps_k == 1 else WARPS * tiles_per_warp * 16 * mt * 8 * 4)
        if epi == E_SWIGLU:
            assert N % 16 == 0
        v = [0] * SLOTS
        v[0], v[1] = K_GEMM, M
        v[2], v[3] = _p(x), _p(xf)
        if norm is not None:
            v[4], v[5] = _p(norm.w["weight"]), _f(norm.eps)
        v[6], v[7], v[8], v[9], v[10], v[11] = _p(W), _p(bias), _p(out), epi, N, K
        v[12] = (xf if xf is not None else x).stride(0) if (xf is not None or x is not None) else 0
        v[13], v[14] = W.stride(0), out.stride(0)
        v[15], v[16], v[17], v[18], v[19] = warps_k, k_per_warp, xs_stride, n_tiles, tiles_per_warp
        if conv is not None:
            bcx, cw, cb, states, item_slot, Lc = conv
            v[20], v[21], v[22], v[23], v[24], v[25], v[26] = _p(bcx), _p(cw), _p(cb), _p(states), states.stride(0), Lc, _p(item_slot)
        if upd is not None:
            bcx, states, Lc, d, item_slot = upd
            v[27], v[28], v[29], v[30], v[31], v[32] = _p(bcx), _p(states), states.stride(0), Lc, d, _p(item_slot)
        return v, smem

    def _build(self, ctx, views, split):
        m, dev = self.model, self.device
        M, d, V = ctx.n_rows, m.spec.hidden_size, m.spec.vocab_size
        bf, f32 = torch.bfloat16, torch.float32
        keep: List[torch.Tensor] = []

        def buf(shape, dtype):
            t = torch.zeros(shape, dtype=dtype, device=dev)
            keep.append(t)
            return t
        x_res = buf((M, d), f32)
        logits = buf((M, V), f32)
        bcx_buf = buf((M, 3 * d), bf)                       # in-projection output: B | C | X
        qkv_w = max([8] + [(b.mixer.H + 2 * b.mixer.G) * b.mixer.hd for b in m.blocks if isinstance(b.mixer, Attention)])
        qkv_buf = buf((M * qkv_w,), bf)
        ff = max(b.ffn.ff for b in m.blocks)
        z = buf((M, ff), bf)
        att_q = att_o = None
        stages, smem = [], 0

        def add(rec):
            nonlocal smem
            if isinstance(rec, tuple):
                rec, need = rec
                smem = max(smem, need)
            stages.append(rec)
        emb = m.embedding
        v = [0] * SLOTS
        v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7] = K_EMBED, M, _p(ctx.tokens), _p(emb.w["weight"]), _p(x_res), d, emb.vocab, _p(ctx.status)
        add(v)
        split_len, max_splits = split
        for n, run in enumerate(m.schedule):
            b = m.blocks[run.layer]
            view = views[n]
            upd = None
            if isinstance(b.mixer, ShortConv):
                c = b.mixer
                assert isinstance(view, StateView)
                bcx = bcx_buf
                add(self._gemm(M, c.w["in_proj.weight"], bcx, E_STORE, xf=x_res, norm=b.norm1, bias=c.w.get("in_proj.bias")))
                add(self._gemm(M, c.w["out_proj.weight"], x_res, E_ACC, bias=c.w.get("out_proj.bias"),
                               conv=(bcx, c.w["conv.weight"], c.w.get("conv.bias"), view.states, ctx.item_slot, c.taps)))
                upd = (bcx, view.states, c.taps, d, ctx.item_slot)
            else:
                a = b.mixer
                assert isinstance(view, PagedView)
                width = (a.H + 2 * a.G) * a.hd
                qkv = qkv_buf[:M * width].view(M, width)
                if att_q is None:
                    att_q, att_o = buf((M, a.H, a.hd), bf), buf((M, a.H * a.hd), bf)
                add(self._gemm(M, a.w["qkv.weight"], qkv, E_STORE, xf=x_res, norm=b.norm1))
                v = [0] * SLOTS
                v[0], v[1], v[2] = K_ROPE, M, _p(qkv)
                v[3], v[4], v[5] = _p(a.w.get("q_norm.weight")), _p(a.w.get("k_norm.weight")), _f(a.eps)
                v[6], v[7] = _p(a.position.inv_freq), ops.PAIRINGS[a.position.pairing]
                v[8], v[9], v[10], v[11] = _p(ctx.positions), _p(ctx.row_slot), _p(view.block_table), view.block_table.shape[1]
                v[12], v[13], v[14], v[15] = _p(view.pool), view.layer, view.pool.shape[1], view.page_tokens
                v[16], v[17], v[18], v[19] = _p(att_q), a.H, a.G, _p(ctx.status)
                add(v)
                scratch, counters = ops.reserve_decode_scratch(dev, M, a.H, a.G, a.hd, max_splits)
                v = [0] * SLOTS
                v[0], v[1], v[2], v[3], v[4], v[5] = K_ATTN, M, _p(att_q), _p(view.pool), _p(view.block_table), view.block_table.shape[1]
                v[6], v[7], v[8], v[9], v[10] = _p(ctx.positions), _p(ctx.row_slot), _p(att_o), _p(scratch), _p(counters)
                v[11], v[12], v[13], v[14], v[15] = a.H, a.G, view.page_tokens, view.layer, view.pool.shape[1]
                v[16], v[17], v[18], v[19] = _f(a.scale * 1.4426950408889634), int(a.window or 0), split_len, max_splits
                add(v)
                add(self._gemm(M, a.w["out_proj.weight"], x_res, E_ACC, x=att_o))
            f = b.ffn
            add(self._gemm(M, f.w["gate_up.weight"], z[:, :f.ff], E_SWIGLU, xf=x_res, norm=b.norm2, upd=upd))
            add(self._gemm(M, f.w["down.weight"], x_res, E_ACC, x=z[:, :f.ff]))
        add(self._gemm(M, m.head.w["weight"], logits, E_F32, xf=x_res, norm=m.final_norm))
        prog = torch.from_numpy(np.array(stages, dtype=np.int64)).to(dev)
        smem_fn = self._lib().fellm_decode_mega_smem
        smem_fn.restype, smem_fn.argtypes = ctypes.c_int, [ctypes.c_int]
        kinds = [(r[0], r[9], r[10], r[11]) if r[0] == K_GEMM else (r[0], 0, 0, 0) for r in stages]
        return {"program": prog, "n": len(stages), "smem": int(smem_fn(int(smem))), "logits": logits, "keep": keep,
                "kinds": kinds}

    def _lib(self):
        from ..csrc import jit
        return jit.load_module("decode_mega", {"HD": self.hd})

    def kernel_modules(self):
        return [("decode_mega", {"HD": self.hd})] if self.supported else []

    # ------------------------------------------------------------------ run one step
    def takes(self, ctx) -> bool:
        return (self.supported and ctx.all_single and ctx.n_rows <= MAX_ROWS and ctx.logits_all
                and getattr(ctx, "fixed_addresses", False))

    def run(self, ctx, views) -> torch.Tensor:
        """ctx must be the decode context whose arrays live at fixed device addresses.  Returns the
        step's float32 logits [rows, vocab] (a buffer the next step overwrites)."""
        G = max((b.mixer.G for b in self.model.blocks if isinstance(b.mixer, Attention)), default=1)
        split = ops.decode_split(ctx.max_len, ctx.n_rows, G, target=2 * self.n_sm)      # two virtual CTAs per SM
        key = (ctx.n_rows, split, ctx.tokens.data_ptr())
        p = self.programs.get(key)
        if p is None:
            if len(self.programs) > 32:
                self.programs.clear()
            p = self._build(ctx, views, split)
            self.programs[key] = p
        if self._fn is None:
            f = self._lib().fellm_decode_mega
            f.restype = ctypes.c_int
            f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                          ctypes.c_void_p]
            self._fn = f
        trace = None
        if self.trace_next:
            trace = torch.zeros(2 * p["n"], dtype=torch.int64, device=self.device)
            self.last_trace, self.last_kinds, self.trace_next = trace, p["kinds"], False
        code = self._fn(p["program"].data_ptr(), p["n"], self.barrier.data_ptr(), ctx.status.data_ptr(), p["smem"],
                        None if trace is None else trace.data_ptr(), torch.cuda.current_stream().cuda_stream)
        if code:
            raise KernelError(f"decode_mega: launch failed with code {code}")
        self.launches += 1
        return p["logits"]
