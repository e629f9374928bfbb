"""Python faces of the CUDA launchers in fellm_b200/csrc: they check devices, dtypes, shapes and
the sizes a kernel takes, pass raw pointers and the current stream, and turn a launcher's return
code into a KernelError.  There is no CPU path and no library fallback behind any of them.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from .config.errors import KernelError
from .csrc import jit

_c_int, _c_ll, _c_f, _c_p = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
_fns = {}


def _fn(module: str, name: str, argtypes, defines=None):
    # (the cache key is made without the jit's own key: that one reads the environment, and this
    # function runs once per kernel launch)
    key = (module, name, tuple(defines.items()) if defines else None)
    f = _fns.get(key)
    if f is None:
        lib = jit.load_module(module, defines)
        try:
            f = getattr(lib, name)
        except AttributeError:
            raise KernelError(f"kernel library {module} has no entry point {name}") from None
        f.argtypes = list(argtypes)
        f.restype = _c_int
        _fns[key] = f
    return f


try:
    _raw_stream = torch._C._cuda_getCurrentRawStream          # the handle without building a Stream object
except AttributeError:                                         # pragma: no cover
    _raw_stream = None


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_launches = 0


def launch_count() -> int:
    """Launcher calls so far (each is one kernel launch of this package, or a refusal)."""
    return _launches


def _check(code: int, what: str):
    global _launches
    _launches += 1
    if code == 0:
        return
    if code == -1:
        raise KernelError(f"{what}: a size the kernel does not take")
    if code == -2:
        raise KernelError(f"{what}: bad arguments (null pointer or mismatched dtypes)")
    raise KernelError(f"{what}: CUDA error {code}")


def _dev(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("fellm_b200 kernels run on CUDA tensors only (there is no CPU path)")


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _is_bf16(t: torch.Tensor) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise KernelError(f"dtype {t.dtype} is not one the kernels take (bfloat16 or float32)")


def _i32(t, name):
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelError(f"{name} must be a contiguous int32 tensor")


# ------------------------------------------------------------------------------ elementwise

def embed_rows(tokens, table, out, status=None):
    """out[t, :] = float32(table[tokens[t], :]).  A token outside the table writes zeros and sets
    status to 1 (the host checks ids first; the kernel never reads out of bounds)."""
    _dev(tokens, table, out)
    _i32(tokens, "tokens")
    T, d = out.shape
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    assert table.shape[1] == d and tokens.numel() == T
    f = _fn("elementwise", "fellm_embed_rows", [_c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_p(tokens), _p(table), _is_bf16(table), _p(out), T, d, table.shape[0], _p(status), _stream()),
           "embed_rows")
    return out


def rmsnorm(x, w, eps: float, out_dtype, rows=None, out=None):
    """x float32 [T, d], w float32 [d] -> [T or len(rows), d] in out_dtype."""
    _dev(x, w, rows)
    assert x.dtype == torch.float32 and w.dtype == torch.float32 and x.is_contiguous()
    d = x.shape[-1]
    assert w.numel() == d
    n = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _i32(rows, "rows")
    if out is None:
        out = torch.empty((n, d), dtype=out_dtype, device=x.device)
    f = _fn("elementwise", "fellm_rmsnorm", [_c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int, _c_f, _c_p])
    _check(f(_p(x), _p(w), _p(out), _is_bf16(out), _p(rows), n, d, float(eps), _stream()), "rmsnorm")
    return out


def silu_mul(gu, out=None):
    """gu [T, 2F] (gate | up) -> [T, F] = silu(gate) * up."""
    _dev(gu)
    assert gu.is_contiguous() and gu.shape[1] % 2 == 0
    T, F = gu.shape[0], gu.shape[1] // 2
    if out is None:
        out = torch.empty((T, F), dtype=gu.dtype, device=gu.device)
    f = _fn("elementwise", "fellm_silu_mul", [_c_p, _c_p, _c_int, _c_int, _c_int, _c_p])
    _check(f(_p(gu), _p(out), _is_bf16(gu), T, F, _stream()), "silu_mul")
    return out


# ------------------------------------------------------------------------------ matrix products

def gemm_simt(a, w, bias=None, out=None, out_dtype=None, accumulate=False):
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias[N]) with float32 FMA on CUDA cores; with
    accumulate=True, out (float32) += that.  Any mix of bfloat16/float32 a and w."""
    _dev(a, w, bias, out)
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: a is [{M},{K}] but w is {list(w.shape)}")
    assert a.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype or a.dtype, device=a.device)
    assert out.stride(1) == 1 and out.shape == (M, N)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if _is_bf16(out) and not _is_bf16(a):
        raise KernelError("gemm_simt: float32 activations do not round down to a bfloat16 result")
    if accumulate:
        residual_written(out)
    f = _fn("gemm_simt", "fellm_gemm_simt",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_p])
    _check(f(_p(a), _is_bf16(a), _p(w), _is_bf16(w), _p(bias), _p(out), _is_bf16(out), M, N, K,
             a.stride(0), w.stride(0), out.stride(0), int(accumulate), _stream()), "gemm_simt")
    return out


# ------------------------------------------------------------------------------ short convolution

MAX_CONV_TAPS = 8


def shortconv(bcx, w, conv_bias, state, item_slot, item_start, row_item, n_items, all_single, out=None,
              blocked=False):
    """bcx [T, 3d] (B | C | X; blocked: [B16 | C16 | X16] per 16 channels, see block_bcx_rows), w
    float32 [d, Lc], state float32 [slots, Lc-1, d] (a view of one layer's slots; slot stride may
    be larger than (Lc-1)*d).  Returns y [T, d] = C * conv(B*X) and advances each item's state slot."""
    _dev(bcx, w, conv_bias, state, item_slot, item_start, row_item)
    T = bcx.shape[0]
    d, Lc = w.shape
    if not 2 <= Lc <= MAX_CONV_TAPS:
        raise KernelError(f"shortconv: conv_L_cache {Lc} is outside the kernel's range 2..{MAX_CONV_TAPS}")
    assert bcx.shape[1] == 3 * d and bcx.is_contiguous() and w.dtype == torch.float32 and w.is_contiguous()
    assert state.dtype == torch.float32 and state.shape[1:] == (Lc - 1, d)
    assert state.stride(1) == d and state.stride(2) == 1
    for t, nm in ((item_slot, "item_slot"), (item_start, "item_start"), (row_item, "row_item")):
        _i32(t, nm)
    if out is None:
        out = torch.empty((T, d), dtype=bcx.dtype, device=bcx.device)
    f = _fn("shortconv", "fellm_shortconv",
            [_c_p, _c_int, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_p])
    _check(f(_p(bcx), _is_bf16(bcx), _p(w), _p(conv_bias), _p(state), state.stride(0), _p(item_slot),
             _p(item_start), _p(row_item), _p(out), T, n_items, d, Lc, int(all_single), int(blocked), _stream()),
           "shortconv")
    return out


def block_bcx_rows(w):
    """Rows (or entries) [B | C | X] of a ShortConv input projection, d each, reordered into blocks
    of 16 channels: 16 B rows, 16 C rows, 16 X rows.  d must be a multiple of 16."""
    d = w.shape[0] // 3
    assert w.shape[0] == 3 * d and d % 16 == 0
    rest = w.shape[1:]
    return w.reshape(3, d // 16, 16, *rest).transpose(0, 1).reshape(3 * d, *rest).contiguous()


_conv_takes_cache = {}


def conv_product_takes(M: int, N: int, K: int, taps: int) -> bool:
    """Whether gemm_bf16_conv runs a product of these sizes: decode steps of up to 16 requests on the weight-streaming
    kernel (K of 1024..1280 in whole chunks), of 17..64 requests on the tcgen05 product of few rows (channels a multiple
    of 32, up to 4 taps; the kernel itself takes up to 128 rows)."""
    key = (M, N, K, taps)
    hit = _conv_takes_cache.get(key)
    if hit is None:
        if M <= 16:
            f = _fn("gemm_skinny", "fellm_gemm_skinny_conv_takes", [_c_int, _c_int, _c_int, _c_int])
            hit = bool(f(M, N, K, taps))
        else:
            f = _fn("gemm_umma", "fellm_gemm_umma_swap_conv_takes", [_c_int, _c_int, _c_int, _c_int])
            # measured on B200: a step of 32 rows at width 1024 0.629 -> 0.604 ms, of 64 rows 0.849 -> 0.842 ms, but at
            # width 2048 (64 rows) 1.298 -> 1.318 ms: tiles of 96 rows cost the wider product more than the launch saves;
            # at 96 and 128 rows the two ways lie within 2% of each other (width 1024: 1.061 / 1.065 and 1.283 / 1.271
            # ms; width 1536: 1.289 / 1.264 and 1.580 / 1.543 ms), so the kernel of its own stays there
            hit = bool(_swap_rows(M, N) and FUSE_SWAP_CONV and M <= SWAP_CONV_MAX_ROWS and K <= SWAP_CONV_MAX_K and f(M, N, K, taps))
        _conv_takes_cache[key] = hit
    return hit


def gemm_bf16_conv(x, w_blocked, bias, conv_w, conv_bias, state, row_slot, *, norm=None, out=None, row_scale=None):
    """A decode step's ShortConv input product and gated convolution in one launch: every row of x
    is one token of its own request (row_slot[i] = its state slot).  x bfloat16 [M, K], or with
    norm=(weight, eps) the float32 residual rows to be RMS-normed on the way in, or with
    row_scale=(ssq, parts, eps) the pre-weighted input of a handed-on norm; w_blocked [3d, K]
    and bias in block_bcx_rows order.  Returns y bfloat16 [M, d]; the states move on by one token."""
    _dev(x, w_blocked, bias, conv_w, conv_bias, state, row_slot)
    M, K = x.shape
    N = w_blocked.shape[0]
    d, taps = conv_w.shape
    assert N == 3 * d and w_blocked.dtype == torch.bfloat16 and w_blocked.stride(1) == 1 and x.stride(1) == 1
    assert conv_w.dtype == torch.float32 and conv_w.is_contiguous()
    assert state.dtype == torch.float32 and state.shape[1:] == (taps - 1, d) and state.stride(1) == d and state.stride(2) == 1
    _i32(row_slot, "row_slot")
    if out is None:
        out = torch.empty((M, d), dtype=torch.bfloat16, device=x.device)
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1
    if M > 16:
        # 17..64 requests: the tcgen05 product of few rows, the convolution in its owners' epilogue
        if norm is not None or x.dtype != torch.bfloat16:
            raise KernelError("gemm_bf16_conv: more than 16 rows take bfloat16 rows (normed before, or a handed-on norm's)")
        if not conv_product_takes(M, N, K, taps):
            raise KernelError(f"gemm_bf16_conv does not take a product of {M} x {N} x {K} with {taps} taps")
        if row_scale is not None:
            _announce_row_scale(row_scale, M, N, K, own_plan=True)
        f = _fn("gemm_umma", "fellm_gemm_umma_swap_conv",
                [_c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
        _check(f(_p(x), _p(w_blocked), _p(bias), _p(conv_w), _p(conv_bias), _p(state), state.stride(0), _p(row_slot), taps,
                 _p(out), M, N, K, x.stride(0), w_blocked.stride(0), out.stride(0), _p(umma_status(x.device)), _stream()),
               "gemm_umma_swap_conv")
        return out
    _announce_next("gemm_skinny", w_blocked, M)
    if row_scale is not None:
        assert norm is None
        _announce_row_scale(row_scale, M, N, K, own_plan=True)
    f = _fn("gemm_skinny", "fellm_gemm_skinny_conv",
            [_c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_p, _c_ll, _c_p, _c_int, _c_p, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_p])
    if norm is not None:
        assert x.dtype == torch.float32 and norm[0].dtype == torch.float32
        code = f(None, _p(x), _p(norm[0]), float(norm[1]), _p(w_blocked), _p(bias), _p(conv_w), _p(conv_bias), _p(state),
                 state.stride(0), _p(row_slot), taps, _p(out), M, N, K, x.stride(0), w_blocked.stride(0), out.stride(0),
                 _stream())
    else:
        assert x.dtype == torch.bfloat16
        code = f(_p(x), None, None, 0.0, _p(w_blocked), _p(bias), _p(conv_w), _p(conv_bias), _p(state),
                 state.stride(0), _p(row_slot), taps, _p(out), M, N, K, x.stride(0), w_blocked.stride(0), out.stride(0),
                 _stream())
    _check(code, "gemm_skinny_conv")
    return out


# ------------------------------------------------------------------------------ attention

PAIRINGS = {"adjacent": 0, "split_half": 1}


def qk_rope_write(qkv, q_w, k_w, eps, inv_freq, pairing, positions, row_slot, block_table, pool, layer,
                  page_tokens, H, G, hd, write_kv=True, status=None, q_out=None, rot_dim=None):
    """qkv [T, (H+2G)*hd] -> q_out [T, H, hd] (per-head RMSNorm, rotary), and k (normed, rotated)
    and v written to pool[page, layer, 0/1, g, slot, :].  q_w/k_w None: no QK norm; inv_freq None:
    no rotation; rot_dim (default hd): the first rot_dim elements of a head are rotated, with
    inv_freq [rot_dim/2].  pool: [pages, layers, 2, G, page_tokens, hd]; block_table [slots, width] is indexed
    by row_slot[t], the slot of the request row t belongs to."""
    _dev(qkv, q_w, k_w, inv_freq, positions, row_slot, block_table, pool)
    T = qkv.shape[0]
    if hd % 2:
        raise KernelError(f"attention: head_dim {hd} must be even")
    assert qkv.is_contiguous() and qkv.shape[1] == (H + 2 * G) * hd
    if write_kv:
        assert pool.is_contiguous() and pool.dtype == qkv.dtype
        assert pool.shape[2:] == (2, G, page_tokens, hd), (pool.shape, G, page_tokens, hd)
        _i32(block_table, "block_table")
    _i32(positions, "positions"), _i32(row_slot, "row_slot")
    if q_out is None:
        q_out = torch.empty((T, H, hd), dtype=qkv.dtype, device=qkv.device)
    rot_dim = hd if rot_dim is None else int(rot_dim)
    if inv_freq is not None:
        if rot_dim % 2 or not 2 <= rot_dim <= hd:
            raise KernelError(f"rotary dimension {rot_dim} must be even and within the head size {hd}")
        if inv_freq.dtype != torch.float32 or inv_freq.numel() != rot_dim // 2:
            raise KernelError(f"inv_freq must hold {rot_dim // 2} float32 values, got {inv_freq.numel()}")
    f = _fn("qk_rope_write", "fellm_qk_rope_write",
            [_c_p, _c_int, _c_p, _c_p, _c_f, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_p, _c_int, _c_int,
             _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p, _c_p])
    _check(f(_p(qkv), _is_bf16(qkv), _p(q_w), _p(k_w), float(eps), _p(inv_freq), PAIRINGS[pairing],
             _p(positions), _p(row_slot), _p(block_table) if write_kv else None,
             block_table.shape[1] if write_kv else 0, _p(pool) if write_kv else None,
             _is_bf16(pool) if write_kv else _is_bf16(qkv), layer, pool.shape[1] if write_kv else 1,
             page_tokens, _p(q_out), T, H, G, hd, rot_dim, int(write_kv), _p(status), _stream()), "qk_rope_write")
    return q_out


def paged_attention_simt(q, pool, block_table, positions, row_slot, layer, scale, window=None, out=None):
    """q [T, H, hd]; pool [pages, layers, 2, G, page_tokens, hd].  Row t attends to the cache
    positions 0..positions[t] (or the last `window` of them) of its item.  Returns [T, H*hd]."""
    _dev(q, pool, block_table, positions, row_slot)
    T, H, hd = q.shape
    G, page_tokens = pool.shape[3], pool.shape[4]
    if hd > 256:
        raise KernelError(f"attention: head_dim {hd} is above the kernel's maximum 256")
    if H % G:
        raise KernelError(f"attention: {H} heads are not a multiple of {G} kv heads")
    assert q.is_contiguous() and pool.is_contiguous() and pool.shape[5] == hd
    _i32(block_table, "block_table"), _i32(positions, "positions"), _i32(row_slot, "row_slot")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    f = _fn("attention_simt", "fellm_paged_attention_simt",
            [_c_p, _c_int, _c_p, _c_int, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_int, _c_f, _c_int, _c_p])
    _check(f(_p(q), _is_bf16(q), _p(pool), _is_bf16(pool), _p(block_table), block_table.shape[1],
             _p(positions), _p(row_slot), _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
             float(scale), int(window or 0), _stream()), "paged_attention_simt")
    return out


# ------------------------------------------------------------------------------ tensor-core products

_EPI_STORE, _EPI_ACC, _EPI_SWIGLU, _EPI_F32 = 0, 1, 2, 3
SKINNY_MAX_ROWS = 32      # measured on B200 (350M shapes): above 32 rows the tcgen05 product wins on every shape
_GEMM_ARGS = [_c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p]
_SKINNY_ARGS = [_c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p]
NORM_FUSE_MAX_ROWS = 16


def fast_gemm_modules():
    return [("gemm_skinny", None), ("gemm_tiled", None), ("gemm_umma", None)]


_umma_status = {}
USE_UMMA = os.environ.get("FELLM_B200_UMMA", "1") != "0"
USE_UMMA_SWAP = os.environ.get("FELLM_B200_UMMA_SWAP", "1") != "0"
FUSE_SWAP_CONV = os.environ.get("FELLM_B200_FUSE_SWAP_CONV", "1") != "0"     # the convolution in that product's epilogue (17..64 rows)
SWAP_CONV_MAX_K = int(os.environ.get("FELLM_B200_SWAP_CONV_MAX_K", 1536))
SWAP_CONV_MAX_ROWS = int(os.environ.get("FELLM_B200_SWAP_CONV_MAX_ROWS", 64))
SWAP_MIN_ROWS = int(os.environ.get("FELLM_B200_SWAP_MIN_ROWS", 17))     # fewer rows: the weight-streaming kernel (norm and convolution fused)
SWAP_MAX_ROWS = int(os.environ.get("FELLM_B200_SWAP_MAX_ROWS", 128))     # more rows: the persistent tcgen05 product (width 1024, 128 rows: 1.68 ms a step there, 1.28 here)
SWAP_MAX_N = 16384                                                       # wider (the vocabulary head): the persistent tcgen05 product


def umma_status(device) -> torch.Tensor:
    """Device int32 the tcgen05 product sets when one of its bounded waits ran out (101 TMA
    producer, 102 MMA issuer, 103 epilogue); zero otherwise."""
    key = torch.device(device).index or 0
    t = _umma_status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _umma_status[key] = t
    return t


def check_umma_status(device):
    """Reads the status word (synchronises)."""
    t = _umma_status.get(torch.device(device).index or 0)
    if t is not None:
        code = int(t.item())
        if code:
            t.zero_()
            if code == 302:
                raise KernelError("decode attention: a row's position has no cache page mapped")
            what = ("the TMA decode attention" if code == 301 else
                    "the tcgen05 prefill attention" if 311 <= code <= 317 else
                    "the tcgen05 product of few rows" if 111 <= code <= 113 else
                    "the tcgen05 product on CTA pairs" if 121 <= code <= 124 else
                    "the tcgen05 product with K over two CTAs" if 131 <= code <= 134 else "the tcgen05 product")
            raise KernelError(f"{what} gave up waiting on a barrier (role {code})")


def fast_gemm_takes(x, w) -> bool:
    """The tensor-core kernels read 16-byte vectors along K."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1)


def norm_fusable(x_f32, w, norm_w) -> bool:
    """Whether RMSNorm of the float32 rows x can run inside the product with w (few rows, the whole
    K range in one CTA's shared memory)."""
    M, K = x_f32.shape
    return (M <= NORM_FUSE_MAX_ROWS and w.dtype == torch.bfloat16 and x_f32.dtype == torch.float32
            and norm_w.dtype == torch.float32 and K % 8 == 0 and K <= 8192 and w.stride(0) % 8 == 0
            and x_f32.stride(1) == 1 and x_f32.stride(0) % 4 == 0 and w.stride(1) == 1
            and not _wide_on_umma(M, w.shape[0], K))


WIDE_GENERAL_N = int(os.environ.get("FELLM_B200_WIDE_GENERAL_N", 32768))


def _wide_on_umma(M: int, N: int, K: int) -> bool:
    """A very wide product (a vocabulary head) of 9..16 rows that the single-shot weight-streaming kernel does not
    take (K = 1536: six slices, no power of two of K warps) runs on the persistent tcgen05 product behind an
    RMSNorm kernel of its own: the general weight-streaming kernel with two row tiles is bound by its instructions
    there (measured on B200, [65536 x 1536]: 83 us at 16 rows, 32 us at 8, 31 us of bytes)."""
    return (USE_UMMA and 8 < M <= 16 and N >= WIDE_GENERAL_N and K % 8 == 0
            and not _single_shot(M, N, K, False) and not _single_shot(M, N, K, True))


_single_shot_cache = {}

# The matrix each bfloat16 product's successor reads, by the data pointer of the product's own matrix:
# a product's launch tells its kernel, whose CTAs ask the L2 for it before they wait for the kernel in
# front of them.  Filled by register_weight_chain(); empty: nobody prefetches.
_next_weight = {}
WEIGHT_PREFETCH = os.environ.get("FELLM_B200_WEIGHT_PREFETCH", "1") != "0"
PREFETCH_MAX_BYTES = int(os.environ.get("FELLM_B200_WEIGHT_PREFETCH_MAX_MB", 48)) << 20     # well inside the L2's 126 MB


def register_weight_chain(weights):
    """weights: the bfloat16 matrices of a decode step in the order its products read them (the last
    is followed by the first: the next step).  Replaces what was registered before for these matrices."""
    ws = [w for w in weights if w is not None and w.dtype == torch.bfloat16 and w.is_cuda and w.is_contiguous()]
    for w, nxt in zip(ws, ws[1:] + ws[:1]):
        _next_weight[w.data_ptr()] = (nxt.data_ptr(), min(nxt.numel() * 2, PREFETCH_MAX_BYTES))


PREFETCH_MAX_ROWS = 16     # measured on B200: 2% off a step of 1 or 8 rows, 1-6% ON a step of 64 (its products are short of bandwidth, not of latency)


def _announce_next(module: str, w, rows: int):
    """Tells the module's next launch which matrix comes after w."""
    if WEIGHT_PREFETCH and _next_weight and rows <= PREFETCH_MAX_ROWS:
        nxt = _next_weight.get(w.data_ptr())
        if nxt is not None:
            _fn(module, "fellm_next_weights", [_c_p, _c_ll])(nxt[0], nxt[1])


def _single_shot(M: int, N: int, K: int, norm: bool) -> bool:
    key = (M, N, K, norm)
    hit = _single_shot_cache.get(key)
    if hit is None:
        f = _fn("gemm_skinny", "fellm_gemm_skinny_single_shot", [_c_int, _c_int, _c_int, _c_int])
        hit = _single_shot_cache[key] = bool(f(M, N, K, int(norm)))
    return hit


# ---- an RMSNorm handed on from the product that writes the residual stream to the product that reads it
#
# In a decode step of up to 16 rows every product is a few microseconds long, and a product that first has
# to norm float32 rows (read them, sum the squares, scale, round) spends a third of that before its first
# MMA.  So the product that ADDS into the residual stream can do the norm's work for its successor: beside
# x += ..., it leaves xg = bfloat16(x * g) (g: the next norm's weights) and the sums of x^2 of every 16
# columns.  The successor stages xg like any bfloat16 input and multiplies its finished sums by the rows'
# factors 1 / sqrt(sum x^2 / K + eps): RMSNorm(x) W^T with the factor taken out of the product.
#
# Who writes and who reads is settled by the caller: expect_norm(x, g) says "the next product that adds
# into x is followed by an RMSNorm with weights g"; norm_handoff(x, g) gives the reader what was left, if
# it is still good (same tensor, same weights, nothing written to x since).
NORM_HANDOFF = os.environ.get("FELLM_B200_NORM_HANDOFF", "1") != "0"
HANDOFF_MAX_ROWS = 128       # up to 16 rows: the weight-streaming kernel on both sides; 17..128: the tcgen05 product of few rows
_handoff_bufs = {}          # device -> (xg bfloat16 [16 * width], ssq float32 [16 * width / 16], width)
_handoff_retired = []
_expected_norm = None       # (data_ptr of x, norm weights)
_handoff = None             # NormHandoff: what the last such product left


class NormHandoff:
    __slots__ = ("x_ptr", "version", "rows", "norm_ptr", "xg", "ssq", "parts")


def reserve_norm_handoff(device, width: int):
    """Room for handed-on norms of rows up to `width` wide (called before the first step, so that nothing
    is allocated under a captured graph).  Without it no norm is handed on."""
    device = torch.device(device)
    if device.type != "cuda" or width % 16 or width > 2048:        # the kernel takes up to 128 parts of 16 columns
        return
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    have = _handoff_bufs.get(device)
    if have is None or have[2] < width:
        if have is not None:
            _handoff_retired.append(have)      # graphs captured with the old buffers may still be replayed
        _handoff_bufs[device] = (torch.zeros(HANDOFF_MAX_ROWS * width, dtype=torch.bfloat16, device=device),
                                 torch.zeros(HANDOFF_MAX_ROWS * width // 16, dtype=torch.float32, device=device), width)
        forget_norm_handoff()


def forget_norm_handoff():
    global _expected_norm, _handoff
    _expected_norm = _handoff = None


def expect_norm(x, norm_w):
    """The next product that adds into x (float32 [rows, d]) is followed by RMSNorm with norm_w [d]."""
    global _expected_norm
    _expected_norm = None
    if (NORM_HANDOFF and x.is_cuda and x.dtype == torch.float32 and x.shape[0] <= HANDOFF_MAX_ROWS
            and norm_w.dtype == torch.float32 and norm_w.numel() == x.shape[1] and norm_w.is_contiguous()):
        bufs = _handoff_bufs.get(x.device)
        if bufs is not None and bufs[2] >= x.shape[1]:
            _expected_norm = (x.data_ptr(), norm_w)


def residual_written(out):
    """Every kernel call that adds into a float32 tensor says so: what was handed on for it is stale.
    Returns the norm expected after this write (expect_norm), if one was announced for this tensor."""
    global _handoff, _expected_norm
    if _handoff is not None and _handoff.x_ptr == out.data_ptr():
        _handoff = None
    exp, _expected_norm = _expected_norm, None          # an expectation is for the very next write
    return exp if (exp is not None and exp[0] == out.data_ptr()) else None


def norm_handoff(x, norm_w):
    """What the last product that added into x left for RMSNorm(x, norm_w), or None."""
    h = _handoff
    if (h is None or h.x_ptr != x.data_ptr() or h.version != x._version or h.rows != x.shape[0]
            or h.norm_ptr != norm_w.data_ptr()):
        return None
    return h


def _swap_rows(M: int, N: int) -> bool:
    """Whether gemm_bf16 gives a product of M rows and N columns to the tcgen05 product of few rows."""
    return USE_UMMA and USE_UMMA_SWAP and max(SWAP_MIN_ROWS, 17) <= M <= SWAP_MAX_ROWS and N <= SWAP_MAX_N


def row_scale_takes(M: int, N: int, K: int) -> bool:
    """Whether a product of these sizes can take a handed-on norm's input: up to 16 rows the single-shot
    weight-streaming kernel, 17..128 rows the tcgen05 product of few rows."""
    if K % 8:
        return False
    if M <= 16:
        return _single_shot(M, N, K, False)
    return _swap_rows(M, N)


def _announce_handoff(exp, out, M: int, N: int, K: int, norm_fused: bool):
    """Before an accumulate product of the weight-streaming kernel: if its successor's norm is known (exp)
    and the kernel can do it, tell the kernel and note what it leaves."""
    global _handoff
    if exp is None or M > HANDOFF_MAX_ROWS or not out.is_contiguous() or norm_fused:
        return
    if M <= 16:
        if N % 16 or not _single_shot(M, N, K, False):
            return
        module, per_part = "gemm_skinny", 16
    else:
        if N % 128 or not _swap_rows(M, N):
            return
        module, per_part = "gemm_umma", 128
    xg, ssq, width = _handoff_bufs[out.device]
    _handoff = None                      # the buffers are about to be rewritten
    f = _fn(module, f"fellm_{module}_next_norm", [_c_p, _c_p, _c_int, _c_p])
    f(_p(exp[1]), _p(xg), N, _p(ssq))
    h = NormHandoff()
    h.x_ptr, h.version, h.rows, h.norm_ptr = out.data_ptr(), out._version, M, exp[1].data_ptr()
    h.xg, h.ssq, h.parts = xg[:M * N].view(M, N), ssq, N // per_part
    return h


def _announce_row_scale(row_scale, M: int, N: int, K: int, own_plan: bool = False):
    ssq, parts, eps = row_scale
    if not own_plan and not row_scale_takes(M, N, K):
        raise KernelError(f"a product of {M} x {N} x {K} does not take a handed-on norm")
    assert ssq.dtype == torch.float32 and ssq.numel() >= M * parts
    module = "gemm_skinny" if M <= 16 else "gemm_umma"
    _fn(module, f"fellm_{module}_row_scale", [_c_p, _c_int, _c_f])(_p(ssq), int(parts), float(eps))


def gemm_bf16(x, w, bias=None, *, out=None, out_dtype=None, accumulate=False, swiglu=False, norm=None, row_scale=None):
    """out = x[M,K] @ w[N,K]^T (+bias) on tensor cores, bfloat16 in, float32 sums.
    accumulate: out (float32 [M,N]) += ; swiglu: w's rows are interleaved in blocks of 8 gate / 8 up
    and out is bfloat16 [M, N/2] = silu(gate)*up; out_dtype float32: float32 store.
    norm=(weight float32 [K], eps): x is the float32 residual stream and is RMS-normed on its way
    into the product (see norm_fusable).
    row_scale=(ssq, parts, eps): x is the pre-weighted input of a handed-on norm (norm_handoff)."""
    global _handoff
    _dev(x, w, bias, out)
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm: x is [{M},{K}] but w is {list(w.shape)}")
    if norm is not None:
        if not norm_fusable(x, w, norm[0]):
            raise KernelError("gemm_bf16: this product cannot take a fused RMSNorm")
    elif not fast_gemm_takes(x, w):
        raise KernelError(f"gemm_bf16: K={K} and the row strides must be multiples of 8 bfloat16 elements")
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N
    if accumulate:
        epi = _EPI_ACC
        assert out is not None and out.dtype == torch.float32 and out.shape == (M, N)
    elif swiglu:
        epi = _EPI_SWIGLU
        if N % 16:
            raise KernelError(f"gemm_bf16: the gate/up matrix needs a multiple of 16 rows, got {N}")
        if out is None:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        assert out.dtype == torch.bfloat16 and out.shape == (M, N // 2)
    elif (out_dtype or (out.dtype if out is not None else torch.bfloat16)) == torch.float32:
        epi = _EPI_F32
        if out is None:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
    else:
        epi = _EPI_STORE
        if out is None:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        assert out.dtype == torch.bfloat16
    assert out.stride(1) == 1
    if M == 0:
        return out
    umma_ok = (USE_UMMA and norm is None and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
               and (epi != _EPI_SWIGLU or out.stride(0) % 8 == 0))
    # few rows: the weight-streaming kernel; up to 64 rows: it too where its single-shot form takes the
    # product (all of W requested at once by every SM), else up to 32 rows except for very wide products
    # (measured at 64 rows: 14 us against 26 us for [1024, 4608], 8 against 9-11 for K = 1024, but 13
    # against 11 for the 9216 rows of gate/up, which stays with tcgen05 beyond 32 rows)
    expected = residual_written(out) if accumulate else None
    if umma_ok and USE_UMMA_SWAP and SWAP_MIN_ROWS <= M <= SWAP_MAX_ROWS and N <= SWAP_MAX_N and (row_scale is None or M > 16):
        # a decode step of 17..128 rows: tcgen05 with the weights as the MMA's 128 rows
        _announce_next("gemm_umma", w, M)
        if row_scale is not None:
            _announce_row_scale(row_scale, M, N, K)
        left = _announce_handoff(expected, out, M, N, K, False) if M > 16 else None
        gemm_umma_swap(x, w, bias, out=out, epi=epi, written=True)
        if left is not None:
            _handoff = left
        return out
    skinny = M <= 64 and ((M <= 16 and not (umma_ok and _wide_on_umma(M, N, K))) or not umma_ok
                          or (_single_shot(M, N, K, norm is not None) and (M <= 32 or N < 8192))
                          or (M <= SKINNY_MAX_ROWS and N < 8192))
    if row_scale is not None and (not skinny or M > 16):
        raise KernelError(f"a product of {M} x {N} x {K} does not take a handed-on norm")
    if skinny:
        _announce_next("gemm_skinny", w, M)
        if row_scale is not None:
            _announce_row_scale(row_scale, M, N, K)
        left = _announce_handoff(expected, out, M, N, K, norm is not None) if M <= 16 else None
        f = _fn("gemm_skinny", "fellm_gemm_skinny", _SKINNY_ARGS)
        if norm is not None:
            code = f(None, _p(x), _p(norm[0]), float(norm[1]), _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0),
                     w.stride(0), out.stride(0), _stream())
        else:
            code = f(_p(x), None, None, 0.0, _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0), w.stride(0),
                     out.stride(0), _stream())
        _check(code, "gemm_skinny")
        if left is not None:
            _handoff = left
    elif umma_ok:
        f = _fn("gemm_umma", "fellm_gemm_umma", _GEMM_ARGS[:-1] + [_c_p, _c_p])
        _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0), w.stride(0), out.stride(0),
                 _p(umma_status(x.device)), _stream()), "gemm_umma")
    else:
        f = _fn("gemm_tiled", "fellm_gemm_tiled", _GEMM_ARGS)
        _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, N, K, x.stride(0), w.stride(0), out.stride(0), _stream()),
               "gemm_tiled")
    return out


_argmax_scratch_cache = {}
FUSED_ARGMAX = os.environ.get("FELLM_B200_FUSED_ARGMAX", "1") != "0"


def head_argmax_scratch(M: int, N: int, K: int, norm: bool) -> int:
    """8-byte keys gemm_bf16_argmax needs for a product of these sizes; 0: it does not take it (more than
    16 rows, or sizes the single-shot product leaves to the general kernel)."""
    key = (M, N, K, norm)
    hit = _argmax_scratch_cache.get(key)
    if hit is None:
        f = _fn("gemm_skinny", "fellm_gemm_skinny_argmax_scratch", [_c_int, _c_int, _c_int, _c_int])
        f.restype = _c_ll
        hit = _argmax_scratch_cache[key] = int(f(M, N, K, int(norm)))
    return hit


def gemm_bf16_argmax(x, w, bias, keys, out_tokens, *, norm=None, row_scale=None):
    """out_tokens[m] = argmax_n (x W^T + bias)[m, n], ties to the lower n, without storing the [M, N]
    logits: the vocabulary head of a greedy decode step of up to 16 rows.  x bfloat16 [M, K], or with
    norm=(weight, eps) the float32 residual rows, or with row_scale=(ssq, parts, eps) the pre-weighted input
    of a handed-on norm; keys: int64 scratch of head_argmax_scratch() entries; out_tokens int32 [>= M]."""
    _dev(x, w, bias, keys, out_tokens)
    M, K = x.shape
    N = w.shape[0]
    need = head_argmax_scratch(M, N, K, norm is not None)
    if not need or w.dtype != torch.bfloat16 or w.stride(1) != 1 or x.stride(1) != 1:
        raise KernelError(f"gemm_bf16_argmax does not take a product of {M} x {N} x {K}")
    assert keys.dtype == torch.int64 and keys.numel() >= need and out_tokens.dtype == torch.int32 and out_tokens.numel() >= M
    _announce_next("gemm_skinny", w, M)
    if row_scale is not None:
        assert norm is None
        _announce_row_scale(row_scale, M, N, K)
    f = _fn("gemm_skinny", "fellm_gemm_skinny_argmax",
            [_c_p, _c_p, _c_p, _c_f, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_p])
    if norm is not None:
        assert x.dtype == torch.float32 and norm[0].dtype == torch.float32
        code = f(None, _p(x), _p(norm[0]), float(norm[1]), _p(w), _p(bias), _p(keys), _p(out_tokens), M, N, K,
                 x.stride(0), w.stride(0), _stream())
    else:
        assert x.dtype == torch.bfloat16
        code = f(_p(x), None, None, 0.0, _p(w), _p(bias), _p(keys), _p(out_tokens), M, N, K, x.stride(0), w.stride(0),
                 _stream())
    _check(code, "gemm_skinny_argmax")
    global _launches
    _launches += 1                      # the product and the pick of the best key
    return out_tokens


def gemm_umma_swap(x, w, bias=None, *, out, epi: int, written: bool = False):
    """The tcgen05 product for up to 128 rows (weights as the MMA's rows, K split over a cluster),
    callable by itself.  epi: 0 store bfloat16, 1 add into float32, 2 SiLU(gate)*up, 3 store float32."""
    M, K = x.shape
    if epi == _EPI_ACC and not written:
        residual_written(out)
    f = _fn("gemm_umma", "fellm_gemm_umma_swap", _GEMM_ARGS[:-1] + [_c_p, _c_p])
    _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, w.shape[0], K, x.stride(0), w.stride(0), out.stride(0),
             _p(umma_status(x.device)), _stream()), "gemm_umma_swap")
    return out


def gemm_tiled(x, w, bias=None, *, out, epi: int):
    """The mma.sync product, callable by itself (tests compare the tcgen05 product with it)."""
    M, K = x.shape
    if epi == _EPI_ACC:
        residual_written(out)
    f = _fn("gemm_tiled", "fellm_gemm_tiled", _GEMM_ARGS)
    _check(f(_p(x), _p(w), _p(bias), _p(out), epi, M, w.shape[0], K, x.stride(0), w.stride(0), out.stride(0), _stream()),
           "gemm_tiled")
    return out


def interleave_gate_up(gate, up):
    """[F,K] gate and up -> [2F,K] with rows in blocks of 16: 8 gate rows, then the 8 up rows of the
    same features (what the SiLU(gate)*up epilogues expect).  F must be a multiple of 8."""
    F, K = gate.shape
    assert F % 8 == 0 and up.shape == gate.shape
    return torch.stack([gate.reshape(F // 8, 8, K), up.reshape(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()


# ------------------------------------------------------------------------------ attention dispatch

_decode_scratch = {}
_decode_scratch_retired = []      # replaced buffers stay alive: a CUDA graph captured earlier still names them


def decode_scratch_need(max_rows: int, heads: int, kv_heads: int, head_dim: int, n_ctx: int):
    """(floats, counters) the split-KV decode kernel can ask for with up to max_rows rows and
    contexts up to n_ctx: the largest over every row count of what attention_decode reserves."""
    floats = 0
    for rows in range(1, max(max_rows, 1) + 1):
        for bucket in range(1024, max(n_ctx, 1) + 1024, 1024):       # the split is chosen per 1024 of context
            _, max_splits = decode_split(bucket, rows, kv_heads)
            floats = max(floats, rows * heads * max_splits * (head_dim + 2))
    return floats, max(max_rows, 1) * kv_heads


def reserve_decode_scratch(device, rows: int, heads: int, kv_heads: int, head_dim: int, max_splits: int, *,
                           floats: int = 0, counters: int = 0):
    """Scratch of the split-KV decode kernel: partial results of every (row, head, key range) and
    one counter per (row, kv head).  An engine sizes it once, before its first step, for the
    largest step it can run (floats=, counters= from decode_scratch_need); a later call that needs
    more (kernels called by hand at other sizes) gets a new buffer, never during a graph capture,
    and the old one is kept alive for the graphs that were captured with it."""
    need = max(rows * heads * max_splits * (head_dim + 2), floats, 1 << 21)     # at least 8 MB: growth is rare
    need_c = max(rows * kv_heads, counters, 1 << 16)
    device = torch.device(device)
    cur = _decode_scratch.get(device)
    if cur is None or cur[0].numel() < need or cur[1].numel() < need_c:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("decode attention scratch must be reserved before graph capture")
        if cur is not None:
            _decode_scratch_retired.append(cur)
        scratch = torch.empty(max(need, cur[0].numel() if cur else 0), dtype=torch.float32, device=device)
        counters_t = torch.zeros(max(need_c, cur[1].numel() if cur else 0), dtype=torch.int32, device=device)
        _decode_scratch[device] = (scratch, counters_t)
    return _decode_scratch[device]


# CTAs the split of decode attention aims at: one wave of the TMA kernel (three CTAs of 68 KB to an
# SM).  Measured on B200, 16 layers of width 1024, context 2048 (4000): batch 8 379 (411) us a step
# with 444, 387 (438) with 592, 399 (417) with 300; batch 32 764 with 444, 822 with 592.
DECODE_TARGET_CTAS = int(os.environ.get("FELLM_B200_DECODE_TARGET", 0))     # 0: three CTAs for every SM of the device
BIG_BATCH_SPLITS = int(os.environ.get("FELLM_B200_DECODE_BIG_SPLITS", 2))
DECODE_STAGES = int(os.environ.get("FELLM_B200_DECODE_STAGES", 0))           # 0: by the step's size (decode_stages)
_sm_count = {}


def sm_count(device=None) -> int:
    """SMs of the device (of a B200, 148, where no GPU is present: the planners are checked on CPU too)."""
    if not torch.cuda.is_available():
        return 148
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def decode_target_ctas() -> int:
    return DECODE_TARGET_CTAS or 3 * sm_count()


SPLIT_WHOLE_ROUNDS = os.environ.get("FELLM_B200_SPLIT_ROUNDS", "1") != "0"
DECODE_MAX_RANGES = int(os.environ.get("FELLM_B200_DECODE_MAX_RANGES", 8))        # of contexts up to 8 x 512 keys (0: no limit)
USE_TMA_DECODE = os.environ.get("FELLM_B200_TMA_DECODE", "1") != "0"
FUSE_DECODE_ROPE = os.environ.get("FELLM_B200_FUSE_ROPE", "1") != "0"
USE_TMA_PREFILL = os.environ.get("FELLM_B200_TMA_PREFILL", "1") != "0"
USE_UMMA_PREFILL = os.environ.get("FELLM_B200_UMMA_ATTN", "1") != "0"
UMMA_PREFILL_MIN_ROWS = int(os.environ.get("FELLM_B200_UMMA_ATTN_MIN_ROWS", 1))    # (token, head) rows of the longest item


def decode_stages(rows: int, kv_heads: int) -> int:
    """Half pages a warp of the TMA decode kernel keeps in flight: 4 (a CTA to an SM) for the few CTAs of a
    step of one or two requests, which then ask for most of their keys at once, else 2 (three CTAs to an SM).
    Measured on B200 (16 layers of width 1024, context 2048): batch 1 0.332 ms a step with 4 against 0.356
    with 2; batch 8 0.400 against 0.396; batch 64 1.22 against 0.92."""
    if DECODE_STAGES:
        return DECODE_STAGES
    return 4 if rows * kv_heads <= 16 else 2


def decode_split(max_len: int, rows: int, kv_heads: int, target: int = 0):
    """(split_len, max_splits): key ranges of a multiple of 64 keys, enough of them to fill the
    machine (at most 8, one cluster, while a range then stays within 512 keys).  max_len is
    rounded up to 1024 so that the choice (and a captured graph) holds while contexts grow."""
    bucket = -(-max(max_len, 1) // 1024) * 1024
    items = max(rows * kv_heads, 1)
    if not target:
        target = decode_target_ctas() // 3 if decode_stages(rows, kv_heads) == 4 else decode_target_ctas()
    want = max(1, target // items)
    if DECODE_MAX_RANGES and bucket <= DECODE_MAX_RANGES * 512:
        # up to 8 ranges are one cluster and merge through its shared memory: worth more than further ranges while a
        # range stays within two pages a warp (measured on B200, context 2,050..2,250: batch 1 0.316 -> 0.310 ms a step
        # with 8 ranges instead of 16, batch 4 0.3415 -> 0.340 with 6 instead of 12)
        want = min(want, DECODE_MAX_RANGES)
    if items > target:
        want = BIG_BATCH_SPLITS      # more than a wave even unsplit: halves, so that the last wave is a short one
    split_len = max(64, -(-(-(-bucket // want)) // 64) * 64)
    if split_len > 256 and SPLIT_WHOLE_ROUNDS:
        split_len = -(-split_len // 256) * 256      # whole rounds of the kernel's four warps, a page each
    return split_len, -(-bucket // split_len)


def _mma_checks(q, pool, what):
    T, H, hd = q.shape
    if q.dtype != torch.bfloat16 or pool.dtype != torch.bfloat16:
        raise KernelError(f"{what} takes bfloat16 queries and cache")
    if hd % 16 or not 16 <= hd <= 256:
        raise KernelError(f"{what}: head_dim {hd} must be a multiple of 16 in 16..256")
    G = pool.shape[3]
    if H % G:
        raise KernelError(f"{what}: {H} heads are not a multiple of {G} kv heads")
    assert q.is_contiguous() and pool.is_contiguous() and pool.shape[5] == hd
    return T, H, G, hd, pool.shape[4]


def decode_fuses_rope(H: int, G: int, hd: int, page_tokens: int, pool) -> bool:
    """Whether attention_decode can take the QKV product's output itself (fuse=...): the TMA kernel's sizes."""
    return (USE_TMA_DECODE and FUSE_DECODE_ROPE and hd == 64 and page_tokens == 64 and G > 0 and H % G == 0
            and H // G <= 16 and pool.numel() // hd < 2 ** 31)


def attention_decode(q, pool, block_table, positions, row_slot, layer, scale, window, max_len, out=None, fuse=None):
    """One query row per request (bfloat16): split-KV decode attention on tensor cores.
    q [T, H, hd] -> [T, H*hd].  The kernel library is compiled for this head size.
    fuse=(qkv [T, (H+2G)*hd], q_w, k_w, eps, inv_freq, pairing) with q=None (see decode_fuses_rope):
    the kernel norms and rotates q and k itself and writes k and v into the cache."""
    if fuse is not None:
        qkv = fuse[0]
        G, hd, page_tokens = pool.shape[3], pool.shape[5], pool.shape[4]
        T = qkv.shape[0]
        H = qkv.shape[1] // hd - 2 * G
        assert q is None and qkv.dtype == torch.bfloat16 and qkv.is_contiguous() and decode_fuses_rope(H, G, hd, page_tokens, pool)
        _dev(qkv, pool, block_table, positions, row_slot, fuse[1], fuse[2], fuse[4])
        assert pool.dtype == torch.bfloat16 and pool.is_contiguous()
    else:
        _dev(q, pool, block_table, positions, row_slot)
        T, H, G, hd, page_tokens = _mma_checks(q, pool, "attention_decode")
    split_len, max_splits = decode_split(max_len, T, G)
    scratch, counters = reserve_decode_scratch(pool.device, T, H, G, hd, max_splits)
    if out is None:
        out = torch.empty((T, H * hd), dtype=torch.bfloat16, device=pool.device)
    if fuse is not None or (USE_TMA_DECODE and hd == 64 and page_tokens == 64 and H // G <= 16 and pool.numel() // hd < 2 ** 31):
        # pages of 64 tokens at head size 64: whole tiles by TMA
        f = _fn("attention_mma", "fellm_attn_decode_tma",
                [_c_p, _c_p, ctypes.c_longlong, _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int,
                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_f, _c_p, _c_int,
                 _c_int, _c_p], defines={"HD": hd})
        if fuse is not None:
            qkv, q_w, k_w, eps, inv_freq, pairing = fuse
            extra = (_p(qkv), _p(q_w), _p(k_w), float(eps), _p(inv_freq), PAIRINGS[pairing])
        else:
            extra = (None, None, None, 0.0, None, 0)
        _check(f(_p(q), _p(pool), pool.shape[0], _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
                 _p(out), _p(scratch), _p(counters), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
                 int(window or 0), split_len, max_splits, _p(umma_status(pool.device)), *extra, decode_stages(T, G),
                 _stream()), "attention_decode (TMA)")
        return out
    f = _fn("attention_mma", "fellm_attn_decode_mma",
            [_c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_f, _c_int, _c_int, _c_int, _c_p], defines={"HD": hd})
    _check(f(_p(q), _p(pool), _p(block_table), block_table.shape[1], _p(positions), _p(row_slot), _p(out),
             _p(scratch), _p(counters), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
             int(window or 0), split_len, max_splits, _stream()), "attention_decode")
    return out


def attention_prefill(q, pool, block_table, positions, row_slot, item_start, n_items, max_item_rows, layer, scale,
                      window, out=None):
    """Portions of prompts (items of any length, one token included) on tensor cores (bfloat16).
    Rows of item i are item_start[i]..item_start[i+1] with consecutive positions."""
    _dev(q, pool, block_table, positions, row_slot, item_start)
    T, H, G, hd, page_tokens = _mma_checks(q, pool, "attention_prefill")
    if H // G > 64:
        raise KernelError(f"attention_prefill: {H // G} heads per kv head exceed the kernel's 64")
    _i32(item_start, "item_start")
    if out is None:
        out = torch.empty((T, H * hd), dtype=q.dtype, device=q.device)
    if (USE_UMMA_PREFILL and hd == 64 and page_tokens == 64 and not window and pool.numel() // hd < 2 ** 31
            and 128 % (H // G) == 0 and max_item_rows * (H // G) >= UMMA_PREFILL_MIN_ROWS):
        # tcgen05: 128 (token, head) rows a CTA, S and P V in tensor memory
        f = _fn("attention_umma", "fellm_attn_prefill_umma",
                [_c_p, _c_p, ctypes.c_longlong, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int,
                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p])
        _check(f(_p(q), _p(pool), pool.shape[0], _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
                 _p(item_start), n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
                 float(scale), 0, _p(umma_status(q.device)), _stream()), "attention_prefill (tcgen05)")
        return out
    if USE_TMA_PREFILL and hd == 64 and page_tokens == 64 and not window and pool.numel() // hd < 2 ** 31:
        # a key tile is a page: K and V by bulk tensor copies
        f = _fn("attention_mma", "fellm_attn_prefill_tma",
                [_c_p, _c_p, ctypes.c_longlong, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int,
                 _c_int, _c_int, _c_int, _c_int, _c_f, _c_int, _c_p, _c_p], defines={"HD": hd})
        _check(f(_p(q), _p(pool), pool.shape[0], _p(block_table), block_table.shape[1], _p(positions), _p(row_slot),
                 _p(item_start), n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1],
                 float(scale), 0, _p(umma_status(q.device)), _stream()), "attention_prefill (TMA)")
        return out
    f = _fn("attention_mma", "fellm_attn_prefill_mma",
            [_c_p, _c_p, _c_p, _c_int, _c_p, _c_p, _c_p, _c_int, _c_int, _c_p, _c_int, _c_int, _c_int, _c_int, _c_int,
             _c_int, _c_int, _c_f, _c_int, _c_p], defines={"HD": hd})
    _check(f(_p(q), _p(pool), _p(block_table), block_table.shape[1], _p(positions), _p(row_slot), _p(item_start),
             n_items, max_item_rows, _p(out), T, H, G, hd, page_tokens, layer, pool.shape[1], float(scale),
             int(window or 0), _stream()), "attention_prefill")
    return out


def attention_modules(dtype: str, head_dim: int):
    mods = [("attention_simt", None)]
    if dtype == "bfloat16":
        mods.append(("attention_mma", {"HD": head_dim}))
        if head_dim == 64 and USE_UMMA_PREFILL:
            mods.append(("attention_umma", None))
    return mods


def paged_attention(q, cache, ctx, scale, window=None):
    """Attention of the step's rows over their items' cache pages; picks the kernel: the float32
    engine runs on CUDA cores; bfloat16 on tensor cores, split over the keys when every item
    brings one token."""
    if q.dtype == torch.bfloat16:
        if ctx.all_single:
            return attention_decode(q, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                                    scale, window, ctx.max_len)
        return attention_prefill(q, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, ctx.item_start,
                                 ctx.n_items, ctx.max_item_rows, cache.layer, scale, window)
    return paged_attention_simt(q, cache.pool, cache.block_table, ctx.positions, ctx.row_slot, cache.layer,
                                scale, window)


# ------------------------------------------------------------------------------ sampling

def sample_params_size() -> int:
    f = _fn("sampling", "fellm_sample_params_size", [])
    return int(f())


def sample(logits, params_dev, counts, bias_tok, bias_val, out_tokens, out_probs=None, update_counts=True):
    """One block per row of float32 logits [B, V]; params_dev: B packed records (see
    fellm_b200/sampling/sampler.py).  counts [slots, V] int32 or None."""
    _dev(logits, params_dev, counts, bias_tok, bias_val, out_tokens, out_probs)
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and out_tokens.dtype == torch.int32
    if counts is not None:
        assert counts.dtype == torch.int32 and counts.shape[1] == V and counts.is_contiguous()
    f = _fn("sampling", "fellm_sample", [_c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p, _c_p, _c_p, _c_int, _c_p])
    _check(f(_p(logits), B, V, _p(params_dev), _p(counts), _p(bias_tok), _p(bias_val), _p(out_tokens),
             _p(out_probs), int(update_counts), _stream()), "sample")
    return out_tokens


def argmax_rows(logits, pval, pidx, out_tokens):
    """Greedy tokens of float32 logits [B, V], ties to the lower id; pval/pidx: scratch [B*64]."""
    _dev(logits, pval, pidx, out_tokens)
    B, V = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous() and pval.numel() >= B * 64 and pidx.numel() >= B * 64
    f = _fn("sampling", "fellm_argmax_rows", [_c_p, _c_int, _c_int, _c_p, _c_p, _c_p, _c_p])
    _check(f(_p(logits), B, V, _p(pval), _p(pidx), _p(out_tokens), _stream()), "argmax_rows")
    return out_tokens


def count_tokens(counts, slots, tokens):
    _dev(counts, slots, tokens)
    _i32(slots, "slots"), _i32(tokens, "tokens")
    f = _fn("sampling", "fellm_count_tokens", [_c_p, _c_int, _c_p, _c_p, _c_int, _c_p])
    _check(f(_p(counts), counts.shape[1], _p(slots), _p(tokens), tokens.numel(), _stream()), "count_tokens")
