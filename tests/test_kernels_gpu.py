"""Each kernel alone against its plain reference, at sizes other than the tiny models'."""
import math

import pytest
import torch

import plain_lfm2 as P
from fellm_b200 import ops
from fellm_b200.config import KernelError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-6) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-3)


@pytest.mark.parametrize("table_dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(table_dtype):
    table = torch.randn(1001, 200, device=DEV).to(table_dtype)
    toks = i32([0, 1000, 17, 17, 512])
    out = torch.empty(5, 200, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed_rows(toks, table, out, status)
    assert torch.equal(out, table[toks.long()].float()) and int(status) == 0
    ops.embed_rows(i32([3, 1001, -1, 4, 5]), table, out, status)       # outside the table: zeros + status
    assert int(status) == 1 and float(out[1].abs().sum()) == 0 and torch.equal(out[0], table[3].float())


@pytest.mark.parametrize("d", [48, 200, 514, 1000, 1536, 4100])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm(d, out_dtype):
    x = torch.randn(37, d, device=DEV) * 3
    w = torch.rand(d, device=DEV) + 0.5
    got = ops.rmsnorm(x, w, 1e-6, out_dtype)
    want = P.rmsnorm(x.cpu(), w.cpu(), 1e-6)
    assert torch.allclose(got.float().cpu(), want, **tol(out_dtype))
    rows = i32([36, 0, 5])
    got = ops.rmsnorm(x, w, 1e-6, out_dtype, rows=rows)
    assert torch.allclose(got.float().cpu(), want[[36, 0, 5]], **tol(out_dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_silu_mul(dtype):
    gu = (torch.randn(19, 2 * 328, device=DEV) * 2).to(dtype)
    got = ops.silu_mul(gu)
    g, u = gu.float().cpu()[:, :328], gu.float().cpu()[:, 328:]
    assert torch.allclose(got.float().cpu(), (g / (1 + torch.exp(-g))) * u, **tol(dtype))


@pytest.mark.parametrize("M,N,K", [(1, 100, 72), (7, 515, 144), (64, 64, 16), (130, 200, 333), (257, 96, 1000)])
@pytest.mark.parametrize("a_dt,w_dt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                       (torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)])
def test_gemm_simt(M, N, K, a_dt, w_dt):
    a = torch.randn(M, K, device=DEV).to(a_dt)
    w = (torch.randn(N, K, device=DEV) * 0.1).to(w_dt)
    bias = torch.randn(N, device=DEV)
    want = a.double().cpu() @ w.double().cpu().T
    got = ops.gemm_simt(a, w, out_dtype=torch.float32)
    assert torch.allclose(got.double().cpu(), want, rtol=1e-5, atol=1e-5 * math.sqrt(K))
    got = ops.gemm_simt(a, w, bias, out_dtype=torch.float32)
    assert torch.allclose(got.double().cpu(), want + bias.double().cpu(), rtol=1e-5, atol=1e-5 * math.sqrt(K))
    res = torch.randn(M, N, device=DEV)
    out = res.clone()
    ops.gemm_simt(a, w, out=out, accumulate=True)
    assert torch.allclose(out.double().cpu(), res.double().cpu() + want, rtol=1e-5, atol=1e-5 * math.sqrt(K))
    if a_dt == torch.bfloat16:
        got = ops.gemm_simt(a, w)
        assert got.dtype == torch.bfloat16 and torch.allclose(got.double().cpu(), want, rtol=1e-2, atol=1e-2)


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    a = torch.randn(70, 200, device=DEV)
    w = torch.randn(150, 200, device=DEV)
    full = ops.gemm_simt(a, w)
    one = ops.gemm_simt(a[33:34].contiguous(), w)
    assert torch.equal(full[33:34], one)


def conv_reference(bcx, w, bias, state):
    """One request: state [Lc-1, d] then the portion's rows; returns y and the new state."""
    T, d = bcx.shape[0], w.shape[0]
    lc = w.shape[1]
    B, C, X = bcx[:, :d], bcx[:, d:2 * d], bcx[:, 2 * d:]
    hist = torch.cat([state, B * X], dim=0)
    y = torch.empty(T, d)
    for t in range(T):
        conv = hist[t + lc - 1] * w[:, lc - 1]
        for j in range(lc - 1):
            conv = conv + hist[t + j] * w[:, j]
        if bias is not None:
            conv = conv + bias
        y[t] = C[t] * conv
    return y, hist[-(lc - 1):].clone()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,lc,use_bias", [(40, 2, False), (200, 3, True), (136, 5, False), (72, 8, True), (1024, 3, False),
                                           (144, 4, True)])
def test_shortconv_portions_and_state(dtype, d, lc, use_bias):
    torch.manual_seed(d + lc)
    lens = [1, lc - 1, 1, 40, 2, 9]                       # shorter than the history, equal to it, longer
    slots = [5, 0, 3, 1, 6, 2]
    T = sum(lens)
    bcx = torch.randn(T, 3 * d, device=DEV).to(dtype)
    w = torch.randn(d, lc, device=DEV)
    bias = torch.randn(d, device=DEV) if use_bias else None
    state = torch.randn(8, 2, lc - 1, d, device=DEV)      # [slots, layers, Lc-1, d]; layer 1 is ours
    before = state.clone()
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    row_item = [i for i, n in enumerate(lens) for _ in range(n)]
    y = ops.shortconv(bcx, w, bias, state[:, 1], i32(slots), i32(starts), i32(row_item), len(lens), False)
    for i, n in enumerate(lens):
        ref_y, ref_s = conv_reference(bcx[starts[i]:starts[i + 1]].float().cpu(), w.cpu(),
                                      None if bias is None else bias.cpu(), before[slots[i], 1].cpu())
        assert torch.allclose(y[starts[i]:starts[i + 1]].float().cpu(), ref_y, **tol(dtype)), (i, n)
        assert torch.allclose(state[slots[i], 1].cpu(), ref_s, rtol=1e-6, atol=1e-6), (i, n)
    assert torch.equal(state[:, 0], before[:, 0]) and torch.equal(state[7], before[7])     # nothing else touched
    if d % 16 == 0:
        # the same columns in blocks of 16 channels (16 B, 16 C, 16 X): the same outputs and states, to the bit
        st3 = before.clone()
        bcx_blocked = ops.block_bcx_rows(bcx.t().contiguous()).t().contiguous()
        y3 = ops.shortconv(bcx_blocked, w, bias, st3[:, 1], i32(slots), i32(starts), i32(row_item), len(lens), False,
                           blocked=True)
        assert torch.equal(y3, y) and torch.equal(st3, state)
    # portions one token at a time give bit-equal outputs and state (float32)
    if dtype == torch.float32:
        st2 = before.clone()
        y2 = torch.empty_like(y)
        for i, n in enumerate(lens):
            for t in range(n):
                r = starts[i] + t
                y2[r:r + 1] = ops.shortconv(bcx[r:r + 1].contiguous(), w, bias, st2[:, 1], i32([slots[i]]),
                                            i32([0, 1]), i32([0]), 1, True)
        assert torch.equal(y2, y) and torch.equal(st2, state)


@pytest.mark.parametrize("M,d,K,lc,use_bias,use_norm", [(8, 1024, 1024, 3, False, True), (1, 1024, 1024, 3, True, True),
                                                         (13, 2048, 1280, 4, True, False), (16, 48, 1152, 8, False, True),
                                                         (5, 1024, 1024, 2, False, False)])
def test_decode_conv_product_equals_product_then_convolution(M, d, K, lc, use_bias, use_norm):
    """A decode step's ShortConv input product with the convolution in its epilogue: the same y and
    the same states, to the bit, as the product and the convolution kernel one after the other."""
    torch.manual_seed(M + d)
    assert ops.conv_product_takes(M, 3 * d, K, lc) and not ops.conv_product_takes(129, 3 * d, K, lc)
    assert not ops.conv_product_takes(M, 3 * d, 2048, lc)            # (17..128 rows are another kernel's: the next test)
    w_in = ops.block_bcx_rows((torch.randn(3 * d, K, device=DEV) * 0.05).bfloat16())
    b_in = ops.block_bcx_rows(torch.randn(3 * d, device=DEV)) if use_bias else None
    conv_w = torch.randn(d, lc, device=DEV)
    conv_b = torch.randn(d, device=DEV) if use_bias else None
    state = torch.randn(20, 2, lc - 1, d, device=DEV)
    slots = torch.randperm(20)[:M].tolist()
    nw = torch.rand(K, device=DEV) + 0.5
    x = torch.randn(M, K, device=DEV) * 2
    if not use_norm:
        x = x.bfloat16()
    norm = (nw, 1e-5) if use_norm else None
    st_a, st_b = state.clone(), state.clone()
    for step in range(3):                                   # the state is carried from launch to launch
        y = ops.gemm_bf16_conv(x, w_in, b_in, conv_w, conv_b, st_a[:, 1], i32(slots), norm=norm)
        bcx = ops.gemm_bf16(x, w_in, b_in, norm=norm)
        ref = ops.shortconv(bcx, conv_w, conv_b, st_b[:, 1], i32(slots), i32(list(range(M + 1))), i32(list(range(M))),
                            M, True, blocked=True)
        assert torch.equal(y, ref), (step, (y.float() - ref.float()).abs().max())
        assert torch.equal(st_a, st_b), step
        x = x * 0.9 + 0.1
    untouched = [s for s in range(20) if s not in slots]
    assert torch.equal(st_a[untouched], state[untouched]) and torch.equal(st_a[:, 0], state[:, 0])


def test_shortconv_refuses_too_many_taps():
    with pytest.raises(KernelError, match="outside the kernel's range"):
        ops.shortconv(torch.zeros(1, 48, device=DEV), torch.zeros(16, 9, device=DEV), None,
                      torch.zeros(1, 8, 16, device=DEV), i32([0]), i32([0, 1]), i32([0]), 1, True)


def build_cache(keys, values, page_tokens, pages_order, dtype, n_layers=2, layer=1):
    """keys/values [C, G, hd] of one request -> pool and block table with the given physical pages."""
    C, G, hd = keys.shape
    n_pages = max(pages_order) + 2
    pool = torch.randn(n_pages, n_layers, 2, G, page_tokens, hd, device=DEV).to(dtype)     # garbage elsewhere
    table = torch.full((3, len(pages_order) + 2), -1, dtype=torch.int32, device=DEV)
    for p in range(C):
        page = pages_order[p // page_tokens]
        pool[page, layer, 0, :, p % page_tokens] = keys[p].to(dtype)
        pool[page, layer, 1, :, p % page_tokens] = values[p].to(dtype)
    table[1, :len(pages_order)] = i32(pages_order)
    return pool, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,page_tokens,window", [(6, 3, 16, 8, None), (8, 1, 80, 16, None), (4, 4, 128, 64, None),
                                                       (5, 5, 48, 16, 37), (16, 2, 256, 32, 100)])
def test_paged_attention_simt(dtype, H, G, hd, page_tokens, window):
    torch.manual_seed(H * hd)
    C = 300
    keys, values = torch.randn(C, G, hd), torch.randn(C, G, hd)
    n_pg = -(-C // page_tokens)
    order = list(reversed(range(3, 3 + n_pg)))            # pages far from logical order
    pool, table = build_cache(keys, values, page_tokens, order, dtype)
    q_pos = [0, 1, page_tokens - 1, page_tokens, 2 * page_tokens - 1, 150, 298, 299]
    q = torch.randn(len(q_pos), H, hd)
    got = ops.paged_attention_simt(q.to(DEV).to(dtype), pool, table, i32(q_pos), i32([1] * len(q_pos)), 1,
                                   hd ** -0.5, window)
    kc, vc = keys.to(dtype).float(), values.to(dtype).float()
    want = P.paged_attention_rows(q.to(dtype).float(), kc, vc, torch.tensor(q_pos), scale=hd ** -0.5, window=window)
    assert torch.allclose(got.float().cpu().reshape(-1, H, hd), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("far", [0, 63, 64, 255, 256, 511])
def test_attention_finds_one_far_key(dtype, far):
    """Among 600 keys one is made to stand out (a page's last slot, the next page's first, the very
    first key): the output must be that key's value."""
    H, G, hd, pt, C = 4, 2, 64, 64, 600
    keys, values = torch.randn(C, G, hd) * 0.1, torch.randn(C, G, hd)
    q = torch.randn(1, H, hd) * 0.1
    direction = torch.randn(hd)
    direction = direction / direction.norm()
    keys[far] = direction * 30.0
    q[0] = direction * 30.0
    pool, table = build_cache(keys, values, pt, list(range(1, 1 + -(-C // pt))), dtype)
    got = ops.paged_attention_simt(q.to(DEV).to(dtype), pool, table, i32([C - 1]), i32([1]), 1, hd ** -0.5)
    got = got.float().cpu().reshape(H, hd)
    for h in range(H):
        assert torch.allclose(got[h], values[far, h // 2].to(dtype).float(), atol=2e-2), (far, h)


@pytest.mark.parametrize("window", [16, 17, 64])
def test_attention_window_edge(window):
    """The key just outside the window must not count, the one just inside must."""
    H, G, hd, pt, C = 2, 1, 32, 16, 200
    keys, values = torch.randn(C, G, hd) * 0.1, torch.randn(C, G, hd)
    d = torch.randn(hd); d = d / d.norm()
    q = (d * 30.0).repeat(1, H, 1)
    pos = C - 1
    for edge, inside in ((pos - window, False), (pos - window + 1, True)):
        k2 = keys.clone(); k2[edge] = d * 30.0
        pool, table = build_cache(k2, values, pt, list(range(1, 1 + -(-C // pt))), torch.float32)
        got = ops.paged_attention_simt(q.to(DEV), pool, table, i32([pos]), i32([1]), 1, hd ** -0.5, window)
        hit = torch.allclose(got.cpu().reshape(H, hd)[0], values[edge, 0], atol=1e-3)
        assert hit == inside, (window, edge, inside)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,pairing,qk_norm,rope", [(4, 2, 16, "adjacent", True, True), (6, 1, 48, "split_half", True, True),
                                                         (3, 3, 80, "adjacent", False, True), (8, 2, 128, "split_half", True, False),
                                                         (2, 2, 256, "split_half", True, True)])
def test_qk_rope_write(dtype, H, G, hd, pairing, qk_norm, rope):
    torch.manual_seed(hd)
    T, pt, eps, theta = 11, 8, 1e-6, 10000.0
    qkv = torch.randn(T, (H + 2 * G) * hd).to(dtype)
    positions = [0, 1, 7, 8, 9, 100, 3000, 15, 16, 23, 24]
    slots = [0, 0, 0, 0, 0, 1, 1, 2, 2, 2, 2]
    qw, kw = torch.rand(hd) + 0.5, torch.rand(hd) + 0.5
    inv = P.rope_inv_freq(theta, hd)
    table = torch.full((3, 400), -1, dtype=torch.int32)
    nxt = 1
    for p, s in zip(positions, slots):
        if table[s, p // pt] < 0:
            table[s, p // pt] = nxt; nxt += 1
    pool = torch.zeros(nxt + 1, 3, 2, G, pt, hd, device=DEV, dtype=dtype)
    q = ops.qk_rope_write(qkv.to(DEV), qw.to(DEV) if qk_norm else None, kw.to(DEV) if qk_norm else None, eps,
                          inv.to(DEV) if rope else None, pairing, i32(positions), i32(slots), table.to(DEV), pool, 2,
                          pt, H, G, hd)
    x = qkv.float()
    qr, kr, vr = x[:, :H * hd].reshape(T, H, hd), x[:, H * hd:(H + G) * hd].reshape(T, G, hd), x[:, (H + G) * hd:].reshape(T, G, hd)
    if qk_norm:
        qr, kr = P.rmsnorm(qr, qw, eps), P.rmsnorm(kr, kw, eps)
    if rope:
        pos_t = torch.tensor(positions)
        qr, kr = P.rope_apply(qr, pos_t, inv, pairing), P.rope_apply(kr, pos_t, inv, pairing)
    t = tol(dtype)
    assert torch.allclose(q.float().cpu(), qr, **t)
    for r, (p, s) in enumerate(zip(positions, slots)):
        page = int(table[s, p // pt])
        assert torch.allclose(pool[page, 2, 0, :, p % pt].float().cpu(), kr[r], **t), r
        assert torch.allclose(pool[page, 2, 1, :, p % pt].float().cpu(), vr[r], **t), r
    assert float(pool[:, :2].abs().sum()) == 0 and float(pool[0].abs().sum()) == 0      # other layers, other pages


def test_qk_rope_write_flags_a_missing_page():
    H, G, hd = 2, 1, 16
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    pool = torch.zeros(2, 1, 2, G, 8, hd, device=DEV)
    table = torch.full((1, 4), -1, dtype=torch.int32, device=DEV)
    ops.qk_rope_write(torch.randn(1, 4 * hd, device=DEV), None, None, 1e-6, None, "adjacent", i32([3]), i32([0]),
                      table, pool, 0, 8, H, G, hd, status=status)
    assert int(status) == 2 and float(pool.abs().sum()) == 0


# ------------------------------------------------------------------ tensor-core kernels (bfloat16)

def _gemm_case(M, N, K, seed=0):
    g = torch.Generator().manual_seed(seed + M * 7 + N * 3 + K)
    x = (torch.randn(M, K, generator=g)).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    return x, w, x.double() @ w.double().T


# M <= 16 runs the weight-streaming kernel, 17..32 it or the tcgen05 product by width, larger M the tcgen05 product
# (the decode-sized ones up to 16 rows take its single-shot form: a slab per warp, 8..10 chunks of K per warp)
# (wide products of a larger model: several slabs a warp, K = 8192 over a cluster of two; many rows and a wide N:
# the tcgen05 product in 128 x 256 tiles, also with a ragged last tile)
# (K slices over clusters of 3, 5 and 7 ranks: widths of 1536, 7168, 3072 and 6400 = 20 x 320 = 4 warps x 5 ranks)
GEMM_SHAPES = [(1, 3072, 1024), (8, 1024, 4608), (13, 1024, 1024), (16, 2048, 2048), (9, 1536, 4608), (8, 6144, 2048),
               (8, 4608, 1536), (16, 1536, 7168), (3, 1536, 1536), (12, 9216, 3072), (5, 1024, 6400),
               (16, 2048, 8192), (40, 6144, 2048), (3, 515, 144), (2048, 2048, 1024), (2048, 2000, 136), (17, 96, 72), (33, 200, 328), (64, 1024, 1024),
               (64, 2048, 200), (5, 65536, 64), (65, 144, 144), (128, 515, 320), (300, 1000, 1000), (2048, 256, 136)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_bf16_store_acc_f32(M, N, K):
    x, w, want = _gemm_case(M, N, K)
    xd, wd = x.to(DEV), w.to(DEV)
    bias = torch.randn(N, device=DEV)
    tol_abs = 4e-3 * math.sqrt(K) * 0.05 * 4                  # bfloat16 products are exact; float32 sums
    got = ops.gemm_bf16(xd, wd, out_dtype=torch.float32)
    assert got.dtype == torch.float32 and torch.allclose(got.double().cpu(), want, rtol=1e-4, atol=1e-4)
    got = ops.gemm_bf16(xd, wd, bias, out_dtype=torch.float32)
    assert torch.allclose(got.double().cpu(), want + bias.double().cpu(), rtol=1e-4, atol=1e-4)
    got = ops.gemm_bf16(xd, wd)
    assert got.dtype == torch.bfloat16 and torch.allclose(got.double().cpu(), want, rtol=1e-2, atol=tol_abs)
    res = torch.randn(M, N, device=DEV)
    out = res.clone()
    ops.gemm_bf16(xd, wd, out=out, accumulate=True)
    assert torch.allclose(out.double().cpu(), res.double().cpu() + want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("M,F,K", [(1, 4608, 1024), (8, 4608, 1024), (11, 2048, 2048), (8, 8192, 2048), (8, 7168, 1536), (14, 1024, 3072),
                                   (200, 512, 1024), (520, 1024, 1536), (130, 96, 600), (2048, 4608, 1024), (1900, 1000, 200), (64, 4608, 1024), (50, 1024, 2048), (8, 320, 144), (40, 64, 72), (64, 200, 136), (100, 328, 200), (513, 192, 64)])
def test_gemm_bf16_swiglu_epilogue(M, F, K):
    g = torch.Generator().manual_seed(F)
    x = torch.randn(M, K, generator=g).bfloat16()
    wg, wu = (torch.randn(F, K, generator=g) * 0.1).bfloat16(), (torch.randn(F, K, generator=g) * 0.1).bfloat16()
    gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
    want = (gate / (1 + torch.exp(-gate))) * up
    w = ops.interleave_gate_up(wg.to(DEV), wu.to(DEV))
    assert w.shape == (2 * F, K) and torch.equal(w[0], wg[0].to(DEV)) and torch.equal(w[8], wu[0].to(DEV))
    got = ops.gemm_bf16(x.to(DEV), w, swiglu=True)
    assert got.shape == (M, F) and got.dtype == torch.bfloat16
    assert torch.allclose(got.double().cpu(), want, rtol=1.2e-2, atol=2e-3)


def test_gemm_bf16_refuses_unaligned_k():
    x = torch.randn(4, 100, device=DEV).bfloat16()
    w = torch.randn(32, 100, device=DEV).bfloat16()
    assert not ops.fast_gemm_takes(x, w)
    with pytest.raises(KernelError, match="multiples of 8"):
        ops.gemm_bf16(x, w)


def test_gemm_skinny_same_bits_every_run():
    x, w, _ = _gemm_case(8, 1024, 4608)
    a = ops.gemm_bf16(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    b = ops.gemm_bf16(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert torch.equal(a, b)                                # the cluster reduces in rank order


@pytest.mark.parametrize("H,G,hd,page_tokens,window", [(16, 8, 64, 64, None), (6, 1, 48, 16, None), (4, 4, 128, 32, None),
                                                       (24, 8, 64, 64, None), (8, 1, 16, 16, 70), (5, 5, 80, 8, None),
                                                       (2, 1, 256, 64, 300), (32, 8, 64, 16, None), (6, 1, 32, 64, None),
                                                       (16, 1, 64, 64, 100), (34, 2, 64, 64, None), (8, 4, 64, 64, 700)])
def test_attention_decode_split_kv(H, G, hd, page_tokens, window):
    """Rows of different lengths, each its own request, pages out of order, key ranges that end
    inside pages (what lies behind the last key in its page is NaN): against the plain attention.
    Head size 64 with pages of 64 tokens and up to 16 heads per kv head takes the TMA kernel."""
    torch.manual_seed(H + hd)
    lens = [1, 2, 63, 64, 65, 200, 777, 1500]
    T = len(lens)
    n_pg = [-(-n // page_tokens) for n in lens]
    total = sum(n_pg)
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(1)).tolist()
    pool = torch.randn(total + 1, 2, 2, G, page_tokens, hd, device=DEV).bfloat16()
    table = torch.full((T + 2, max(n_pg) + 1), -1, dtype=torch.int32)
    keys, values, at = [], [], 0
    for r, n in enumerate(lens):
        k, v = torch.randn(n, G, hd).bfloat16(), torch.randn(n, G, hd).bfloat16()
        keys.append(k); values.append(v)
        for p in range(n_pg[r]):
            page = perm[at] + 1; at += 1
            table[r + 1, p] = page
            lo, hi = p * page_tokens, min(n, (p + 1) * page_tokens)
            pool[page, 1, 0, :, :hi - lo] = k[lo:hi].transpose(0, 1).to(DEV)
            pool[page, 1, 1, :, :hi - lo] = v[lo:hi].transpose(0, 1).to(DEV)
            pool[page, 1, :, :, hi - lo:] = float("nan")
    q = torch.randn(T, H, hd).bfloat16()
    got = ops.attention_decode(q.to(DEV), pool, table.to(DEV), i32([n - 1 for n in lens]), i32(list(range(1, T + 1))),
                               1, hd ** -0.5, window, max(lens))
    got = got.float().cpu().reshape(T, H, hd)
    for r, n in enumerate(lens):
        want = P.paged_attention_rows(q[r:r + 1].float(), keys[r].float(), values[r].float(), torch.tensor([n - 1]),
                                      scale=hd ** -0.5, window=window)
        assert torch.allclose(got[r], want[0], rtol=2e-2, atol=2e-2), (r, n, (got[r] - want[0]).abs().max())
    # the same rows in one launch and alone give the same bits when the key ranges are the same
    again = ops.attention_decode(q.to(DEV), pool, table.to(DEV), i32([n - 1 for n in lens]), i32(list(range(1, T + 1))),
                                 1, hd ** -0.5, window, max(lens))
    assert torch.equal(again.float().cpu().reshape(T, H, hd), got)


@pytest.mark.parametrize("H,G,pairing,qk_norm,rope,window", [(16, 8, "split_half", True, True, None), (6, 2, "adjacent", True, True, None),
                                                              (16, 1, "adjacent", False, True, 90), (4, 4, "split_half", True, False, None)])
def test_attention_decode_takes_the_qkv_product_itself(H, G, pairing, qk_norm, rope, window):
    """Head size 64, pages of 64 tokens: the decode kernel norms and rotates q and k and writes k and v
    into the cache itself; against qk_rope_write followed by the same kernel, outputs and cache."""
    hd, pt = 64, 64
    torch.manual_seed(H * 7 + G)
    lens = [1, 2, 33, 64, 65, 129, 700, 1500]                # the step's own position: first of a page, of a half, inside
    T = len(lens)
    n_pg = [-(-n // pt) for n in lens]
    perm = torch.randperm(sum(n_pg), generator=torch.Generator().manual_seed(2)).tolist()
    pool = torch.randn(sum(n_pg) + 1, 2, 2, G, pt, hd, device=DEV).bfloat16()
    table = torch.full((T + 2, max(n_pg) + 1), -1, dtype=torch.int32)
    at = 0
    for r, n in enumerate(lens):
        for p in range(n_pg[r]):
            table[r + 1, p] = perm[at] + 1; at += 1
        last = int(table[r + 1, (n - 1) // pt])
        pool[last, 1, :, :, (n - 1) % pt:] = float("nan")     # the step's own row and what lies behind it
    qkv = torch.randn(T, (H + 2 * G) * hd, device=DEV).bfloat16()
    qw, kw = (torch.rand(hd, device=DEV) + 0.5, torch.rand(hd, device=DEV) + 0.5) if qk_norm else (None, None)
    inv = P.rope_inv_freq(10000.0, hd).to(DEV) if rope else None
    pos, slots, tab = i32([n - 1 for n in lens]), i32(list(range(1, T + 1))), table.to(DEV)
    assert ops.decode_fuses_rope(H, G, hd, pt, pool)
    pool_a, pool_b = pool.clone(), pool.clone()
    got = ops.attention_decode(None, pool_a, tab, pos, slots, 1, hd ** -0.5, window, max(lens),
                               fuse=(qkv, qw, kw, 1e-6, inv, pairing))
    ops.check_umma_status(DEV)
    q = ops.qk_rope_write(qkv, qw, kw, 1e-6, inv, pairing, pos, slots, tab, pool_b, 1, pt, H, G, hd)
    want = ops.attention_decode(q, pool_b, tab, pos, slots, 1, hd ** -0.5, window, max(lens))
    assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), (got.float() - want.float()).abs().max()
    for r, n in enumerate(lens):
        page, row = int(table[r + 1, (n - 1) // pt]), (n - 1) % pt
        a, b = pool_a[page, 1, :, :, row].float(), pool_b[page, 1, :, :, row].float()
        assert torch.equal(a[1], b[1]), r                                        # v: copied
        assert torch.allclose(a[0], b[0], rtol=1e-2, atol=1e-2), (r, (a[0] - b[0]).abs().max())      # k: one bfloat16 rounding apart at most
    keep = torch.ones_like(pool_a, dtype=torch.bool)
    for r, n in enumerate(lens):
        keep[int(table[r + 1, (n - 1) // pt]), 1, :, :, (n - 1) % pt] = False
    assert torch.equal(torch.nan_to_num(pool_a[keep]), torch.nan_to_num(pool[keep]))       # nothing else written


@pytest.mark.parametrize("far", [0, 63, 64, 1023, 1024, 2999])
def test_attention_decode_finds_one_far_key(far):
    H, G, hd, pt, C = 16, 8, 64, 64, 3000
    keys, values = torch.randn(C, G, hd) * 0.1, torch.randn(C, G, hd)
    d = torch.randn(hd); d = d / d.norm()
    keys[far] = d * 30.0
    q = (d * 30.0).repeat(1, H, 1)
    pool, table = build_cache(keys, values, pt, list(range(1, 1 + -(-C // pt))), torch.bfloat16)
    got = ops.attention_decode(q.to(DEV).bfloat16(), pool, table, i32([C - 1]), i32([1]), 1, hd ** -0.5, None, C)
    got = got.float().cpu().reshape(H, hd)
    for h in range(H):
        assert torch.allclose(got[h], values[far, h // 2].bfloat16().float(), atol=2e-2), (far, h)


@pytest.mark.parametrize("M,N,K", [(1, 3072, 1024), (8, 640, 144), (16, 200, 328), (3, 65536, 64), (8, 9216, 1024), (12, 3072, 1024),
                                   (16, 4096, 2048), (5, 512, 1280), (7, 256, 4096), (8, 6144, 2048)])
def test_gemm_bf16_fused_rmsnorm_prologue(M, N, K):
    g = torch.Generator().manual_seed(N)
    x = torch.randn(M, K, generator=g) * 2
    nw = torch.rand(K, generator=g) + 0.5
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    xn = P.rmsnorm(x, nw, 1e-5).bfloat16()                       # the normed rows are rounded to bfloat16
    want = xn.double() @ w.double().T
    assert ops.norm_fusable(x.to(DEV), w.to(DEV), nw.to(DEV))
    got = ops.gemm_bf16(x.to(DEV), w.to(DEV), out_dtype=torch.float32, norm=(nw.to(DEV), 1e-5))
    # a normed value that sits on a bfloat16 rounding boundary may round the other way: allow one such flip
    assert torch.allclose(got.double().cpu(), want, rtol=2e-3, atol=2e-2 * 0.05 * math.sqrt(K) / 8)
    unfused = ops.gemm_bf16(ops.rmsnorm(x.to(DEV), nw.to(DEV), 1e-5, torch.bfloat16), w.to(DEV), out_dtype=torch.float32)
    assert torch.allclose(got, unfused, rtol=2e-3, atol=2e-2 * 0.05 * math.sqrt(K) / 8)
    assert not ops.norm_fusable(torch.zeros(17, K, device=DEV), w.to(DEV), nw.to(DEV))


@pytest.mark.parametrize("H,G,hd,page_tokens,window", [(16, 8, 64, 64, None), (6, 1, 48, 16, None), (4, 4, 128, 32, None),
                                                       (24, 8, 64, 16, None), (8, 1, 16, 16, 70), (5, 5, 80, 8, None),
                                                       (2, 1, 256, 64, 300), (20, 1, 32, 16, None), (4, 4, 64, 64, None),
                                                       (32, 1, 64, 64, None), (16, 8, 64, 64, 120), (12, 4, 64, 64, None),
                                                       (16, 1, 64, 64, None)])
@pytest.mark.parametrize("tcgen05", [True, False])
def test_attention_prefill_mma(H, G, hd, page_tokens, window, tcgen05, monkeypatch):
    """Items of mixed lengths in one launch (a portion that starts mid-sequence, a whole prompt, a
    single decoded token, two tokens), pages out of order, NaN behind each item's last key in its
    page, against the plain attention.  Head size 64 with pages of 64 tokens and no window takes
    the tcgen05 kernel where the heads of a kv head divide its 128 rows, else (or with it switched
    off) the TMA kernel on mma.sync."""
    takes = hd == 64 and page_tokens == 64 and not window
    if not tcgen05 and not takes:
        pytest.skip("the same kernel either way")
    monkeypatch.setattr(ops, "USE_UMMA_PREFILL", tcgen05)
    torch.manual_seed(H * 3 + hd)
    ctx_before = [150, 0, 700, 33, 0]           # cached positions before this step's rows
    new = [97, 130, 1, 2, 64]                   # rows each item brings
    n = len(new)
    total = [a + b for a, b in zip(ctx_before, new)]
    n_pg = [-(-t // page_tokens) for t in total]
    perm = torch.randperm(sum(n_pg), generator=torch.Generator().manual_seed(2)).tolist()
    pool = torch.randn(sum(n_pg) + 1, 2, 2, G, page_tokens, hd, device=DEV).bfloat16()
    table = torch.full((n + 1, max(n_pg) + 1), -1, dtype=torch.int32)
    keys, values, at = [], [], 0
    for r in range(n):
        k, v = torch.randn(total[r], G, hd).bfloat16(), torch.randn(total[r], G, hd).bfloat16()
        keys.append(k); values.append(v)
        for p in range(n_pg[r]):
            page = perm[at] + 1; at += 1
            table[r + 1, p] = page
            lo, hi = p * page_tokens, min(total[r], (p + 1) * page_tokens)
            pool[page, 1, 0, :, :hi - lo] = k[lo:hi].transpose(0, 1).to(DEV)
            pool[page, 1, 1, :, :hi - lo] = v[lo:hi].transpose(0, 1).to(DEV)
            pool[page, 1, :, :, hi - lo:] = float("nan")
    T = sum(new)
    q = torch.randn(T, H, hd).bfloat16()
    starts = [0]
    for x in new:
        starts.append(starts[-1] + x)
    positions = [ctx_before[r] + j for r in range(n) for j in range(new[r])]
    row_slot = [r + 1 for r in range(n) for _ in range(new[r])]
    got = ops.attention_prefill(q.to(DEV), pool, table.to(DEV), i32(positions), i32(row_slot), i32(starts), n,
                                max(new), 1, hd ** -0.5, window)
    got = got.float().cpu().reshape(T, H, hd)
    for r in range(n):
        rows = slice(starts[r], starts[r + 1])
        want = P.paged_attention_rows(q[rows].float(), keys[r].float(), values[r].float(),
                                      torch.tensor(positions[rows]), scale=hd ** -0.5, window=window)
        assert torch.allclose(got[rows], want, rtol=2e-2, atol=2e-2), (r, (got[rows] - want).abs().max())
    # and the float32-arithmetic kernel agrees on the same cache
    simt = ops.paged_attention_simt(q.to(DEV), pool, table.to(DEV), i32(positions), i32(row_slot), 1, hd ** -0.5, window)
    assert torch.allclose(simt.float().cpu().reshape(T, H, hd), got, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("far,qpos", [(0, 999), (63, 999), (64, 999), (935, 999), (936, 1000), (999, 999)])
@pytest.mark.parametrize("tcgen05", [True, False])
def test_attention_prefill_finds_one_far_key(far, qpos, tcgen05, monkeypatch):
    """One key stands out among a thousand; the query block straddles it or lies far behind it."""
    monkeypatch.setattr(ops, "USE_UMMA_PREFILL", tcgen05)
    H, G, hd, pt, C = 4, 2, 64, 64, 1001
    keys, values = torch.randn(C, G, hd) * 0.1, torch.randn(C, G, hd)
    d = torch.randn(hd); d = d / d.norm()
    keys[far] = d * 30.0
    n_new = 70
    q = torch.randn(n_new, H, hd) * 0.1
    row = qpos - (C - n_new)
    q[row] = d * 30.0
    pool, table = build_cache(keys, values, pt, list(range(1, 1 + -(-C // pt))), torch.bfloat16)
    positions = list(range(C - n_new, C))
    got = ops.attention_prefill(q.to(DEV).bfloat16(), pool, table, i32(positions), i32([1] * n_new), i32([0, n_new]), 1,
                                n_new, 1, hd ** -0.5, None)
    got = got.float().cpu().reshape(n_new, H, hd)
    for h in range(H):
        assert torch.allclose(got[row, h], values[far, h // 2].bfloat16().float(), atol=2e-2), (far, h)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 256), (65, 144, 144), (300, 1000, 1000), (2048, 1024, 4608),
                                   (513, 3072, 1024), (1000, 200, 72), (64, 1024, 4608), (64, 1024, 1024), (48, 3072, 1024),
                                   (128, 2048, 1000), (33, 1000, 4608),
                                   (520, 1536, 7168), (130, 200, 4096), (600, 1024, 1024), (65, 9000, 512), (200, 1000, 520)])
def test_gemm_umma_tcgen05(M, N, K):
    """The tcgen05 / TMEM / TMA product by itself: against float64, against the mma.sync product,
    and its bounded waits must not have run out.  (Products of up to 64 rows that the weight-streaming
    kernel takes in one shot run there instead: the same checks hold.)"""
    x, w, want = _gemm_case(M, N, K, seed=5)
    xd, wd = x.to(DEV), w.to(DEV)
    got = ops.gemm_bf16(xd, wd, out_dtype=torch.float32)
    ops.check_umma_status(DEV)
    assert torch.allclose(got.double().cpu(), want, rtol=1e-4, atol=1e-4), (got.double().cpu() - want).abs().max()
    ref = torch.empty(M, N, device=DEV)
    ops.gemm_tiled(xd, wd, out=ref, epi=3)
    assert torch.allclose(got, ref, rtol=1e-4, atol=1e-4)            # the same products, summed in another order
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV)
    out = res.clone()
    ops.gemm_bf16(xd, wd, bias, out=out, accumulate=True)
    assert torch.allclose(out.double().cpu(), res.double().cpu() + want + bias.double().cpu(), rtol=1e-4, atol=1e-4)
    ops.check_umma_status(DEV)
    assert torch.equal(ops.gemm_bf16(xd, wd, out_dtype=torch.float32), got)       # the same bits every run


@pytest.mark.parametrize("M", [9, 12, 16])
def test_a_vocabulary_head_of_9_to_16_rows_off_the_single_shot_kernel(M):
    """A very wide product whose K the single-shot weight-streaming kernel does not take (1536 = six slices), at 9..16
    rows: the persistent tcgen05 product behind an RMSNorm kernel, not the general weight-streaming kernel with the
    norm inside.  Through linear(), as the head calls it; against the plain norm and a float64 product."""
    from fellm_b200.parts.linear import LazyNorm, linear
    from fellm_b200.parts.rmsnorm import RMSNorm
    N, K, eps = 65536, 1536, 1e-5
    assert ops._wide_on_umma(M, N, K) and not ops._wide_on_umma(8, N, K) and not ops._wide_on_umma(M, N, 1024)
    g = torch.Generator().manual_seed(M)
    x = (torch.randn(M, K, generator=g) * 2).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    norm = RMSNorm(dtype="bfloat16", size=K, eps=eps)
    norm.w = {"weight": (torch.rand(K, generator=g) + 0.5).to(DEV)}
    assert not ops.norm_fusable(x, w, norm.w["weight"]) and ops.norm_fusable(x[:8], w, norm.w["weight"])
    got = linear(LazyNorm(x, norm, torch.bfloat16), w, out_dtype=torch.float32)
    ops.check_umma_status(DEV)
    xb = ops.rmsnorm(x, norm.w["weight"], eps, torch.bfloat16)
    assert torch.allclose(xb.float().cpu(), P.rmsnorm(x.cpu(), norm.w["weight"].cpu(), eps), rtol=2 ** -7, atol=1e-6)
    want = xb.double().cpu() @ w.double().cpu().T               # the rounded rows: what the product read
    assert torch.allclose(got.double().cpu(), want, rtol=1e-4, atol=1e-4)
    few = linear(LazyNorm(x[:8], norm, torch.bfloat16), w, out_dtype=torch.float32)        # 8 rows: the norm inside
    assert torch.allclose(few, got[:8], rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("M,N,K", [(33, 200, 328), (48, 1024, 1024), (64, 2048, 200), (64, 515, 144)])
def test_gemm_skinny_up_to_64_rows(M, N, K, monkeypatch):
    """The weight-streaming kernel takes up to 64 rows (it is the fallback where the tcgen05 product cannot run)."""
    monkeypatch.setattr(ops, "USE_UMMA", False)
    x, w, want = _gemm_case(M, N, K, seed=9)
    got = ops.gemm_bf16(x.to(DEV), w.to(DEV), out_dtype=torch.float32)
    assert torch.allclose(got.double().cpu(), want, rtol=1e-4, atol=1e-4)


def build_cache_pages(keys, values, page_tokens, dtype, first_live_page=0, n_layers=2, layer=1):
    """Like build_cache, without a loop over positions: pages in reverse physical order, NaN in the
    pages before `first_live_page`, which the block table marks as given back (-1)."""
    C, G, hd = keys.shape
    n_pg = -(-C // page_tokens)
    pad = n_pg * page_tokens - C
    kp = torch.cat([keys, torch.full((pad, G, hd), float("nan"))]).reshape(n_pg, page_tokens, G, hd).transpose(1, 2)
    vp = torch.cat([values, torch.full((pad, G, hd), float("nan"))]).reshape(n_pg, page_tokens, G, hd).transpose(1, 2)
    pool = torch.randn(n_pg + 2, n_layers, 2, G, page_tokens, hd).to(dtype)
    phys = [n_pg - p for p in range(n_pg)]                       # logical page p lives in page n_pg - p
    pool[phys, layer, 0] = kp.to(dtype)
    pool[phys, layer, 1] = vp.to(dtype)
    table = torch.full((3, n_pg + 2), -1, dtype=torch.int32)
    table[1, :n_pg] = torch.tensor(phys, dtype=torch.int32)
    if first_live_page:
        pool[phys[:first_live_page], layer] = float("nan")
        table[1, :first_live_page] = -1
    return pool.to(DEV), table.to(DEV)


@pytest.mark.parametrize("hd,pt", [(64, 64), (32, 16)])
@pytest.mark.parametrize("window", [16, 17, 64, 100])
def test_attention_decode_window_edge(hd, pt, window):
    """The tensor-core decode kernels (TMA at head size 64 / pages of 64, cp.async otherwise): the key
    just outside the window must not count, the one just inside must.  The window's first key lies
    inside a page, on a page's first slot, in the request's first page, or in a later key range of
    the split; the pages wholly behind the window are given back (-1 in the block table, NaN in the
    pool) as the cache manager does."""
    H, G, C = 4, 2, 1500
    torch.manual_seed(window + hd)
    keys, values = torch.randn(C, G, hd) * 0.1, torch.randn(C, G, hd)
    d = torch.randn(hd); d = d / d.norm()
    q = (d * 30.0).repeat(1, H, 1).to(DEV).bfloat16()
    boundary = 10 * pt + window - 1                          # window starts on a page's first slot
    for pos in (window - 1, window, window + 3, boundary, boundary + 1, boundary - 1, 1400, C - 1):
        for edge, inside in ((pos - window, False), (pos - window + 1, True)):
            if edge < 0:
                continue
            k2 = keys.clone(); k2[edge] = d * 30.0
            for trimmed in (False, True):
                dead = max(0, pos - window + 1) // pt if trimmed else 0      # what the manager gave back before this query
                pool, table = build_cache_pages(k2[:pos + 1], values[:pos + 1], pt, torch.bfloat16, first_live_page=dead)
                got = ops.attention_decode(q, pool, table, i32([pos]), i32([1]), 1, hd ** -0.5, window, C)
                got = got.float().cpu().reshape(H, hd)
                assert not torch.isnan(got).any(), (pos, edge, trimmed)
                hit = torch.allclose(got[0], values[edge, 0].bfloat16().float(), atol=3e-2)
                assert hit == inside, (window, pos, edge, inside, trimmed)
    ops.check_umma_status(DEV)


@pytest.mark.parametrize("hd,pt", [(64, 64), (32, 16), (48, 8)])
@pytest.mark.parametrize("window", [16, 17, 64, 100])
def test_attention_prefill_window_edge(hd, pt, window):
    """The same for a prompt portion on tensor cores: rows of one portion whose windows start in
    different pages (the first row's in an earlier page than the last row's)."""
    H, G, C, n_new = 4, 2, 700, 70
    torch.manual_seed(window + hd + 1)
    keys, values = torch.randn(C, G, hd) * 0.1, torch.randn(C, G, hd)
    d = torch.randn(hd); d = d / d.norm()
    positions = list(range(C - n_new, C))
    for row in (0, 1, 37, n_new - 1):
        pos = positions[row]
        for edge, inside in ((pos - window, False), (pos - window + 1, True)):
            k2 = keys.clone(); k2[edge] = d * 30.0
            q = torch.randn(n_new, H, hd) * 0.1
            q[row] = d * 30.0
            dead = max(0, positions[0] - window + 1) // pt              # behind the FIRST row's window
            pool, table = build_cache_pages(k2, values, pt, torch.bfloat16, first_live_page=dead)
            got = ops.attention_prefill(q.to(DEV).bfloat16(), pool, table, i32(positions), i32([1] * n_new), i32([0, n_new]),
                                        1, n_new, 1, hd ** -0.5, window)
            got = got.float().cpu().reshape(n_new, H, hd)
            assert not torch.isnan(got).any(), (row, edge)
            hit = torch.allclose(got[row, 0], values[edge, 0].bfloat16().float(), atol=3e-2)
            assert hit == inside, (window, row, edge, inside)


@pytest.mark.parametrize("M", [1, 16, 17, 33, 40, 48, 63, 64, 65, 96, 100, 128])
@pytest.mark.parametrize("N,K", [(1024, 1024), (1024, 4608), (3072, 1024), (9216, 1024), (2048, 2048), (200, 136), (515, 328),
                                 (128, 64), (6144, 2048), (1536, 7168)])
def test_gemm_umma_swap_few_rows(M, N, K):
    """The tcgen05 product of a decode step of up to 128 rows (weights as the MMA's 128 rows, tokens as
    its columns, K over a cluster): every epilogue against float64, the same bits on every run, and
    its bounded waits must not have run out.  Sizes with ragged tiles in N and in K included."""
    x, w, want = _gemm_case(M, N, K, seed=11)
    xd, wd = x.to(DEV), w.to(DEV)
    got = torch.full((M, N), float("nan"), device=DEV)
    ops.gemm_umma_swap(xd, wd, out=got, epi=3)
    ops.check_umma_status(DEV)
    assert torch.allclose(got.double().cpu(), want, rtol=1e-4, atol=1e-4), (got.double().cpu() - want).abs().max()
    again = torch.empty_like(got)
    ops.gemm_umma_swap(xd, wd, out=again, epi=3)
    assert torch.equal(again, got)                                    # ranks are summed in rank order
    bias = torch.randn(N, device=DEV)
    res = torch.randn(M, N, device=DEV)
    out = res.clone()
    ops.gemm_umma_swap(xd, wd, bias, out=out, epi=1)
    assert torch.allclose(out.double().cpu(), res.double().cpu() + want + bias.double().cpu(), rtol=1e-4, atol=1e-4)
    outb = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    ops.gemm_umma_swap(xd, wd, out=outb, epi=0)
    assert torch.allclose(outb.double().cpu(), want, rtol=1e-2, atol=4e-3 * math.sqrt(K) * 0.2)
    if N % 16 == 0:
        F = N // 2
        g = torch.Generator().manual_seed(F)
        wg, wu = (torch.randn(F, K, generator=g) * 0.1).bfloat16(), (torch.randn(F, K, generator=g) * 0.1).bfloat16()
        gate, up = x.double() @ wg.double().T, x.double() @ wu.double().T
        z = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_umma_swap(xd, ops.interleave_gate_up(wg.to(DEV), wu.to(DEV)), out=z, epi=2)
        assert torch.allclose(z.double().cpu(), (gate / (1 + torch.exp(-gate))) * up, rtol=1.2e-2, atol=2e-3)
    ops.check_umma_status(DEV)


@pytest.mark.parametrize("M,N,K,use_norm", [(1, 65536, 1024, True), (8, 65536, 1024, True), (16, 65536, 1024, False), (5, 4096, 1024, True),
                                            (8, 65536, 2048, True), (3, 8192, 1536, False)])
def test_head_argmax_without_logits(M, N, K, use_norm):
    """The vocabulary head of a greedy decode step: the single-shot product leaves every CTA's best
    (value, index) of each row, a second kernel picks the row's best; against argmax of the logits the
    same product stores, with ties (equal largest logits far apart) going to the lower id."""
    g = torch.Generator().manual_seed(N + M)
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    w[N - 7] = w[11]                                               # two equal rows: whichever is largest ties with its twin
    x = torch.randn(M, K, generator=g) * 2
    x[0] = w[11].float() * 50.0                                    # row 0 points at the twins: the lower id must win
    nw = torch.rand(K, generator=g) + 0.5 if use_norm else None
    need = ops.head_argmax_scratch(M, N, K, use_norm)
    assert ops.head_argmax_scratch(17, N, K, use_norm) == 0
    if need == 0:                                                  # sizes the single-shot product leaves to the general kernel
        with pytest.raises(KernelError, match="does not take"):
            ops.gemm_bf16_argmax(x.bfloat16().to(DEV), w.to(DEV), None, torch.zeros(8, dtype=torch.int64, device=DEV),
                                 torch.zeros(M, dtype=torch.int32, device=DEV))
        assert K != 1024                                           # the 350M head is taken
        return
    keys = torch.zeros(need, dtype=torch.int64, device=DEV)
    toks = torch.full((M + 2,), -5, dtype=torch.int32, device=DEV)
    if use_norm:
        if M == 1 and K == 1024:
            x[0] = x[0] / nw                                       # the norm's weight must not turn row 0 away from the twins
        logits = ops.gemm_bf16(x.to(DEV), w.to(DEV), out_dtype=torch.float32, norm=(nw.to(DEV), 1e-5))
        ops.gemm_bf16_argmax(x.to(DEV), w.to(DEV), None, keys, toks, norm=(nw.to(DEV), 1e-5))
    else:
        logits = ops.gemm_bf16(x.bfloat16().to(DEV), w.to(DEV), out_dtype=torch.float32)
        ops.gemm_bf16_argmax(x.bfloat16().to(DEV), w.to(DEV), None, keys, toks)
    want = torch.argmax(logits, dim=1).int()                       # the first maximum
    assert torch.equal(toks[:M], want), (toks[:M], want)
    assert int(toks[M]) == -5                                      # nothing written past the rows
    if not use_norm or (M == 1 and K == 1024):
        assert int(want[0]) == 11 and float(logits[0, 11]) == float(logits[0, N - 7])


@pytest.mark.parametrize("M,N,K,d_next", [(8, 1024, 1024, 3072), (1, 1024, 4608, 9216), (16, 2048, 2048, 6144), (5, 1024, 1024, 65536),
                                           (13, 512, 1280, 512), (8, 2048, 8192, 2048), (8, 1536, 1536, 4608), (16, 1536, 7168, 14336),
                                           (17, 1024, 4608, 9216), (40, 1024, 1024, 3072), (64, 2048, 2048, 6144), (33, 1536, 1536, 4608),
                                           (24, 128, 64, 200), (65, 1024, 1024, 3072), (128, 1024, 4608, 9216), (100, 2048, 2048, 6144)])
def test_rmsnorm_handed_on_from_the_adding_product(M, N, K, d_next):
    """The product that adds into the residual rows leaves them weighted for the next RMSNorm, with the sums of
    squares in parts; the next product scales its sums by the rows' factors.  Against the plain norm and product."""
    g = torch.Generator().manual_seed(M * N + K)
    res = (torch.randn(M, N, generator=g) * 3).to(DEV)
    res[M // 2, 7] = 90.0                                          # one value that dominates its row's sum of squares
    y = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    w_out = (torch.randn(N, K, generator=g) * 0.05).bfloat16().to(DEV)
    nw = (torch.rand(N, generator=g) + 0.5).to(DEV)
    ops.forget_norm_handoff()
    ops.reserve_norm_handoff(DEV, 2048)
    plain_sum = res.clone()
    ops.gemm_bf16(y, w_out, out=plain_sum, accumulate=True)        # nothing announced: nothing handed on
    assert ops.norm_handoff(plain_sum, nw) is None
    ops.expect_norm(res, nw)
    ops.gemm_bf16(y, w_out, out=res, accumulate=True)
    assert torch.equal(res, plain_sum)
    h = ops.norm_handoff(res, nw)
    # up to 16 rows the weight-streaming kernel does it (a part = 16 columns), beyond that the tcgen05 product (128)
    assert h is not None and h.rows == M and h.parts == N // (16 if M <= 16 else 128)      # (17..128 rows)
    assert ops.norm_handoff(res, nw.clone()) is None and ops.norm_handoff(res.clone(), nw) is None
    assert torch.equal(h.xg, (res * nw).bfloat16())
    ssq = h.ssq[:M * h.parts].view(M, h.parts)
    assert torch.allclose(ssq, (res * res).view(M, h.parts, N // h.parts).sum(-1), rtol=1e-5)
    # the consumers: every epilogue, against RMSNorm then product in float64
    eps = 1e-5
    xn = P.rmsnorm(res.cpu(), nw.cpu(), eps)
    n2 = d_next
    w = (torch.randn(n2, N, generator=g) * 0.05).bfloat16()
    bias = torch.randn(n2, generator=g)
    want = xn.double() @ w.double().T + bias.double()
    scale = (h.ssq, h.parts, eps)
    # Two references.  (1) Float64 sums of the very bfloat16 operands a kernel read: only the float32 accumulation
    # (2^-24 a term, far fewer in practice) and the row factor's float32 lie between.  (2) The unrounded norm: the
    # rounding of a normed value to bfloat16 is at most 2^-8 of it and, over a row, adds like independent errors
    # of standard deviation <= 2^-8 / sqrt(3); seven of those for every element, on top of (1).
    wd = w.double()
    r = 1.0 / torch.sqrt((res.double().cpu() ** 2).mean(-1, keepdim=True) + eps)
    xg = h.xg.double().cpu()
    exact_handed = (xg @ wd.T) * r + bias.double()
    acc = 2e-6 * ((xg.abs() @ wd.abs().T) * r + bias.abs().double()) + 1e-6
    rounding = 7 * 2.0 ** -8 / math.sqrt(3) * torch.sqrt((xn.double() ** 2) @ (wd ** 2).T) + acc
    assert ops.row_scale_takes(M, n2, N)
    got = ops.gemm_bf16(h.xg, w.to(DEV), bias.to(DEV), out_dtype=torch.float32, row_scale=scale)
    assert bool(((got.double().cpu() - exact_handed).abs() <= acc).all())
    assert bool(((got.double().cpu() - want).abs() <= rounding).all())
    # the norm inside the product (up to 16 rows) or in front of it rounds x*r*g, the handed-on rows are x*g rounded
    if M <= 16:
        fused = ops.gemm_bf16(res, w.to(DEV), bias.to(DEV), out_dtype=torch.float32, norm=(nw, eps))
    else:
        xb = ops.rmsnorm(res, nw, eps, torch.bfloat16)
        fused = ops.gemm_bf16(xb, w.to(DEV), bias.to(DEV), out_dtype=torch.float32)
        exact_normed = xb.double().cpu() @ wd.T + bias.double()
        assert bool(((fused.double().cpu() - exact_normed).abs() <= acc).all())
    assert bool(((fused.double().cpu() - want).abs() <= rounding).all())
    got_b = ops.gemm_bf16(h.xg, w.to(DEV), bias.to(DEV), row_scale=scale)
    assert torch.equal(got_b, got.bfloat16())
    if n2 <= 16384 and n2 % 16 == 0:
        wi = ops.interleave_gate_up(w[:n2 // 2].to(DEV), w[n2 // 2:].to(DEV))
        got_s = ops.gemm_bf16(h.xg, wi, swiglu=True, row_scale=scale)
        gu = exact_handed - bias.double()
        gate, up = gu[:, :n2 // 2], gu[:, n2 // 2:]
        ref_s = torch.nn.functional.silu(gate) * up
        # gate and up are each within `acc` of these sums; SiLU's slope is at most 1.1; the product is rounded to
        # bfloat16
        ag, au = acc[:, :n2 // 2], acc[:, n2 // 2:]
        bound = (ag * 1.1 * up.abs() + au * torch.nn.functional.silu(gate).abs() + ag * au
                 + ref_s.abs() * 2.0 ** -8 + 1e-6)
        assert bool(((got_s.double().cpu() - ref_s).abs() <= bound).all())
    if M <= 16:
        need = ops.head_argmax_scratch(M, n2, N, False)
        assert need
        keys = torch.zeros(need, dtype=torch.int64, device=DEV)
        toks = torch.full((M,), -1, dtype=torch.int32, device=DEV)
        ops.gemm_bf16_argmax(h.xg, w.to(DEV), bias.to(DEV), keys, toks, row_scale=scale)
        assert torch.equal(toks.long(), got.argmax(-1))
    # a write into the rows ends what was handed on; so does a torch-side update
    assert ops.norm_handoff(res, nw) is not None
    res += 1
    assert ops.norm_handoff(res, nw) is None
    ops.expect_norm(res, nw)
    ops.gemm_bf16(y, w_out, out=res, accumulate=True)
    assert ops.norm_handoff(res, nw) is not None
    ops.gemm_bf16(y, w_out, out=res, accumulate=True)              # a second product, nothing announced for it
    assert ops.norm_handoff(res, nw) is None
    ops.forget_norm_handoff()


@pytest.mark.parametrize("M", [1, 8, 9, 15, 16])
def test_handed_on_norm_into_the_convolution_product(M):
    """(At 9 to 16 rows and width 1024 the kernel's dynamic shared memory is exactly 48 KB: with its static part
    it needs the opt-in.)"""
    d, lc = 1024, 3
    g = torch.Generator().manual_seed(5)
    res = (torch.randn(M, d, generator=g) * 2).to(DEV)
    y = torch.randn(M, d, generator=g).bfloat16().to(DEV)
    w_out = (torch.randn(d, d, generator=g) * 0.05).bfloat16().to(DEV)
    nw = (torch.rand(d, generator=g) + 0.5).to(DEV)
    w_in = ops.block_bcx_rows((torch.randn(3 * d, d, generator=g) * 0.05).bfloat16().to(DEV))
    conv_w = torch.randn(d, lc, generator=g).to(DEV)
    state = torch.randn(12, 1, lc - 1, d, generator=g).to(DEV)
    state = torch.randn(20, 1, lc - 1, d, generator=g).to(DEV)
    slots = i32(torch.randperm(20, generator=g)[:M].tolist())
    ops.forget_norm_handoff()
    ops.reserve_norm_handoff(DEV, 2048)
    ops.expect_norm(res, nw)
    ops.gemm_bf16(y, w_out, out=res, accumulate=True)
    h = ops.norm_handoff(res, nw)
    st_a, st_b = state.clone(), state.clone()
    got = ops.gemm_bf16_conv(h.xg, w_in, None, conv_w, None, st_a[:, 0], slots, row_scale=(h.ssq, h.parts, 1e-5))
    bcx = ops.gemm_bf16(h.xg, w_in, row_scale=(h.ssq, h.parts, 1e-5))
    ref = ops.shortconv(bcx, conv_w, None, st_b[:, 0], slots, i32(list(range(M + 1))), i32(list(range(M))), M, True, blocked=True)
    assert torch.equal(got, ref) and torch.equal(st_a, st_b)
    fused = ops.gemm_bf16(res, w_in, norm=(nw, 1e-5))
    assert torch.allclose(bcx.float(), fused.float(), rtol=2e-2, atol=2e-2)
    ops.forget_norm_handoff()


@pytest.mark.parametrize("M,d,K,lc,use_bias,handed_on", [(17, 1024, 1024, 3, False, True), (64, 1024, 1024, 3, False, True), (40, 2048, 2048, 4, True, False),
                                                          (33, 1536, 1536, 2, True, True), (24, 96, 72, 3, False, False), (50, 1024, 4608, 3, False, False),
                                                          (128, 1024, 1024, 3, False, True), (97, 1024, 1024, 3, True, False)])
def test_decode_conv_product_of_17_to_128_rows_equals_product_then_convolution(M, d, K, lc, use_bias, handed_on, monkeypatch):
    """A decode step's ShortConv input product of 17..128 requests with the convolution in the epilogue of the tcgen05
    product of few rows (tiles of 96 weight rows = two blocks of 16 channels): the same y and the same states, to the
    bit, as that product and the convolution kernel one after the other; also behind a handed-on norm."""
    g = torch.Generator().manual_seed(M + d + lc)
    monkeypatch.setattr(ops, "SWAP_CONV_MAX_K", 8192)        # (the engine takes it up to K = 1536 and 64 rows; the
    monkeypatch.setattr(ops, "SWAP_CONV_MAX_ROWS", 128)      # kernel any K and up to 128 rows)
    monkeypatch.setattr(ops, "_conv_takes_cache", {})
    assert ops.conv_product_takes(M, 3 * d, K, lc)
    assert not ops.conv_product_takes(129, 3 * d, K, lc) and not ops.conv_product_takes(M, 3 * d, K, 5)
    w_in = ops.block_bcx_rows((torch.randn(3 * d, K, generator=g) * 0.05).bfloat16().to(DEV))
    b_in = ops.block_bcx_rows(torch.randn(3 * d, generator=g).to(DEV)) if use_bias else None
    conv_w = torch.randn(d, lc, generator=g).to(DEV)
    conv_b = torch.randn(d, generator=g).to(DEV) if use_bias else None
    state = torch.randn(140, 2, lc - 1, d, generator=g).to(DEV)
    slots = torch.randperm(140, generator=g)[:M].tolist()
    scale = None
    if handed_on:
        assert K == d
        res = (torch.randn(M, K, generator=g) * 2).to(DEV)
        y0 = torch.randn(M, K, generator=g).bfloat16().to(DEV)
        w0 = (torch.randn(K, K, generator=g) * 0.05).bfloat16().to(DEV)
        nw = (torch.rand(K, generator=g) + 0.5).to(DEV)
        ops.forget_norm_handoff()
        ops.reserve_norm_handoff(DEV, 2048)
        ops.expect_norm(res, nw)
        ops.gemm_bf16(y0, w0, out=res, accumulate=True)
        h = ops.norm_handoff(res, nw)
        assert h is not None
        x, scale = h.xg, (h.ssq, h.parts, 1e-5)
    else:
        x = torch.randn(M, K, generator=g).bfloat16().to(DEV)
    st_a, st_b = state.clone(), state.clone()
    for step in range(3):                                   # the state is carried from launch to launch
        y = ops.gemm_bf16_conv(x, w_in, b_in, conv_w, conv_b, st_a[:, 1], i32(slots), row_scale=scale)
        bcx = ops.gemm_bf16(x, w_in, b_in, row_scale=scale)
        ref = ops.shortconv(bcx, conv_w, conv_b, st_b[:, 1], i32(slots), i32(list(range(M + 1))), i32(list(range(M))),
                            M, True, blocked=True)
        assert torch.equal(y, ref), (step, (y.float() - ref.float()).abs().max())
        assert torch.equal(st_a, st_b), step
        if not handed_on:
            x = (x.float() * 0.9 + 0.1).bfloat16()
    untouched = [s for s in range(140) if s not in slots]
    assert torch.equal(st_a[untouched], state[untouched]) and torch.equal(st_a[:, 0], state[:, 0])
    ops.forget_norm_handoff()
