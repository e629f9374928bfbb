"""The decode-attention entry point for callers that cannot allocate device memory
(fellm_b200/csrc/attention_decode_static.h): called through its exported C symbol, twice in a
row, against the engine's own decode attention and against the plain attention of
tests/plain_lfm2.py.  Collected last on purpose: if it fails under `-x`, every other test has
already run."""
import ctypes

import pytest
import torch

import plain_lfm2 as P
from fellm_b200 import ops
from fellm_b200.csrc import jit

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_FLOATS = 1 << 20


def entry(hd):
    lib = jit.load_module("attention_decode_static", {"HD": hd})
    f = lib.fellm_attn_decode_static
    c_p, c_i, c_f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    f.argtypes = [c_p, c_p, c_p, c_i, c_p, c_p, c_p, c_i, c_i, c_i, c_i, c_i, c_i, c_i, c_f, c_i, c_i, c_i, c_p,
                  ctypes.c_char_p, c_i]
    f.restype = c_i
    return f


def case(seed, lens, H, G, hd, pt):
    g = torch.Generator().manual_seed(seed)
    T = len(lens)
    n_pg = [-(-n // pt) for n in lens]
    pool = torch.randn(sum(n_pg) + 1, 2, 2, G, pt, hd, generator=g).bfloat16().to(DEV)
    table = torch.full((T, max(n_pg)), -1, dtype=torch.int32)
    page = 1
    for r in range(T):
        for p in range(n_pg[r]):
            table[r, p] = page
            page += 1
        if lens[r] % pt:
            pool[page - 1, 1, :, :, lens[r] % pt:] = float("nan")       # behind the row's last key: never read
    q = torch.randn(T, H, hd, generator=g).bfloat16().to(DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    slot = torch.arange(T, dtype=torch.int32, device=DEV)
    return q, pool, table.to(DEV), pos, slot


def run_static(f, q, pool, table, pos, slot, layer, scale, split_len, max_splits, free_before=None):
    T, H, hd = q.shape
    out = torch.full((T, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    err = ctypes.create_string_buffer(256)
    if free_before is not None:
        torch.cuda.synchronize()
        free_before.append(torch.cuda.mem_get_info()[0])
    rc = f(q.data_ptr(), pool.data_ptr(), table.data_ptr(), table.shape[1], pos.data_ptr(), slot.data_ptr(),
           out.data_ptr(), T, H, pool.shape[3], hd, pool.shape[4], layer, pool.shape[1], scale, 0, split_len,
           max_splits, torch.cuda.current_stream().cuda_stream, err, 256)
    return rc, err.value.decode(), out


def plain_rows(q, pool, table, lens, layer, scale):
    """The plain attention (tests/plain_lfm2.py) over each row's own keys, gathered from its pages."""
    T, H, hd = q.shape
    pt = pool.shape[4]
    out = torch.empty(T, H * hd)
    for r, n in enumerate(lens):
        pages = table[r, :-(-n // pt)].long().cpu()
        kv = pool[pages.to(pool.device), layer].float().cpu()          # [pages, 2, G, pt, hd]
        k = kv[:, 0].permute(0, 2, 1, 3).reshape(-1, kv.shape[2], hd)[:n]
        v = kv[:, 1].permute(0, 2, 1, 3).reshape(-1, kv.shape[2], hd)[:n]
        out[r] = P.paged_attention_rows(q[r:r + 1].float().cpu(), k, v, torch.tensor([n - 1]), scale=scale).reshape(-1)
    return out


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    H, G, hd, pt = 16, 8, 64, 64
    f = entry(hd)
    for n_call, (seed, lens) in enumerate(((1, [1, 64, 65, 700, 1500, 3000]), (2, [2999, 5, 130]))):
        q, pool, table, pos, slot = case(seed, lens, H, G, hd, pt)          # the second call reuses the arrays
        split_len, max_splits = ops.decode_split(max(lens), len(lens), G)
        want = ops.attention_decode(q, pool, table, pos, slot, 1, hd ** -0.5, None, max(lens))
        free = []
        rc, msg, got = run_static(f, q, pool, table, pos, slot, 1, hd ** -0.5, split_len, max_splits, free)
        assert rc == 0, msg
        torch.cuda.synchronize()
        if n_call:      # the first call may load the kernel image; after it the device's free memory stays put
            assert abs(torch.cuda.mem_get_info()[0] - free[0]) <= (2 << 20)
        assert not torch.isnan(got.float()).any()
        assert torch.allclose(got.float(), want.float(), rtol=2e-2, atol=2e-2), (got.float() - want.float()).abs().max()
        plain = plain_rows(q, pool, table, lens, 1, hd ** -0.5)
        assert torch.allclose(got.float().cpu(), plain, rtol=2e-2, atol=2e-2), (got.float().cpu() - plain).abs().max()


def test_fewer_key_ranges_than_the_longest_row_has_still_gives_the_right_rows():
    """max_splits below ceil((largest position + 1) / split_len): the last range takes the keys
    behind it (the header's rule); every row is written and right."""
    H, G, hd, pt = 16, 8, 64, 64
    f = entry(hd)
    lens = [900, 64, 3, 450]
    q, pool, table, pos, slot = case(7, lens, H, G, hd, pt)
    plain = plain_rows(q, pool, table, lens, 1, hd ** -0.5)
    for split_len, max_splits in ((128, 3), (256, 1), (64, 15)):
        rc, msg, got = run_static(f, q, pool, table, pos, slot, 1, hd ** -0.5, split_len, max_splits)
        assert rc == 0, msg
        assert not torch.isnan(got.float()).any(), (split_len, max_splits)
        assert torch.allclose(got.float().cpu(), plain, rtol=2e-2, atol=2e-2), (split_len, max_splits)


def test_refuses_what_does_not_fit_with_a_reason():
    H, G, hd, pt = 16, 8, 64, 64
    f = entry(hd)
    q, pool, table, pos, slot = case(3, [100] * 64, H, G, hd, pt)
    too_many = SCRATCH_FLOATS // (64 * H * (hd + 2)) + 1
    rc, msg, _ = run_static(f, q, pool, table, pos, slot, 1, hd ** -0.5, 64, too_many)
    assert rc == -3 and "scratch floats" in msg and str(SCRATCH_FLOATS) in msg
    rc, msg, _ = run_static(f, q[:, :, :32].contiguous(), pool, table, pos, slot, 1, hd ** -0.5, 64, 2)
    assert rc == -1 and "head size" in msg
