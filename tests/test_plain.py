"""The plain implementation itself: FeLLM's own test vectors and the properties its kernel tests
check (crates/backend-cpu/src/kernels/{shortconv,norm,rope,swiglu,softmax}.rs test modules)."""
import math

import torch

import plain_lfm2 as P
import tiny


def test_shortconv_identity_vector_from_fellm():
    # crates/backend-cpu/src/kernels/shortconv.rs:113-154: identity projections, d=4, Lc=3,
    # x=[1,2,3,4], state rows [10,20,30,40],[5,6,7,8], conv taps chosen so that y=[1,8,27,64] and the
    # new state is [5,6,7,8],[1,4,9,16].  With B=C=X=x: bx = x*x, y = x * (bx*w2 + s0*w0 + s1*w1).
    d, lc = 4, 3
    x = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    w_in = torch.cat([torch.eye(d)] * 3, dim=0)
    w_out = torch.eye(d)
    w_conv = torch.zeros(d, lc)
    w_conv[:, lc - 1] = 1.0                       # only the current tap: conv = bx
    y = P.shortconv_mixer(x, w_in, w_conv, w_out)
    assert torch.allclose(y, torch.tensor([[1.0, 8.0, 27.0, 64.0]]))
    # the rolling state is the sequence's own history: feeding [s0/., s1/., x] as a 3-token
    # sequence whose bx values are the state rows reproduces the one-token recurrence
    state = torch.tensor([[10.0, 20.0, 30.0, 40.0], [5.0, 6.0, 7.0, 8.0]])
    w_conv2 = torch.tensor([[0.5, 0.25, 1.0]] * d)
    bx = x[0] * x[0]
    expect = x[0] * (bx * 1.0 + state[0] * 0.5 + state[1] * 0.25)
    seq = torch.cat([state.sqrt(), x], dim=0)     # bx_t = seq_t^2 with identity projections
    y3 = P.shortconv_mixer(seq, w_in, w_conv2, w_out)
    assert torch.allclose(y3[2], expect, rtol=1e-5)


def test_rmsnorm_unit_rms_and_weight():
    x = torch.randn(5, 48)
    y = P.rmsnorm(x, torch.ones(48), 1e-6)
    assert torch.allclose((y * y).mean(-1), torch.ones(5), atol=1e-3)      # norm.rs:55-81
    w = torch.rand(48) + 0.5
    assert torch.allclose(P.rmsnorm(x, w, 1e-6), y * w, atol=1e-6)


def test_rope_position_zero_is_identity_and_norm_kept():
    inv = P.rope_inv_freq(10000.0, 32)
    assert inv.dtype == torch.float32 and inv[0] == 1.0
    assert math.isclose(float(inv[1]), 10000.0 ** (-2 / 32), rel_tol=1e-6)
    x = torch.randn(3, 2, 32)
    for pairing in ("adjacent", "split_half"):
        assert torch.equal(P.rope_apply(x, torch.zeros(3, dtype=torch.long), inv, pairing), x)   # rope.rs:64-77
        y = P.rope_apply(x, torch.tensor([1, 7, 300]), inv, pairing)
        assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)
    # the two pairings rotate different element pairs
    a = P.rope_apply(x, torch.tensor([1, 7, 300]), inv, "adjacent")
    b = P.rope_apply(x, torch.tensor([1, 7, 300]), inv, "split_half")
    assert not torch.allclose(a, b)


def test_rope_relative():
    # q.k after rotation depends on the distance only
    inv = P.rope_inv_freq(1e4, 16)
    q, k = torch.randn(1, 1, 16), torch.randn(1, 1, 16)
    def dot(pq, pk):
        return float((P.rope_apply(q, torch.tensor([pq]), inv, "split_half")
                      * P.rope_apply(k, torch.tensor([pk]), inv, "split_half")).sum())
    assert math.isclose(dot(5, 2), dot(105, 102), rel_tol=1e-4, abs_tol=1e-5)


def test_swiglu_zero_and_formula():
    d, f = 8, 12
    wg, wu, wd = torch.randn(f, d), torch.randn(f, d), torch.randn(d, f)
    assert torch.equal(P.swiglu(torch.zeros(2, d), wg, wu, wd), torch.zeros(2, d))    # silu(0) = 0
    h = torch.randn(2, d)
    want = (torch.nn.functional.silu(h @ wg.T) * (h @ wu.T)) @ wd.T
    assert torch.allclose(P.swiglu(h, wg, wu, wd), want, atol=1e-5)


def test_ff_dim_rule():
    assert P.ff_dim(dict(block_ff_dim=6656, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256)) == 4608
    assert P.ff_dim(dict(block_ff_dim=10752, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256)) == 7168
    assert P.ff_dim(dict(block_ff_dim=12288, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=256)) == 8192
    assert P.ff_dim(dict(block_ff_dim=480, block_auto_adjust_ff_dim=True, block_ffn_dim_multiplier=1.0, block_multiple_of=64)) == 320
    assert P.ff_dim(dict(block_ff_dim=192)) == 192


def test_attention_matches_naive_softmax_and_window():
    # attention_correctness.rs:90-171 compares an online softmax with a naive one; here the plain
    # paged yardstick against the plain mixer's inner loop
    T, H, G, hd = 9, 4, 2, 8
    q, k, v = torch.randn(T, H, hd), torch.randn(T, G, hd), torch.randn(T, G, hd)
    pos = torch.arange(T)
    out = P.paged_attention_rows(q, k, v, pos, scale=hd ** -0.5)
    for t in (0, 4, 8):
        for h in range(H):
            s = (k[:t + 1, h // 2] @ q[t, h]) * hd ** -0.5
            want = torch.softmax(s, 0) @ v[:t + 1, h // 2]
            assert torch.allclose(out[t, h], want, atol=1e-5)
    w = P.paged_attention_rows(q, k, v, pos, scale=hd ** -0.5, window=3)
    s = (k[6:9, 0] @ q[8, 0]) * hd ** -0.5
    assert torch.allclose(w[8, 0], torch.softmax(s, 0) @ v[6:9, 0], atol=1e-5)


def test_forward_is_causal_and_tied_head():
    cfg, w = tiny.plain_model("A")
    toks = tiny.tokens("A", 20, 3)
    full = P.forward(cfg, w, toks)
    part = P.forward(cfg, w, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-5)
    assert full.shape == (20, cfg["vocab_size"])
    assert "lm_head.weight" not in w                      # A is tied
    cfgb, wb = tiny.plain_model("B")
    assert "lm_head.weight" in wb and wb["model.layers.0.conv.conv.bias"].shape == (144,)
    assert P.layer_kinds(cfgb)[2] == "full_attention" and P.ff_dim(cfgb) == 320


def test_greedy_takes_lowest_id_on_ties():
    logits = torch.tensor([0.0, 2.0, 2.0, 1.0])
    assert int(torch.argmax(logits)) == 1                 # sampling.rs:588-604


def test_sample_distribution_filters():
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 2.0])
    d = P.sample_distribution(logits, temperature=1.0, top_k=2)
    assert d[0] > 0 and d[4] > 0 and d[1] == 0 and math.isclose(float(d.sum()), 1.0, rel_tol=1e-6)
    d = P.sample_distribution(logits, temperature=1.0, top_k=1 + 1, top_p=0.4)
    assert d[0] == 1.0                                    # first of the tie reaches 0.4 alone
    d = P.sample_distribution(logits, temperature=0.5, min_p=0.2)
    e = torch.exp((logits - 2.0) / 0.5)
    keep = e / e.sum() >= 0.2 * (e / e.sum()).max()
    assert torch.equal(d > 0, keep)
