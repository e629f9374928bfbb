"""Plain, slow LFM2 (ShortConv hybrid) forward pass: whole sequences, no cache.

This file is the yardstick the engine is compared with.  It is written from the
formulas of orielhaim/FeLLM's CPU kernels and graph builder (each function cites
the file and lines it restates).  FeLLM's own model code is Rust and cannot be
compiled or imported here (no cargo/rustc on the machine), so this file rests on
those formulas alone; the one hand-computed vector FeLLM's ShortConv unit test
carries (crates/backend-cpu/src/kernels/shortconv.rs:113-154) is replayed in
tests/test_plain.py.

Nothing here is shared with the product path: it has its own config reading, its
own safetensors reader, and one function per part.  Everything is float32 on the
CPU, sequence at a time, quadratic attention, and generation recomputes the whole
sequence for every new token.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16,
              "I32": torch.int32, "I64": torch.int64}


def read_safetensors(path) -> dict:
    """Minimal reader: 8-byte little-endian header length, JSON header, raw data.

    Container checks follow plugins/dspark/src/checkpoint.rs:59-118.
    """
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = memoryview(raw)[8 + hlen:]
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=dt).reshape(meta["shape"])
        out[name] = t
    return out


def load_folder(folder):
    """(config dict, {name: float32 tensor}) of a model folder."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: v.to(torch.float32) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# --------------------------------------------------------------------------- sizes

def ff_dim(cfg: dict) -> int:
    """Feed-forward width.  FeLLM reads an already final feed_forward_length
    (crates/fellm-model/src/probe.rs:232); config.json carries block_ff_dim and the
    auto-adjust rule: F=floor(2F/3); F=floor(mult*F); round up to multiple_of."""
    f = int(cfg["block_ff_dim"])
    if cfg.get("block_auto_adjust_ff_dim", False):
        f = int(2 * f / 3)
        mult = cfg.get("block_ffn_dim_multiplier", None)
        if mult is not None:
            f = int(mult * f)
        mo = int(cfg.get("block_multiple_of", 256))
        f = mo * ((f + mo - 1) // mo)
    return f


def layer_kinds(cfg: dict) -> list:
    """Per-layer mixer kind, from layer_types or full_attn_idxs
    (FeLLM infers it from which tensors a block has, probe.rs:340-363)."""
    n = int(cfg["num_hidden_layers"])
    if cfg.get("layer_types") is not None:
        return list(cfg["layer_types"])
    idx = set(cfg["full_attn_idxs"])
    return ["full_attention" if i in idx else "conv" for i in range(n)]


def head_dim(cfg: dict) -> int:
    """probe.rs:225-227: key_length, else d / heads."""
    return int(cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"])


# --------------------------------------------------------------------------- parts

def rmsnorm(x, w, eps):
    """y = x * 1/sqrt(mean(x^2)+eps) * w, product order x*scale*w
    (crates/backend-cpu/src/kernels/norm.rs:6-39)."""
    scale = 1.0 / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return x * scale * w


def rope_inv_freq(theta: float, rope_dim: int):
    """inv_freq[i] = theta^(-2i/rope_dim) in float32 (crates/fellm-model/src/rope.rs:13-21)."""
    i = torch.arange(rope_dim // 2, dtype=torch.float32)
    exp = -(2.0 * i) / float(rope_dim)
    return torch.pow(torch.tensor(float(theta), dtype=torch.float32), exp)


def rope_apply(x, positions, inv_freq, pairing: str):
    """x [T, heads, hd]; angle = float32(pos) * inv_freq; a' = a*c - b*s, b' = a*s + b*c on
    pairs (2i, 2i+1) ('adjacent') or (i, i+rope_dim/2) ('split_half') of the first
    rope_dim = 2*len(inv_freq) <= hd elements of each head; the rest stays as it is
    (crates/backend-cpu/src/kernels/rope.rs:28-62)."""
    rope_dim = 2 * inv_freq.numel()
    if rope_dim < x.shape[-1]:
        return torch.cat([rope_apply(x[..., :rope_dim], positions, inv_freq, pairing), x[..., rope_dim:]], dim=-1)
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]      # [T, hd/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    half = x.shape[-1] // 2
    if pairing == "adjacent":
        a, b = x[..., 0::2], x[..., 1::2]
    elif pairing == "split_half":
        a, b = x[..., :half], x[..., half:]
    else:
        raise ValueError(pairing)
    a2, b2 = a * c - b * s, a * s + b * c
    out = torch.empty_like(x)
    if pairing == "adjacent":
        out[..., 0::2], out[..., 1::2] = a2, b2
    else:
        out[..., :half], out[..., half:] = a2, b2
    return out


def shortconv_mixer(xn, w_in, w_conv, w_out, b_in=None, b_conv=None, b_out=None):
    """Gated short causal depthwise convolution over a whole sequence xn [T, d].

    [B; C; X] = W_in xn (thirds, in that order); bx = B*X;
    conv[t,c] = bx[t,c]*w[c,Lc-1] + sum_{j<Lc-1} bx[t-(Lc-1)+j, c]*w[c,j] with zeros before
    the first token; y = W_out (C * conv)
    (crates/backend-cpu/src/kernels/shortconv.rs:61-106; FeLLM runs it one token at a time with
    a rolling state, which over a sequence that starts from a zero state is this sum).
    Biases (conv_bias=true) are added to W_in xn, to conv before the C gate, and to W_out(.)."""
    T, d = xn.shape
    w_conv = w_conv.reshape(d, -1)
    lc = w_conv.shape[1]
    bcx = xn @ w_in.T
    if b_in is not None:
        bcx = bcx + b_in
    B, C, X = bcx[:, :d], bcx[:, d:2 * d], bcx[:, 2 * d:]
    bx = B * X
    padded = torch.cat([torch.zeros(lc - 1, d), bx], dim=0)            # padded[t + lc-1] = bx[t]
    conv = bx * w_conv[:, lc - 1]
    for j in range(lc - 1):
        conv = conv + padded[j:j + T] * w_conv[:, j]
    if b_conv is not None:
        conv = conv + b_conv
    y = (C * conv) @ w_out.T
    if b_out is not None:
        y = y + b_out
    return y


def attention_mixer(xn, positions, wq, wk, wv, wo, q_norm_w, k_norm_w, *, n_heads, n_kv_heads,
                    hd, eps, inv_freq, pairing, window=None):
    """GQA attention with per-head QK RMSNorm and RoPE over a whole sequence xn [T, d].

    q,k,v = W xn -> RMSNorm per head on q,k (one [hd] weight each, eps = norm eps) -> RoPE on q,k
    -> s = q.k / sqrt(hd), kv head g = h // (H/G), causal (a query at position p sees keys 0..p,
    or the last `window` of them) -> softmax in float32 -> sum p v -> W_o
    (crates/fellm-model/src/graph.rs:2014-2246; crates/fellm-plugin-abi/src/attention_provider.rs:175-237)."""
    T = xn.shape[0]
    q = (xn @ wq.T).reshape(T, n_heads, hd)
    k = (xn @ wk.T).reshape(T, n_kv_heads, hd)
    v = (xn @ wv.T).reshape(T, n_kv_heads, hd)
    q = rope_apply(rmsnorm(q, q_norm_w, eps), positions, inv_freq, pairing)
    k = rope_apply(rmsnorm(k, k_norm_w, eps), positions, inv_freq, pairing)
    rep = n_heads // n_kv_heads
    scale = 1.0 / math.sqrt(hd)
    out = torch.empty(T, n_heads, hd)
    pi, pj = positions[:, None], positions[None, :]
    visible = pj <= pi
    if window is not None:
        visible = visible & (pj > pi - window)
    for h in range(n_heads):
        g = h // rep
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = s.masked_fill(~visible, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out.reshape(T, n_heads * hd) @ wo.T


def swiglu(hn, w_gate, w_up, w_down):
    """f = W_down (silu(W_gate h) * W_up h), silu(g) = g / (1 + exp(-g))
    (crates/backend-cpu/src/kernels/swiglu.rs:4-16; graph.rs:2260-2287)."""
    g = hn @ w_gate.T
    u = hn @ w_up.T
    return ((g / (1.0 + torch.exp(-g))) * u) @ w_down.T


def block(x, positions, cfg, w, i, kind, inv_freq):
    """h = x + Mixer(RMSNorm(x)); out = h + FFN(RMSNorm(h)) (graph.rs:1650-1777)."""
    p = f"model.layers.{i}."
    eps = float(cfg.get("norm_eps", 1e-5))
    xn = rmsnorm(x, w[p + "operator_norm.weight"], eps)
    if kind == "conv":
        bias = bool(cfg.get("conv_bias", False))
        y = shortconv_mixer(
            xn, w[p + "conv.in_proj.weight"], w[p + "conv.conv.weight"], w[p + "conv.out_proj.weight"],
            w[p + "conv.in_proj.bias"] if bias else None,
            w[p + "conv.conv.bias"] if bias else None,
            w[p + "conv.out_proj.bias"] if bias else None)
    elif kind == "full_attention":
        y = attention_mixer(
            xn, positions, w[p + "self_attn.q_proj.weight"], w[p + "self_attn.k_proj.weight"],
            w[p + "self_attn.v_proj.weight"], w[p + "self_attn.out_proj.weight"],
            w[p + "self_attn.q_layernorm.weight"], w[p + "self_attn.k_layernorm.weight"],
            n_heads=int(cfg["num_attention_heads"]), n_kv_heads=int(cfg["num_key_value_heads"]),
            hd=head_dim(cfg), eps=eps, inv_freq=inv_freq,
            pairing=cfg.get("rope_pairing", "split_half"))
    else:
        raise ValueError(f"unknown layer type {kind!r}")
    h = x + y
    hn = rmsnorm(h, w[p + "ffn_norm.weight"], eps)
    f = swiglu(hn, w[p + "feed_forward.w1.weight"], w[p + "feed_forward.w3.weight"],
               w[p + "feed_forward.w2.weight"])
    return h + f


def forward(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence (graph.rs:19-132): embedding (no scaling),
    blocks, final RMSNorm, head (the embedding matrix when tied)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x = w["model.embed_tokens.weight"][tokens]
    inv_freq = rope_inv_freq(float(cfg["rope_theta"]), head_dim(cfg))
    for i, kind in enumerate(layer_kinds(cfg)):
        x = block(x, positions, cfg, w, i, kind, inv_freq)
    xf = rmsnorm(x, w["model.embedding_norm.weight"], float(cfg.get("norm_eps", 1e-5)))
    tied = bool(cfg.get("tie_word_embeddings", cfg.get("tie_embedding", True)))
    head = w["model.embed_tokens.weight"] if tied else w["lm_head.weight"]
    return xf @ head.T


def greedy(cfg: dict, w: dict, prompt, n_new: int) -> list:
    """n_new greedy tokens; ties go to the lower id (crates/fellm-runtime/src/sampling.rs:588-604).
    Recomputes the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = forward(cfg, w, seq)[-1]
        tok = int(torch.argmax(logits))          # torch.argmax returns the first maximum
        out.append(tok)
        seq.append(tok)
    return out


# ------------------------------------------------------------------ kernels' yardsticks

def paged_attention_rows(q, k_all, v_all, q_pos, *, scale, window=None):
    """q [R, H, hd] float32 with absolute positions q_pos [R]; k_all, v_all [C, G, hd] the
    request's keys/values at positions 0..C-1.  Returns [R, H, hd]."""
    R, H, hd = q.shape
    G = k_all.shape[1]
    rep = H // G
    out = torch.empty(R, H, hd)
    kpos = torch.arange(k_all.shape[0])
    for r in range(R):
        vis = kpos <= q_pos[r]
        if window is not None:
            vis = vis & (kpos > q_pos[r] - window)
        for h in range(H):
            g = h // rep
            s = (k_all[:, g, :] @ q[r, h, :]) * scale
            s = s.masked_fill(~vis, float("-inf"))
            out[r, h] = torch.softmax(s, dim=0) @ v_all[:, g, :]
    return out


def sample_distribution(logits, *, temperature, top_k=0, top_p=1.0, min_p=0.0):
    """The processed distribution FeLLM draws from
    (crates/fellm-runtime/src/sampling.rs:325-394,396-478): logits/temperature -> keep the k
    best (ties: lower id first) -> softmax over them -> drop p < min_p * p_max, renormalise ->
    shortest prefix (by descending p) whose mass reaches top_p, renormalise."""
    V = logits.numel()
    z = logits.to(torch.float32) / max(temperature, torch.finfo(torch.float32).eps)
    k = top_k if 0 < top_k < V else V
    order = sorted(range(V), key=lambda i: (-float(z[i]), i))[:k]
    vals = torch.tensor([float(z[i]) for i in order])
    p = torch.exp(vals - vals.max())
    p = p / p.sum()
    keep = list(range(len(order)))
    if 0.0 < min_p < 1.0:
        thr = float(p[0]) * min_p
        keep = [j for j in keep if float(p[j]) >= thr]
        p = p[keep] / p[keep].sum()
        order = [order[j] for j in keep]
    if 0.0 < top_p < 1.0:
        cum, cut = 0.0, len(order)
        for j in range(len(order)):
            cum += float(p[j])
            if cum >= top_p:
                cut = j + 1
                break
        order, p = order[:cut], p[:cut] / p[:cut].sum()
    dist = torch.zeros(V)
    for j, i in enumerate(order):
        dist[i] = p[j]
    return dist
