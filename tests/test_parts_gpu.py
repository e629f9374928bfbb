"""Each part alone against its plain function; and the seams: a toy mixer with state of its own,
defined here, registered, built and stepped without touching the framework's files; a layer that
runs twice; a layer that reads another layer's cache; a windowed attention layer whose pages come
back."""
import json

import pytest
import torch

import plain_lfm2 as P
import tiny
from fellm_b200.cache import CacheManager
from fellm_b200.config import EngineOptions, register_architecture
from fellm_b200.engine import Engine, StepItem
from fellm_b200.engine.step import StepBuffers
from fellm_b200.models import normed, register_arrangement
from fellm_b200.parts import (FeedForward, FixedState, LayerSpec, Mixer, ModelSpec, ParamDecl, PartSpec, PositionEncoding, Run,
                              build_part, register_part)
from fellm_b200.weights import write_model_folder

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]


def tdtype(d):
    return torch.float32 if d == "float32" else torch.bfloat16


def near(got, want, dtype):
    """The engine's own criterion (tests/tiny.py): largest error against the largest magnitude."""
    return tiny.close(got, want, dtype)[0]


def bound(category, spec, dtype, seed=0):
    """A part with random tensors in the dtypes the loader would keep; returns (part, float32 CPU copies)."""
    part = build_part(category, spec, dtype)
    g = torch.Generator().manual_seed(seed)
    raw = {}
    for local, decl in part.param_decls().items():
        if decl.init[0] == "ones":
            t = 1.0 + 0.2 * torch.randn(decl.shape, generator=g)
        else:
            t = torch.randn(decl.shape, generator=g) * (0.3 if decl.role == "vector" else 0.08)
        raw[local] = t.bfloat16().float()
    kept = {k: v.to(DEV, torch.float32 if (part.decls[k].role == "vector" or dtype == "float32") else torch.bfloat16)
            for k, v in raw.items()}
    part.bind(kept)
    return part, raw


class Harness:
    """A cache manager and step buffers for one mixer, driven by hand."""

    def __init__(self, need, dtype, page_tokens=8):
        self.cache = CacheManager([need], page_tokens=page_tokens, max_tokens=512, max_requests=4, n_ctx=512,
                                  dtype=tdtype(dtype), device=DEV)
        self.buf = StepBuffers(600, 4, DEV)

    def ctx(self, items):
        """items: [(req, n_tokens)]; tokens are not used by a mixer."""
        import numpy as np
        c = self.cache
        starts, slots, lens, pos, ri, rs = [0], [], [], [], [], []
        for i, (req, n) in enumerate(items):
            if not c.has(req):
                c.add_request(req)
            c.reserve(req, n)
            p0, s = c.length(req), c.slot(req)
            pos += list(range(p0, p0 + n)); ri += [i] * n; rs += [s] * n
            starts.append(starts[-1] + n); slots.append(s); lens.append(p0 + n)
        ctx = self.buf.fill(np.zeros(len(pos)), np.array(pos), np.array(ri), np.array(rs), starts, slots, lens, [],
                            max(n for _, n in items), max(lens))
        c.flush()
        views = c.views(ctx.item_slot)
        for req, n in items:
            c.advance(req, n)
        return ctx, views[0]


@pytest.mark.parametrize("dtype", DTYPES)
def test_rmsnorm_part(dtype):
    part, raw = bound("norm", PartSpec.make("rmsnorm", size=200, eps=1e-6), dtype)
    x = torch.randn(9, 200)
    got = part.forward(x.to(DEV), tdtype(dtype))
    assert near(got.float().cpu(), P.rmsnorm(x, raw["weight"], 1e-6), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    emb, raw = bound("embedding", PartSpec.make("table", vocab=301, size=72), dtype)
    toks = torch.tensor([0, 300, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(emb.forward(toks).cpu(), raw["weight"][toks.long().cpu()])
    head, hraw = bound("head", PartSpec.make("linear", vocab=301, size=72, tied=False), dtype)
    xf = torch.randn(3, 72).bfloat16().float()
    got = head.forward(xf.to(DEV, tdtype(dtype)))
    assert got.dtype == torch.float32 and near(got.cpu(), xf @ hraw["weight"].T, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    part, raw = bound("feed_forward", PartSpec.make("swiglu", size=72, ff=200), dtype)
    hn = torch.randn(13, 72).bfloat16().float()
    out = torch.randn(13, 72, device=DEV)
    res = out.clone().cpu()
    part.forward(hn.to(DEV, tdtype(dtype)), None, out)
    want = res + P.swiglu(hn, raw["gate.weight"], raw["up.weight"], raw["down.weight"])
    assert near(out.cpu(), want, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,bias", [(3, False), (4, True), (2, True)])
def test_shortconv_part_whole_and_cut(dtype, taps, bias):
    d = 72
    part, raw = bound("mixer", PartSpec.make("shortconv", size=d, taps=taps, bias=bias), dtype, seed=taps)
    xn = torch.randn(30, d).bfloat16().float()
    want = P.shortconv_mixer(xn, raw["in_proj.weight"], raw["conv.weight"], raw["out_proj.weight"],
                             raw.get("in_proj.bias"), raw.get("conv.bias"), raw.get("out_proj.bias"))
    h = Harness(part.cache_need(), dtype)
    for cuts in ([30], [1, 1, 1, 2, 25], [7, 3, 1, 19]):
        req = f"r{len(cuts)}"
        out = torch.zeros(30, d, device=DEV)
        at = 0
        for n in cuts:
            ctx, view = h.ctx([(req, n)])
            part.forward(xn[at:at + n].to(DEV, tdtype(dtype)), ctx, view, out[at:at + n])
            at += n
        assert near(out.cpu(), want, dtype), cuts
        h.cache.release(req)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,hd,pairing,window", [(4, 2, 16, "adjacent", None), (6, 1, 48, "split_half", None),
                                                    (4, 4, 32, "split_half", 11)])
def test_attention_part_whole_and_cut(dtype, H, G, hd, pairing, window):
    d, eps, theta = 72, 1e-6, 10000.0
    spec = PartSpec.make("attention", size=d, heads=H, kv_heads=G, head_dim=hd, qk_norm=True, norm_eps=eps,
                         position=PartSpec.make("rope", rot_dim=hd, theta=theta, pairing=pairing), window=window)
    part, raw = bound("mixer", spec, dtype, seed=hd)
    T = 41
    xn = torch.randn(T, d).bfloat16().float()
    want = P.attention_mixer(xn, torch.arange(T), raw["q_proj.weight"], raw["k_proj.weight"], raw["v_proj.weight"],
                             raw["out_proj.weight"], raw["q_norm.weight"], raw["k_norm.weight"], n_heads=H,
                             n_kv_heads=G, hd=hd, eps=eps, inv_freq=P.rope_inv_freq(theta, hd), pairing=pairing,
                             window=window)
    h = Harness(part.cache_need(), dtype)
    for cuts in ([T], [3, 2, 9, 1, 1, 25], [16, 16, 9]):
        req = f"r{len(cuts)}{cuts[0]}"
        out = torch.zeros(T, d, device=DEV)
        at = 0
        for n in cuts:
            ctx, view = h.ctx([(req, n)])
            part.forward(xn[at:at + n].to(DEV, tdtype(dtype)), ctx, view, out[at:at + n])
            at += n
        assert near(out.cpu(), want, dtype), cuts
        if window:
            g = h.cache.paged[0]
            assert g.first_page[h.cache.slot(req)] == (T - window + 1) // 8        # pages behind the window came back
        h.cache.release(req)
    h.cache.audit()


# ----------------------------------------------------------------------------------------------
# Another position encoding, defined here: rotary over the first `rot_dim` elements of a head only,
# with every frequency divided by `factor` (the shape of a linear position scaling).  An attention
# mixer asks a position part for inv_freq, pairing and rot_dim and for nothing else.

@register_part("position", "toy_scaled_partial_rope")
class ScaledPartialRope(PositionEncoding):
    def __init__(self, *, dtype, rot_dim, theta, factor, pairing):
        super().__init__()
        self.rot_dim, self.pairing = rot_dim, pairing
        self.inv_freq = P.rope_inv_freq(theta, rot_dim) / factor

    def to(self, device):
        self.inv_freq = self.inv_freq.to(device)
        return self


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rot,pairing,kind", [(32, 16, "adjacent", "rope"), (32, 16, "split_half", "rope"),
                                                 (64, 32, "split_half", "rope"), (48, 20, "adjacent", "toy"),
                                                 (64, 64, "split_half", "toy")])
def test_attention_part_with_partial_rotary_and_another_position_encoding(dtype, hd, rot, pairing, kind):
    """rot_dim < head_dim (FeLLM's rope_dim <= head_dim, crates/backend-cpu/src/kernels/rope.rs:37-44):
    the elements behind rot_dim are normed and not rotated.  Page size 64 at head size 64 makes the
    decode cuts take the kernel that rotates inside attention when rot_dim == head_dim, and the
    separate rotation kernel otherwise."""
    d, H, G, eps, theta = 72, 4, 2, 1e-5, 10000.0
    if kind == "rope":
        pos = PartSpec.make("rope", rot_dim=rot, theta=theta, pairing=pairing)
        inv = P.rope_inv_freq(theta, rot)
    else:
        pos = PartSpec.make("toy_scaled_partial_rope", rot_dim=rot, theta=theta, factor=4.0, pairing=pairing)
        inv = P.rope_inv_freq(theta, rot) / 4.0
    spec = PartSpec.make("attention", size=d, heads=H, kv_heads=G, head_dim=hd, qk_norm=True, norm_eps=eps,
                         position=pos, window=None)
    part, raw = bound("mixer", spec, dtype, seed=hd + rot)
    assert part.rot_dim == rot
    T = 37
    xn = torch.randn(T, d).bfloat16().float()
    want = P.attention_mixer(xn, torch.arange(T), raw["q_proj.weight"], raw["k_proj.weight"], raw["v_proj.weight"],
                             raw["out_proj.weight"], raw["q_norm.weight"], raw["k_norm.weight"], n_heads=H,
                             n_kv_heads=G, hd=hd, eps=eps, inv_freq=inv, pairing=pairing)
    # the rotation matters: without it the result is another one
    flat = P.attention_mixer(xn, torch.arange(T), raw["q_proj.weight"], raw["k_proj.weight"], raw["v_proj.weight"],
                             raw["out_proj.weight"], raw["q_norm.weight"], raw["k_norm.weight"], n_heads=H,
                             n_kv_heads=G, hd=hd, eps=eps, inv_freq=inv * 0, pairing=pairing)
    assert not near(flat, want, dtype)
    h = Harness(part.cache_need(), dtype, page_tokens=64 if hd == 64 else 8)
    for cuts in ([T], [20] + [1] * 17, [5, 2, 30]):
        req = f"r{len(cuts)}"
        out = torch.zeros(T, d, device=DEV)
        at = 0
        for n in cuts:
            ctx, view = h.ctx([(req, n)])
            part.forward(xn[at:at + n].to(DEV, tdtype(dtype)), ctx, view, out[at:at + n])
            at += n
        assert near(out.cpu(), want, dtype), cuts
        h.cache.release(req)


def test_a_position_part_that_does_not_fit_the_head_is_refused():
    from fellm_b200.config import ConfigError
    for rot in (80, 18 + 1):
        spec = PartSpec.make("attention", size=72, heads=4, kv_heads=2, head_dim=64, qk_norm=True, norm_eps=1e-5,
                             position=PartSpec.make("toy_scaled_partial_rope", rot_dim=rot, theta=1e4, factor=1.0,
                                                    pairing="adjacent"), window=None)
        with pytest.raises(ConfigError, match="rotary dimension"):
            build_part("mixer", spec, "bfloat16")


# ----------------------------------------------------------------------------------------------
# A toy mixer with state of its own: y_t = W (sum of xn over the request's tokens 0..t).  Its
# state is the running sum, one float32 vector per request.  Nothing of it is in the framework.

@register_part("mixer", "toy_running_sum")
class RunningSum(Mixer):
    def __init__(self, *, dtype, size):
        super().__init__()
        self.size = size
        self.decls = {"proj.weight": ParamDecl((size, size))}

    def cache_need(self):
        return FixedState((self.size,))

    def forward(self, xn, ctx, cache, out, reads_only=False):
        starts, slots = ctx.item_start.tolist(), cache.item_slot.tolist()
        for i, slot in enumerate(slots):
            x = xn[starts[i]:starts[i + 1]].float()
            run = cache.states[slot] + torch.cumsum(x, dim=0)
            cache.states[slot] = run[-1]
            out[starts[i]:starts[i + 1]] += run @ self.w["proj.weight"].float().T
        return out


def toy_spec(cfg):
    d, hd = cfg["hidden_size"], cfg["head_dim"]
    pos = PartSpec.make("rope", rot_dim=hd, theta=cfg["rope_theta"], pairing="split_half")
    def layer(i, mixer):
        p = f"layers.{i}."
        return LayerSpec(PartSpec.make("rmsnorm", prefix=p + "n1.", size=d, eps=1e-5), mixer,
                         PartSpec.make("rmsnorm", prefix=p + "n2.", size=d, eps=1e-5),
                         PartSpec.make("swiglu", prefix=p + "ff.", size=d, ff=cfg["ff"]))
    att = dict(size=d, heads=cfg["heads"], kv_heads=cfg["kv_heads"], head_dim=hd, qk_norm=False, norm_eps=1e-5,
               position=pos, window=None)
    layers = [layer(0, PartSpec.make("toy_running_sum", prefix="layers.0.toy.", size=d)),
              layer(1, PartSpec.make("attention", prefix="layers.1.att.", **att)),
              layer(2, PartSpec.make("attention", prefix="layers.2.att.", shares_cache=True, **att))]
    # layer 1 runs twice (each run with a cache of its own); layer 2 reads the cache of the first run
    schedule = [Run(0), Run(1), Run(2, cache_of=1), Run(1), Run(0)]
    return ModelSpec("ToyForCausalLM", d, cfg["vocab_size"], cfg["max_position"],
                     PartSpec.make("table", prefix="emb.", vocab=cfg["vocab_size"], size=d), layers,
                     PartSpec.make("rmsnorm", prefix="norm.", size=d, eps=1e-5),
                     PartSpec.make("linear", prefix="head.", vocab=cfg["vocab_size"], size=d, tied=True), schedule)


class ToyConfig(dict):
    def to_dict(self):
        return dict(self)


register_architecture("ToyForCausalLM", lambda d: ToyConfig(d), toy_spec)
TOY = dict(architectures=["ToyForCausalLM"], vocab_size=97, hidden_size=48, head_dim=16, heads=3, kv_heads=1,
           ff=80, rope_theta=10000.0, max_position=256)


def toy_plain(w, tokens):
    """The toy model, whole sequence, in plain torch."""
    d, hd, H, G = 48, 16, 3, 1
    x = w["emb.weight"][torch.tensor(tokens)]
    T = len(tokens)
    inv = P.rope_inv_freq(10000.0, hd)
    pos = torch.arange(T)

    def ffn(x, i):
        hn = P.rmsnorm(x, w[f"layers.{i}.n2.weight"], 1e-5)
        return x + P.swiglu(hn, w[f"layers.{i}.ff.gate.weight"], w[f"layers.{i}.ff.up.weight"], w[f"layers.{i}.ff.down.weight"])

    def toy(x):
        xn = P.rmsnorm(x, w["layers.0.n1.weight"], 1e-5)
        return ffn(x + torch.cumsum(xn, 0) @ w["layers.0.toy.proj.weight"].T, 0)

    def qkv(xn, i, with_kv=True):
        q = P.rope_apply((xn @ w[f"layers.{i}.att.q_proj.weight"].T).reshape(T, H, hd), pos, inv, "split_half")
        if not with_kv:
            return q, None, None
        k = P.rope_apply((xn @ w[f"layers.{i}.att.k_proj.weight"].T).reshape(T, G, hd), pos, inv, "split_half")
        v = (xn @ w[f"layers.{i}.att.v_proj.weight"].T).reshape(T, G, hd)
        return q, k, v

    def attend(x, i, q, k, v):
        a = P.paged_attention_rows(q, k, v, pos, scale=hd ** -0.5).reshape(T, H * hd)
        return ffn(x + a @ w[f"layers.{i}.att.out_proj.weight"].T, i)

    x = toy(x)
    q, k1, v1 = qkv(P.rmsnorm(x, w["layers.1.n1.weight"], 1e-5), 1)
    x = attend(x, 1, q, k1, v1)
    q, _, _ = qkv(P.rmsnorm(x, w["layers.2.n1.weight"], 1e-5), 2, with_kv=False)
    x = attend(x, 2, q, k1, v1)                       # reads the first run's keys and values
    q, k, v = qkv(P.rmsnorm(x, w["layers.1.n1.weight"], 1e-5), 1)
    x = attend(x, 1, q, k, v)                         # layer 1 again, own cache
    # the toy layer again: a second running sum, its own state
    xn = P.rmsnorm(x, w["layers.0.n1.weight"], 1e-5)
    x = ffn(x + torch.cumsum(xn, 0) @ w["layers.0.toy.proj.weight"].T, 0)
    return P.rmsnorm(x, w["norm.weight"], 1e-5) @ w["emb.weight"].T


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_registers_builds_and_steps(dtype, tmp_path):
    folder = write_model_folder(tmp_path / "toy", TOY, 3)
    eng = Engine.open(folder, EngineOptions(dtype=dtype, n_ctx=0, max_requests=4, max_tokens=512, page_tokens=16,
                                            cuda_graphs=False))
    needs = eng.model.cache_needs()
    assert needs[2] is None and needs[0] == FixedState((48,)) and needs[1] == needs[3]
    assert len(eng.cache.paged) == 1 and eng.cache.paged[0].pool.shape[1] == 2       # two runs keep keys
    assert len(eng.cache.fixed) == 1 and eng.cache.fixed[0].states.shape[1] == 2     # two runs keep a sum
    w = {k: v.float() for k, v in P.read_safetensors(folder / "model.safetensors").items()}
    toks = [int(t) for t in torch.randint(0, 97, (50,), generator=torch.Generator().manual_seed(1))]
    want = toy_plain(w, toks)
    for cuts in ([50], [7, 1, 1, 2, 30, 9]):
        eng.add_request("t")
        rows, at = [], 0
        for n in cuts:
            rows.append(eng.step([StepItem("t", toks[at:at + n], list(range(n)))]))
            at += n
        eng.release("t")
        ok, err, tolr = tiny.close(torch.cat(rows), want, dtype)
        assert ok, (cuts, err, tolr)
    eng.check_status()


# ----------------------------------------------------------------------------------------------
# A second toy architecture for the seams the first one leaves out, all of it defined here:
#   * a mixer that keeps TWO states of different shapes (a running sum and the last token's
#     input; FeLLM's GatedDeltaNet keeps a convolution history and a matrix the same way,
#     crates/fellm-model/src/graph.rs:792-806): cache_need() returns a list, forward() gets a list;
#   * a feed-forward with routing: a float32 router picks one of E experts per token;
#   * a block arrangement of its own: one norm, mixer and feed-forward side by side
#     (x += mixer(n(x)) + ffn(n(x))), registered by name;
#   * a layer without a feed-forward.

@register_part("mixer", "toy_sum_and_last")
class SumAndLast(Mixer):
    def __init__(self, *, dtype, size):
        super().__init__()
        self.size = size
        self.decls = {"sum.weight": ParamDecl((size, size)), "last.weight": ParamDecl((size, size))}

    def cache_need(self):
        return [FixedState((self.size,)), FixedState((1, self.size))]

    def forward(self, xn, ctx, cache, out, reads_only=False):
        sums, last = cache
        starts, slots = ctx.item_start.tolist(), sums.item_slot.tolist()
        for i, slot in enumerate(slots):
            x = xn[starts[i]:starts[i + 1]].float()
            run = sums.states[slot] + torch.cumsum(x, dim=0)
            prev = torch.cat([last.states[slot], x[:-1]], dim=0)          # the input of the token before
            sums.states[slot] = run[-1]
            last.states[slot] = x[-1:]
            out[starts[i]:starts[i + 1]] += run @ self.w["sum.weight"].float().T + prev @ self.w["last.weight"].float().T
        return out


@register_part("feed_forward", "toy_routed")
class Routed(FeedForward):
    def __init__(self, *, dtype, size, ff, experts):
        super().__init__()
        self.decls = {"router.weight": ParamDecl((experts, size), role="vector")}      # kept float32
        for e in range(experts):
            self.decls[f"experts.{e}.up.weight"] = ParamDecl((ff, size))
            self.decls[f"experts.{e}.down.weight"] = ParamDecl((size, ff))
        self.experts = experts

    def forward(self, hn, ctx, out):
        h = hn.float()
        pick = torch.argmax(h @ self.w["router.weight"].T, dim=-1)                      # router logits in float32
        for e in range(self.experts):
            rows = (pick == e).nonzero().flatten()
            if rows.numel():
                z = torch.relu(h[rows] @ self.w[f"experts.{e}.up.weight"].float().T)
                out[rows] += z @ self.w[f"experts.{e}.down.weight"].float().T
        return out


@register_arrangement("toy_parallel")
def _parallel(block, x, ctx, cache, act_dtype, reads_only):
    xn = block.norm1.forward(x, act_dtype)               # both branches read the block's input
    block.mixer.forward(xn, ctx, cache, x, reads_only=reads_only)
    block.ffn.forward(xn, ctx, x)


def toy2_spec(cfg):
    d = cfg["hidden_size"]
    norm = lambda p: PartSpec.make("rmsnorm", prefix=p, size=d, eps=1e-6)
    layers = [
        LayerSpec(norm("l0.n."), PartSpec.make("toy_sum_and_last", prefix="l0.mix.", size=d), None,
                  PartSpec.make("toy_routed", prefix="l0.ff.", size=d, ff=cfg["ff"], experts=cfg["experts"]),
                  arrangement="toy_parallel"),
        LayerSpec(norm("l1.n."), PartSpec.make("toy_running_sum", prefix="l1.mix.", size=d)),     # no feed-forward
        LayerSpec(norm("l2.n1."), PartSpec.make("toy_sum_and_last", prefix="l2.mix.", size=d), norm("l2.n2."),
                  PartSpec.make("swiglu", prefix="l2.ff.", size=d, ff=cfg["ff"]))]
    return ModelSpec("Toy2ForCausalLM", d, cfg["vocab_size"], cfg["max_position"],
                     PartSpec.make("table", prefix="emb.", vocab=cfg["vocab_size"], size=d), layers,
                     norm("norm."), PartSpec.make("linear", prefix="head.", vocab=cfg["vocab_size"], size=d, tied=False))


register_architecture("Toy2ForCausalLM", lambda d: ToyConfig(d), toy2_spec)
TOY2 = dict(architectures=["Toy2ForCausalLM"], vocab_size=61, hidden_size=40, ff=56, experts=3, max_position=128)


def toy2_plain(w, tokens):
    x = w["emb.weight"][torch.tensor(tokens)]

    def sum_and_last(xn, p):
        prev = torch.cat([torch.zeros(1, xn.shape[1]), xn[:-1]], dim=0)
        return torch.cumsum(xn, 0) @ w[p + "sum.weight"].T + prev @ w[p + "last.weight"].T

    xn = P.rmsnorm(x, w["l0.n.weight"], 1e-6)
    pick = torch.argmax(xn @ w["l0.ff.router.weight"].T, dim=-1)
    ff = torch.zeros_like(x)
    for t in range(len(tokens)):
        e = int(pick[t])
        ff[t] = torch.relu(xn[t] @ w[f"l0.ff.experts.{e}.up.weight"].T) @ w[f"l0.ff.experts.{e}.down.weight"].T
    x = x + sum_and_last(xn, "l0.mix.") + ff
    x = x + torch.cumsum(P.rmsnorm(x, w["l1.n.weight"], 1e-6), 0) @ w["l1.mix.proj.weight"].T
    x = x + sum_and_last(P.rmsnorm(x, w["l2.n1.weight"], 1e-6), "l2.mix.")
    hn = P.rmsnorm(x, w["l2.n2.weight"], 1e-6)
    x = x + P.swiglu(hn, w["l2.ff.gate.weight"], w["l2.ff.up.weight"], w["l2.ff.down.weight"])
    return P.rmsnorm(x, w["norm.weight"], 1e-6) @ w["head.weight"].T


def test_two_states_a_routed_feed_forward_and_an_arrangement_of_its_own(tmp_path):
    """float32 only: the expert a token goes to must not flip on rounding."""
    folder = write_model_folder(tmp_path / "toy2", TOY2, 5)
    eng = Engine.open(folder, EngineOptions(dtype="float32", n_ctx=0, max_requests=4, max_tokens=256, page_tokens=16,
                                            cuda_graphs=False))
    needs = eng.model.cache_needs()
    assert needs[0] == [FixedState((40,)), FixedState((1, 40))] and needs[1] == FixedState((40,))
    # the running sums of all three layers share one group, the last-token vectors another
    shapes = sorted(tuple(g.states.shape[1:]) for g in eng.cache.fixed)
    assert shapes == [(2, 1, 40), (3, 40)] and not eng.cache.paged
    assert eng.model.blocks[1].ffn is None and eng.model.blocks[0].norm2 is None
    w = {k: v.float() for k, v in P.read_safetensors(folder / "model.safetensors").items()}
    toks = [int(t) for t in torch.randint(0, 61, (33,), generator=torch.Generator().manual_seed(2))]
    want = toy2_plain(w, toks)
    other = [int(t) for t in torch.randint(0, 61, (9,), generator=torch.Generator().manual_seed(3))]
    for cuts in ([33], [5, 1, 1, 2, 24], [1] * 33):
        eng.add_request("t"), eng.add_request("o")          # a second request beside it, so that slots matter
        rows, at = [], 0
        for j, n in enumerate(cuts):
            items = [StepItem("t", toks[at:at + n], list(range(n)))]
            if j < len(other):
                items.insert(0, StepItem("o", [other[j]], []))
            rows.append(eng.step(items))
            at += n
        eng.release("t"), eng.release("o")
        ok, err, tolr = tiny.close(torch.cat(rows), want, "float32")
        assert ok, (cuts, err, tolr)
    eng.check_status()
