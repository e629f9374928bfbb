"""A model assembled from a ModelSpec: embedding, blocks of (norm, mixer, norm, feed-forward),
final norm and head, run in the order the spec's schedule gives.

The forward pass here is the body of the step function: it runs exactly the rows of one
StepContext, reads and writes the caches through the views it is given, and computes the final
norm and the head only for the rows whose logits are wanted (FeLLM skips final_norm + lm_head for
mid-prompt tokens the same way, crates/fellm-runtime/src/compiled.rs:425-434).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.errors import ConfigError
from ..parts.base import ParamDecl, build_part
from ..parts.linear import LazyNorm
from ..parts.spec import ModelSpec


def _normed(x, norm, consumer, act_dtype):
    """The consumer's input: normed now, or left to the consumer's first product."""
    if getattr(consumer, "takes_lazy_norm", False):
        return LazyNorm(x, norm, act_dtype)
    return norm.forward(x, act_dtype)


ARRANGEMENTS = {}


def register_arrangement(name: str):
    """Decorator: `fn(block, x, ctx, cache, act_dtype, reads_only)` wires a block's parts for
    LayerSpec.arrangement == name.  x is the float32 residual stream [T, d] and is updated in
    place (mixers and feed-forwards ADD into the tensor they are given as `out`); `block` has
    .norm1, .mixer, .norm2, .ffn (None where the spec names none) and, during the call,
    .norm_after: the norm that reads x after this block (the next block's first, or the final one;
    None where that is not known).  An arrangement may tell a norm that it comes next
    (`norm.expect(x)`) right before the part whose last act is to add into x."""
    def deco(fn):
        ARRANGEMENTS[name] = fn
        return fn
    return deco


def normed(x, norm, consumer, act_dtype):
    """The consumer's input: normed now, or left to the consumer's first product."""
    return _normed(x, norm, consumer, act_dtype)


@register_arrangement("prenorm")
def _prenorm(block, x, ctx, cache, act_dtype, reads_only):
    """x += mixer(norm1(x)); x += ffn(norm2(x))   (crates/fellm-model/src/graph.rs:1650-1777)."""
    h = _normed(x, block.norm1, block.mixer, act_dtype)
    after_mixer = block.norm2 if block.ffn is not None else block.norm_after
    if after_mixer is not None:
        after_mixer.expect(x)
    block.mixer.forward(h, ctx, cache, x, reads_only=reads_only)
    if block.ffn is not None:
        h = _normed(x, block.norm2, block.ffn, act_dtype)
        if block.norm_after is not None:
            block.norm_after.expect(x)
        block.ffn.forward(h, ctx, x)


class Block:
    """One layer's parts; how they are wired is looked up by the spec's arrangement name."""

    def __init__(self, spec, dtype: str):
        if spec.arrangement not in ARRANGEMENTS:
            raise ConfigError(f"unknown block arrangement {spec.arrangement!r}; registered: "
                              f"{', '.join(sorted(ARRANGEMENTS))}")
        self.spec = spec
        self.arrange = ARRANGEMENTS[spec.arrangement]
        self.norm1 = build_part("norm", spec.norm1, dtype) if spec.norm1 is not None else None
        self.mixer = build_part("mixer", spec.mixer, dtype)
        self.norm2 = build_part("norm", spec.norm2, dtype) if spec.norm2 is not None else None
        self.ffn = build_part("feed_forward", spec.ffn, dtype) if spec.ffn is not None else None
        self.norm_after = None

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def forward(self, x, ctx, cache, act_dtype, reads_only=False, norm_after=None):
        """x: float32 residual stream [T, d], updated in place."""
        self.norm_after = norm_after
        self.arrange(self, x, ctx, cache, act_dtype, reads_only)
        return x


class Model:
    def __init__(self, spec: ModelSpec, dtype: str):
        self.spec, self.dtype = spec, dtype
        self.act_dtype = torch.bfloat16 if dtype == "bfloat16" else torch.float32
        self.embedding = build_part("embedding", spec.embedding, dtype)
        self.blocks: List[Block] = [Block(ls, dtype) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype)
        self.head = build_part("head", spec.head, dtype)
        self.schedule = list(spec.schedule)

    # ---- parameters
    def all_parts(self):
        parts = [self.embedding]
        for b in self.blocks:
            parts += b.parts()
        return parts + [self.final_norm, self.head]

    def param_table(self) -> Dict[str, tuple]:
        """{tensor name in the file: (part, local name, ParamDecl)} over all parts."""
        table = {}
        for part in self.all_parts():
            for local, decl in part.param_decls().items():
                name = part.spec.tensor_name(local)
                if name in table:
                    raise ConfigError(f"two parts claim the tensor {name}")
                table[name] = (part, local, decl)
        return table

    def tied_aliases(self) -> Dict[str, str]:
        """{name a file may also carry: name of the tensor it must equal}.  A tied head owns no
        tensor, but files written from a state dict often store the head all the same, as a copy of
        the embedding matrix (FeLLM reads `output.weight` when it is there and ties otherwise,
        crates/fellm-model/src/graph.rs:29-34); such a copy is accepted if it is one."""
        if getattr(self.head, "tied", False):
            return {self.head.spec.tensor_name("weight"): self.embedding.spec.tensor_name("weight")}
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]):
        """tensors: {file name: tensor already on the device, in its kept dtype}."""
        per_part: Dict[int, dict] = {}
        for name, (part, local, _) in self.param_table().items():
            per_part.setdefault(id(part), {})[local] = tensors[name]
        for part in self.all_parts():
            if part is self.head and getattr(part, "tied", False):
                continue
            part.bind(per_part.get(id(part), {}))
        if getattr(self.head, "tied", False):
            self.head.bind({"weight": self.embedding.w["weight"]})

    def kernel_modules(self):
        mods = []
        for part in self.all_parts():
            mods += part.kernel_modules(self.dtype)
        return mods

    def weight_chain(self):
        """The matrices of one step in the order its products read them (the schedule's order)."""
        chain = []
        for run in self.schedule:
            b = self.blocks[run.layer]
            chain += b.mixer.weight_order()
            if b.ffn is not None:
                chain += b.ffn.weight_order()
        return chain + self.head.weight_order()

    def cache_needs(self):
        """Per schedule entry: the mixer's cache need, or None when the entry reads another's."""
        return [None if run.cache_of is not None else self.blocks[run.layer].mixer.cache_need()
                for run in self.schedule]

    # ---- the step's body
    def forward(self, ctx, caches, greedy_tokens=None) -> torch.Tensor:
        """ctx: StepContext; caches[n]: the cache view of schedule entry n.  Returns float32
        logits [len(ctx.logit_rows), vocab] (an empty tensor when none are wanted).
        greedy_tokens (int32, device): the caller only wants the greedy token of every wanted row; where the
        head can give them without the logits it writes greedy_tokens[:wanted] and None is returned."""
        ops.forget_norm_handoff()
        x = self.embedding.forward(ctx.tokens, ctx.status)
        for n, run in enumerate(self.schedule):
            src = n if run.cache_of is None else run.cache_of
            if n + 1 < len(self.schedule):
                norm_after = self.blocks[self.schedule[n + 1].layer].norm1
            else:
                norm_after = self.final_norm if (ctx.logits_all and ctx.n_logit_rows) else None
            self.blocks[run.layer].forward(x, ctx, caches[src], self.act_dtype,
                                           reads_only=run.cache_of is not None, norm_after=norm_after)
        if ctx.n_logit_rows == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=x.device)
        if ctx.logits_all and getattr(self.head, "takes_lazy_norm", False):
            xf = LazyNorm(x, self.final_norm, self.act_dtype)
        else:
            xf = self.final_norm.forward(x, self.act_dtype, rows=ctx.logit_rows)
        if greedy_tokens is not None and self.head.forward_greedy(xf, greedy_tokens):
            return None
        return self.head.forward(xf)


def build_model(spec: ModelSpec, dtype: str) -> Model:
    return Model(spec, dtype)
