"""The data that describes a model: which parts each layer is made of, with which sizes,
under which tensor names, and in which order the layers run.

FeLLM keeps the same facts in `ModelSpec`/`LayerSpec{mix, ffn, attn_ordinal, conv_ordinal}`
(crates/fellm-model/src/probe.rs:36-56,86-181) and turns them into an op graph
(crates/fellm-model/src/graph.rs:1607-1778).  Here the description stays data all the way down:
an architecture's `build_spec` fills it in and `fellm_b200.models.build_model` assembles parts
from it, so a layer-by-layer mix of mixers and feed-forwards needs no code.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its kind (a key of the part registries in fellm_b200.parts.base), its sizes and
    constants, and the tensor name in the weight file of each of its parameters
    (`names[local] = file name`; a local name that is absent keeps `prefix + local`)."""
    kind: str
    params: Tuple[Tuple[str, object], ...] = ()
    prefix: str = ""
    names: Tuple[Tuple[str, str], ...] = ()

    @staticmethod
    def make(kind: str, prefix: str = "", names: Optional[Dict[str, str]] = None, **params):
        return PartSpec(kind, tuple(sorted(params.items())), prefix,
                        tuple(sorted((names or {}).items())))

    def kwargs(self) -> dict:
        return dict(self.params)

    def tensor_name(self, local: str) -> str:
        return dict(self.names).get(local, self.prefix + local)


@dataclass(frozen=True)
class LayerSpec:
    """One block.  `arrangement` names how the parts are wired, a key of
    fellm_b200.models.model.ARRANGEMENTS (`register_arrangement` adds one):
    'prenorm': h = x + mixer(norm1(x)); out = h + ffn(norm2(h))   (graph.rs:1650-1777).
    norm1, norm2 and ffn may be None where an arrangement has no use for them (a layer without a
    feed-forward, a block with one norm)."""
    norm1: Optional[PartSpec]
    mixer: PartSpec
    norm2: Optional[PartSpec] = None
    ffn: Optional[PartSpec] = None
    arrangement: str = "prenorm"


@dataclass(frozen=True)
class Run:
    """One entry of the order in which layers run.  `layer` indexes ModelSpec.layers and may
    appear in several entries (the same weights run again, with a cache of their own).
    `cache_of`, when set, is the index of an EARLIER entry whose cache this entry reads instead
    of keeping one."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: List[LayerSpec]
    final_norm: PartSpec
    head: PartSpec
    schedule: List[Run] = field(default_factory=list)

    def __post_init__(self):
        if not self.schedule:
            self.schedule = [Run(i) for i in range(len(self.layers))]
        for n, run in enumerate(self.schedule):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"schedule entry {n} names layer {run.layer} of {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < n:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {run.cache_of}, "
                                     "which does not run before it")
                if self.schedule[run.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {n} reads the cache of entry {run.cache_of}, "
                                     "which keeps none of its own")
