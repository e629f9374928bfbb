from . import attention, embedding, rmsnorm, rope, shortconv, swiglu  # noqa: F401  (registers the parts)
from .base import (EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Embedding,
                   FeedForward, FixedState, Head, Mixer, Norm, PagedKV, ParamDecl, Part, PositionEncoding,
                   build_part, register_part)
from .spec import LayerSpec, ModelSpec, PartSpec, Run
