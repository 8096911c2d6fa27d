from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS,
                   Arrangement, CacheNeed, Embedding, FeedForward, Head, LayerBinding, Mixer, Norm,
                   Part, PositionEncoding, TensorDecl)
from . import (norm, rope, attention, swiglu, block, embedding, branch, sink_attention,  # noqa: F401
               recurrent, polynorm, hyper, latent_attention, moe)                                          # (register kinds)
