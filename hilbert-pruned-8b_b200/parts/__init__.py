from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, BuildContext,
                   CacheNeed, FeedForward, Mixer, Norm, ParamSpec, Part, PositionEncoding, Registry, StateNeed, TOKEN_FILTERS, TokenFilter)
from . import (attention, block, decay_memory, dense_ffn, dyt, embedding, head_memory, latent_attention, layernorm, mlstm, moe, parallel, pool_attention, rmsnorm, rope,  # noqa: F401
               selective_scan, short_conv, sink_attention, swiglu)  # noqa: F401  (register the built-in parts)
from .block import Block

__all__ = ["Block", "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS",
           "BuildContext", "CacheNeed", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part", "PositionEncoding",
           "Registry", "StateNeed", "TOKEN_FILTERS", "TokenFilter"]
