"""Parts a model is put together from.  Importing the package registers the built-in kinds."""
from . import (attention, block, delta, embedding, hyper, latent, linear_state, matrix_memory, mlp, moe,  # noqa: F401
               norm, norm_attention, reentry, rope, selective_state, window_attention)                # (registration)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, CacheView, Embedding,
                   FeedForward, GroupView, Head, Mixer, Norm, Part, PositionEncoding, StepContext, lookup,
                   register_part)
from .spec import (CacheParts, FixedState, LayerCall, LayerSpec, ModelBlueprint, PagedKV, PagedLatent, PartSpec, Reentry,
                   TensorSpec)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "CacheView",
           "Embedding", "FeedForward", "GroupView", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "StepContext", "lookup", "register_part", "CacheParts", "FixedState", "LayerCall", "LayerSpec", "ModelBlueprint",
           "PagedKV", "PagedLatent", "PartSpec", "Reentry", "TensorSpec"]
