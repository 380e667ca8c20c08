"""Parts a layer is put together from. Importing the package registers the
built-in ones."""
from .base import (Block, CacheView, Embedding, FeedForward, Head, KVRequest, Mixer, Norm, Part, PositionEncoding,
                   Residual, StateRequest, TensorSpec, build_part, known_parts, register_block,
                   register_embedding, register_ffn, register_head, register_mixer, register_norm,
                   register_position)
from . import (attention, attention_latent, attention_projnorm, block, block_postnorm, delta, embedding,  # noqa: F401
               feedforward, feedforward_dense, feedforward_routed, mamba, norms, norms_layer, position,  # (registration)
               retention)
from .embedding import LinearHead, TokenEmbedding
