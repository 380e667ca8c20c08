"""Parts a layer is put together from. Importing the package registers the
built-in ones."""
from .base import (Block, CacheView, Embedding, FeedForward, Head, KVRequest, Mixer, Norm, Part, PositionEncoding,
                   Residual, StateRequest, TensorSpec, build_part, known_parts, register_block,
                   register_embedding, register_ffn, register_head, register_mixer, register_norm,
                   register_position)
from . import (attention, attention_projnorm, block, block_postnorm, delta, embedding, feedforward,  # noqa: F401
               feedforward_dense, mamba, norms, norms_layer, position)                                  # (registration)
from .embedding import LinearHead, TokenEmbedding
