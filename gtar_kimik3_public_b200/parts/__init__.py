"""Parts of a model: norms, position encodings, mixers, feed-forwards, blocks, embedding and head.
Importing the package registers the built-in parts."""

from . import (  # noqa: F401
    attention, block, delta_rule, embedding, experts, latent_attention, linear_attention, mlp, norms, rope, scored_attention,
    side_by_side, wide_norm_attention,
)
from .base import (  # noqa: F401
    Block, FeedForward, KVRequest, Mixer, Norm, Part, PositionEncoding, RowsRequest, StateRequest, StepContext, TensorSpec,
    build_part, known_parts, register_part,
)
