"""Parts of a model: embeddings, norms, mixers, feed-forwards, position encodings, heads and the arrangements
of a block, each behind a registry."""
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, INPUT_FILTERS, JOINTS, MIXERS, NORMS, POSITIONS, CacheNeed,
                   Embedding, FeedForward, Head, InputFilter, Joint, Mixer, Norm, NormedDelta, PairDelta, ParamDecl, Part,
                   Position, StateNeed, WeightedRows)
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from . import attention, block, channel_delta, ends, feed_forward, latent_attention, mlstm, norm, rope, stream  # noqa: F401  (registers the built-in kinds)
