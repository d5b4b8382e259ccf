"""Parts of a model; importing the package registers the built-in ones."""
from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, PagedKVSpec, StateSpec, NormedActivations,
                   ResidualSink, CastActivations, StreamWrite,
                   register_part, make_part, part_factory, registered_parts)
from . import norm, rope, attention, mlp, block, embedding, linear_attention, diff_attention, delta_rule, wkv, latent_attention, moe, sigmoid_attention, softmax_attention, side_by_side  # noqa: F401  (registration)
