"""Layer parts and their registries.  Importing this package registers the built-in kinds."""
from .base import Part, TensorDecl
from .registry import (build_block, build_embedding, build_feed_forward, build_mixer, build_norm, build_position,
                       register_block, register_embedding, register_feed_forward, register_mixer, register_norm,
                       register_position, registered)
from . import (norm, position, attention, feedforward, embedding, recurrent, latent_attention,  # noqa: F401  (registration)
               experts, state_space)
from .block import Block, PostNormBlock, PreNormBlock, SandwichBlock, ScaledParts
from .norm import NormedDelta, StreamCopy
from .linear import Linear
from .position import PositionEncoding

__all__ = ["Part", "TensorDecl", "Block", "PreNormBlock", "SandwichBlock", "NormedDelta", "StreamCopy", "PostNormBlock", "ScaledParts", "Linear", "PositionEncoding",
           "build_block", "build_embedding", "build_feed_forward", "build_mixer", "build_norm", "build_position",
           "register_block", "register_embedding", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "registered"]
