"""Parts a decoder is assembled from.  Importing the package registers the built-in kinds."""

from .base import (Block, FeedForward, LayerCall, LayerSpec, Mixer, ModelPlan, Norm, NormedUpdate, Part, PartSpec,
                   PositionEncoding, StreamCall, StreamOp, WeightSpec, build_part, register_part, registered,
                   settle_update)
from . import (attention, block, embedding, glu, latent_attention, layernorm, reentry, rmsnorm, rope, ssd,  # noqa: F401
               swiglu)                                                                       # (registration)

__all__ = ["Block", "FeedForward", "LayerCall", "LayerSpec", "Mixer", "ModelPlan", "Norm", "NormedUpdate", "Part",
           "PartSpec", "PositionEncoding", "StreamCall", "StreamOp", "WeightSpec", "build_part", "register_part",
           "registered", "settle_update"]
