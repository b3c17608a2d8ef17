# importing the modules registers the built-in parts
from . import (attention, block, conv_attention, experts, feed_forward, latent_attention, linear_state,  # noqa: F401
               norm, position, token_side)
from .base import (
    BuildContext,
    ParamSpec,
    Part,
    ResidualStream,
    StepContext,
    build_part,
    register_part,
    unregister_part,
)
from .model import DecoderModel

__all__ = [
    "BuildContext",
    "DecoderModel",
    "ParamSpec",
    "Part",
    "ResidualStream",
    "StepContext",
    "build_part",
    "register_part",
    "unregister_part",
]
