from .base import (LayerCache, Mixer, Part, StateNeed, build_part, register_part,
                   registered_parts, unregister_part)
from . import norm, rope, attention, mlp, block   # registers the built-in kinds
from .model import DecoderModel, tensor_specs

__all__ = ["LayerCache", "Mixer", "Part", "StateNeed", "build_part", "register_part",
           "registered_parts", "unregister_part", "DecoderModel", "tensor_specs"]
