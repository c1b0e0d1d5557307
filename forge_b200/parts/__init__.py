from .base import (CATEGORIES, CompositeCacheSpec, KVCacheSpec, Part, Runtime, StateSpec, build_part, register_part, registered_parts,
                   unregister_part)
from . import (attention, block, embedding, feedforward, headmix_attention, latent_attention, norm, position,  # noqa: F401  (register
               recurrent, routed, scored_attention, side_by_side)                                            # the built-in parts)
from .block import build_block
from .linear import Linear

__all__ = ["CATEGORIES", "CompositeCacheSpec", "KVCacheSpec", "StateSpec", "Part", "Runtime", "Linear", "build_part", "build_block",
           "register_part", "registered_parts", "unregister_part"]
