from . import (attention, block, differential_attention, embedding, feed_forward, head,  # noqa: F401  (register)
               latent_attention, linear_recurrence, matrix_memory, norms, positions, retention,
               side_by_side, time_mix, window_attention)
from .interfaces import (Block, Embedding, FeedForward, Head, KVSpec, LayerCache, Mixer, Norm,
                         PositionEncoding, StateSpec)
from .linear import Linear
from .registry import build_part, part_factory, register_part, registered_parts

__all__ = ["Block", "Embedding", "FeedForward", "Head", "KVSpec", "LayerCache", "Mixer", "Norm",
           "PositionEncoding", "StateSpec", "Linear", "build_part", "part_factory",
           "register_part", "registered_parts"]
