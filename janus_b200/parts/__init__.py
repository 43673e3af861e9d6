from . import (attention, block, capped_attention, connection, delta_rule, diff_attention, feedforward,  # noqa: F401
               gated_linear, latent_attention, lightning, mamba2, norm, parallel, rope, routed, shared_kv_attention, transforms)      # (registers the built-in kinds)
from .base import (Connection, FeedForward, KVSpec, LayerSpec, Mixer, ModelSpec, Norm, Part, PartSpec,
                   PositionEncoding, ScheduleEntry, StateSpec, make_part, register_part,
                   registered_parts)

__all__ = [
    "Connection", "FeedForward", "KVSpec", "LayerSpec", "Mixer", "ModelSpec", "Norm", "Part", "PartSpec",
    "PositionEncoding", "ScheduleEntry", "StateSpec", "make_part", "register_part", "registered_parts",
]
