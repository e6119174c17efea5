"""The parts a model is assembled from.  Importing the package registers the built-in kinds."""
from . import (attention, block, conv_attention, delta_rule, distance_attention, feedforward, gated_recurrence,  # noqa: F401
               latent_attention, matrix_memory, norm, position, rotated_attention, routed_experts, selective_scan, side_by_side, sink_attention)
from .base import (BLOCKS, Block, EMBEDDING, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, ROTATION,  # noqa: F401
                   CacheNeed, ModelContext, Rotation, Part, StepContext, Workspace, register_block, register_feed_forward,
                   register_mixer, register_norm, register_position_encoding)
