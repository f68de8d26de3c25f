"""Parts a layer is put together from, and their registries."""
from . import attention, block, embedding, ffn, norm, position  # noqa: F401  (register the built-in parts)
from .base import BuildContext, KVRequest, ResidualStream, StateRequest
from .registry import (arrangement_class, embedding_class, feed_forward_class, head_class, mixer_class, norm_class,
                       position_class, register_arrangement, register_embedding, register_feed_forward,
                       register_head, register_mixer, register_norm, register_position, unregister)
from .spec import (EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerSpec, MixerSpec, ModelPlan, NormSpec,
                   PositionSpec, ScheduleEntry)
