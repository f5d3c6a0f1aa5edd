"""Parts a model is put together from; importing this package registers the built-in kinds."""
from . import (attention, block, capped_attention, channel_delta, embedding, gated_delta, gated_linear, latent_attention, mlp, moe, norm, rotary,  # noqa: F401
               side_by_side, ssd, wkv)  # noqa: F401  (registration)
from .base import Part, StepContext, TensorWant, build_part, register_part  # noqa: F401
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry  # noqa: F401
