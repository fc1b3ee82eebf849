from . import attention, block, delta_rule, embedding, feed_forward, gated_attention, hyper, latent_attention, mingru, mixed_attention, norms, parallel, positions, shaped_attention, wkv  # noqa: F401  (register parts)
from .base import (
    CacheSpecs,
    KVCacheSpec,
    Part,
    PartSpec,
    StateSpec,
    build_part,
    register_part,
    registered_parts,
)
from .context import CacheView, HostBatch, StepContext, Workspace
from .model import LayerCall, Model, ModelRecipe

__all__ = [
    "CacheSpecs",
    "CacheView",
    "HostBatch",
    "KVCacheSpec",
    "LayerCall",
    "Model",
    "ModelRecipe",
    "Part",
    "PartSpec",
    "StateSpec",
    "StepContext",
    "Workspace",
    "build_part",
    "register_part",
    "registered_parts",
]
