from .base import (BatchAnnotation, CacheBinding, CacheNeed, GatedDelta, GroupView, KVNeed, ResidualStream, Runtime, ScaledTerms, StateNeed,
                   StepContext, build_part, part_class, register_part, registered)
from . import attention, block, embedding, feed_forward, latent_attention, norm, parallel, position, recurrent  # register the parts
from .linear import Linear
from .model import DecoderModel, declared_tensors

__all__ = ["BatchAnnotation", "CacheBinding", "CacheNeed", "DecoderModel", "GatedDelta", "GroupView", "KVNeed", "Linear",
           "ResidualStream", "Runtime", "ScaledTerms", "StateNeed", "StepContext", "build_part",
           "declared_tensors", "part_class", "register_part", "registered"]
