"""Inference and rollout utilities (public names of ``rwkvtune/inference/__init__.py:5-52``)."""
from .batch_generator import BatchGenerator, GenerationConfig
from .core import TokenSampler
from .generator import TextGenerator
from .grpo_batch_generator import GRPOBatchGenerator
from .pipeline import InferencePipeline
from .scheduler_core import SchedulerCore, SeqStatus, SequenceState, create_scheduler_core
from .state_cache import AutoConfig, CacheConfig, CacheLevel, CacheStats, StateCache, create_state_cache
from .structured_output import JsonObjectEnforcer, JsonSchemaEnforcer, create_enforcer, is_structured_output_available

__all__ = ["InferencePipeline", "TextGenerator", "BatchGenerator", "GenerationConfig", "GRPOBatchGenerator", "TokenSampler",
           "SchedulerCore", "SequenceState", "SeqStatus", "create_scheduler_core", "JsonSchemaEnforcer",
           "JsonObjectEnforcer", "create_enforcer", "is_structured_output_available", "StateCache", "CacheConfig",
           "CacheLevel", "CacheStats", "AutoConfig", "create_state_cache"]
