"""omniserver_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

One architecture (the Qwen2 text decoder of Qwen2-VL), from a model folder to generated tokens:
typed configuration and registry, weights by tensor name, layers put together from parts, a paged
cache with page groups and per-request state slots, one step function for mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels.  The public names follow
omniserve/__init__.py:7-23.
"""

from .config import EngineConfig
from .engine import (LLMEngine, ModelRunner, Request, SamplingParams, Scheduler, SchedulerConfig, Sequence, Status,
                     StepDelta, StepEntry, build_runner)

__all__ = ["LLMEngine", "StepDelta", "ModelRunner", "Request", "SamplingParams", "Sequence", "Status", "Scheduler",
           "SchedulerConfig", "EngineConfig", "StepEntry", "build_runner"]
__version__ = "0.1.0"
