"""zedinfer_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) to generated tokens: typed configuration and an
architecture registry, weights bound by name, layers assembled from parts, a paged cache manager,
one step function, a continuous-batching scheduler, sampling, and hand-written CUDA kernels.
"""
from .config import GenerationConfig, SchedulerConfig

__version__ = "0.1.0"


def __getattr__(name):
    # the engine classes import torch and the kernels; load them on first use
    if name in ("InferenceEngine", "InferenceRequest", "EngineCore", "StepEntry", "GenerationResult"):
        from . import engine
        return getattr(engine, name)
    raise AttributeError(name)


__all__ = ["GenerationConfig", "SchedulerConfig", "InferenceEngine", "InferenceRequest", "EngineCore", "StepEntry",
           "GenerationResult", "__version__"]
