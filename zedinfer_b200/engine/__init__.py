from .core import EngineCore, StepEntry
from .engine import InferenceEngine, RequestFuture
from .model import Model
from .request import GenerationResult, GenerationStats, InferenceRequest, RequestPhase
from .scheduler import ScheduledBatch, Scheduler

__all__ = ["EngineCore", "StepEntry", "InferenceEngine", "RequestFuture", "Model", "GenerationResult",
           "GenerationStats", "InferenceRequest", "RequestPhase", "ScheduledBatch", "Scheduler"]
