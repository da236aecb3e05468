from .loading import LoadedModel, build_model, load_model
from .public import CacheConfig, Engine, EngineRequestHandle
from .replay import Replay
from .runner import Runner, StepEntry
from .scheduler import (BatchingConfig, Phase, QueueFullError, Request, RequestTimeoutError,
                        Scheduled, Scheduler)

__all__ = ["LoadedModel", "build_model", "load_model", "CacheConfig", "Engine",
           "EngineRequestHandle", "Replay", "Runner", "StepEntry", "BatchingConfig", "Phase",
           "QueueFullError", "Request", "RequestTimeoutError", "Scheduled", "Scheduler"]
