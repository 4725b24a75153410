from .batch import BatchError, StepEntry, pack_step
from .step import ModelRunner
from .loading import build_model, load_runner
from .scheduler import Request, Scheduled, Scheduler
from .engine import Engine

__all__ = ["BatchError", "StepEntry", "pack_step", "ModelRunner", "build_model", "load_runner",
           "Request", "Scheduled", "Scheduler", "Engine"]
