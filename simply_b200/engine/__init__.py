"""Engine: step function, scheduler, generation and trace replay."""

from simply_b200.engine.batch import StepContext, StepEntry
from simply_b200.engine.engine import Engine, GenerationResult
from simply_b200.engine.scheduler import Request, Scheduler, Status

__all__ = ["Engine", "GenerationResult", "Request", "Scheduler", "Status", "StepContext",
           "StepEntry"]
