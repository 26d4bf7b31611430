"""Model assembly, the step function, the generation loop, replay and the entry point."""

from .engine import Engine
from .generate import BatchLimits, GenerationError, Generator, plan_batches
from .session import Session
from .step import StepEntry, StepError, Stepper

__all__ = ["Engine", "BatchLimits", "GenerationError", "Generator", "plan_batches", "Session", "StepEntry",
           "StepError", "Stepper"]
