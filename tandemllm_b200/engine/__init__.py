"""The step function, the scheduler above it, and the Python entry point."""

from .engine import Engine, EngineArgs
from .scheduler import Request, Scheduled, Scheduler
from .step import KernelFault, StepEntry, StepFunction

__all__ = ["Engine", "EngineArgs", "Request", "Scheduled", "Scheduler", "KernelFault", "StepEntry", "StepFunction"]
