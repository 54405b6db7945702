"""The step function, the scheduler above it, and the Python entry point."""
from .context import Span, StepContext, Workspace
from .engine import Engine, Generation, build_model, load_model, parse_dtype, random_model
from .scheduler import Planned, Request, RequestError, Scheduler, StopReason
from .step import Runner, StepEntry, StepError

__all__ = ["Span", "StepContext", "Workspace", "Engine", "Generation", "build_model", "load_model", "parse_dtype",
           "random_model", "Planned", "Request", "RequestError", "Scheduler", "StopReason", "Runner", "StepEntry",
           "StepError"]
