from .engine import Engine, build_runner, generate
from .replay import TraceReplayer, replay_stream
from .request import GenerationResult, Request, StepRecord
from .scheduler import Scheduler, StepPlan
from .step import ModelRunner, PagedKVBinding, StateBinding, StepContext, StepEntry

__all__ = ["Engine", "build_runner", "generate", "TraceReplayer", "replay_stream", "GenerationResult", "Request",
           "StepRecord", "Scheduler", "StepPlan", "ModelRunner", "PagedKVBinding", "StateBinding", "StepContext", "StepEntry"]
