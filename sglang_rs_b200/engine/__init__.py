from .runner import ModelRunner, StepContext, StepEntry, StepInputError, StepPlanner
from .scheduler import Request, ScheduledEntry, Scheduler, SchedulerConfig, StepOutput

__all__ = ["ModelRunner", "StepContext", "StepEntry", "StepInputError", "StepPlanner", "Request", "ScheduledEntry", "Scheduler",
           "SchedulerConfig", "StepOutput", "Engine"]


def __getattr__(name):
    if name == "Engine":
        from .engine import Engine
        return Engine
    raise AttributeError(name)
