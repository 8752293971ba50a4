from .runner import ModelRunner, StepContext, StepEntry, StepInputError

__all__ = ["ModelRunner", "StepContext", "StepEntry", "StepInputError"]
