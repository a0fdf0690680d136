from .step import ModelRunner, StepContext, StepEntry, StepError

__all__ = ["ModelRunner", "StepContext", "StepEntry", "StepError"]
