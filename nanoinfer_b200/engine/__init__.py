from .runner import BadToken, ContextFull, ModelRunner, StepError, StepItem, TooManyRows

__all__ = ["BadToken", "ContextFull", "ModelRunner", "StepError", "StepItem", "TooManyRows"]
