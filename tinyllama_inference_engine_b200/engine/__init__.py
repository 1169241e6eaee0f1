from .batch import StepContext, StepEntry

__all__ = ["StepContext", "StepEntry"]
