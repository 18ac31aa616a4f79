from .step import StepEntry, StepError, StepRunner

__all__ = ["StepEntry", "StepError", "StepRunner"]
