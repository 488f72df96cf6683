from .step import ModelRunner, OutOfPages, StepEntry

__all__ = ["ModelRunner", "OutOfPages", "StepEntry"]
