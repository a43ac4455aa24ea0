from .batch import GroupStep, StepContext, StepEntry, Workspace
from .runner import ModelRunner

__all__ = ["GroupStep", "ModelRunner", "StepContext", "StepEntry", "Workspace"]
