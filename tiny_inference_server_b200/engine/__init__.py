from .batch import StepContext, StepEntry, build_step
from .runner import DeviceFault, ModelRunner

__all__ = ["StepContext", "StepEntry", "build_step", "DeviceFault", "ModelRunner"]
