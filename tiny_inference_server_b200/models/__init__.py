"""Registered architectures."""
from .base import Model, ScheduleEntry, StepOutput
from . import gqa_mtp  # noqa: F401  (registers "gqa_mtp_transformer")

__all__ = ["Model", "ScheduleEntry", "StepOutput"]
