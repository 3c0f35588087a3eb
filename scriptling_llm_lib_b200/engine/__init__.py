from .layout import ModelLayout, ScheduleEntry, sequential_schedule
from .model import DecoderModel
from .step import DTYPES, Engine, Sequence, StepContext, StepEntry, StepError

__all__ = ["ModelLayout", "ScheduleEntry", "sequential_schedule", "DecoderModel", "Engine", "Sequence", "StepContext",
           "StepEntry", "StepError", "DTYPES"]
