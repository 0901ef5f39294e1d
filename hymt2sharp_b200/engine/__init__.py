from .spec import ModelSpec, Run
from .model import DecoderModel
from .engine import Engine, EngineError, StepEntry

__all__ = ["ModelSpec", "Run", "DecoderModel", "Engine", "EngineError", "StepEntry"]
