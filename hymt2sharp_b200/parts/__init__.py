from .base import (CATEGORIES, MixerSlot, PartSpec, Prenormed, RotaryEpilogue, StepContext, build_part, register_part)
from . import norm, rope, attention, swiglu, block  # noqa: F401  (registers the built-in kinds)
from .linear import Linear, compute_form, matmul

__all__ = ["CATEGORIES", "MixerSlot", "PartSpec", "Prenormed", "RotaryEpilogue", "StepContext", "build_part", "register_part", "Linear",
           "compute_form", "matmul"]
