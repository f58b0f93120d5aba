"""The parts layers are made of.  Importing the package registers the built-in ones."""
from . import attention, block, embedding, ffn, norm, rope, shortconv  # noqa: F401
from .base import (BuildEnv, FeedForward, KVSpec, LayerSpec, Mixer, ModelPlan, Part, PartSpec,  # noqa: F401
                   ScheduleEntry, StateSpec, TensorSpec)
