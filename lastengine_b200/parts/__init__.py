"""The parts layers are made of.  Importing the package registers the built-in ones."""
from . import (attention, block, embedding, ffn, gate, latent_attention, norm, pooled_attention, recurrent,  # noqa: F401
               retention, rope, shortconv)  # noqa: F401
from .base import (BuildEnv, FeedForward, KVSpec, LatentSpec, LayerSpec, Mixer, ModelPlan, Part, PartSpec,  # noqa: F401
                   ScheduleEntry, StateSpec, StreamAdd, TensorSpec)
