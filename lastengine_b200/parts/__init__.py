"""The parts layers are made of.  Importing the package registers the built-in ones."""
from . import (attention, block, composite, embedding, ffn, gate, gated_scan, latent_attention, mixed_attention,  # noqa: F401
               norm, pooled_attention, recurrent, retention, rope, shortconv)  # noqa: F401
from .base import (BuildEnv, FeedForward, KVSpec, LatentSpec, LayerSpec, Mixer, ModelPlan, Part, PartSpec,  # noqa: F401
                   ScheduleEntry, StateSpec, StreamAdd, TensorSpec)
