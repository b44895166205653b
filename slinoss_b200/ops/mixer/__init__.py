"""Mixer-level operators: in_proj split and the gated RMSNorm tail."""

from .projection import split_mixer_projection
from .tail import mixer_tail, mixer_gated_norm

__all__ = ["split_mixer_projection", "mixer_tail", "mixer_gated_norm"]
