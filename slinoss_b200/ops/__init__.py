"""CUDA operators of the SLinOSS mixer hot path (sm_100a)."""

from .v2x2ssd import v2x2ssd, v2x2ssd_cute, v2x2ssd_decode
from .scanprep import scanprep_b200, conv_scanprep_b200, causal_conv_silu_b200
from .mixer import mixer_tail, split_mixer_projection

__all__ = ["v2x2ssd", "v2x2ssd_cute", "v2x2ssd_decode", "scanprep_b200", "conv_scanprep_b200",
           "causal_conv_silu_b200", "mixer_tail", "split_mixer_projection"]
