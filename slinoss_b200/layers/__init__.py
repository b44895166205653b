"""Layers of the SLinOSS mixer path (CUDA-backed)."""

from .backend import (B200CConv1dBackend, B200MixerDecodeBackend, B200ScanBackend,
                      B200ScanPrepBackend, CConv1dBackend, MixerDecodeBackend, MixerDecodeInputs,
                      ScanBackend, ScanInputs, ScanPrepBackend, ScanPrepInputs)
from .mixer import SLinOSSMixer
from .mlp import SLinOSSMLP, SLinOSSMLPConfig
from .norm import RMSNorm
from .scanprep import SLinOSSScanPrep
from .state import ScanState, SLinOSSMixerState

__all__ = ["B200CConv1dBackend", "B200MixerDecodeBackend", "B200ScanBackend",
           "B200ScanPrepBackend", "CConv1dBackend", "MixerDecodeBackend", "MixerDecodeInputs",
           "ScanBackend", "ScanInputs", "ScanPrepBackend", "ScanPrepInputs", "SLinOSSMixer",
           "SLinOSSMLP", "SLinOSSMLPConfig", "RMSNorm", "SLinOSSScanPrep", "ScanState",
           "SLinOSSMixerState"]
