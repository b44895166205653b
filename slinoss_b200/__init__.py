"""slinoss_b200: the SLinOSS v2x2ssd scan and its mixer hot path on B200 (sm_100a).

Module tree mirrors the reference package for the parts it replaces:
``slinoss_b200.ops.v2x2ssd``, ``slinoss_b200.ops.scanprep``, ``slinoss_b200.ops.mixer``,
``slinoss_b200.layers`` and ``slinoss_b200.blocks``.  Every operator launches
hand-written CUDA kernels through the C ABI of ``include/slinoss_b200.h``; there is
no CPU path and no fallback when the library is missing.
"""

from .blocks import (SLinOSSBlock, SLinOSSBlockConfig, SLinOSSMixerConfig, SLinOSSStack,
                     SLinOSSStackConfig)
from .layers import (RMSNorm, ScanState, SLinOSSMixer, SLinOSSMixerState, SLinOSSMLP,
                     SLinOSSMLPConfig, SLinOSSScanPrep)

__version__ = "0.1.0"

__all__ = ["RMSNorm", "ScanState", "SLinOSSBlock", "SLinOSSBlockConfig", "SLinOSSMixer",
           "SLinOSSMixerConfig", "SLinOSSMixerState", "SLinOSSMLP", "SLinOSSMLPConfig",
           "SLinOSSScanPrep", "SLinOSSStack", "SLinOSSStackConfig"]
