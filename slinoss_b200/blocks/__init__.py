"""Blocks and stacks built around the CUDA-backed SLinOSS mixer.

``SLinOSSBlock`` is a pre-norm residual block (mixer branch, optional FFN branch); ``SLinOSSStack`` a sequence of
blocks with a final norm; the ``*Config`` records and the three schedule helpers describe them; the ``*State``
records carry the streaming state of the mixers for segmented training and decoding.  On CUDA the norms, the
FFN activation and (optionally) the whole FFN branch run on this package's row kernels, see ``ops.block``.
"""

from .block import SLinOSSBlock
from .config import (SLinOSSBlockConfig, SLinOSSMixerConfig, SLinOSSMLPConfig, SLinOSSStackConfig,
                     sandwich_block_schedule, scaled_budget_schedule, uniform_block_schedule)
from .stack import SLinOSSStack
from .state import SLinOSSBlockState, SLinOSSStackState

__all__ = [
    "SLinOSSBlock", "SLinOSSStack",
    "SLinOSSBlockConfig", "SLinOSSStackConfig", "SLinOSSMixerConfig", "SLinOSSMLPConfig",
    "SLinOSSBlockState", "SLinOSSStackState",
    "uniform_block_schedule", "sandwich_block_schedule", "scaled_budget_schedule",
]
