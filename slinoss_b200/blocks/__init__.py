"""Blocks and stacks built around the CUDA-backed SLinOSS mixer."""

from .block import SLinOSSBlock
from .config import (SLinOSSBlockConfig, SLinOSSMLPConfig, SLinOSSMixerConfig, SLinOSSStackConfig,
                     sandwich_block_schedule, scaled_budget_schedule, uniform_block_schedule)
from .stack import SLinOSSStack
from .state import SLinOSSBlockState, SLinOSSStackState

__all__ = ["SLinOSSBlock", "SLinOSSBlockConfig", "SLinOSSBlockState", "SLinOSSMLPConfig",
           "SLinOSSMixerConfig", "SLinOSSStack", "SLinOSSStackConfig", "SLinOSSStackState",
           "sandwich_block_schedule", "scaled_budget_schedule", "uniform_block_schedule"]
