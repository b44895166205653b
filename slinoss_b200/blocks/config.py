"""Typed configuration of blocks and stacks (field-for-field the reference's
dataclasses, slinoss/blocks/config.py:23-163, so configs are interchangeable)."""

from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Literal

from ..layers.mlp import SLinOSSMLPConfig

NormKind = Literal["rmsnorm", "layernorm"]
FinalNormKind = Literal["rmsnorm", "layernorm", "none"]


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


@dataclass(frozen=True, slots=True)
class SLinOSSMixerConfig:
    d_state: int = 128
    expand: float = 2.0
    d_head: int = 64
    d_conv: int = 4
    chunk_size: int = 64
    bc_groups: int | None = None
    dt_min: float = 5.0e-3
    dt_max: float = 1.0e-1
    dt_init_floor: float = 5.0e-3
    alpha_min: float = 0.0
    alpha_max: float = 20.0
    theta_init_min: float = 0.05
    theta_init_max: float = 2.0
    theta_mod_scale: float = 1.0
    r_min: float = 0.8
    r_max: float = 1.0
    eps: float = 1.0e-8

    def __post_init__(self) -> None:
        for name in ("d_state", "expand", "d_head", "d_conv", "chunk_size"):
            _require(getattr(self, name) > 0, f"{name} must be positive. Got {getattr(self, name)}.")
        if self.bc_groups is not None:
            _require(self.bc_groups > 0, f"bc_groups must be positive. Got {self.bc_groups}.")
        _require(0.0 <= self.alpha_min < self.alpha_max,
                 "alpha_min/alpha_max must satisfy 0 <= min < max. Got "
                 f"{self.alpha_min}, {self.alpha_max}.")
        _require(self.theta_mod_scale >= 0.0,
                 f"theta_mod_scale must be non-negative. Got {self.theta_mod_scale}.")

    def build_kwargs(self) -> dict[str, object]:
        return asdict(self)


@dataclass(frozen=True, slots=True)
class SLinOSSBlockConfig:
    d_model: int
    mixer: SLinOSSMixerConfig = field(default_factory=SLinOSSMixerConfig)
    ffn: SLinOSSMLPConfig | None = field(default_factory=SLinOSSMLPConfig)
    norm_kind: NormKind = "rmsnorm"
    norm_eps: float = 1.0e-5
    residual_in_fp32: bool = True
    residual_dropout: float = 0.0

    def __post_init__(self) -> None:
        _require(self.d_model > 0, f"d_model must be positive. Got {self.d_model}.")
        _require(self.norm_kind in ("rmsnorm", "layernorm"), f"Unsupported norm_kind: {self.norm_kind!r}.")
        _require(self.norm_eps > 0.0, f"norm_eps must be positive. Got {self.norm_eps}.")
        _require(0.0 <= self.residual_dropout < 1.0,
                 f"residual_dropout must lie in [0, 1). Got {self.residual_dropout}.")


def uniform_block_schedule(block: SLinOSSBlockConfig, *, n_layers: int):
    _require(n_layers > 0, f"n_layers must be positive. Got {n_layers}.")
    return tuple(block for _ in range(n_layers))


def sandwich_block_schedule(*, stem, middle, tail, n_layers: int):
    _require(n_layers > 0, f"n_layers must be positive. Got {n_layers}.")
    if n_layers <= 2:
        return (stem, tail)[:n_layers]
    return (stem, *(middle for _ in range(n_layers - 2)), tail)


def _lerp(a: float, b: float, i: int, n: int) -> float:
    return float(a) if n <= 1 else float(a + (b - a) * i / (n - 1))


def scaled_budget_schedule(base: SLinOSSBlockConfig, *, n_layers: int, mixer_expand_range=None,
                           ffn_expand_range=None, residual_dropout_range=None):
    """Linearly interpolates mixer expand, FFN expand and residual dropout over depth."""
    _require(n_layers > 0, f"n_layers must be positive. Got {n_layers}.")
    if ffn_expand_range is not None and base.ffn is not None:
        _require(base.ffn.hidden_dim is None,
                 "scaled_budget_schedule can only scale FFN expand when base.ffn.hidden_dim is not fixed.")
    out = []
    for i in range(n_layers):
        mixer, ffn, drop = base.mixer, base.ffn, base.residual_dropout
        if mixer_expand_range is not None:
            mixer = replace(mixer, expand=_lerp(*mixer_expand_range, i, n_layers))
        if ffn_expand_range is not None and ffn is not None:
            ffn = replace(ffn, expand=_lerp(*ffn_expand_range, i, n_layers))
        if residual_dropout_range is not None:
            drop = _lerp(*residual_dropout_range, i, n_layers)
        out.append(replace(base, mixer=mixer, ffn=ffn, residual_dropout=drop))
    return tuple(out)


@dataclass(frozen=True, slots=True)
class SLinOSSStackConfig:
    blocks: tuple[SLinOSSBlockConfig, ...]
    final_norm_kind: FinalNormKind = "rmsnorm"
    final_norm_eps: float = 1.0e-5
    gradient_checkpointing: bool = False

    def __post_init__(self) -> None:
        _require(bool(self.blocks), "SLinOSSStackConfig requires at least one block.")
        d_model = self.blocks[0].d_model
        for i, blk in enumerate(self.blocks[1:], start=1):
            _require(blk.d_model == d_model,
                     "All block configs in a stack must share d_model. "
                     f"Block 0 has {d_model}, block {i} has {blk.d_model}.")
        _require(self.final_norm_kind in ("rmsnorm", "layernorm", "none"),
                 f"Unsupported final_norm_kind: {self.final_norm_kind!r}.")
        _require(self.final_norm_eps > 0.0, f"final_norm_eps must be positive. Got {self.final_norm_eps}.")

    @property
    def d_model(self) -> int:
        return self.blocks[0].d_model

    @classmethod
    def uniform(cls, block: SLinOSSBlockConfig, *, n_layers: int,
                final_norm_kind: FinalNormKind = "rmsnorm", final_norm_eps: float = 1.0e-5,
                gradient_checkpointing: bool = False) -> "SLinOSSStackConfig":
        return cls(blocks=uniform_block_schedule(block, n_layers=n_layers),
                   final_norm_kind=final_norm_kind, final_norm_eps=final_norm_eps,
                   gradient_checkpointing=gradient_checkpointing)


__all__ = ["FinalNormKind", "NormKind", "SLinOSSBlockConfig", "SLinOSSMLPConfig",
           "SLinOSSMixerConfig", "SLinOSSStackConfig", "sandwich_block_schedule",
           "scaled_budget_schedule", "uniform_block_schedule"]
