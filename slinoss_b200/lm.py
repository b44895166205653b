"""Causal language-model shell around ``SLinOSSStack`` and its data-parallel training step.

Token embedding -> ``SLinOSSStack`` -> tied output head, cross-entropy on shifted ids: the shape of
the reference's performance harness (scripts/perf/_training_model.py:204-252, minus its positional
table: the configuration this package is benchmarked on feeds the stack with token embeddings
only) and of its example (examples/blocks_lm.py:18-55).  The stack itself calls the CUDA kernels
of this package; embedding, head and loss are library calls (torch).
"""

from __future__ import annotations

import torch
from torch import nn
from torch.nn import functional as F

from . import shard
from .blocks import SLinOSSBlockConfig, SLinOSSMixerConfig, SLinOSSStack, SLinOSSStackConfig
from .layers import SLinOSSMLPConfig


def lm_stack_config(d_model: int = 2048, n_layers: int = 24, d_state: int = 64, d_head: int = 64,
                    ffn_expand: float = 4.0) -> SLinOSSStackConfig:
    """The stacked-LM benchmark configuration: ``n_layers`` blocks of mixer (inner width = model
    width, ``d_model / d_head`` heads) + GELU MLP of ``ffn_expand`` x, RMSNorm everywhere."""
    block = SLinOSSBlockConfig(
        d_model=d_model,
        mixer=SLinOSSMixerConfig(d_state=d_state, expand=1.0, d_head=d_head, chunk_size=64),
        ffn=SLinOSSMLPConfig(kind="gelu", expand=ffn_expand))
    return SLinOSSStackConfig.uniform(block, n_layers=n_layers)


class SLinOSSLM(nn.Module):
    """``ids (batch, T) -> logits (batch, T, vocab)``; the head shares the embedding matrix."""

    def __init__(self, vocab_size: int, stack_config: SLinOSSStackConfig, *, init_std: float = 0.02,
                 device=None, dtype=None) -> None:
        super().__init__()
        self.vocab_size, self.d_model = int(vocab_size), int(stack_config.d_model)
        self.token_embed = nn.Embedding(vocab_size, self.d_model, device=device, dtype=dtype)
        self.backbone = SLinOSSStack(stack_config, device=device, dtype=dtype)
        self.init_std = init_std
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Random init with one standard deviation for the embedding and every Linear weight;
        the mixer's own parameters (skip, conv, scan-preparation biases) keep their init."""
        nn.init.normal_(self.token_embed.weight, mean=0.0, std=self.init_std)
        for m in self.backbone.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, mean=0.0, std=self.init_std)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        if ids.ndim != 2:
            raise ValueError(f"Expected ids shape (batch, T), got {tuple(ids.shape)}.")
        return F.linear(self.hidden(ids), self.token_embed.weight)

    def hidden(self, ids: torch.Tensor, *, sequence_group=None) -> torch.Tensor:
        x = self.token_embed(ids)
        return self.backbone(x) if sequence_group is None else self.backbone(x, sequence_group=sequence_group)

    def loss(self, ids: torch.Tensor, *, sequence_group=None) -> torch.Tensor:
        """Mean next-token cross-entropy of ``ids`` (float32).  The last position has no target, so
        its row is dropped before the head GEMM rather than from the logits.

        With ``sequence_group`` the TIME axis of ``ids`` is sharded over the ranks of that process group in rank
        order: a rank's last position is scored against the next rank's first token, and the value returned is
        this rank's SHARE of the mean over the whole sequence (its summed cross-entropy over the global number
        of positions) - the shares add up to the loss and their gradients add up to its gradient, so parameter
        gradients are to be SUMMED over the group."""
        if sequence_group is None:
            rows = self.hidden(ids)[:, :-1].reshape(-1, self.d_model)
            logits = F.linear(rows, self.token_embed.weight)
            return F.cross_entropy(logits.float(), ids[:, 1:].reshape(-1))
        import torch.distributed as dist
        world, rank = dist.get_world_size(sequence_group), dist.get_rank(sequence_group)
        firsts = [torch.empty_like(ids[:, :1]) for _ in range(world)]
        dist.all_gather(firsts, ids[:, :1].contiguous(), group=sequence_group)
        hidden = self.hidden(ids, sequence_group=sequence_group)
        if rank + 1 < world:
            rows, targets = hidden, torch.cat((ids[:, 1:], firsts[rank + 1]), dim=1)
        else:
            rows, targets = hidden[:, :-1], ids[:, 1:]
        count = torch.tensor([targets.numel()], device=ids.device, dtype=torch.float64)
        dist.all_reduce(count, group=sequence_group)
        logits = F.linear(rows.reshape(-1, self.d_model), self.token_embed.weight)
        return F.cross_entropy(logits.float(), targets.reshape(-1), reduction="sum") / count.item()


def decay_groups(model: nn.Module, weight_decay: float):
    """AdamW parameter groups: no decay for 1-D parameters and those tagged ``_no_weight_decay``
    (the mixer's ``d_skip``), as the reference's harness does."""
    decay, plain = [], []
    for p in model.parameters():
        if not p.requires_grad:
            continue
        (plain if (p.ndim < 2 or getattr(p, "_no_weight_decay", False)) else decay).append(p)
    return [{"params": decay, "weight_decay": weight_decay}, {"params": plain, "weight_decay": 0.0}]


class DataParallelTrainer:
    """One training step = forward, backward (gradient buckets all-reduced behind it), clip, AdamW.
    One instance per rank; every rank feeds its own shard of the batch."""

    def __init__(self, model: SLinOSSLM, *, lr: float = 3e-4, weight_decay: float = 0.05,
                 grad_clip: float = 1.0, bucket_bytes: int = 32 << 20, reduce: bool = True,
                 sequence_parallel: bool = False) -> None:
        """``sequence_parallel``: the ranks do not hold different sequences but consecutive TIME slices of the
        same sequences (``ids`` = this rank's slice); the loss shares' gradients then ADD over the ranks, which
        the averaging reducer delivers when every share is scaled by the world size first."""
        self.model, self.grad_clip = model, grad_clip
        self.sequence_parallel = bool(sequence_parallel)
        fused = self.fused = next(model.parameters()).is_cuda
        self.opt = torch.optim.AdamW(decay_groups(model, weight_decay), lr=lr, betas=(0.9, 0.95),
                                     fused=fused)
        self.reducer = shard.GradBucketReducer(model.parameters(), bucket_bytes=bucket_bytes) \
            if reduce else None

    def step(self, ids: torch.Tensor) -> torch.Tensor:
        self.opt.zero_grad(set_to_none=True)
        if self.sequence_parallel:
            import torch.distributed as dist
            loss = self.model.loss(ids, sequence_group=dist.group.WORLD)
            (loss * dist.get_world_size()).backward()
        else:
            loss = self.model.loss(ids)
            loss.backward()
        if self.reducer is not None:
            self.reducer.finish()
        if self.grad_clip and self.grad_clip > 0:
            self._clip()
        self.opt.step()
        loss = loss.detach()
        if self.sequence_parallel:       # the shares add up to the loss of the whole sequences
            import torch.distributed as dist
            loss = loss.clone()
            dist.all_reduce(loss)
        return loss

    def _clip(self) -> None:
        """Global-norm clipping.  With the fused optimizer the coefficient is not applied as a pass over
        the gradients: the optimizer kernel divides every gradient by ``grad_scale`` as it reads it
        (the hook loss scaling uses), so ``grad_scale = 1 / coefficient`` clips with no extra traffic
        and no host synchronisation."""
        grads = [p.grad for p in self.model.parameters() if p.grad is not None]
        if not self.fused:
            torch.nn.utils.clip_grad_norm_(self.model.parameters(), self.grad_clip)
            return
        norms = torch._foreach_norm(grads, 2.0)
        total = torch.linalg.vector_norm(torch.stack([n.float() for n in norms]), 2.0)
        # clip_grad_norm_'s coefficient is min(1, clip / (total + 1e-6)); grad_scale is its reciprocal
        self.opt.grad_scale = torch.clamp((total + 1e-6) / self.grad_clip, min=1.0).reshape(())
        self.last_grad_norm = total


__all__ = ["DataParallelTrainer", "SLinOSSLM", "decay_groups", "lm_stack_config"]
