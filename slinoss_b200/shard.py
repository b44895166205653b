"""Data-parallel plumbing of the scan and the mixer: one process per GPU.

Every (batch, head) stream of the scan is independent, so a job over N GPUs is N
processes that each own a slice of the batch and never exchange data on the scan
path; the only collectives are the host-side ones here:

* ``reduce_step_ms``   - step time of the job = MAX over ranks (device-timed per rank);
* ``job_throughput``   - units of all ranks divided by that time;
* ``allreduce_mean_``  - weight-gradient averaging when the mixer is *trained* data
  parallel (weights replicated, batch sharded), one flat bucket per dtype so that the
  cost is launch-latency bound, not per-tensor bound.

All functions take CPU or CUDA tensors and work with the ``gloo`` and ``nccl`` backends
of ``torch.distributed``; with no process group they degrade to the single-process
meaning (world size 1).
"""

from __future__ import annotations

from typing import Iterable, Optional, Sequence

import torch

try:  # torch.distributed is always built in the wheels this package targets
    import torch.distributed as dist
except ImportError:  # pragma: no cover
    dist = None


def _active(group=None) -> bool:
    return dist is not None and dist.is_available() and dist.is_initialized()


def world_size(group=None) -> int:
    return dist.get_world_size(group) if _active(group) else 1


def rank(group=None) -> int:
    return dist.get_rank(group) if _active(group) else 0


def shard_bounds(n_units: int, world: int, r: int) -> tuple[int, int]:
    """Half-open range ``[lo, hi)`` of the units rank ``r`` owns when ``n_units``
    independent units (batch entries, (batch, head) streams ...) are dealt out to
    ``world`` ranks as evenly as possible: the first ``n_units % world`` ranks get one
    more.  The ranges of all ranks are disjoint and cover ``[0, n_units)``."""
    if world < 1 or not (0 <= r < world):
        raise ValueError(f"rank {r} is outside a world of {world}.")
    if n_units < 0:
        raise ValueError(f"n_units must be non-negative. Got {n_units}.")
    base, extra = divmod(n_units, world)
    lo = r * base + min(r, extra)
    return lo, lo + base + (1 if r < extra else 0)


def shard_batch(tensors: Sequence[Optional[torch.Tensor]], world: int, r: int, dim: int = 0):
    """Slices every tensor (None passes through) along ``dim`` to rank ``r``'s range.
    Slices are made contiguous: the C ABI takes dense tensors only."""
    out = []
    for t in tensors:
        if t is None:
            out.append(None)
            continue
        lo, hi = shard_bounds(t.shape[dim], world, r)
        out.append(t.narrow(dim, lo, hi - lo).contiguous())
    return out


def rank_seed(seed: int, r: int) -> int:
    """Seed of rank ``r``'s synthetic shard (weak scaling: every rank draws its own)."""
    return int(seed) * 1000003 + int(r)


def reduce_step_ms(ms: float, device: torch.device | str = "cpu", group=None) -> float:
    """MAX over ranks of a per-rank duration (the job is as slow as its slowest rank)."""
    if not _active(group):
        return float(ms)
    t = torch.tensor([float(ms)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


def job_throughput(units_this_rank: int, step_ms: float, device: torch.device | str = "cpu",
                   group=None) -> tuple[float, int, float]:
    """Whole-job units/s: SUM of the ranks' units over the MAX of their step times.
    Returns ``(units_per_second, total_units, max_ms)``."""
    if not _active(group):
        return units_this_rank / (step_ms * 1e-3), int(units_this_rank), float(step_ms)
    t = torch.tensor([float(units_this_rank)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    mx = reduce_step_ms(step_ms, device, group)
    return float(t.item()) / (mx * 1e-3), int(round(t.item())), mx


def allreduce_mean_(grads: Iterable[Optional[torch.Tensor]], group=None) -> None:
    """In place: every gradient becomes its mean over the ranks.  Gradients are packed
    into one flat buffer per (dtype, device) so each bucket is a single collective."""
    if not _active(group):
        return
    n = dist.get_world_size(group)
    buckets: dict = {}
    for g in grads:
        if g is not None:
            buckets.setdefault((g.dtype, g.device), []).append(g)
    for (dtype, device), items in buckets.items():
        acc_dtype = torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype
        flat = torch.cat([g.reshape(-1).to(acc_dtype) for g in items])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        flat.div_(n)
        off = 0
        for g in items:
            k = g.numel()
            g.copy_(flat[off:off + k].view_as(g).to(dtype))
            off += k
