"""Data-parallel plumbing of the scan and the mixer: one process per GPU.

Every (batch, head) stream of the scan is independent, so a job over N GPUs is N
processes that each own a slice of the batch and never exchange data on the scan
path; the only collectives are the host-side ones here:

* ``reduce_step_ms``   - step time of the job = MAX over ranks (device-timed per rank);
* ``job_throughput``   - units of all ranks divided by that time;
* ``allreduce_mean_``  - weight-gradient averaging when the mixer is *trained* data
  parallel (weights replicated, batch sharded), one flat bucket per dtype so that the
  cost is launch-latency bound, not per-tensor bound;
* ``GradBucketReducer`` - the same averaging for a large model: gradients are packed into
  buckets of a few tens of megabytes in the order the backward pass produces them and every
  bucket's all-reduce starts from an autograd hook on a side stream as soon as its last
  gradient exists, so the collective runs behind the rest of the backward pass.

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


class GradBucketReducer:
    """Bucketed, overlapped gradient averaging for data-parallel training (one process per GPU,
    weights replicated, batch sharded): the collective of the stacked-LM training configuration.

    Parameters are dealt into buckets of about ``bucket_bytes`` in REVERSE registration order,
    which is the order in which the backward pass finishes their gradients.  A
    ``post_accumulate_grad`` hook counts the gradients of a bucket; the last one packs the bucket
    into its flat buffer on a side stream (ordered after the stream that produced the gradients)
    and starts the all-reduce there without waiting.  ``finish()`` starts whatever is left
    (a parameter that got no gradient counts as zeros, so that every rank issues the same
    collectives), waits and orders the calling stream after all of it.  The averaged gradients are
    left in ``p.grad`` as VIEWS of the buckets' flat buffers (no copy back: the buffers are refilled
    by the next backward pass, by which time the optimizer has consumed them); the average is taken
    by the collective itself where the backend has ``ReduceOp.AVG`` (NCCL), else by one in-place
    division per bucket.  With a ``reduce_dtype`` other than the parameters' the result is copied
    back instead.  With no process group the class does nothing (world size 1).

    Works with ``nccl`` (CUDA tensors, real overlap) and ``gloo`` (CPU tensors)."""

    def __init__(self, params: Iterable[torch.nn.Parameter], *, bucket_bytes: int = 32 << 20,
                 group=None, reduce_dtype: Optional[torch.dtype] = None) -> None:
        self.group = group
        self.params = [p for p in params if p.requires_grad]
        self.reduce_dtype = reduce_dtype
        self.buckets: list[dict] = []
        self._bucket_of: dict[int, dict] = {}
        self._hooks = []
        self._stream = None
        # the collective averages by itself where the backend can (NCCL); gloo has no AVG
        self._avg = _active(group) and dist.get_backend(group) == "nccl"
        open_bucket: dict = {}
        for p in reversed(self.params):
            dt = reduce_dtype or p.dtype
            key = (dt, p.device)
            b = open_bucket.get(key)
            nbytes = p.numel() * torch.empty((), dtype=dt).element_size()
            if b is None or (b["bytes"] + nbytes > bucket_bytes and b["params"]):
                b = {"params": [], "bytes": 0, "numel": 0, "dtype": dt, "device": p.device, "flat": None,
                     "ready": 0, "handle": None}
                self.buckets.append(b)
                open_bucket[key] = b
            b["params"].append(p)
            b["bytes"] += nbytes
            b["numel"] += p.numel()
            self._bucket_of[id(p)] = b
        if _active(group):
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    # -- hooks ------------------------------------------------------------------------------
    def _on_grad(self, p: torch.Tensor) -> None:
        b = self._bucket_of[id(p)]
        b["ready"] += 1
        if b["ready"] == len(b["params"]):
            self._launch(b)

    def _side_stream(self, device):
        if device.type != "cuda":
            return None
        if self._stream is None:
            self._stream = torch.cuda.Stream(device)
        return self._stream

    def _launch(self, b: dict) -> None:
        if b["flat"] is None:
            b["flat"] = torch.empty(b["numel"], dtype=b["dtype"], device=b["device"])
        side = self._side_stream(b["device"])

        def pack_and_start():
            off = 0
            for p in b["params"]:
                n = p.numel()
                dst = b["flat"][off:off + n]
                if p.grad is None:
                    dst.zero_()
                else:
                    dst.copy_(p.grad.reshape(-1))
                off += n
            op = dist.ReduceOp.AVG if self._avg else dist.ReduceOp.SUM
            b["handle"] = dist.all_reduce(b["flat"], op=op, group=self.group, async_op=True)

        if side is None:
            pack_and_start()
        else:
            side.wait_stream(torch.cuda.current_stream(b["device"]))
            with torch.cuda.stream(side):
                pack_and_start()

    # -- end of the backward pass -----------------------------------------------------------
    def finish(self) -> None:
        """Call after ``backward()``: completes every bucket and leaves the averaged gradients
        in ``p.grad``."""
        if not _active(self.group):
            return
        n = dist.get_world_size(self.group)
        for b in self.buckets:
            if b["handle"] is None:
                self._launch(b)
        for b in self.buckets:
            side = self._side_stream(b["device"])
            ctx = torch.cuda.stream(side) if side is not None else _NullContext()
            with ctx:
                b["handle"].wait()
                if not self._avg:
                    b["flat"].div_(n)
                off = 0
                for p in b["params"]:
                    k = p.numel()
                    piece = b["flat"][off:off + k].view(p.shape)
                    if p.grad is not None:
                        if piece.dtype == p.dtype:
                            p.grad = piece              # a view of the bucket: no copy back
                        else:
                            p.grad.copy_(piece)
                    off += k
            b["handle"], b["ready"] = None, 0
        if self._stream is not None:
            torch.cuda.current_stream(self._stream.device).wait_stream(self._stream)

    def remove(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks = []


class _NullContext:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False
