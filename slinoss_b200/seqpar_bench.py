"""Timing of the sequence-parallel scan (one time slice per GPU) against the plain op on the same slice.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m slinoss_b200.seqpar_bench --steps 10 --warmup 3

Every rank holds ``--T`` tokens of the config-1 streams (batch 8 x heads 16, P 64, N 64, bf16), so the
sequence is N x T tokens long.  One step = forward + backward of the sharded scan (two local passes each way
and one exchange of state-sized tensors); time = MAX over ranks, CUDA events.  Prints one JSON line on rank 0
with the plain op's time on one slice beside it and the parity of the sharded result against a single-GPU
scan of the gathered sequence (``--check``, small T only).
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import shard
from .ops.v2x2ssd import v2x2ssd_cute, v2x2ssd_sequence_parallel
from .synthetic import make_scan_case


def stack_leg(args, world, rank, dev, barrier):
    """Forward + backward of a stack of blocks whose input is sharded in time (``sequence_group``), against the
    same stack on rank 0 over the whole sequence."""
    import torch.distributed as dist
    import slinoss_b200 as sb
    torch.manual_seed(0)
    blk = sb.SLinOSSBlockConfig(d_model=1024, mixer=sb.SLinOSSMixerConfig(d_state=64, expand=2.0, d_head=64),
                                ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=4.0))
    stack = sb.SLinOSSStack(sb.SLinOSSStackConfig.uniform(blk, n_layers=args.stack), device=dev,
                            dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(1)
    batch = min(args.batch, 2)
    x_full = torch.randn(batch, args.T * world, 1024, generator=g).to(torch.bfloat16)
    w_full = torch.randn(batch, args.T * world, 1024, generator=g).to(torch.bfloat16)
    sl = slice(rank * args.T, (rank + 1) * args.T)
    x = x_full[:, sl].to(dev).requires_grad_(True)
    w = w_full[:, sl].to(dev)
    group = dist.group.WORLD if world > 1 else None

    def step():
        stack.zero_grad(set_to_none=True)
        out = stack(x, sequence_group=group)
        (gx,) = torch.autograd.grad((out.float() * w.float()).sum(), x)
        return out, gx

    for _ in range(args.warmup):
        step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = shard.reduce_step_ms(e0.elapsed_time(e1) / args.steps, dev)
    out, gx = step()
    err = None
    if rank == 0 and args.T * world <= 16384:
        xw = x_full.to(dev).requires_grad_(True)
        ow = stack(xw)
        (gw,) = torch.autograd.grad((ow.float() * w_full.to(dev).float()).sum(), xw)
        rel = lambda a, b: float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))
        err = max(rel(out.detach(), ow[:, sl].detach()), rel(gx, gw[:, sl]))
    if rank == 0:
        line = {"what": f"stack of {args.stack} blocks, forward + backward, time axis sharded over the GPUs",
                "config": f"batch {batch} x T {args.T} per GPU ({args.T * world} in all), d_model 1024, 32 heads x 64, "
                          "N 64, GELU FFN x4, bf16",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "tokens_per_s": batch * args.T * world / (ms * 1e-3),
                "max_rel_err_vs_single_gpu_stack_on_the_whole_sequence": err}
        text = json.dumps(line)
        print(text, flush=True)
        if args.out:
            with open(args.out, "w") as f:
                f.write(text + "\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--T", type=int, default=4096, help="tokens per rank")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--stack", type=int, default=0, metavar="LAYERS",
                    help="time a stack of LAYERS blocks (d_model 1024, 32 heads x 64, N 64, GELU FFN x4) on the "
                         "sharded sequence instead of the bare scan")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("slinoss_b200.seqpar_bench needs CUDA devices: the kernels have no CPU path.")
    import torch.distributed as dist
    world, rank = int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.stack > 0:
        stack_leg(args, world, rank, dev, barrier)
        if world > 1:
            dist.destroy_process_group()
        return
    check = args.T * world <= 16384
    if check:   # the same long sequence on every rank (same seed), of which a rank keeps its slice
        full = make_scan_case(args.batch, args.heads, args.T * world, 64, 64, dtype=torch.bfloat16, seed=0)
        sl = slice(rank * args.T, (rank + 1) * args.T)
        mine = [t[:, :, sl].contiguous().to(dev) for t in full.tensors()]
        dY = full.dY[:, :, sl].contiguous().to(dev)
    else:       # long sequences: every rank draws its own slice (timing only)
        part = make_scan_case(args.batch, args.heads, args.T, 64, 64, dtype=torch.bfloat16, seed=rank)
        mine = [t.to(dev) for t in part.tensors()]
        dY = part.dY.to(dev)
    leaves = [t.clone().requires_grad_(True) for t in mine]

    def step_sharded():
        Y, end, _, _ = v2x2ssd_sequence_parallel(*leaves, chunk_size=64)
        return Y, torch.autograd.grad(Y, leaves, dY)

    def step_plain():
        Y = v2x2ssd_cute(*leaves, chunk_size=64)
        return Y, torch.autograd.grad(Y, leaves, dY)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            fn()
        e1.record()
        barrier()
        return shard.reduce_step_ms(e0.elapsed_time(e1) / args.steps, dev)

    ms_sharded = timed(step_sharded)
    ms_plain = timed(step_plain)
    # parity: rank 0 scans the whole sequence alone and compares its own slice of Y and of the gradients
    err = None
    if check:
        Y, grads = step_sharded()
        if rank == 0:
            whole = [t.to(dev).clone().requires_grad_(True) for t in full.tensors()]
            Yw = v2x2ssd_cute(*whole, chunk_size=64)
            gw = torch.autograd.grad(Yw, whole, full.dY.to(dev))
            rel = lambda a, b: float((a.double() - b.double()).abs().max() / b.double().abs().max().clamp_min(1e-30))
            err = max([rel(Y, Yw[:, :, sl])] + [rel(g, w[:, :, sl]) for g, w in zip(grads, gw)])
    if rank == 0:
        tokens = args.batch * args.T * world
        line = {"what": "sequence-parallel v2x2ssd forward+backward (time axis sharded over the GPUs)",
                "config": f"batch {args.batch} x heads {args.heads} x T {args.T} per GPU ({args.T * world} in all), "
                          "P 64, N 64, bf16",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_sharded, "tokens_per_s": tokens / (ms_sharded * 1e-3),
                "ms_plain_op_on_one_slice": ms_plain, "cost_vs_plain": ms_sharded / ms_plain,
                "max_rel_err_vs_single_gpu_scan_of_the_whole_sequence": err}
        text = json.dumps(line)
        print(text, flush=True)
        if args.out:
            with open(args.out, "w") as f:
                f.write(text + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
