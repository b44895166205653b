"""Training step of the stacked language model, data parallel over the GPUs of one node.

    python -m slinoss_b200.lm_bench --steps 5 --warmup 3                      # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m slinoss_b200.lm_bench --steps 5 --warmup 3                         # eight GPUs

Model: token embedding -> ``SLinOSSStack`` (24 blocks of mixer + GELU MLP 4x, RMSNorm, d_model 2048,
32 heads x 64, N 64) -> tied head, vocabulary 32000, random init (std 0.02), bf16 parameters.
Data: uniform random token ids, 4 sequences of 4096 tokens PER GPU (global batch 32 on 8 GPUs).
Every rank runs forward, backward, gradient all-reduce (NCCL, buckets started from autograd hooks
on a side stream so that they run behind the rest of the backward pass), clipping and AdamW.

Rank 0 prints one JSON line: tokens/s of the whole job, step time (MAX over ranks, CUDA events), the
same step without the all-reduce, and their difference = the EXPOSED part of the collective.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import shard
from . import _C
from .lm import DataParallelTrainer, SLinOSSLM, lm_stack_config


def timed_steps(trainer, ids, steps, warmup, barrier):
    losses = []
    for _ in range(warmup):
        losses.append(trainer.step(ids))
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        losses.append(trainer.step(ids))
    e1.record()
    barrier()
    return e0.elapsed_time(e1) / steps, [float(x) for x in losses]


def kernel_table(trainer, ids, rows: int, steps: int = 2) -> None:
    """Device time per kernel over ``steps`` training steps: ms per step, share, launches per step."""
    import sys
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(steps):
            trainer.step(ids)
        torch.cuda.synchronize()
    table = [(e.device_time_total / (1e3 * steps), e.count // steps, e.key)
             for e in prof.key_averages() if e.device_time_total > 0 and e.device_type.name == "CUDA"]
    table.sort(reverse=True)
    total = sum(t for t, _, _ in table)
    print(f"device time per step {total:.1f} ms", file=sys.stderr)
    for t, n, key in table[:rows]:
        print(f"{t:8.2f} ms {100 * t / total:5.1f}% x{n:5d} {key[:120]}", file=sys.stderr)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=0, help="informational; the launcher sets WORLD_SIZE")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--batch-per-gpu", type=int, default=4)
    ap.add_argument("--bucket-mb", type=int, default=32)
    ap.add_argument("--ffn-remat", choices=["full", "rows", "none"], default=None,
                    help="what the FFN branch rebuilds in the backward pass (default: the block's own)")
    ap.add_argument("--sequence-parallel", action="store_true",
                    help="the ranks hold consecutive time slices of the same --batch-per-gpu sequences (context "
                         "length = --seq x ranks) instead of different sequences")
    ap.add_argument("--kernel-table", type=int, default=0, metavar="ROWS",
                    help="after the timed steps, profile two more steps (torch profiler) on rank 0 and print "
                         "the ROWS kernels with the most device time to stderr")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("slinoss_b200.lm_bench needs CUDA devices: the kernels have no CPU path.")
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    torch.manual_seed(0)                         # identical replicas on every rank
    cfg = lm_stack_config(args.d_model, args.layers)
    model = SLinOSSLM(args.vocab, cfg, device=dev, dtype=torch.bfloat16)
    if args.ffn_remat is not None:
        for blk in model.backbone.blocks:
            blk.ffn_remat = args.ffn_remat
    ffn_remat = model.backbone.blocks[0].ffn_remat
    n_params = sum(p.numel() for p in model.parameters())
    seqpar = args.sequence_parallel and world > 1
    if seqpar:   # the same long sequences on every rank, of which a rank keeps its time slice
        g = torch.Generator(device=dev).manual_seed(1)
        ids = torch.randint(0, args.vocab, (args.batch_per_gpu, args.seq * world), generator=g, device=dev)
        ids = ids[:, rank * args.seq:(rank + 1) * args.seq].contiguous()
    else:
        g = torch.Generator(device=dev).manual_seed(shard.rank_seed(1, rank))
        ids = torch.randint(0, args.vocab, (args.batch_per_gpu, args.seq), generator=g, device=dev)

    trainer = DataParallelTrainer(model, bucket_bytes=args.bucket_mb << 20, reduce=world > 1,
                                  sequence_parallel=seqpar)
    ms, losses = timed_steps(trainer, ids, args.steps, args.warmup, barrier)
    ms = shard.reduce_step_ms(ms, dev)
    ms_plain = None
    if world > 1:                                # the same step with the collective taken out
        trainer.reducer.remove()
        n_buckets = len(trainer.reducer.buckets)
        trainer.reducer = None
        ms_plain, _ = timed_steps(trainer, ids, args.steps, 1, barrier)
        ms_plain = shard.reduce_step_ms(ms_plain, dev)
    else:
        n_buckets = 0
    mem_gb = torch.cuda.max_memory_allocated(dev) / 2 ** 30
    if args.kernel_table > 0 and rank == 0 and world == 1:
        kernel_table(trainer, ids, args.kernel_table)
    if rank == 0:
        tokens = world * args.batch_per_gpu * args.seq
        line = {
            "what": "stacked-LM training step (forward, backward, gradient all-reduce, clip, AdamW)",
            "config": {"layers": args.layers, "d_model": args.d_model, "heads": args.d_model // 64,
                       "d_state": 64, "vocab": args.vocab, "seq": args.seq,
                       "batch_per_gpu": args.batch_per_gpu, "global_batch": world * args.batch_per_gpu,
                       "dtype": "bf16", "parameters": n_params, "ffn_remat": ffn_remat,
                       "sharding": (f"sequence parallel: {args.batch_per_gpu} sequences of {args.seq * world} tokens, "
                                    "one time slice per GPU") if seqpar else "data parallel", "data": "synthetic uniform ids"},
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "tokens_per_s": tokens / (ms * 1e-3),
            "ms_per_step_without_allreduce": ms_plain,
            "exposed_allreduce_ms": None if ms_plain is None else ms - ms_plain,
            "allreduce": {"buckets": n_buckets, "bucket_mb": args.bucket_mb,
                          "bytes": 2 * n_params, "backend": "nccl" if world > 1 else None},
            "loss_first": losses[0], "loss_last": losses[args.warmup + args.steps - 1],
            "peak_memory_gb": mem_gb,
            "device_status": _C.device_status(),   # 0 unless a bounded device-side wait expired
        }
        text = json.dumps(line)
        print(text, flush=True)
        if args.out:
            with open(args.out, "w") as f:
                f.write(text + "\n")
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
