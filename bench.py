"""Benchmark of the v2x2ssd scan forward+backward (BASELINE config 1) on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One "step" = one forward + one backward pass of the scan over one batch of synthetic
input (batch 8, heads 16, T 4096, P 64, N 64, chunk 64, bf16 operands, float32 state)
per GPU.  Every rank owns an independent shard of (batch, head) streams, so there is
no data-path collective ("weak" scaling: per-GPU work is fixed).  Rank 0 prints ONE
JSON line:

  value / ms_per_step   device-timed (CUDA events on the launching stream, max over
                        ranks) with inputs resident in HBM, through the C ABI launchers
  e2e                   the same step through the public op with HOST (pinned) buffers:
                        host->device copies of all inputs and device->host copies of Y and
                        all gradients are inside the timed region (the batch is fed in slices of one
                        batch entry x half the heads on a copy-in stream, two op streams and a
                        copy-out stream, so that both copy directions and the kernels overlap)
  roofline              the dominant kernel (the backward sweep): its algorithmic bytes / its
                        CUDA-event time vs the measured HBM copy bandwidth
                        (MEASURED_PEAKS.json); "step" and "fwd" give the same figure for the
                        whole step and for the forward kernel
  cpu_baseline          the C/OpenMP port of the reference's sequential scan (oracle/),
                        timed on the host cores on a bounded sample (N=1, rank 0 only)
  others                the other configurations of the hot path, measured on rank 0's GPU after the
                        headline legs: config 3 (decode of 1024 consecutive tokens, eager and as
                        one CUDA graph) and config 2 (the mixer layer forward+backward and its four
                        row-kernel calls; under --gpus N every rank owns batch 8/N of it) and, at
                        N=1, the config-1 streams with 128 state columns (the mixer's default) and the
                        CPU restatement of configs 3 and 2 timed on the host cores (bounded samples)

``--impl reference`` times only that CPU port on WHOLE steps of the same workload with all host
threads (set explicitly: a launcher may export OMP_NUM_THREADS=1) and prints the same line with
``"impl": "reference"``.  Its metric is a throughput, so the figure does not depend on --gpus.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

CFG = dict(batch=8, heads=16, T=4096, P=64, N=64, chunk=64)
METRIC = "v2x2ssd fwd+bwd tokens/s"
FALLBACK_HBM_GBS = 6650.0
TRAFFIC_FILE = ROOT / "profiles" / "scan_tc_bwd_traffic.json"


def kernel_source_digest() -> str:
    """sha256 over the tensor-core scan sources: ties a profiler figure to the kernels it was taken on."""
    import hashlib
    h = hashlib.sha256()
    for name in ("scan_tc.cu", "scan_tc_fwd.cuh", "scan_tc_bwd.cuh", "tc_common.cuh"):
        h.update((ROOT / "slinoss_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def ncu_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the backward sweep at this
    workload, as recorded beside the ncu summary (a profiler figure, not measured live here).
    Null when the kernels have changed since the capture."""
    try:
        rec = json.loads(TRAFFIC_FILE.read_text())
    except Exception:
        return None, None
    if rec.get("kernel_source_digest") != kernel_source_digest():
        return None, f"{TRAFFIC_FILE.name}: taken on other kernel sources ({rec.get('kernel_source_digest')})"
    return int(rec["dram_bytes_per_launch"]), f"{TRAFFIC_FILE.name}: {rec.get('how', '')}"


def algorithmic_bytes(c) -> dict:
    """Each input read once, each output written once (bf16 operands, float32 M/K)."""
    bht = c["batch"] * c["heads"] * c["T"]
    u = bht * c["P"] * 2
    bc = bht * 2 * c["N"] * 2
    m, k = bht * 2 * 4, bht * 4 * 4
    fwd = u + 2 * bc + m + k + u
    bwd = (u + 2 * bc + m + k) + u + (u + 2 * bc + m + k)
    return {"fwd": fwd, "bwd": bwd, "total": fwd + bwd}


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.path = index, None, f"/tmp/slinoss_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline(sample_heads: int = 16, repeats: int = 1) -> dict:
    """Times the C/OpenMP oracle port (forward + backward) on a slice of the workload:
    batch 1, ``sample_heads`` heads, full T/P/N.  Returns tokens/s on the host cores."""
    from oracle import scan_c
    from slinoss_b200.synthetic import make_scan_case
    c = CFG
    scan_c.set_num_threads(os.cpu_count() or 1)   # explicit: a launcher may have exported OMP_NUM_THREADS=1
    case = make_scan_case(1, sample_heads, c["T"], c["P"], c["N"], dtype=torch.bfloat16, seed=0)
    arrs = [t.float().numpy() for t in case.tensors()]
    dY = case.dY.float().numpy()
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        scan_c.forward(*arrs)
        scan_c.backward(*arrs, dY)
        best = min(best, time.perf_counter() - t0)
    tokens = c["T"]  # batch 1
    # the full workload has batch*heads streams; this sample has sample_heads of them
    scale = c["batch"] * c["heads"] / sample_heads
    full_step_s = best * scale
    return {"value": c["batch"] * c["T"] / full_step_s, "unit": "tokens/s", "cores": scan_c.num_threads(),
            "kind": "port",
            "sample": f"fwd+bwd of batch 1 x {sample_heads} heads x T {c['T']} (1/{scale:.0f} of a step) "
                      f"in {best:.2f} s, scaled linearly", "sample_seconds": best}


def cpu_baseline_others() -> dict:
    """The CPU restatement of configs 3 and 2 timed on the host cores on bounded samples (seconds each):
    decode = the C/OpenMP port's one-token update over a carried state; the mixer's row-wise stages (conv +
    scan preparation, gated RMSNorm tail) = the torch CPU oracle, forward + backward."""
    from oracle import mixer_torch as mt
    from oracle import scan_c
    cores = scan_c.set_num_threads(os.cpu_count() or 1)
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(0)
    r = lambda *sh: torch.randn(*sh, generator=g)
    # ---- config 3: one token, batch 16 of 256 (state 16 x 32 x 64 x 128 float32)
    b, h, P, N = 16, 32, 64, 64
    state = (0.1 * r(b, h, P, 2 * N)).numpy()
    args = [r(b, h, 1, P).numpy(), torch.stack([0.95 * torch.ones(b, h, 1), 0.1 * torch.ones(b, h, 1)], -1).numpy(),
            (0.05 * r(b, h, 1, 2, 2)).numpy(), (r(b, h, 1, 2 * N) / 8).numpy(), (r(b, h, 1, 2 * N) / 8).numpy()]
    bp, up = np.zeros((b, h, 2 * N), np.float32), np.zeros((b, h, P), np.float32)
    steps, t0 = 0, time.perf_counter()
    while steps < 8 or time.perf_counter() - t0 < 2.0:
        _, state = scan_c.forward(*args, initial_states=state, B_prev=bp, U_prev=up)
        steps += 1
    dec_s = (time.perf_counter() - t0) / steps
    # ---- config 2: batch 1 x T 512 of the 8 x 2048 rows (d_inner 2048 = 32 heads x 64, N 64)
    T, H = 512, 32
    cfg = {"dt_min": 5e-3, "dt_max": 1e-1, "alpha_min": 0.0, "alpha_max": 20.0, "theta_init_min": 0.05,
           "theta_init_max": 2.0, "theta_mod_scale": 1.0, "r_min": 0.8, "r_max": 1.0, "eps": 1e-8}
    value, params, bc = r(1, T, H * P).requires_grad_(), r(1, T, 3 * H).requires_grad_(), r(1, T, H, 4, N).requires_grad_()
    w, bias = (0.3 * r(H * P, 4)).requires_grad_(), r(H * P).requires_grad_()
    biases = [r(H).requires_grad_() for _ in range(4)] + [torch.ones(H)]
    gate, wn = r(1, T, H * P).requires_grad_(), torch.ones(H * P, requires_grad=True)
    d_skip = torch.ones(H, requires_grad=True)

    def rows_step():
        v, _ = mt.causal_conv_silu(value, w, bias)
        U, M, K, Bo, Co = mt.scanprep(v, params, bc, cfg, *biases, d_head=P)
        out = mt.gated_rmsnorm(U, gate, wn, 1e-5, skip_input=U, d_skip=d_skip)    # (U stands in for the scan output)
        (out.square().sum() + M.square().sum() + K.square().sum() + Bo.square().sum() + Co.square().sum()).backward()

    rows_step()
    n, t0 = 0, time.perf_counter()
    while n < 2 or time.perf_counter() - t0 < 2.0:
        rows_step()
        n += 1
    rows_s = (time.perf_counter() - t0) / n
    return {"kind": "port", "cores": cores,
            "config3_decode": {"value": 256 / (dec_s * 256 / b), "unit": "tokens/s",
                               "sample": f"one-token update of batch {b} x 32 heads (1/16 of the batch), "
                                         f"{dec_s * 1e3:.2f} ms, scaled linearly to batch 256"},
            "config2_rows": {"value": 8 * 2048 / (rows_s * 8 * 2048 / T), "unit": "tokens/s",
                             "sample": f"conv + scan preparation + gated RMSNorm tail, forward + backward, of 1 x {T} "
                                       f"rows (1/32 of the rows), {rows_s * 1e3:.1f} ms, scaled linearly; "
                                       "GEMMs and the scan itself not included"}}


def run_reference_arm(args, rank):
    """The reference's CPU path for this workload = the C/OpenMP port of its sequential scan
    (forward + analytic backward), on WHOLE steps of config 1 with every host core.  The number
    of steps is capped so that the run ends within a few minutes; the line says how many ran."""
    if rank != 0:
        return
    from oracle import scan_c
    from slinoss_b200.synthetic import make_scan_case
    c = CFG
    cores = scan_c.set_num_threads(os.cpu_count() or 1)
    case = make_scan_case(c["batch"], c["heads"], c["T"], c["P"], c["N"], dtype=torch.bfloat16, seed=0)
    arrs = [t.float().numpy() for t in case.tensors()]
    dY = case.dY.float().numpy()
    budget_s, times = 150.0, []
    t_begin = time.perf_counter()
    for i in range(max(1, args.warmup // 3) + max(2, args.steps)):
        t0 = time.perf_counter()
        scan_c.forward(*arrs)
        scan_c.backward(*arrs, dY)
        dt = time.perf_counter() - t0
        if i >= max(1, args.warmup // 3):
            times.append(dt)            # (the first pass warms caches and the thread pool)
        if len(times) >= 2 and time.perf_counter() - t_begin + dt > budget_s:
            break
    step_s = statistics.mean(times)
    value = c["batch"] * c["T"] / step_s
    base = {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{len(times)} whole steps (batch {c['batch']} x {c['heads']} heads x T {c['T']}), "
                      f"{step_s:.2f} s each, not scaled"}
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": len(times), "steps_requested": args.steps, "warmup": 1,
            "ms_per_step": step_s * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": workload_config(args.gpus),
            "note": "host throughput of one whole step; a throughput does not grow with --gpus, so at "
                    "N > 1 compare it with the GPU arm's value / N",
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def workload_config(n):
    return {"workload": "BASELINE config 1: v2x2ssd fwd+bwd, batch 8 x heads 16 x T 4096, P 64, N 64, "
                        "chunk 64, bf16 operands, float32 state/accumulation, per GPU",
            "sharding": f"{n} independent shards of (batch, head) streams, no collective",
            "l2": "inputs of one step (415 MB) exceed the 126 MB L2; no explicit flush",
            **CFG}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tc"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--T", type=int, default=0, help="override the sequence length (smaller cases)")
    ap.add_argument("--no-others", action="store_true", help="skip the config 2 / config 3 legs")
    ap.add_argument("--e2e-head-parts", type=int, default=0,
                    help="end-to-end leg: slices per batch entry along heads (0 = 2 on one GPU, 1 when "
                         "several ranks share the host)")
    ap.add_argument("--e2e-op-streams", type=int, default=2,
                    help="end-to-end leg: streams the op runs on, slices alternate between them")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return
    if args.T > 0:
        CFG["T"] = args.T
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU path.")
    args.warmup = max(args.warmup, 3)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    from slinoss_b200 import _C, shard
    from slinoss_b200.ops.v2x2ssd import v2x2ssd_cute
    from slinoss_b200.synthetic import make_scan_case

    c = CFG
    case_h = make_scan_case(c["batch"], c["heads"], c["T"], c["P"], c["N"], dtype=torch.bfloat16,
                            seed=shard.rank_seed(0, rank))
    case = case_h.to(dev)
    U, M, K, B, C, dY = case.U, case.M, case.K, case.B, case.C, case.dY

    def step_device():
        # what autograd does: the forward keeps its chunk-start states for the backward
        _, fin, st = _C.scan_fwd(U, M, K, B, C, None, None, None, chunk_size=c["chunk"],
                                 y_dtype=torch.bfloat16, want_final=False, path=args.path,
                                 save_states=True)
        _C.scan_bwd(U, M, K, B, C, None, None, None, dY, None, chunk_size=c["chunk"], path=args.path,
                    saved=(st, fin))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_device()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    fwd_ms = bwd_ms = 0.0
    t_start = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    barrier()
    launches_before = _C.kernel_launches()
    t_start.record()
    for _ in range(args.steps):
        step_device()
    t_end.record()
    barrier()
    launches_timed = _C.kernel_launches() - launches_before
    total_ms = t_start.elapsed_time(t_end)
    # per-phase split (separate short loop so that the events do not perturb the headline)
    for _ in range(min(args.steps, 5)):
        e0.record()
        _, fin, st = _C.scan_fwd(U, M, K, B, C, None, None, None, chunk_size=c["chunk"],
                                 y_dtype=torch.bfloat16, want_final=False, path=args.path,
                                 save_states=True)
        e1.record()
        _C.scan_bwd(U, M, K, B, C, None, None, None, dY, None, chunk_size=c["chunk"], path=args.path,
                    saved=(st, fin))
        e2.record()
        torch.cuda.synchronize()
        fwd_ms += e0.elapsed_time(e1)
        bwd_ms += e1.elapsed_time(e2)
    fwd_ms /= min(args.steps, 5)
    bwd_ms /= min(args.steps, 5)

    # ---- end to end through the public op with host buffers --------------------------------
    # The batch is fed in slices; host->device copies, the op (forward + autograd backward) and
    # device->host copies run on three streams, so the two PCIe directions and the kernels
    # overlap.  Every step moves ALL inputs in and ALL results (Y and the five gradients) out.
    pin = lambda t: t.pin_memory()
    h_in = [pin(t) for t in (case_h.U, case_h.M, case_h.K, case_h.B, case_h.C, case_h.dY)]
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d_in = [torch.empty_like(t, device=dev) for t in h_in]
    # one slice = one batch entry x a block of heads: short pipeline fill and drain
    hp = args.e2e_head_parts if args.e2e_head_parts > 0 else (2 if world == 1 else 1)
    hp = max(1, min(hp, c["heads"]))
    hs = c["heads"] // hp
    slices = [(slice(b, b + 1), slice(h * hs, (h + 1) * hs if h + 1 < hp else c["heads"]))
              for b in range(c["batch"]) for h in range(hp)]
    out_shapes = [(case_h.U.shape, torch.bfloat16), (case_h.U.shape, torch.bfloat16),
                  (case_h.M.shape, torch.float32), (case_h.K.shape, torch.float32),
                  (case_h.B.shape, torch.bfloat16), (case_h.C.shape, torch.bfloat16)]   # Y, dU, dM, dK, dB, dC
    h_out = [torch.empty(s, dtype=dt).pin_memory() for s, dt in out_shapes]
    d2h = sum(t.numel() * t.element_size() for t in h_out)
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    s_ops = [torch.cuda.Stream(dev) for _ in range(max(1, args.e2e_op_streams))]
    main_stream = torch.cuda.current_stream(dev)

    # per-slice views and autograd leaves are built once, outside the step
    views = [([d[sl] for d in d_in], [h[sl] for h in h_in], [h[sl] for h in h_out]) for sl in slices]
    leaves_of = [[v.detach().requires_grad_(True) for v in dv[:5]] for dv, _, _ in views]

    def copy_only():
        """The same bytes over the same streams without the op: the host-link bound of the step."""
        for s in (s_in, s_out):
            s.wait_stream(main_stream)
        for dv, hv, ho in views:
            with torch.cuda.stream(s_in):
                for d, h in zip(dv, hv):
                    d.copy_(h, non_blocking=True)
            with torch.cuda.stream(s_out):
                for h, d in zip(ho, (dv[0], dv[0], dv[1], dv[2], dv[3], dv[4])):
                    h.copy_(d, non_blocking=True)
        for s in (s_in, s_out):
            main_stream.wait_stream(s)

    def step_e2e():
        for s in (s_in, s_out, *s_ops):
            s.wait_stream(main_stream)
        for i, (dv, hv, ho) in enumerate(views):
            s_op = s_ops[i % len(s_ops)]
            with torch.cuda.stream(s_in):
                for d, h in zip(dv, hv):
                    d.copy_(h, non_blocking=True)
                ev_in = torch.cuda.Event(); ev_in.record(s_in)
            with torch.cuda.stream(s_op):
                s_op.wait_event(ev_in)
                leaves = leaves_of[i]
                Y = v2x2ssd_cute(*leaves, chunk_size=c["chunk"], path=args.path)
                grads = torch.autograd.grad(Y, leaves, dv[5])
                outs = (Y.detach(), *grads)
                ev_op = torch.cuda.Event(); ev_op.record(s_op)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_op)
                for h, o in zip(ho, outs):
                    o.record_stream(s_out)
                    h.copy_(o, non_blocking=True)
        for s in (s_in, s_out, *s_ops):
            main_stream.wait_stream(s)

    e2e_steps = max(2, min(args.steps, 5))
    for _ in range(2):
        step_e2e()
    barrier()
    t_start.record()
    for _ in range(e2e_steps):
        step_e2e()
    t_end.record()
    barrier()
    e2e_ms = t_start.elapsed_time(t_end)
    clocks = sampler.stop() if rank == 0 else None   # sampled over the device-timed and the end-to-end loops
    copy_only()
    barrier()
    t_start.record()
    for _ in range(e2e_steps):
        copy_only()
    t_end.record()
    barrier()
    copy_ms = t_start.elapsed_time(t_end)

    # ---- the other configurations of the hot path (rank-local figures; rank 0's are reported) ----
    others = None
    if not args.no_others and args.path != "simt" and args.T == 0:
        del d_in, h_in, h_out, views, leaves_of
        torch.cuda.empty_cache()
        from slinoss_b200 import measure
        measure.PRINT_LINES = False
        bshare = max(1, 8 // world)
        others = {
            "config3_decode": measure.measure_decode_sequence(0, dev, steps=1024, batch=256)
                              + measure.measure_mixer_step(20, dev, batch=256),
            "config2_mixer": measure.measure_mixer(12, dev, batch=bshare)
                             + measure.measure_scanprep(10, dev, batch=bshare)
                             + measure.measure_tail(10, dev, batch=bshare),
            "scan_d_state_128": measure.measure_scan_n128(10, dev) if world == 1 else None,
            "cpu_baseline": cpu_baseline_others() if (world == 1 and not args.no_cpu_baseline) else None,
            "note": "config 3: 1024 consecutive tokens, fresh inputs per token; config 2: batch "
                    f"{bshare} per GPU (8 sharded over {world} rank(s)); figures of rank 0's GPU",
        }
        barrier()

    # the job is as slow as its slowest rank: MAX over ranks of every device-timed figure
    total_ms, e2e_ms, fwd_ms, bwd_ms, copy_ms = (shard.reduce_step_ms(v, dev)
                                                 for v in (total_ms, e2e_ms, fwd_ms, bwd_ms, copy_ms))
    if rank == 0:
        tokens_step = world * c["batch"] * c["T"]
        ms_step = total_ms / args.steps
        ab = algorithmic_bytes(c)
        peak, peak_kind = measured_peak()
        achieved = ab["total"] / (ms_step * 1e-3) / 1e9
        bwd_gbs = ab["bwd"] / (bwd_ms * 1e-3) / 1e9
        traffic, traffic_source = ncu_traffic() if (args.path != "simt" and args.T == 0) else (None, None)
        line = {
            "metric": METRIC, "value": tokens_step / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(world),
            "e2e": {"value": tokens_step / (e2e_ms / e2e_steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / e2e_steps, "slices": len(slices),
                    "copy_only_ms_per_step": copy_ms / e2e_steps,
                    "note": "copy_only = the same host<->device bytes over the same streams without the op: "
                            "the host-link bound of this step on this box"},
            "gpu_launches": launches_timed,
            "roofline": {"bound": "hbm", "kernel": "backward sweep (scan_tc_bwd_kernel + its scalar finish)",
                         "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
                         "traffic": traffic, "traffic_source": traffic_source,
                         "peak_source": peak_kind, "algorithmic_bytes": ab["bwd"], "ms": bwd_ms,
                         "share_of_step": bwd_ms / (fwd_ms + bwd_ms),
                         "step": {"ms": ms_step, "algorithmic_bytes": ab["total"], "achieved": achieved,
                                  "frac": achieved / peak},
                         "fwd": {"ms": fwd_ms, "algorithmic_bytes": ab["fwd"],
                                 "achieved": ab["fwd"] / (fwd_ms * 1e-3) / 1e9,
                                 "frac": ab["fwd"] / (fwd_ms * 1e-3) / 1e9 / peak}},
            "clocks": clocks,
            "kernel_path": args.path,
            # 0 unless a bounded device-side wait of the tensor-core kernels expired during this run
            "device_status": _C.device_status(),
        }
        if others is not None:
            line["others"] = others
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(sample_heads=8)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
