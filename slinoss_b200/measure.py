"""Device timing of every C-ABI entry point at the sizes of the reference's configs.

    python -m slinoss_b200.measure [--what decode,decode_sequence,mixer_step,scanprep,tail,mixer,scan] [--iters 20]

Prints one JSON line per measured call: CUDA-event time (mean of ``iters`` back-to-back
launches after warm-up, on the launching stream), the call's algorithmic bytes (every
input read once, every output written once) and the fraction of the HBM roofline that
makes.  ``bench.py`` is the headline (scan forward+backward at config 1); this module
covers the other rows of the hot path: decode (config 3), fused conv + scan preparation
and the mixer tail at the mixer configuration (config 2), and the whole mixer layer.

Inputs are seeded synthetic tensors of the configs' shapes and value ranges.  All inputs of a
call exceed the 126 MB L2 except where noted in the line (``"l2"``).
"""

from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
FALLBACK_HBM_GBS = 6650.0


def hbm_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def time_ms(fn, iters: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


PRINT_LINES = True   # `python -m slinoss_b200.measure` prints; bench.py collects the returned lines instead


def emit(line):
    if PRINT_LINES:
        print(json.dumps(line), flush=True)
    return line


def report(name, ms, algo_bytes, config, extra=None):
    peak, kind = hbm_peak()
    gbs = algo_bytes / (ms * 1e-3) / 1e9
    line = {"call": name, "ms": ms, "algorithmic_bytes": algo_bytes, "achieved_gbs": gbs,
            "peak_gbs": peak, "peak_source": kind, "frac": gbs / peak, "config": config}
    if extra:
        line.update(extra)
    return emit(line)


# ---------------------------------------------------------------------------------------
def measure_decode(iters, dev, batch=None, N=64):
    """Config 3: batch 256, heads 32, P 64, N 64 (or the mixer's default 128), bf16 vectors, float32 state."""
    from . import _C
    g = torch.Generator().manual_seed(0)
    b, h, P = (256 if N == 64 else 128), 32, 64
    r = lambda *s: torch.randn(*s, generator=g)
    U = r(b, h, P).to(torch.bfloat16).to(dev)
    Bv = (r(b, h, 2 * N) / N ** 0.5).to(torch.bfloat16).to(dev)
    Cv = (r(b, h, 2 * N) / N ** 0.5).to(torch.bfloat16).to(dev)
    rad = torch.clamp(torch.exp(-torch.nn.functional.softplus(r(b, h))), 0.9, 0.999)
    th = (torch.rand(b, h, generator=g) * 2 - 1) * torch.pi
    M = torch.stack([rad * torch.cos(th), rad * torch.sin(th)], -1).contiguous().to(dev)
    K = (0.05 * r(b, h, 2, 2)).to(dev)
    state = (0.1 * r(b, h, P, 2 * N)).to(dev)
    state2 = torch.empty_like(state)
    Bp, Up = torch.zeros_like(Bv), torch.zeros_like(U)
    cfg = f"config 3: batch {b} x heads 32 x P 64 x N {N}, one token"

    def out_of_place():
        _C.scan_decode(U, M, K, Bv, Cv, state, Bp, Up, y_dtype=torch.bfloat16, state_out=state2)

    def in_place():
        _C.scan_decode(U, M, K, Bv, Cv, state, Bp, Up, y_dtype=torch.bfloat16, state_out=state)

    algo = nbytes(state, state2, U, Bv, Cv, M, K, Bp, Up) + nbytes(U)
    lines = [report("sl_v2x2ssd_decode (state out of place)", time_ms(out_of_place, iters), algo, cfg),
             report("sl_v2x2ssd_decode (state in place)", time_ms(in_place, iters), algo, cfg)]

    # the same call as a serving loop would issue it: 16 tokens captured once in a CUDA graph
    # (state ping-pongs between two buffers), then replayed
    tokens = 16

    def loop():
        a, b2 = state, state2
        for _ in range(tokens):
            _C.scan_decode(U, M, K, Bv, Cv, a, Bp, Up, y_dtype=torch.bfloat16, state_out=b2)
            a, b2 = b2, a

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        loop()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        loop()
    ms = time_ms(graph.replay, max(2, iters // 4)) / tokens
    lines.append(report("sl_v2x2ssd_decode (CUDA-graph replay of 16 tokens, per token)", ms, algo, cfg,
                        {"us_per_sequence_token": ms * 1e3 / b, "tokens_per_s": b / (ms * 1e-3)}))
    return lines


def measure_decode_sequence(iters, dev, steps=1024, batch=256):
    """Config 3 as the reference's decode harness runs it (scripts/perf/_training_decode.py:182-214):
    ``steps`` CONSECUTIVE tokens with fresh per-token inputs over the carried float32 state, one pair
    of CUDA events around all of them; eager launches, then the whole sequence replayed from one CUDA
    graph.  Per-token inputs are drawn on the device (5.3 MB per token)."""
    from . import _C
    h, P, N = 32, 64, 64
    g = torch.Generator(device=dev).manual_seed(3)
    r = lambda *s: torch.randn(*s, generator=g, device=dev)
    U = r(steps, batch, h, P).to(torch.bfloat16)
    Bv = (r(steps, batch, h, 2 * N) / N ** 0.5).to(torch.bfloat16)
    Cv = (r(steps, batch, h, 2 * N) / N ** 0.5).to(torch.bfloat16)
    rad = torch.clamp(torch.exp(-torch.nn.functional.softplus(r(steps, batch, h))), 0.9, 0.999)
    th = (torch.rand(steps, batch, h, generator=g, device=dev) * 2 - 1) * torch.pi
    M = torch.stack([rad * torch.cos(th), rad * torch.sin(th)], -1).contiguous()
    K = 0.05 * r(steps, batch, h, 2, 2)
    state0 = 0.1 * r(batch, h, P, 2 * N)
    state = state0.clone()
    zeroB, zeroU = torch.zeros_like(Bv[0]), torch.zeros_like(U[0])
    Y = torch.empty(steps, batch, h, P, dtype=torch.bfloat16, device=dev)

    def sequence():
        for t in range(steps):      # the carried taps are the previous token's B and U
            bp, up = (zeroB, zeroU) if t == 0 else (Bv[t - 1], U[t - 1])
            y, _ = _C.scan_decode(U[t], M[t], K[t], Bv[t], Cv[t], state, bp, up,
                                  y_dtype=torch.bfloat16, state_out=state)
            Y[t].copy_(y)

    algo = 2 * nbytes(state) + nbytes(U[0], Bv[0], Cv[0], M[0], K[0], zeroB, zeroU) + nbytes(U[0])
    cfg = f"config 3: batch {batch} x heads 32 x P 64 x N 64, {steps} consecutive tokens, fresh inputs per token"
    lines = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sequence()                     # warm-up pass
    torch.cuda.synchronize()
    state.copy_(state0)
    e0.record(); sequence(); e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    extra = lambda m: {"us_per_step": m * 1e3, "tokens_per_s": batch / (m * 1e-3), "steps": steps}
    lines.append(report("decode sequence, eager launches (per step; includes the copy of y)", ms, algo, cfg, extra(ms)))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        sequence()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sequence()
    state.copy_(state0)
    graph.replay()
    torch.cuda.synchronize()
    state.copy_(state0)
    e0.record(); graph.replay(); e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    lines.append(report("decode sequence, one CUDA graph of all steps (per step)", ms, algo, cfg, extra(ms)))
    return lines


def _mixer_tensors(dev, batch=8, T=2048, heads=32, P=64, N=64):
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g)
    d_inner = heads * P
    proj = r(batch, T, 2 * d_inner).to(torch.bfloat16).to(dev)      # gate | value, as in_proj leaves them
    gate, value = proj[..., :d_inner], proj[..., d_inner:]
    params = r(batch, T, 3 * heads).to(torch.bfloat16).to(dev)
    bc = r(batch, T, heads, 4, N).to(torch.bfloat16).to(dev)
    w = (0.3 * r(d_inner, 4)).to(torch.bfloat16).to(dev)
    bias = (0.1 * r(d_inner)).to(torch.bfloat16).to(dev)
    return gate, value, params, bc, w, bias


def measure_scanprep(iters, dev, batch=8):
    """Config 2 sizes: batch 8, T 2048, heads 32, P 64, N 64, conv width 4, bf16."""
    from . import _C
    from .layers import SLinOSSScanPrep
    heads, P, N = 32, 64, 64
    gate, value, params, bc, w, bias = _mixer_tensors(dev, batch=batch)
    owner = SLinOSSScanPrep(n_heads=heads, d_state=N, d_head=P, device=dev)
    biases = tuple(getattr(owner, k).detach().float().contiguous()
                   for k in ("dt_bias", "alpha_bias", "theta_mod_bias", "theta_bias", "theta_sign"))
    cfg = _C.make_config(owner)
    name = f"config 2: batch {batch} x T 2048 x heads 32 x P 64 x N 64, conv width 4, bf16"
    outs = _C.scanprep_conv_fwd(value, w, bias, None, params, bc, biases, cfg, heads=heads, P=P,
                                want_state=True)
    U, M, K, Bo, Co, nstate = outs
    vbytes = value.shape[0] * value.shape[1] * value.shape[2] * 2
    algo_f = vbytes + nbytes(params, bc, w, bias, U, M, K, Bo, Co, nstate)
    lines = [report("sl_scanprep_conv_fwd (conv + SiLU + scan preparation, 3 kernels)",
                    time_ms(lambda: _C.scanprep_conv_fwd(value, w, bias, None, params, bc, biases, cfg,
                                                         heads=heads, P=P, want_state=True), iters),
                    algo_f, name)]
    dU, dM, dK = torch.randn_like(U), torch.randn_like(M), torch.randn_like(K)
    dB, dC = torch.randn_like(Bo), torch.randn_like(Co)
    res = _C.scanprep_conv_bwd(value, w, bias, None, params, bc, biases, cfg, dU, dM, dK, dB, dC,
                               heads=heads, P=P)
    algo_b = vbytes + nbytes(params, bc, w, bias, dU, dM, dK, dB, dC, res["d_value"], res["d_params"],
                             res["d_bc"])
    lines.append(report("sl_scanprep_conv_bwd (3 kernels; includes zeroing of the float32 accumulators)",
                        time_ms(lambda: _C.scanprep_conv_bwd(value, w, bias, None, params, bc, biases, cfg,
                                                             dU, dM, dK, dB, dC, heads=heads, P=P), iters),
                        algo_b, name))
    return lines


def measure_tail(iters, dev, batch=8):
    from . import _C
    heads, P = 32, 64
    gate, value, *_ = _mixer_tensors(dev, batch=batch)
    g = torch.Generator().manual_seed(1)
    Y = torch.randn(batch, heads, 2048, P, generator=g).to(torch.bfloat16).to(dev)
    Uskip = torch.randn(batch, heads, 2048, P, generator=g).to(torch.bfloat16).to(dev)
    d_skip = torch.ones(heads, device=dev)
    wn = torch.ones(heads * P, device=dev, dtype=torch.bfloat16)
    name = f"config 2: batch {batch} x T 2048 x d_inner 2048 (32 heads x 64), bf16"
    normed = _C.mixer_tail_fwd(Y, gate, Uskip, d_skip, wn, 1e-5)
    gbytes = gate.shape[0] * gate.shape[1] * gate.shape[2] * 2
    lines = [report("sl_mixer_tail_fwd", time_ms(lambda: _C.mixer_tail_fwd(Y, gate, Uskip, d_skip, wn, 1e-5), iters),
                    nbytes(Y, Uskip, normed) + gbytes, name)]
    dn = torch.randn_like(normed)
    outs = _C.mixer_tail_bwd(Y, gate, Uskip, d_skip, wn, 1e-5, dn)
    lines.append(report("sl_mixer_tail_bwd (includes zeroing of the float32 accumulators)",
                        time_ms(lambda: _C.mixer_tail_bwd(Y, gate, Uskip, d_skip, wn, 1e-5, dn), iters),
                        nbytes(Y, Uskip, dn, outs[0], outs[1], outs[2]) + gbytes, name))
    return lines


def measure_mixer(iters, dev, batch=8):
    """Whole mixer layer, forward + backward, config 2 (GEMMs are cuBLAS; tensor-pipe bound)."""
    import slinoss_b200 as sb
    torch.manual_seed(0)
    mixer = sb.SLinOSSMixer(1024, d_state=64, expand=2, d_head=64, d_conv=4, chunk_size=64).to(dev).to(torch.bfloat16)
    x = torch.randn(batch, 2048, 1024, device=dev, dtype=torch.bfloat16, requires_grad=True)

    def step():
        out = mixer(x)
        out.backward(out)
        mixer.zero_grad(set_to_none=True)
        x.grad = None

    ms = time_ms(step, max(3, iters // 4))
    flops = 3 * 2 * batch * 2048 * 1024 * (12384 + 2048)    # in_proj + out_proj, fwd + 2x bwd
    return [emit({"call": "SLinOSSMixer forward+backward (config 2)", "ms": ms,
                  "tokens_per_s": batch * 2048 / (ms * 1e-3), "gemm_tflops_equivalent": flops / (ms * 1e-3) / 1e12,
                  "config": f"x ({batch}, 2048, 1024) bf16, d_inner 2048, 32 heads x 64, N 64, d_conv 4"})]


def measure_mixer_step(iters, dev, batch=256, N=64):
    """One decode token of the whole mixer (d_model 1024, 32 heads x 64, N 64, conv width 4, bf16) at
    the decode configuration's batch: in_proj, the one-launch fused step, out_proj.  Eager through
    ``SLinOSSMixer.step`` and replayed from the CUDA-graph engine; the traffic that bounds it is the
    float32 state read and written once (2 x 268 MB at batch 256)."""
    import slinoss_b200 as sb
    from .engine import MixerDecodeEngine
    torch.manual_seed(0)
    m = sb.SLinOSSMixer(1024, d_state=N, expand=2, d_head=64, d_conv=4, chunk_size=64).to(dev).to(torch.bfloat16)
    x = torch.randn(batch, 1024, device=dev, dtype=torch.bfloat16)
    algo = 2 * batch * 32 * 64 * 2 * N * 4
    cfg = f"SLinOSSMixer.step: batch {batch}, d_model 1024, 32 heads x 64, N {N}, d_conv 4, bf16"
    lines = []
    with torch.no_grad():
        _, state = m.step(x, None)

        def eager():
            m.step(x, state, inplace=True)

        ms = time_ms(eager, max(iters, 20))
        lines.append(report("SLinOSSMixer.step, eager (in_proj + fused step + out_proj, per token)", ms, algo, cfg,
                            {"us_per_step": ms * 1e3, "tokens_per_s": batch / (ms * 1e-3)}))
        eng = MixerDecodeEngine(m, batch)
        ms = time_ms(lambda: eng.step(x), max(iters, 20))
        lines.append(report("MixerDecodeEngine.step, CUDA-graph replay (per token)", ms, algo, cfg,
                            {"us_per_step": ms * 1e3, "tokens_per_s": batch / (ms * 1e-3)}))
        m.decode_backend.fused = False
        _, state2 = m.step(x, None)
        ms = time_ms(lambda: m.step(x, state2, inplace=True), max(iters, 20))
        lines.append(report("SLinOSSMixer.step with separate launches (conv, scan preparation, decode, tail)", ms, algo,
                            cfg, {"us_per_step": ms * 1e3, "tokens_per_s": batch / (ms * 1e-3)}))
    return lines


def measure_scan(iters, dev):
    """Config 1 scan forward / backward through the C ABI (the figures bench.py headlines)."""
    from . import _C
    from .synthetic import make_scan_case
    c = make_scan_case(8, 16, 4096, 64, 64, dtype=torch.bfloat16, seed=0).to(dev)
    name = "config 1: batch 8 x heads 16 x T 4096 x P 64 x N 64, bf16"
    fwd = lambda: _C.scan_fwd(c.U, c.M, c.K, c.B, c.C, None, None, None, chunk_size=64,
                              y_dtype=torch.bfloat16, want_final=False, save_states=True)
    _, fin, st = fwd()
    bht = 8 * 16 * 4096
    # the same size with grouped B/C (4 heads per group) and with carried taps + carried state:
    # what segmented (streaming-state) training and bc_groups < heads models run
    g = make_scan_case(8, 16, 4096, 64, 64, groups=4, dtype=torch.bfloat16, seed=1, streaming=True,
                       with_init=True).to(dev)
    _, gfin, gst = _C.scan_fwd(g.U, g.M, g.K, g.B, g.C, g.initial_states, g.B_prev, g.U_prev, chunk_size=64,
                               y_dtype=torch.bfloat16, want_final=True, save_states=True)
    gname = name + ", 4 groups of B/C, carried state and taps"
    gbytes = bht * (1456 - 2 * 256 + 2 * 64) + 2 * 8 * 16 * 64 * 128 * 4   # B, C, dB, dC shrink 4x; + z0, d_initial
    grouped = [report("sl_v2x2ssd_bwd (grouped B/C, carried state and taps; saved chunk states)",
                      time_ms(lambda: _C.scan_bwd(g.U, g.M, g.K, g.B, g.C, g.initial_states, g.B_prev, g.U_prev,
                                                  g.dY, None, chunk_size=64, saved=(gst, gfin)), iters),
                      gbytes, gname)]
    # the same step through the public op and autograd (device-resident tensors): what a training loop calls
    from .ops.v2x2ssd import v2x2ssd_cute
    leaves = [t.clone().requires_grad_(True) for t in c.tensors()]

    def op_step():
        Y = v2x2ssd_cute(*leaves, chunk_size=64)
        torch.autograd.grad(Y, leaves, c.dY)

    through_op = [report("v2x2ssd_cute forward + torch.autograd.grad (public op, tensors on the device)",
                         time_ms(op_step, iters), bht * (792 + 1456), name)]
    return grouped + through_op + [report("sl_v2x2ssd_fwd (saving chunk states)", time_ms(fwd, iters), bht * 792, name),
            report("sl_v2x2ssd_bwd (saved chunk states)",
                   time_ms(lambda: _C.scan_bwd(c.U, c.M, c.K, c.B, c.C, None, None, None, c.dY, None,
                                               chunk_size=64, saved=(st, fin)), iters), bht * 1456, name),
            report("sl_v2x2ssd_bwd (recomputing chunk states)",
                   time_ms(lambda: _C.scan_bwd(c.U, c.M, c.K, c.B, c.C, None, None, None, c.dY, None,
                                               chunk_size=64), iters), bht * 1456, name)]


def measure_ffn_rows(iters, dev, rows=16384, C=2048, hidden=8192):
    """Row-wise kernels of the FFN branch at the stacked-LM size: 4 x 4096 rows of d_model 2048, hidden 8192."""
    from . import _C
    g = torch.Generator().manual_seed(2)
    x = torch.randn(rows, C, generator=g).to(torch.bfloat16).to(dev)
    dy = torch.randn(rows, C, generator=g).to(torch.bfloat16).to(dev)
    w = torch.ones(C, dtype=torch.bfloat16, device=dev)
    proj = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(dev)
    dh = torch.randn(rows, hidden, generator=g).to(torch.bfloat16).to(dev)
    name = f"config 4 rows: {rows} x d_model {C} (hidden {hidden}), bf16"
    rc, rh = rows * C * 2, rows * hidden * 2
    return [report("sl_rmsnorm_fwd", time_ms(lambda: _C.rmsnorm_fwd(x, w, 1e-5), iters), 2 * rc, name),
            report("sl_rmsnorm_bwd (includes zeroing of d_weight)",
                   time_ms(lambda: _C.rmsnorm_bwd(x, w, 1e-5, dy), iters), 3 * rc, name),
            report("sl_ffn_activation_fwd (GELU)", time_ms(lambda: _C.ffn_activation_fwd(proj, "gelu"), iters),
                   2 * rh, name),
            report("sl_ffn_activation_bwd (GELU)", time_ms(lambda: _C.ffn_activation_bwd(proj, dh, "gelu"), iters),
                   3 * rh, name)]


def measure_scan_n128(iters, dev):
    """The config-1 streams with 128 state columns (the mixer's default d_state): two passes over the
    column blocks of B and C."""
    from . import _C
    from .synthetic import make_scan_case
    c = make_scan_case(8, 16, 4096, 64, 128, dtype=torch.bfloat16, seed=0).to(dev)
    name = "batch 8 x heads 16 x T 4096 x P 64 x N 128, bf16"
    fwd = lambda: _C.scan_fwd(c.U, c.M, c.K, c.B, c.C, None, None, None, chunk_size=64,
                              y_dtype=torch.bfloat16, want_final=False, save_states=True)
    _, fin, st = fwd()
    bht = 8 * 16 * 4096
    return [report("sl_v2x2ssd_fwd, N = 128 (saving chunk states)", time_ms(fwd, iters), bht * 1304, name),
            report("sl_v2x2ssd_bwd, N = 128 (saved chunk states)",
                   time_ms(lambda: _C.scan_bwd(c.U, c.M, c.K, c.B, c.C, None, None, None, c.dY, None,
                                               chunk_size=64, saved=(st, fin)), iters), bht * 2480, name)]


WHAT = {"mixer_step_n128": lambda iters, dev: measure_mixer_step(iters, dev, batch=128, N=128), "decode_n128": lambda iters, dev: measure_decode(iters, dev, N=128), "scan_n128": measure_scan_n128, "ffn_rows": measure_ffn_rows, "decode": measure_decode, "decode_sequence": measure_decode_sequence, "mixer_step": measure_mixer_step,
        "scanprep": measure_scanprep, "tail": measure_tail, "mixer": measure_mixer, "scan": measure_scan}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="decode,decode_sequence,mixer_step,scanprep,tail,mixer,scan,scan_n128,ffn_rows")
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("slinoss_b200.measure needs a CUDA device: the kernels have no CPU path.")
    dev = torch.device("cuda", torch.cuda.current_device())
    for k in args.what.split(","):
        WHAT[k.strip()](args.iters, dev)


if __name__ == "__main__":
    main()
