"""ctypes binding of ``libslinoss_b200.so`` (the C-ABI CUDA library).

Two layers live here:

* ``lib()`` loads the shared library built in-tree by ``slinoss_b200.build`` and
  declares the prototypes of every ``sl_*`` symbol of ``include/slinoss_b200.h``.
  There is no fallback: if the library is missing, ``lib()`` raises.
* tensor-level launchers (``scan_fwd``, ``scan_bwd``, ``scan_decode``,
  ``scanprep_conv_fwd`` ...) that allocate outputs and scratch with torch, pass raw
  device pointers and torch's *current stream* to the C functions and turn
  non-zero status codes into exceptions.  The ops in ``slinoss_b200.ops`` only
  talk to these launchers.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libslinoss_b200.so"
_lib = None

SL_F32, SL_BF16, SL_F16 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TC = 0, 1, 2
WS_SCAN_FWD, WS_SCAN_BWD, WS_SCAN_STATES = 0, 1, 4

_DTYPE_CODE = {torch.float32: SL_F32, torch.bfloat16: SL_BF16, torch.float16: SL_F16}
_PATHS = {"auto": PATH_AUTO, "simt": PATH_SIMT, "tc": PATH_TC}


class ScanPrepConfig(ctypes.Structure):
    _fields_ = [(n, c_float) for n in (
        "dt_min", "dt_max", "alpha_min", "alpha_max", "theta_init_min", "theta_init_max",
        "theta_mod_scale", "r_min", "r_max", "eps")]


_P = c_void_p
_PROTOTYPES = {
    "sl_version": (c_int, []),
    "sl_kernel_launches": (ctypes.c_ulonglong, []),
    "sl_device_status": (c_int, []),
    "sl_device_status_reset": (c_int, []),
    "sl_status_string": (ctypes.c_char_p, [c_int]),
    "sl_last_cuda_error": (ctypes.c_char_p, []),
    "sl_workspace_bytes": (c_size_t, [c_int] * 10),
    "sl_v2x2ssd_fwd": (c_int, [_P] * 11 + [c_int] * 10 + [_P, c_size_t, _P]),
    "sl_v2x2ssd_bwd": (c_int, [_P] * 20 + [c_int] * 10 + [_P, c_size_t, _P]),
    "sl_static_scratch_bytes": (c_size_t, []),
    "sl_v2x2ssd_bwd_static": (c_int, [_P] * 18 + [c_int] * 8 + [_P]),
    "sl_v2x2ssd_decode": (c_int, [_P] * 10 + [c_int] * 7 + [_P]),
    "sl_scanprep_conv_fwd": (c_int, [_P, c_int64, _P, _P, _P, _P, c_int, _P, _P, _P, _P, _P, _P, _P,
                                     ctypes.POINTER(ScanPrepConfig), _P, c_int64, c_int64, c_int64,
                                     _P, _P, _P, _P] + [c_int] * 7 + [_P]),
    "sl_scanprep_conv_bwd": (c_int, [_P, c_int64, _P, _P, _P, c_int, _P, _P, _P, _P, _P, _P, _P,
                                     ctypes.POINTER(ScanPrepConfig), _P, c_int64, c_int64, c_int64,
                                     _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]
                             + [c_int] * 7 + [_P]),
    "sl_mixer_decode_step_workspace_bytes": (c_size_t, [c_int] * 3),
    "sl_mixer_decode_step": (c_int, [_P, c_int64, _P, c_int64, _P, _P, _P, _P, _P, c_int, _P, _P, _P, _P, _P,
                                     ctypes.POINTER(ScanPrepConfig), _P, _P, c_float, _P, _P, _P, _P, _P, _P,
                                     c_size_t] + [c_int] * 6 + [_P]),
    "sl_rmsnorm_fwd": (c_int, [_P, _P, c_float, _P, ctypes.c_longlong, c_int, c_int, _P]),
    "sl_rmsnorm_bwd": (c_int, [_P, _P, c_float, _P, _P, _P, ctypes.c_longlong, c_int, c_int, _P]),
    "sl_ffn_activation_fwd": (c_int, [_P, _P, ctypes.c_longlong, c_int, c_int, c_int, _P]),
    "sl_ffn_activation_bwd": (c_int, [_P, _P, _P, ctypes.c_longlong, c_int, c_int, c_int, _P]),
    "sl_mixer_tail_fwd": (c_int, [_P, _P, c_int64, _P, _P, _P, c_float, _P] + [c_int] * 5 + [_P]),
    "sl_mixer_tail_bwd": (c_int, [_P, _P, c_int64, _P, _P, _P, c_float, _P, _P, _P, _P, _P, _P]
                          + [c_int] * 5 + [_P]),
}
EXPORTED_SYMBOLS = tuple(_PROTOTYPES)


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    """The loaded C-ABI library.  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"slinoss_b200: CUDA library {_LIB_PATH} is missing. Build it with "
                "`python -m slinoss_b200.build` (needs nvcc); there is no fallback path.")
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (restype, argtypes) in _PROTOTYPES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def kernel_launches() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib().sl_kernel_launches())


def device_status() -> int:
    """0, or the status code SL_ERR_DEVICE_TIMEOUT (7) if a kernel gave up a bounded wait since
    the last reset; synchronises."""
    return int(lib().sl_device_status())


def device_status_reset() -> int:
    """Site code of the first expired wait (0 = none); clears the record; synchronises."""
    return int(lib().sl_device_status_reset())


def check(status: int, what: str) -> None:
    if status != 0:
        text = lib().sl_status_string(status).decode()
        if status == 6:   # SL_ERR_LAUNCH_FAILED: add the CUDA runtime's own words
            text += f" ({lib().sl_last_cuda_error().decode()})"
        raise RuntimeError(f"slinoss_b200.{what} failed with status {status}: {text}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; expected float32, bfloat16 or float16") from None


def require_cuda(*tensors) -> torch.device:
    """All tensors must live on one CUDA device (the kernels have no CPU path)."""
    dev = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise ValueError("slinoss_b200 kernels require CUDA tensors.")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("All tensors must be on the same device.")
    return dev


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _workspace(kind, dev, batch, heads, groups, T, P, N, chunk, io, path):
    nbytes = lib().sl_workspace_bytes(kind, batch, heads, groups, T, P, N, chunk, io, path)
    if nbytes == 0:
        return None, 0
    return torch.empty(nbytes, dtype=torch.uint8, device=dev), nbytes


def workspace_bytes(kind, batch, heads, groups, T, P, N, chunk, io_dtype, path="auto") -> int:
    return int(lib().sl_workspace_bytes(kind, batch, heads, groups, T, P, N, chunk,
                                        dtype_code(io_dtype), _PATHS[path]))


# ---------------------------------------------------------------------------------
# scan
# ---------------------------------------------------------------------------------
def scan_fwd(U, M, K, B, C, z0, B_prev, U_prev, *, chunk_size, y_dtype, want_final, path="auto",
             save_states=False):
    """Launch ``sl_v2x2ssd_fwd``.  ``U,B,C,B_prev,U_prev`` share one dtype; ``M,K,z0``
    are float32.  Returns ``(Y, final_state or None)``; with ``save_states`` a third item:
    the chunk-state buffer for ``scan_bwd`` (None when the chosen path keeps none)."""
    dev = require_cuda(U, M, K, B, C, z0, B_prev, U_prev)
    batch, heads, T, P = U.shape
    groups, N = B.shape[1], B.shape[3] // 2
    io, pcode = dtype_code(U.dtype), _PATHS[path]
    Y = torch.empty((batch, heads, T, P), dtype=y_dtype, device=dev)
    states = None
    with torch.cuda.device(dev):
        if save_states:
            sbytes = lib().sl_workspace_bytes(WS_SCAN_STATES, batch, heads, groups, T, P, N,
                                              chunk_size, io, pcode)
            if sbytes:
                states = torch.empty(sbytes, dtype=torch.uint8, device=dev)
        final = torch.empty((batch, heads, P, 2 * N), dtype=torch.float32, device=dev) \
            if (want_final or states is not None) else None
        ws, nbytes = _workspace(WS_SCAN_FWD, dev, batch, heads, groups, T, P, N, chunk_size, io, pcode)
        check(lib().sl_v2x2ssd_fwd(
            _ptr(U), _ptr(M), _ptr(K), _ptr(B), _ptr(C), _ptr(z0), _ptr(B_prev), _ptr(U_prev),
            _ptr(Y), _ptr(final), _ptr(states), batch, heads, groups, T, P, N, chunk_size, io,
            dtype_code(y_dtype), pcode, _ptr(ws), nbytes, _stream(dev)), "sl_v2x2ssd_fwd")
    if save_states:
        return Y, final, states
    return Y, final


def scan_bwd(U, M, K, B, C, z0, B_prev, U_prev, dY, d_final, *, chunk_size, path="auto",
             saved=None):
    """Launch ``sl_v2x2ssd_bwd``.  Returns ``(dU, dM, dK, dB, dC, d_initial, dB_prev,
    dU_prev)``; the last three are None when the matching input is absent.  ``saved`` is
    ``(chunk_states, final_state)`` from ``scan_fwd(..., save_states=True)`` or None."""
    dev = require_cuda(U, M, K, B, C, z0, B_prev, U_prev, dY, d_final)
    states, zfinal = saved if (saved is not None and saved[0] is not None) else (None, None)
    batch, heads, T, P = U.shape
    groups, N = B.shape[1], B.shape[3] // 2
    io, pcode = dtype_code(U.dtype), _PATHS[path]
    dU = torch.empty_like(U)
    dM = torch.empty((batch, heads, T, 2), dtype=torch.float32, device=dev)
    dK = torch.empty((batch, heads, T, 2, 2), dtype=torch.float32, device=dev)
    dB = torch.empty_like(B)
    dC = torch.empty_like(C)
    d_init = torch.empty((batch, heads, P, 2 * N), dtype=torch.float32, device=dev) \
        if z0 is not None else None
    dB_prev = torch.empty_like(B_prev) if B_prev is not None else None
    dU_prev = torch.empty_like(U_prev) if U_prev is not None else None
    dy_code = dtype_code(dY.dtype) if dY is not None else io
    with torch.cuda.device(dev):
        ws, nbytes = _workspace(WS_SCAN_BWD, dev, batch, heads, groups, T, P, N, chunk_size, io, pcode)
        check(lib().sl_v2x2ssd_bwd(
            _ptr(U), _ptr(M), _ptr(K), _ptr(B), _ptr(C), _ptr(z0), _ptr(B_prev), _ptr(U_prev),
            _ptr(states), _ptr(zfinal), _ptr(dY), _ptr(d_final), _ptr(dU), _ptr(dM), _ptr(dK),
            _ptr(dB), _ptr(dC), _ptr(d_init), _ptr(dB_prev), _ptr(dU_prev), batch, heads, groups,
            T, P, N, chunk_size, io, dy_code, pcode, _ptr(ws), nbytes, _stream(dev)),
            "sl_v2x2ssd_bwd")
    return dU, dM, dK, dB, dC, d_init, dB_prev, dU_prev


def scan_bwd_static(U, M, K, B, C, z0, B_prev, U_prev, dY, d_final, outs):
    """Launch ``sl_v2x2ssd_bwd_static``: the float32-exact backward with its scratch in the
    library's built-in array, for callers that may not allocate device memory.

    Nothing is allocated here either: ``outs`` is the tuple of caller-provided result
    tensors ``(dU, dM, dK, dB, dC, d_initial, dB_prev, dU_prev)`` (the last three may be
    None).  Calls share the one scratch array, so keep them on one stream."""
    dev = require_cuda(U, M, K, B, C, z0, B_prev, U_prev, dY, d_final, *outs)
    batch, heads, T, P = U.shape
    groups, N = B.shape[1], B.shape[3] // 2
    dy_code = dtype_code(dY.dtype) if dY is not None else dtype_code(U.dtype)
    with torch.cuda.device(dev):
        check(lib().sl_v2x2ssd_bwd_static(
            _ptr(U), _ptr(M), _ptr(K), _ptr(B), _ptr(C), _ptr(z0), _ptr(B_prev), _ptr(U_prev),
            _ptr(dY), _ptr(d_final), *[_ptr(o) for o in outs], batch, heads, groups, T, P, N,
            dtype_code(U.dtype), dy_code, _stream(dev)), "sl_v2x2ssd_bwd_static")
    return outs


def scan_decode(U, M, K, B, C, state, B_prev, U_prev, *, y_dtype, state_out=None):
    """Launch ``sl_v2x2ssd_decode``: one token over the carried float32 state.
    ``state_out`` defaults to a fresh tensor; pass ``state`` itself to update in place."""
    dev = require_cuda(U, M, K, B, C, state, B_prev, U_prev)
    batch, heads, P = U.shape
    groups, N = B.shape[1], B.shape[2] // 2
    Y = torch.empty((batch, heads, P), dtype=y_dtype, device=dev)
    if state_out is None:
        state_out = torch.empty_like(state)
    with torch.cuda.device(dev):
        check(lib().sl_v2x2ssd_decode(
            _ptr(U), _ptr(M), _ptr(K), _ptr(B), _ptr(C), _ptr(state), _ptr(B_prev), _ptr(U_prev),
            _ptr(Y), _ptr(state_out), batch, heads, groups, P, N, dtype_code(U.dtype),
            dtype_code(y_dtype), _stream(dev)), "sl_v2x2ssd_decode")
    return Y, state_out


# ---------------------------------------------------------------------------------
# scan preparation (+ causal conv)
# ---------------------------------------------------------------------------------
def make_config(owner) -> ScanPrepConfig:
    return ScanPrepConfig(owner.dt_min, owner.dt_max, owner.alpha_min, owner.alpha_max,
                          owner.theta_init_min, owner.theta_init_max, owner.theta_mod_scale,
                          owner.r_min, owner.r_max, owner.eps)


def _row_stride(x: torch.Tensor) -> int:
    """Row stride (elements) of a (batch, T, C) tensor whose channels are dense and
    whose batch stride is T * row stride (a column slice of a dense buffer)."""
    if x.stride(2) != 1 or (x.shape[0] > 1 and x.stride(0) != x.shape[1] * x.stride(1)):
        raise ValueError(f"expected a row-strided (batch,T,C) tensor, got strides {x.stride()}")
    return int(x.stride(1)) if x.shape[1] > 1 else max(int(x.stride(1)), int(x.shape[2]))


def as_rows(x: torch.Tensor) -> torch.Tensor:
    """Return ``x`` (batch,T,C) in a layout `_row_stride` accepts, copying only if needed."""
    if x.stride(2) == 1 and (x.shape[0] == 1 or x.stride(0) == x.shape[1] * x.stride(1)) \
            and (x.shape[1] > 1 or x.stride(1) >= x.shape[2]):
        return x
    return x.contiguous()


def scanprep_conv_fwd(value, conv_weight, conv_bias, conv_state, params, bc, biases, cfg, *,
                      heads, P, u_layout="bhtp", want_state=False):
    """Launch ``sl_scanprep_conv_fwd``.

    ``value`` (batch,T,heads*P) row-strided or None; ``params`` (batch,T,3*heads) or None;
    ``bc`` (batch,T,groups,4,N) or None; ``biases`` = (dt_bias, alpha_bias, theta_mod_bias,
    theta_bias, theta_sign).  Returns ``(U, M, K, B, C, next_conv_state)`` with None for
    skipped parts.  ``u_layout`` "bhtp" gives (batch,heads,T,P), "btc" (batch,T,heads*P)."""
    ref = value if value is not None else (params if params is not None else bc)
    dev = require_cuda(value, conv_weight, conv_bias, conv_state, params, bc, *(biases or ()))
    batch, T = ref.shape[0], ref.shape[1]
    io = dtype_code(ref.dtype)
    U = M = K = Bo = Co = nstate = None
    usb = ush = ust = 0
    vstride = 0
    d_conv = 1
    if value is not None:
        value = as_rows(value)
        vstride = _row_stride(value)
        if u_layout == "bhtp":
            U = torch.empty((batch, heads, T, P), dtype=value.dtype, device=dev)
            usb, ush, ust = heads * T * P, T * P, P
        else:
            U = torch.empty((batch, T, heads * P), dtype=value.dtype, device=dev)
            usb, ush, ust = T * heads * P, P, heads * P
        if conv_weight is not None:
            d_conv = int(conv_weight.shape[1])
            if want_state:
                nstate = torch.empty((batch, heads * P, d_conv - 1), dtype=value.dtype, device=dev)
    groups = N = 1
    if bc is not None:
        groups, N = int(bc.shape[2]), int(bc.shape[4])
        Bo = torch.empty((batch, groups, T, 2 * N), dtype=bc.dtype, device=dev)
        Co = torch.empty_like(Bo)
    if params is not None:
        M = torch.empty((batch, heads, T, 2), dtype=torch.float32, device=dev)
        K = torch.empty((batch, heads, T, 2, 2), dtype=torch.float32, device=dev)
    b5 = list(biases) if biases is not None else [None] * 5
    with torch.cuda.device(dev):
        check(lib().sl_scanprep_conv_fwd(
            _ptr(value), vstride, _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state),
            _ptr(nstate), d_conv, _ptr(params), _ptr(bc), *[_ptr(b) for b in b5],
            ctypes.byref(cfg) if cfg is not None else None, _ptr(U), usb, ush, ust, _ptr(M),
            _ptr(K), _ptr(Bo), _ptr(Co), batch, heads, groups, T, P, N, io, _stream(dev)),
            "sl_scanprep_conv_fwd")
    return U, M, K, Bo, Co, nstate


def scanprep_conv_bwd(value, conv_weight, conv_bias, conv_state, params, bc, biases, cfg, dU, dM,
                      dK, dBo, dCo, *, heads, P, u_layout="bhtp", want_dstate=False):
    """Launch ``sl_scanprep_conv_bwd``.  Returns a dict with d_value, d_conv_weight,
    d_conv_bias, d_conv_state, d_params, d_bc, d_dt_bias, d_alpha_bias,
    d_theta_mod_bias, d_theta_bias (None for skipped parts; bias / weight gradients
    are float32 accumulators)."""
    ref = value if value is not None else (params if params is not None else bc)
    dev = require_cuda(value, conv_weight, conv_bias, conv_state, params, bc, dU, dM, dK, dBo, dCo)
    batch, T = ref.shape[0], ref.shape[1]
    io = dtype_code(ref.dtype)
    out = dict.fromkeys(("d_value", "d_conv_weight", "d_conv_bias", "d_conv_state", "d_params",
                         "d_bc", "d_dt_bias", "d_alpha_bias", "d_theta_mod_bias", "d_theta_bias"))
    usb = ush = ust = 0
    vstride = 0
    d_conv = 1
    f32 = dict(dtype=torch.float32, device=dev)
    if dU is not None:
        value = as_rows(value)
        vstride = _row_stride(value)
        dU = dU.contiguous()
        if u_layout == "bhtp":
            usb, ush, ust = heads * T * P, T * P, P
        else:
            usb, ush, ust = T * heads * P, P, heads * P
        out["d_value"] = torch.empty((batch, T, heads * P), dtype=value.dtype, device=dev)
        if conv_weight is not None:
            d_conv = int(conv_weight.shape[1])
            out["d_conv_weight"] = torch.zeros((heads * P, d_conv), **f32)
            out["d_conv_bias"] = torch.zeros((heads * P,), **f32)
            if want_dstate and d_conv > 1:
                out["d_conv_state"] = torch.zeros((batch, heads * P, d_conv - 1),
                                                  dtype=value.dtype, device=dev)
    groups = N = 1
    if dBo is not None:
        groups, N = int(bc.shape[2]), int(bc.shape[4])
        dBo, dCo = dBo.contiguous(), dCo.contiguous()
        out["d_bc"] = torch.empty(bc.shape, dtype=bc.dtype, device=dev)
    if dM is not None:
        dM, dK = dM.contiguous(), dK.contiguous()
        out["d_params"] = torch.empty(params.shape, dtype=params.dtype, device=dev)
        for k in ("d_dt_bias", "d_alpha_bias", "d_theta_mod_bias", "d_theta_bias"):
            out[k] = torch.zeros((heads,), **f32)
    b5 = list(biases) if biases is not None else [None] * 5
    with torch.cuda.device(dev):
        check(lib().sl_scanprep_conv_bwd(
            _ptr(value), vstride, _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state), d_conv,
            _ptr(params), _ptr(bc), *[_ptr(b) for b in b5],
            ctypes.byref(cfg) if cfg is not None else None, _ptr(dU), usb, ush, ust, _ptr(dM),
            _ptr(dK), _ptr(dBo), _ptr(dCo), _ptr(out["d_value"]), _ptr(out["d_conv_weight"]),
            _ptr(out["d_conv_bias"]), _ptr(out["d_conv_state"]), _ptr(out["d_params"]),
            _ptr(out["d_bc"]), _ptr(out["d_dt_bias"]), _ptr(out["d_alpha_bias"]),
            _ptr(out["d_theta_mod_bias"]), _ptr(out["d_theta_bias"]), batch, heads, groups, T, P,
            N, io, _stream(dev)), "sl_scanprep_conv_bwd")
    return out


# ---------------------------------------------------------------------------------
# mixer tail (row-wise part)
# ---------------------------------------------------------------------------------
def mixer_tail_fwd(Y, gate, skip, d_skip, norm_weight, eps):
    """Launch ``sl_mixer_tail_fwd``.  Returns normed (batch,T,heads*P)."""
    dev = require_cuda(Y, gate, skip, d_skip, norm_weight)
    batch, heads, T, P = Y.shape
    gate = as_rows(gate)
    normed = torch.empty((batch, T, heads * P), dtype=Y.dtype, device=dev)
    with torch.cuda.device(dev):
        check(lib().sl_mixer_tail_fwd(
            _ptr(Y), _ptr(gate), _row_stride(gate), _ptr(skip), _ptr(d_skip), _ptr(norm_weight),
            float(eps), _ptr(normed), batch, heads, T, P, dtype_code(Y.dtype), _stream(dev)),
            "sl_mixer_tail_fwd")
    return normed


def mixer_tail_bwd(Y, gate, skip, d_skip, norm_weight, eps, d_normed):
    """Launch ``sl_mixer_tail_bwd``.  Returns ``(dY, d_gate, d_skip_input, d_d_skip,
    d_norm_weight)``; the last two are float32 accumulators."""
    dev = require_cuda(Y, gate, skip, d_skip, norm_weight, d_normed)
    batch, heads, T, P = Y.shape
    gate = as_rows(gate)
    d_normed = d_normed.contiguous()
    dY = torch.empty_like(Y)
    d_gate = torch.empty((batch, T, heads * P), dtype=Y.dtype, device=dev)
    d_skip_in = torch.empty_like(Y) if skip is not None else None
    d_d_skip = torch.zeros((heads,), dtype=torch.float32, device=dev) if skip is not None else None
    d_w = torch.zeros((heads * P,), dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().sl_mixer_tail_bwd(
            _ptr(Y), _ptr(gate), _row_stride(gate), _ptr(skip), _ptr(d_skip), _ptr(norm_weight),
            float(eps), _ptr(d_normed), _ptr(dY), _ptr(d_gate), _ptr(d_skip_in), _ptr(d_d_skip),
            _ptr(d_w), batch, heads, T, P, dtype_code(Y.dtype), _stream(dev)), "sl_mixer_tail_bwd")
    return dY, d_gate, d_skip_in, d_d_skip, d_w


# ---------------------------------------------------------------------------------
# fused decode step of the mixer
# ---------------------------------------------------------------------------------
def mixer_decode_workspace(batch, heads, P, dev) -> torch.Tensor:
    """The zero-initialised scratch ``mixer_decode_step`` needs (allocate once, reuse every token)."""
    n = lib().sl_mixer_decode_step_workspace_bytes(batch, heads, P)
    return torch.zeros(n, dtype=torch.uint8, device=dev)


def mixer_decode_step(gate, value, params, bc, conv_weight, conv_bias, conv_state, biases, cfg, d_skip,
                      norm_weight, eps, state, b_prev_in, b_prev_out, u_prev, workspace, *, heads, P,
                      normed=None):
    """Launch ``sl_mixer_decode_step``.  ``gate`` and ``value`` are (batch, heads*P) views with a row
    stride; ``conv_state``, ``state`` and ``u_prev`` are updated in place; ``b_prev_out`` receives this
    token's b.  Returns ``normed`` (batch, heads*P)."""
    dev = require_cuda(gate, value, params, bc, conv_weight, conv_bias, conv_state, d_skip, norm_weight, state,
                       b_prev_in, b_prev_out, u_prev, workspace)
    batch = int(gate.shape[0])
    groups, N = int(bc.shape[-3]), int(bc.shape[-1])
    if gate.stride(-1) != 1 or value.stride(-1) != 1:
        raise ValueError("gate and value must have dense channels (row-strided views are fine).")
    if normed is None:
        normed = torch.empty((batch, heads * P), dtype=gate.dtype, device=dev)
    d_conv = 1 if conv_weight is None else int(conv_weight.shape[1])
    with torch.cuda.device(dev):
        check(lib().sl_mixer_decode_step(
            _ptr(gate), int(gate.stride(0)), _ptr(value), int(value.stride(0)), _ptr(params), _ptr(bc),
            _ptr(conv_weight), _ptr(conv_bias), _ptr(conv_state), d_conv, *[_ptr(b) for b in biases],
            ctypes.byref(cfg), _ptr(d_skip), _ptr(norm_weight), float(eps), _ptr(state), _ptr(b_prev_in),
            _ptr(b_prev_out), _ptr(u_prev), _ptr(normed), _ptr(workspace), workspace.numel(), batch, heads,
            groups, P, N, dtype_code(gate.dtype), _stream(dev)), "sl_mixer_decode_step")
    return normed


# ---------------------------------------------------------------------------------
# FFN branch: row-wise kernels
# ---------------------------------------------------------------------------------
FFN_KINDS = {"gelu": 0, "swiglu": 1}


def rmsnorm_supported(C: int, dtype: torch.dtype) -> bool:
    v = 4 if dtype == torch.float32 else 8
    return dtype in _DTYPE_CODE and C % v == 0 and C // v <= 256


def rmsnorm_fwd(x, weight, eps):
    """``x (..., C)`` dense -> same shape; launches ``sl_rmsnorm_fwd``."""
    dev = require_cuda(x, weight)
    C = int(x.shape[-1])
    out = torch.empty_like(x)
    with torch.cuda.device(dev):
        check(lib().sl_rmsnorm_fwd(_ptr(x), _ptr(weight), float(eps), _ptr(out), x.numel() // C, C,
                                   dtype_code(x.dtype), _stream(dev)), "sl_rmsnorm_fwd")
    return out


def rmsnorm_bwd(x, weight, eps, d_out):
    """Returns ``(d_x, d_weight float32)``."""
    dev = require_cuda(x, weight, d_out)
    C = int(x.shape[-1])
    d_x = torch.empty_like(x)
    d_w = torch.zeros(C, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(lib().sl_rmsnorm_bwd(_ptr(x), _ptr(weight), float(eps), _ptr(d_out), _ptr(d_x), _ptr(d_w),
                                   x.numel() // C, C, dtype_code(x.dtype), _stream(dev)), "sl_rmsnorm_bwd")
    return d_x, d_w


def ffn_activation_fwd(projected, kind: str):
    """``projected (..., W)`` dense, W = hidden (gelu) or 2*hidden (swiglu) -> ``hidden (..., hidden)``."""
    dev = require_cuda(projected)
    W = int(projected.shape[-1])
    H = W // 2 if kind == "swiglu" else W
    hidden = torch.empty(projected.shape[:-1] + (H,), dtype=projected.dtype, device=dev)
    with torch.cuda.device(dev):
        check(lib().sl_ffn_activation_fwd(_ptr(projected), _ptr(hidden), projected.numel() // W, H,
                                          FFN_KINDS[kind], dtype_code(projected.dtype), _stream(dev)),
              "sl_ffn_activation_fwd")
    return hidden


def ffn_activation_bwd(projected, d_hidden, kind: str):
    dev = require_cuda(projected, d_hidden)
    W = int(projected.shape[-1])
    H = W // 2 if kind == "swiglu" else W
    d_proj = torch.empty_like(projected)
    with torch.cuda.device(dev):
        check(lib().sl_ffn_activation_bwd(_ptr(projected), _ptr(d_hidden), _ptr(d_proj), projected.numel() // W, H,
                                          FFN_KINDS[kind], dtype_code(projected.dtype), _stream(dev)),
              "sl_ffn_activation_bwd")
    return d_proj
