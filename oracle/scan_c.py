"""ctypes wrapper of the C/OpenMP oracle port (numpy float32 in and out).

Test / baseline infrastructure only.  ``forward`` and ``backward`` mirror
``scan_np.v2x2ssm`` and ``scan_np.v2x2ssd_bwd``.
"""

from __future__ import annotations

import ctypes

import numpy as np

from .build_oracle import OUT, build

_lib = None
_fp = ctypes.POINTER(ctypes.c_float)


def lib():
    global _lib
    if _lib is None:
        if not OUT.exists():
            build()
        _lib = ctypes.CDLL(str(OUT))
        _lib.oracle_num_threads.restype = ctypes.c_int
        _lib.oracle_v2x2ssd_fwd.argtypes = [_fp] * 10 + [ctypes.c_int] * 6
        _lib.oracle_v2x2ssd_bwd.argtypes = [_fp] * 18 + [ctypes.c_int] * 6
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> int:
    """Threads the OpenMP loops use from now on (an explicit call overrides OMP_NUM_THREADS)."""
    lib().oracle_set_num_threads(int(n))
    return num_threads()


def _c(x):
    return None if x is None else np.ascontiguousarray(x, dtype=np.float32)


def _p(x):
    return None if x is None else x.ctypes.data_as(_fp)


def forward(U, M, K, B, C, *, initial_states=None, B_prev=None, U_prev=None):
    U, M, K, B, C, z0, Bp, Up = map(_c, (U, M, K, B, C, initial_states, B_prev, U_prev))
    b, h, T, P = U.shape
    g, N = B.shape[1], B.shape[3] // 2
    Y = np.empty_like(U)
    fin = np.empty((b, h, P, 2 * N), np.float32)
    lib().oracle_v2x2ssd_fwd(_p(U), _p(M), _p(K), _p(B), _p(C), _p(z0), _p(Bp), _p(Up), _p(Y),
                             _p(fin), b, h, g, T, P, N)
    return Y, fin


def backward(U, M, K, B, C, dY, *, d_final_state=None, initial_states=None, B_prev=None,
             U_prev=None):
    U, M, K, B, C, z0, Bp, Up, dY, dF = map(
        _c, (U, M, K, B, C, initial_states, B_prev, U_prev, dY, d_final_state))
    b, h, T, P = U.shape
    g, N = B.shape[1], B.shape[3] // 2
    out = {"U": np.zeros_like(U), "M": np.empty_like(M), "K": np.empty_like(K),
           "B": np.zeros_like(B), "C": np.zeros_like(C),
           "initial_states": np.empty((b, h, P, 2 * N), np.float32),
           "B_prev": np.zeros((b, g, 2 * N), np.float32), "U_prev": np.zeros((b, h, P), np.float32)}
    lib().oracle_v2x2ssd_bwd(_p(U), _p(M), _p(K), _p(B), _p(C), _p(z0), _p(Bp), _p(Up), _p(dY),
                             _p(dF), *[_p(out[k]) for k in ("U", "M", "K", "B", "C",
                                                            "initial_states", "B_prev", "U_prev")],
                             b, h, g, T, P, N)
    return out
