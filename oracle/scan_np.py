"""numpy restatement of the v2x2ssd scan (test oracle; not a product path).

The scan keeps, per (batch, head), a complex state ``z[p, n]`` and evaluates

    z_t = m_t z_{t-1} + u_{t-1} (x) (kprev_t b_{t-1}) + u_t (x) (kcurr_t b_t)
    y_t[p] = Re sum_n conj(c_t[n]) z_t[p, n]

Packed layouts follow the reference (slinoss/ops/v2x2ssd/reference.py:11-28):
``U (B,H,T,P)``, ``M (B,H,T,2)``, ``K (B,H,T,2,2)`` with tap 0 = prev and
tap 1 = curr, ``B, C (B,G,T,2N)`` interleaved (re, im) with G dividing H, state
``(B,H,P,2N)``.

Functions
---------
``v2x2ssm``       sequential scan      (reference.py:739-847)
``v2x2ssd``       three-stage chunked  (reference.py:992-1347: chunk_increment,
                  state_passing, chunk_scan, including the log-magnitude /
                  unit-phase prefix policy of reference.py:498-523)
``v2x2ssd_bwd``   analytic adjoint of the sequential scan; the reference obtains
                  the same gradients by autograd through ``v2x2ssd``
                  (tests/test_v2x2ssd_cute.py:1831-1876 in the reference).
"""

from __future__ import annotations

import numpy as np


def _real_dtype(dtype) -> np.dtype:
    dtype = np.dtype(dtype)
    if dtype not in (np.dtype(np.float32), np.dtype(np.float64)):
        raise ValueError(f"compute dtype must be float32 or float64, got {dtype}.")
    return dtype


def _cdtype(rdtype: np.dtype) -> np.dtype:
    return np.dtype(np.complex64) if rdtype == np.float32 else np.dtype(np.complex128)


def as_complex(x: np.ndarray, rdtype) -> np.ndarray:
    """(..., 2N) interleaved (re, im) -> complex (..., N)."""
    x = np.asarray(x, dtype=rdtype)
    return (x[..., 0::2] + 1j * x[..., 1::2]).astype(_cdtype(np.dtype(rdtype)))


def pack_complex(z: np.ndarray, rdtype) -> np.ndarray:
    """complex (..., N) -> (..., 2N) interleaved (re, im)."""
    out = np.empty(z.shape[:-1] + (2 * z.shape[-1],), dtype=rdtype)
    out[..., 0::2] = z.real
    out[..., 1::2] = z.imag
    return out


def _expand_groups(x: np.ndarray, n_heads: int) -> np.ndarray:
    groups = x.shape[1]
    if n_heads % groups != 0:
        raise ValueError(f"groups={groups} must divide heads={n_heads}.")
    rep = n_heads // groups
    return x if rep == 1 else np.repeat(x, rep, axis=1)


def _reduce_groups(x: np.ndarray, groups: int) -> np.ndarray:
    """Sum per-head gradients (B,H,...) over the heads of each BC group."""
    b, h = x.shape[:2]
    rep = h // groups
    if rep == 1:
        return x
    return x.reshape((b, groups, rep) + x.shape[2:]).sum(axis=2)


def _prepare(U, M, K, B, C, initial_states, B_prev, U_prev, rdtype):
    rdtype = _real_dtype(rdtype)
    U = np.asarray(U, dtype=rdtype)
    bsz, H, T, P = U.shape
    D = B.shape[-1]
    N = D // 2
    m = as_complex(np.asarray(M, dtype=rdtype), rdtype)[..., 0]
    k = as_complex(np.asarray(K, dtype=rdtype).reshape(bsz, H, T, 4), rdtype)
    kp, kc = k[..., 0], k[..., 1]
    b = as_complex(_expand_groups(np.asarray(B, dtype=rdtype), H), rdtype)
    c = None if C is None else as_complex(_expand_groups(np.asarray(C, dtype=rdtype), H), rdtype)
    if (B_prev is None) != (U_prev is None):
        raise ValueError("B_prev and U_prev must be passed together (or both omitted).")
    if B_prev is None:
        b0 = np.zeros((bsz, H, N), dtype=_cdtype(rdtype))
        u0 = np.zeros((bsz, H, P), dtype=rdtype)
    else:
        b0 = as_complex(_expand_groups(np.asarray(B_prev, dtype=rdtype), H), rdtype)
        u0 = np.asarray(U_prev, dtype=rdtype)
    if initial_states is None:
        z0 = np.zeros((bsz, H, P, N), dtype=_cdtype(rdtype))
    else:
        z0 = as_complex(np.asarray(initial_states, dtype=rdtype), rdtype)
    b_prev_seq = np.concatenate([b0[:, :, None], b[:, :, :-1]], axis=2)
    u_prev_seq = np.concatenate([u0[:, :, None], U[:, :, :-1]], axis=2)
    return U, m, kp, kc, b, c, b_prev_seq, u_prev_seq, z0, (bsz, H, T, P, N)


def v2x2ssm(U, M, K, B, C, *, initial_states=None, B_prev=None, U_prev=None,
            dtype=np.float64, return_states=False):
    """Sequential scan.  Returns ``(Y, final_state, B_last, U_last)`` in ``dtype``.

    ``T == 0`` returns the carried state unchanged (reference.py:704-736).
    With ``return_states`` the per-token states ``z_t`` (T,B,H,P,N) are appended.
    """
    rdtype = _real_dtype(dtype)
    U_r, m, kp, kc, b, c, bps, ups, z, (bsz, H, T, P, N) = _prepare(
        U, M, K, B, C, initial_states, B_prev, U_prev, rdtype)
    G = np.asarray(B).shape[1]
    if T == 0:
        fin = pack_complex(z, rdtype)
        if B_prev is None:
            return (np.empty((bsz, H, 0, P), rdtype), fin,
                    np.zeros((bsz, G, 2 * N), rdtype), np.zeros((bsz, H, P), rdtype))
        return (np.empty((bsz, H, 0, P), rdtype), fin,
                np.asarray(B_prev, rdtype).copy(), np.asarray(U_prev, rdtype).copy())
    beta_p = kp[..., None] * bps
    beta_c = kc[..., None] * b
    Y = np.empty((bsz, H, T, P), dtype=rdtype)
    states = np.empty((T, bsz, H, P, N), dtype=z.dtype) if return_states else None
    cconj = np.conj(c)
    for t in range(T):
        drive = ups[:, :, t, :, None] * beta_p[:, :, t, None, :] \
            + U_r[:, :, t, :, None] * beta_c[:, :, t, None, :]
        z = m[:, :, t, None, None] * z + drive
        Y[:, :, t] = (cconj[:, :, t, None, :] * z).sum(axis=-1).real
        if return_states:
            states[t] = z
    out = (Y, pack_complex(z, rdtype), np.asarray(B, rdtype)[:, :, -1].copy(),
           U_r[:, :, -1].copy())
    return out + (states,) if return_states else out


def _pad_time(x: np.ndarray, pad: int, axis: int = 2) -> np.ndarray:
    if pad == 0:
        return x
    shape = list(x.shape)
    shape[axis] = pad
    return np.concatenate([x, np.zeros(shape, dtype=x.dtype)], axis=axis)


def chunk_prefix_parts(m_blk: np.ndarray):
    """Stable in-chunk prefix: cumulative log|m| and cumulative unit phase
    (reference.py:498-523).  Exact-zero transitions are rejected."""
    mag = np.abs(m_blk)
    if (mag == 0).any():
        raise ValueError("M must be strictly nonzero in chunked scan paths.")
    logprefix = np.cumsum(np.log(mag), axis=-1)
    phase = np.cumprod(m_blk / mag, axis=-1)
    tiny = np.finfo(mag.dtype).tiny
    phase = phase / np.maximum(np.abs(phase), tiny)
    return logprefix, phase


def v2x2ssd(U, M, K, B, C, *, chunk_size=64, initial_states=None, B_prev=None,
            U_prev=None, dtype=np.float64, return_chunk_starts=False):
    """Chunked scan in the reference's three stages.

    Stage 1 (reference.py:526-548): reverse scan per chunk for the affine
    increment ``inc`` and the chunk transition ``m_chunk``.  Stage 2
    (reference.py:471-489): sequential propagation of chunk-start states.
    Stage 3 (reference.py:1203-1263): in-chunk outputs from the chunk-start
    state (off term) and the causal score matrices (diagonal term); segment
    ratios are formed as ``exp(logp_t - logp_s) * phase_t * conj(phase_s)``.
    """
    rdtype = _real_dtype(dtype)
    if chunk_size <= 0:
        raise ValueError(f"chunk_size must be positive. Got {chunk_size}.")
    U_r, m, kp, kc, b, c, bps, ups, z0, (bsz, H, T, P, N) = _prepare(
        U, M, K, B, C, initial_states, B_prev, U_prev, rdtype)
    if T == 0:
        return v2x2ssm(U, M, K, B, C, initial_states=initial_states, B_prev=B_prev,
                       U_prev=U_prev, dtype=dtype)
    L = int(chunk_size)
    pad = (-T) % L
    nC = (T + pad) // L
    cd = _cdtype(rdtype)
    m_p = np.concatenate([m, np.ones((bsz, H, pad), cd)], axis=2) if pad else m
    beta_p = _pad_time(kp[..., None] * bps, pad)
    beta_c = _pad_time(kc[..., None] * b, pad)
    u_c = _pad_time(U_r, pad)
    u_p = _pad_time(ups, pad)
    c_p = _pad_time(np.conj(c), pad)

    m_blk = m_p.reshape(bsz, H, nC, L)
    bp_blk = beta_p.reshape(bsz, H, nC, L, N)
    bc_blk = beta_c.reshape(bsz, H, nC, L, N)
    uc_blk = u_c.reshape(bsz, H, nC, L, P)
    up_blk = u_p.reshape(bsz, H, nC, L, P)
    c_blk = c_p.reshape(bsz, H, nC, L, N)

    # stage 1: chunk increments by reverse scan
    inc = np.zeros((bsz, H, nC, P, N), cd)
    m_suf = np.ones((bsz, H, nC), cd)
    for t in range(L - 1, -1, -1):
        inc += up_blk[..., t, :, None] * (m_suf[..., None] * bp_blk[..., t, :])[..., None, :]
        inc += uc_blk[..., t, :, None] * (m_suf[..., None] * bc_blk[..., t, :])[..., None, :]
        m_suf = m_suf * m_blk[..., t]
    m_chunk = m_suf

    # stage 2: state passing
    starts = np.empty((bsz, H, nC, P, N), cd)
    z = z0
    for ci in range(nC):
        starts[:, :, ci] = z
        z = m_chunk[:, :, ci, None, None] * z + inc[:, :, ci]
    final = z

    # stage 3: in-chunk outputs
    logp, phase = chunk_prefix_parts(m_blk)
    prefix = np.exp(logp).astype(rdtype) * phase
    q_off = c_blk * prefix[..., None]
    y_off = np.einsum("bhcln,bhcpn->bhclp", q_off, starts).real
    tril = np.tril(np.ones((L, L), dtype=bool))
    logdiff = np.where(tril, logp[..., :, None] - logp[..., None, :], 0.0)
    scale = np.exp(logdiff).astype(rdtype) * phase[..., :, None] * np.conj(phase[..., None, :])
    s_prev = np.where(tril, (np.einsum("bhctn,bhcsn->bhcts", c_blk, bp_blk) * scale).real, 0.0)
    s_curr = np.where(tril, (np.einsum("bhctn,bhcsn->bhcts", c_blk, bc_blk) * scale).real, 0.0)
    y_diag = np.einsum("bhcts,bhcsp->bhctp", s_prev, up_blk) \
        + np.einsum("bhcts,bhcsp->bhctp", s_curr, uc_blk)
    Y = (y_diag + y_off).reshape(bsz, H, T + pad, P)[:, :, :T].astype(rdtype)
    out = (np.ascontiguousarray(Y), pack_complex(final, rdtype),
           np.asarray(B, rdtype)[:, :, -1].copy(), U_r[:, :, -1].copy())
    if return_chunk_starts:
        return out + (pack_complex(starts, rdtype), pack_complex(m_chunk[..., None], rdtype))
    return out


def v2x2ssd_bwd(U, M, K, B, C, dY, *, d_final_state=None, initial_states=None,
                B_prev=None, U_prev=None, dtype=np.float64):
    """Gradients of the scan by the sequential adjoint recurrence.

    With ``G_t`` the gradient w.r.t. ``z_t`` (complex = d/dre + i d/dim):

        G_t      = dy_t (x) c_t + conj(m_{t+1}) G_{t+1}
        G_{T-1}  = dy_{T-1} (x) c_{T-1} + d_final_state
        dc_t[n]  = sum_p dy_t[p] z_t[p,n]
        dm_t     = sum_{p,n} G_t conj(z_{t-1})
        dbc_t[n] = sum_p u_t[p] G_t[p,n],  dbp_t[n] = sum_p u_{t-1}[p] G_t[p,n]
        du_t    += Re sum_n conj(kc_t b_t) G_t,  du_{t-1} += Re sum_n conj(kp_t b_{t-1}) G_t
        dkc_t    = sum_n dbc_t conj(b_t),  dkp_t = sum_n dbp_t conj(b_{t-1})
        db_t    += conj(kc_t) dbc_t,       db_{t-1} += conj(kp_t) dbp_t

    The ``t-1`` terms at ``t = 0`` are the gradients of ``U_prev`` / ``B_prev``
    and ``d_initial = conj(m_0) G_0``.  Grouped ``B``/``C`` gradients are summed
    over the heads of a group.  Returns a dict keyed by input name.
    """
    rdtype = _real_dtype(dtype)
    out = v2x2ssm(U, M, K, B, C, initial_states=initial_states, B_prev=B_prev,
                  U_prev=U_prev, dtype=dtype, return_states=True)
    states = out[4]
    U_r, m, kp, kc, b, c, bps, ups, z0, (bsz, H, T, P, N) = _prepare(
        U, M, K, B, C, initial_states, B_prev, U_prev, rdtype)
    groups = np.asarray(B).shape[1]
    cd = _cdtype(rdtype)
    dY = np.asarray(dY, dtype=rdtype)
    G = np.zeros((bsz, H, P, N), cd) if d_final_state is None \
        else as_complex(np.asarray(d_final_state, dtype=rdtype), rdtype)

    dU = np.zeros((bsz, H, T, P), rdtype)
    dU_prev = np.zeros((bsz, H, P), rdtype)
    dm = np.zeros((bsz, H, T), cd)
    dkp = np.zeros((bsz, H, T), cd)
    dkc = np.zeros((bsz, H, T), cd)
    db = np.zeros((bsz, H, T, N), cd)
    db_prev = np.zeros((bsz, H, N), cd)
    dc = np.zeros((bsz, H, T, N), cd)
    m_next = np.ones((bsz, H), cd)  # final_state is z_{T-1} itself
    for t in range(T - 1, -1, -1):
        z_t = states[t]
        z_prev = states[t - 1] if t > 0 else z0
        G = dY[:, :, t, :, None] * c[:, :, t, None, :] + np.conj(m_next)[..., None, None] * G
        dc[:, :, t] = (dY[:, :, t, :, None] * z_t).sum(axis=2)
        dm[:, :, t] = (G * np.conj(z_prev)).sum(axis=(2, 3))
        dbc = (U_r[:, :, t, :, None] * G).sum(axis=2)
        dbp = (ups[:, :, t, :, None] * G).sum(axis=2)
        beta_c = kc[:, :, t, None] * b[:, :, t]
        beta_p = kp[:, :, t, None] * bps[:, :, t]
        dU[:, :, t] += (np.conj(beta_c)[:, :, None, :] * G).sum(axis=3).real
        du_prev_t = (np.conj(beta_p)[:, :, None, :] * G).sum(axis=3).real
        dkc[:, :, t] = (dbc * np.conj(b[:, :, t])).sum(axis=-1)
        dkp[:, :, t] = (dbp * np.conj(bps[:, :, t])).sum(axis=-1)
        db[:, :, t] += np.conj(kc[:, :, t])[..., None] * dbc
        db_prev_t = np.conj(kp[:, :, t])[..., None] * dbp
        if t > 0:
            dU[:, :, t - 1] += du_prev_t
            db[:, :, t - 1] += db_prev_t
        else:
            dU_prev += du_prev_t
            db_prev += db_prev_t
        m_next = m[:, :, t]
    d_initial = np.conj(m_next)[..., None, None] * G if T > 0 else G

    dK = np.empty((bsz, H, T, 2, 2), rdtype)
    dK[..., 0, 0], dK[..., 0, 1] = dkp.real, dkp.imag
    dK[..., 1, 0], dK[..., 1, 1] = dkc.real, dkc.imag
    dM = np.stack([dm.real, dm.imag], axis=-1).astype(rdtype)
    return {
        "U": dU,
        "M": dM,
        "K": dK,
        "B": _reduce_groups(pack_complex(db, rdtype), groups),
        "C": _reduce_groups(pack_complex(dc, rdtype), groups),
        "initial_states": pack_complex(d_initial, rdtype),
        "B_prev": _reduce_groups(pack_complex(db_prev, rdtype), groups),
        "U_prev": dU_prev,
    }


__all__ = ["as_complex", "pack_complex", "chunk_prefix_parts", "v2x2ssm", "v2x2ssd",
           "v2x2ssd_bwd"]
