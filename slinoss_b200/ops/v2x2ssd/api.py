"""Host side of the v2x2ssd scan: validation, dtype policy, autograd wiring."""

from __future__ import annotations

import torch

from ... import _C

_IO_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _contig(name: str, x: torch.Tensor) -> None:
    if not x.is_contiguous():
        raise ValueError(f"{name} must be contiguous; got strides {x.stride()}.")


def _require(cond: bool, message: str) -> None:
    if not cond:
        raise ValueError(message)


def validate_inputs(U, M, K, B, C, initial_states, B_prev, U_prev):
    """Shape / device / layout contract of the scan.  The conditions and the messages are the
    reference's (``_validate_inputs``, slinoss/ops/v2x2ssd/reference.py:152-234), since callers
    match on them; the checks are grouped here as: the five operands as a set, the per-operand
    rank table, cross-operand extents, then the optional carried tensors.
    Returns ``(batch, heads, T, N, P)``."""
    operands = {"U": U, "M": M, "K": K, "B": B, "C": C}
    values = tuple(operands.values())
    _require(all(torch.is_floating_point(t) for t in values),
             "U, M, K, B, and C must be floating-point tensors.")
    _require(all(t.device == U.device for t in values),
             f"All inputs must be on the same device. Got {[t.device for t in values]}.")
    for name, t in operands.items():
        _contig(name, t)

    # rank (and fixed trailing extents) of every operand
    layout = {"U": (4, (), "(batch,heads,T,P)"), "M": (4, (2,), "(batch,heads,T,2)"),
              "K": (5, (2, 2), "(batch,heads,T,2,2)"), "B": (4, (), "(batch,groups,T,2N)"),
              "C": (4, (), "(batch,groups,T,2N)")}
    for name, (rank, tail, text) in layout.items():
        t = operands[name]
        ok = t.ndim == rank and (not tail or tuple(t.shape[-len(tail):]) == tail)
        _require(ok, f"{name} must be {text}. Got {tuple(t.shape)}.")

    batch, heads, T, P = map(int, U.shape)
    for name in ("M", "K"):
        _require(tuple(operands[name].shape[:3]) == (batch, heads, T),
                 f"Leading (batch,heads,T) dims of {name} must match U.")
    for name in ("B", "C"):
        t = operands[name]
        _require(t.shape[0] == batch and t.shape[2] == T, f"{name} must match U on batch/time dims.")
    D, groups = int(B.shape[-1]), int(B.shape[1])
    _require(D % 2 == 0, f"B/C 2N dim must be divisible by 2. Got {D}.")
    _require(groups > 0, "B/C must have a positive group dimension.")
    _require(heads % groups == 0,
             f"B/C group dimension must divide heads. Got heads={heads}, groups={groups}.")
    _require(tuple(C.shape) == (batch, groups, T, D), "C must match grouped B exactly.")

    # carried tensors
    _require((B_prev is None) == (U_prev is None),
             "B_prev and U_prev must be passed together (or both omitted).")
    carried = []
    if initial_states is not None:
        carried.append(("initial_states", initial_states, (batch, heads, P, D),
                        "initial_states must be (batch,heads,P,2N) "
                        f"={(batch, heads, P, D)}. Got {tuple(initial_states.shape)}.",
                        "initial_states must be on the same device as inputs."))
    if B_prev is not None:
        both = "B_prev and U_prev must be on the same device as inputs."
        carried.append(("B_prev", B_prev, (batch, groups, D),
                        f"B_prev must be (batch,groups,2N)={(batch, groups, D)}. "
                        f"Got {tuple(B_prev.shape)}.", both))
        carried.append(("U_prev", U_prev, (batch, heads, P),
                        f"U_prev must be (batch,heads,P)={(batch, heads, P)}. "
                        f"Got {tuple(U_prev.shape)}.", both))
    for name, t, shape, shape_msg, _ in carried:
        _require(tuple(t.shape) == shape, shape_msg)
    for name, t, _, _, device_msg in carried:
        _contig(name, t)
        _require(t.device == U.device, device_msg)
    return batch, heads, T, D // 2, P


def resolve_dtypes(input_dtypes, compute_dtype, output_dtype, default_output_dtype):
    """Compute / output dtype policy (reference.py:61-82); the CUDA kernels compute
    in float32 only (cute/api.py:91-95)."""
    if compute_dtype is None:
        promoted = input_dtypes[0]
        for dt in input_dtypes[1:]:
            promoted = torch.promote_types(promoted, dt)
        compute_dtype = torch.float32 if promoted in (torch.float16, torch.bfloat16) else promoted
    if compute_dtype not in (torch.float32, torch.float64):
        raise ValueError(f"compute_dtype must be float32 or float64, got {compute_dtype}.")
    if compute_dtype != torch.float32:
        raise ValueError(
            "The sm_100a v2x2ssd kernels support only float32 compute. "
            f"Got compute_dtype={compute_dtype}.")
    odtype = default_output_dtype if output_dtype is None else output_dtype
    if odtype not in (torch.float16, torch.bfloat16, torch.float32, torch.float64):
        raise ValueError(f"output_dtype must be a real floating dtype, got {odtype}.")
    return compute_dtype, odtype


def _empty_outputs(batch, heads, groups, P, D, device, odtype, initial_states, B_prev, U_prev):
    """T == 0: the carried state passes through unchanged (reference.py:704-736)."""
    Y = torch.empty((batch, heads, 0, P), device=device, dtype=odtype)
    final = torch.zeros((batch, heads, P, D), device=device, dtype=odtype) \
        if initial_states is None else initial_states.to(dtype=odtype).contiguous()
    if B_prev is None:
        return (Y, final, torch.zeros((batch, groups, D), device=device, dtype=odtype),
                torch.zeros((batch, heads, P), device=device, dtype=odtype))
    return Y, final, B_prev.to(dtype=odtype).contiguous(), U_prev.to(dtype=odtype).contiguous()


def _io_dtype(U: torch.Tensor) -> torch.dtype:
    return U.dtype if U.dtype in _IO_DTYPES else torch.float32


def _prep(U, M, K, B, C, initial_states, B_prev, U_prev):
    """Cast to what the C ABI takes: U/B/C/B_prev/U_prev in one io dtype, the rest float32."""
    io = _io_dtype(U)
    cast = lambda x, dt: None if x is None else x.detach().to(dtype=dt).contiguous()
    return (cast(U, io), cast(M, torch.float32), cast(K, torch.float32), cast(B, io), cast(C, io),
            cast(initial_states, torch.float32), cast(B_prev, io), cast(U_prev, io))


def assert_nonzero_transitions(M: torch.Tensor) -> None:
    """Raise the reference's error for an exact-zero transition (slinoss/ops/v2x2ssd/reference.py:509-517).

    ``|m_t| > 0`` is a precondition of the chunked (tensor-core) kernels: they form ``log|m|`` and, in the
    merged-tap form, ``kp_{t+1} / m_{t+1}``; a zero transition yields NaN or Inf there (the exact path computes
    a forward pass through it, with dM = 0 at that token).  The ops do not check it themselves, because the
    check synchronises the device (the reference's torch path does it on every call); call this where the
    transitions do not come from the scan preparation, whose radius is bounded below by ``r_min``."""
    if bool((M[..., 0] == 0).logical_and(M[..., 1] == 0).any()):
        raise ValueError(
            "M must be strictly nonzero in chunked scan paths. Exact-zero transitions are outside the "
            "SLinOSS operating region; use v2x2ssm if you need arbitrary zero-transition behavior.")


class _ScanFn(torch.autograd.Function):
    """Saves the inputs (same saved set as slinoss/ops/v2x2ssd/cute/autograd.py:110-118)
    and, optionally, the 16-bit chunk-start states of the tensor-core path, which spare the
    backward its state pre-sweep at the price of one more (batch,heads,T/64,64,128) tensor."""

    @staticmethod
    def forward(ctx, U, M, K, B, C, initial_states, B_prev, U_prev, chunk_size, odtype,
                return_state, path, save_states):
        args = _prep(U, M, K, B, C, initial_states, B_prev, U_prev)
        ctx.set_materialize_grads(False)      # an unused output arrives as None in backward, not as zeros
        y_dtype = odtype if odtype in _IO_DTYPES else torch.float32
        out = _C.scan_fwd(*args, chunk_size=chunk_size, y_dtype=y_dtype, want_final=return_state,
                          path=path, save_states=save_states)
        Y, final = out[0], out[1]
        states = out[2] if len(out) > 2 else None
        ctx.has_saved_states = states is not None
        extra = [states, final] if states is not None else []
        ctx.save_for_backward(*[a for a in args if a is not None], *extra)
        ctx.present = [a is not None for a in args]
        ctx.in_dtypes = [None if x is None else x.dtype
                         for x in (U, M, K, B, C, initial_states, B_prev, U_prev)]
        ctx.chunk_size, ctx.path, ctx.return_state = chunk_size, path, return_state
        Y = Y.to(dtype=odtype)
        if not return_state:
            return Y
        return (Y, final.to(dtype=odtype), B[:, :, -1, :].detach().to(dtype=odtype).contiguous(),
                U[:, :, -1, :].detach().to(dtype=odtype).contiguous())

    @staticmethod
    def backward(ctx, *grads):
        it = iter(ctx.saved_tensors)
        U, M, K, B, C, z0, B_prev, U_prev = [next(it) if p else None for p in ctx.present]
        saved = (next(it), next(it)) if ctx.has_saved_states else None
        dY = grads[0]
        d_final = dB_last = dU_last = None
        if ctx.return_state:
            _, d_final, dB_last, dU_last = grads
        out = [None] * 8
        if dY is not None or d_final is not None:
            half = U.dtype in (torch.bfloat16, torch.float16) and ctx.path != "simt"
            if dY is None and half:
                dY = torch.zeros_like(U)      # only the end state was used: zeros keep the tensor-core sweep
            if dY is not None:
                if half and dY.dtype != U.dtype:
                    # a float32 output was asked of 16-bit operands: the tensor-core sweep takes dY as a 16-bit
                    # operand like U, B and C (the exact sweeps would keep it in float32 at ~20x the time)
                    dY = dY.to(U.dtype)
                elif dY.dtype not in _IO_DTYPES:
                    dY = dY.to(torch.float32)
                dY = dY.contiguous()
            if d_final is not None:
                d_final = d_final.to(torch.float32).contiguous()
            out = list(_C.scan_bwd(U, M, K, B, C, z0, B_prev, U_prev, dY, d_final,
                                   chunk_size=ctx.chunk_size, path=ctx.path, saved=saved))
        if dB_last is not None:
            if out[3] is None:
                out[3] = torch.zeros_like(B)
            out[3][:, :, -1, :].add_(dB_last.to(dtype=out[3].dtype))
        if dU_last is not None:
            if out[0] is None:
                out[0] = torch.zeros_like(U)
            out[0][:, :, -1, :].add_(dU_last.to(dtype=out[0].dtype))
        res = []
        for g, dt, need in zip(out, ctx.in_dtypes, ctx.needs_input_grad[:8]):
            res.append(g.to(dtype=dt) if (g is not None and dt is not None and need) else None)
        return (*res, None, None, None, None, None)


@torch.compiler.disable
def v2x2ssd_cute(U, M, K, B, C, *, chunk_size, initial_states=None, B_prev=None, U_prev=None,
                 compute_dtype=None, output_dtype=None, return_state=False, path="auto",
                 save_chunk_states=True):
    """GPU scan.  Returns ``Y`` or ``(Y, final_state, B_last, U_last)``.

    ``path`` selects the kernel family: "auto" (tensor cores when the shape and dtype
    allow, else the exact float32 recurrence), "simt" or "tc".  ``save_chunk_states``
    (training only) keeps the tensor-core path's 16-bit chunk-start states for the
    backward instead of recomputing them there; False saves only the inputs, like the
    reference."""
    batch, heads, T, N, P = validate_inputs(U, M, K, B, C, initial_states, B_prev, U_prev)
    _C.require_cuda(U)
    if chunk_size <= 0:
        raise ValueError(f"chunk_size must be positive. Got {chunk_size}.")
    _, odtype = resolve_dtypes([U.dtype, M.dtype, K.dtype, B.dtype, C.dtype], compute_dtype,
                               output_dtype, U.dtype)
    if T == 0:
        empty = _empty_outputs(batch, heads, int(B.shape[1]), P, 2 * N, U.device, odtype,
                               initial_states, B_prev, U_prev)
        return empty if return_state else empty[0]
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (U, M, K, B, C, initial_states, B_prev, U_prev))
    if needs_grad:
        return _ScanFn.apply(U, M, K, B, C, initial_states, B_prev, U_prev, int(chunk_size),
                             odtype, bool(return_state), path, bool(save_chunk_states))
    args = _prep(U, M, K, B, C, initial_states, B_prev, U_prev)
    y_dtype = odtype if odtype in _IO_DTYPES else torch.float32
    Y, final = _C.scan_fwd(*args, chunk_size=int(chunk_size), y_dtype=y_dtype,
                           want_final=return_state, path=path)
    Y = Y.to(dtype=odtype)
    if not return_state:
        return Y
    return (Y, final.to(dtype=odtype), B[:, :, -1, :].to(dtype=odtype).contiguous(),
            U[:, :, -1, :].to(dtype=odtype).contiguous())


@torch.compiler.disable
def v2x2ssd(U, M, K, B, C, *, chunk_size=64, initial_states=None, B_prev=None, U_prev=None,
            compute_dtype=None, output_dtype=None, path="auto"):
    """Same call and 4-tuple result as the reference's ``v2x2ssd``."""
    return v2x2ssd_cute(U, M, K, B, C, chunk_size=chunk_size, initial_states=initial_states,
                        B_prev=B_prev, U_prev=U_prev, compute_dtype=compute_dtype,
                        output_dtype=output_dtype, return_state=True, path=path)


@torch.compiler.disable
def v2x2ssd_decode(U, M, K, B, C, *, state, B_prev=None, U_prev=None, output_dtype=None,
                   inplace=False):
    """One decode token.  ``U (batch,heads,P)``, ``M (batch,heads,2)``, ``K (batch,heads,2,2)``,
    ``B, C (batch,groups,2N)``, ``state (batch,heads,P,2N)`` float32.

    Returns ``(Y, next_state, B_last, U_last)`` with the same meaning as one ``T = 1``
    call of the sequential scan (slinoss/ops/v2x2ssd/reference.py:739-847).  With
    ``inplace`` the float32 ``state`` tensor is updated where it lies."""
    if U.ndim != 3 or M.shape != U.shape[:2] + (2,) or K.shape != U.shape[:2] + (2, 2):
        raise ValueError("decode expects U (batch,heads,P), M (batch,heads,2), K (batch,heads,2,2).")
    if B.ndim != 3 or B.shape != C.shape or B.shape[-1] % 2:
        raise ValueError("decode expects B, C (batch,groups,2N).")
    if (B_prev is None) ^ (U_prev is None):
        raise ValueError("B_prev and U_prev must be passed together (or both omitted).")
    batch, heads, P = U.shape
    if state.shape != (batch, heads, P, B.shape[-1]):
        raise ValueError(f"state must be {(batch, heads, P, B.shape[-1])}. Got {tuple(state.shape)}.")
    io = _io_dtype(U)
    odtype = U.dtype if output_dtype is None else output_dtype
    cast = lambda x, dt: None if x is None else x.to(dtype=dt).contiguous()
    if inplace and (state.dtype != torch.float32 or not state.is_contiguous()):
        raise ValueError("in-place decode needs a contiguous float32 state.")
    st = cast(state, torch.float32)
    y_dtype = odtype if odtype in _IO_DTYPES else torch.float32
    Y, nxt = _C.scan_decode(cast(U, io), cast(M, torch.float32), cast(K, torch.float32),
                            cast(B, io), cast(C, io), st, cast(B_prev, io), cast(U_prev, io),
                            y_dtype=y_dtype, state_out=st if inplace else None)
    return Y.to(dtype=odtype), nxt, B, U
