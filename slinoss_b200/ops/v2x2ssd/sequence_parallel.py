"""The scan over a sequence that is split across ranks (one contiguous time slice per rank).

The recurrence is linear in its state: over a slice with transition product ``Pi = prod_t m_t`` the end
state is ``Pi * z_start + f0``, where ``f0`` is the end state of the same slice started from zero.  So a
sequence sharded over W ranks needs ONE exchange of small per-(batch, head) tensors:

    pass A   every rank scans its slice from a zero state                          -> f0_r   (and Pi_r from M)
    exchange all_gather of (f0_r, Pi_r) and of each slice's last token (b, u)      (state-sized, not T-sized)
             z_start_r = sum_{q < r} (prod_{q < s < r} Pi_s) f0_q                  (W - 1 complex scalings)
    pass B   every rank scans its slice again from z_start_r                       -> Y_r, end state

which is the associative ``(prod m, Z)`` exchange the reference's scope notes describe for long contexts
(its own decomposition has the same shape inside one device: ``chunk_increment`` -> ``state_passing`` ->
``chunk_scan``, slinoss/ops/v2x2ssd/reference.py:992-1264).  Both passes are the ordinary differentiable op;
the exchange is differentiable too (gather forward, sum-reduce backward), so ``backward()`` works through
the whole thing and every rank must call it (the exchange's backward is a collective).  The price is a
second pass over the slice; nothing of size T crosses the link.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .api import v2x2ssd_cute


class _Gather(torch.autograd.Function):
    """``stack(all_gather(x))`` forward; backward sums the ranks' gradients of the stack and keeps the
    slot of this rank (all_reduce: available in every backend)."""

    @staticmethod
    def forward(ctx, x, group):
        world = dist.get_world_size(group)
        ctx.group, ctx.rank = group, dist.get_rank(group)
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=group)
        return torch.stack(parts)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g[ctx.rank], None


def previous_rank_value(x, group=None):
    """``x`` of the previous rank of ``group`` (zeros on rank 0), differentiable: what a rank needs of its
    predecessor's slice (the last token of B and U for the scan's carried taps, the last rows of the conv
    input for the causal conv).  Every rank must call it, and its backward, together."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    allx = _Gather.apply(x.contiguous(), group)
    # rank 0 multiplies the (unused) gathered rows by zero: its autograd graph stays attached to the gather
    return (allx[rank - 1] if rank > 0 else allx[0] * 0).contiguous()


def _scale_state(pi, z):
    """Complex scalar ``pi (batch, heads)`` (complex64) times the interleaved complex state ``z (batch, heads, P, 2N)``."""
    zc = torch.view_as_complex(z.reshape(*z.shape[:-1], -1, 2))
    return torch.view_as_real(zc * pi[..., None, None]).reshape(z.shape)


def transition_product(M):
    """``prod_t m_t`` per (batch, heads) as (re, im), formed from summed log-magnitudes and summed angles in
    float64 (never as a running product of small numbers)."""
    m = M.double()
    logmag = 0.5 * torch.log(m[..., 0] ** 2 + m[..., 1] ** 2).sum(-1)
    angle = torch.atan2(m[..., 1], m[..., 0]).sum(-1)
    mag = torch.exp(logmag)
    return torch.stack((mag * torch.cos(angle), mag * torch.sin(angle)), -1).float()


def _gather_packed(parts, group):
    """One differentiable gather for several per-batch tensors of one dtype: returns, per tensor, the stack over
    ranks ``(W, *shape)``."""
    batch = parts[0].shape[0]
    flat = torch.cat([p.reshape(batch, -1) for p in parts], dim=1)
    allx = _Gather.apply(flat, group)                                  # (W, batch, sum of widths)
    outs, off = [], 0
    for p in parts:
        n = p[0].numel()
        outs.append(allx[:, :, off:off + n].reshape(allx.shape[0], *p.shape))
        off += n
    return outs


@torch.compiler.disable
def v2x2ssd_sequence_parallel(U, M, K, B, C, *, chunk_size=64, group=None, initial_states=None, B_prev=None,
                              U_prev=None, output_dtype=None, path="auto", single_rank_exchange=False):
    """Scan of a sequence whose time axis is sharded over the ranks of ``group`` in rank order.

    Arguments are this rank's slice, in the layouts of ``v2x2ssd``; ``initial_states``, ``B_prev`` and
    ``U_prev`` describe what precedes the WHOLE sequence and are read on rank 0 only.  Returns
    ``(Y, end_state, B_last, U_last)`` of this rank's slice (``end_state`` float32); the last rank's are those of
    the whole sequence.  Without an initialised process group (or with one rank) this is the plain op, unless
    ``single_rank_exchange`` asks for the two passes and the exchange anyway (a group of one: for tests and
    profiles of the path on a single device)."""
    if not (dist.is_available() and dist.is_initialized()) or \
            (dist.get_world_size(group) == 1 and not single_rank_exchange):
        Y, fin, bl, ul = v2x2ssd_cute(U, M, K, B, C, chunk_size=chunk_size, initial_states=initial_states,
                                      B_prev=B_prev, U_prev=U_prev, output_dtype=output_dtype,
                                      return_state=True, path=path)
        return Y, fin.float(), bl, ul
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    if U.shape[2] < 1:
        raise ValueError("every rank needs at least one token of the sequence.")
    # ---- the token before each slice: the previous rank's last (b, u), one exchange for both ------------
    b_all, u_all = _gather_packed([B[:, :, -1, :], U[:, :, -1, :]], group)
    if rank > 0:
        Bp, Up = b_all[rank - 1].contiguous(), u_all[rank - 1].contiguous()   # (batch, groups, 2N), (batch, heads, P)
    else:                                                              # zeros, attached to the gather's graph
        Bp, Up = (b_all[0] * 0).contiguous(), (u_all[0] * 0).contiguous()
    z_first = None
    if rank == 0:
        if B_prev is not None:
            Bp, Up = Bp + B_prev, Up + U_prev
        z_first = initial_states
    # ---- pass A: the slice from a zero state ------------------------------------------------------------
    _, f0, _, _ = v2x2ssd_cute(U, M, K, B, C, chunk_size=chunk_size, initial_states=z_first, B_prev=Bp, U_prev=Up,
                               output_dtype=torch.float32, return_state=True, path=path)
    f_all, pi_all = _gather_packed([f0.float(), transition_product(M)], group)   # (W, batch, heads, P, 2N), (W, batch, heads, 2)
    pi_c = torch.view_as_complex(pi_all.contiguous())                  # (W, batch, heads)
    # ---- the state at the start and at the end of this rank's slice -----------------------------------------
    # (the term multiplied by zero keeps every rank's autograd graph attached to the gather, whose backward is
    # a collective, whatever part of it this rank's result uses)
    start = f_all[rank] * 0 if rank == 0 else f_all[0]
    for q in range(1, rank):
        start = _scale_state(pi_c[q], start) + f_all[q]
    end = f_all[0] if rank == 0 else _scale_state(pi_c[rank], start) + f_all[rank]
    if rank + 1 < world:
        start = start + 0.0 * (f_all[rank + 1:].sum() + pi_all[rank + 1:].sum())
    if rank == 0 and initial_states is not None:
        start = start + initial_states.float()
    # ---- pass B: the slice from its true start state -------------------------------------------------------
    Y = v2x2ssd_cute(U, M, K, B, C, chunk_size=chunk_size, initial_states=start.contiguous(), B_prev=Bp, U_prev=Up,
                     output_dtype=output_dtype, return_state=False, path=path)
    return Y, end, B[:, :, -1, :], U[:, :, -1, :]


__all__ = ["previous_rank_value", "transition_product", "v2x2ssd_sequence_parallel"]
