"""The N > 1 path on CPU: two ``gloo`` ranks, one process each.

The scan shards by batch with no data-path collective; what a multi-GPU job adds is the
host plumbing of ``slinoss_b200.shard`` (who owns which streams, MAX-over-ranks timing,
SUM-over-ranks throughput) and, when the mixer is trained data parallel, the averaging of
the replicated weights' gradients.  Each rank runs the package's real host code above the
C ABI with the oracle-backed launchers of tests/fake_cabi.py underneath.
"""

import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from slinoss_b200 import shard

WORLD = 2


class _Patch:
    """The one method of pytest's monkeypatch that FakeCABI.install uses."""

    @staticmethod
    def setattr(obj, name, value):
        setattr(obj, name, value)


def _init(rank, store_path):
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("gloo", init_method=f"file://{store_path}", rank=rank, world_size=WORLD)
    torch.manual_seed(0)
    torch.set_num_threads(1)
    from tests.fake_cabi import FakeCABI
    return FakeCABI().install(_Patch)


def _rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


# ---------------------------------------------------------------------------------------
def _scan_worker(rank, store_path, out_path):
    _init(rank, store_path)
    from oracle import scan_np
    from slinoss_b200.ops.v2x2ssd import v2x2ssd_cute
    from slinoss_b200.synthetic import make_scan_case
    try:
        full = make_scan_case(4, 2, 40, 4, 4, seed=3)            # the same bits on every rank
        mine = shard.shard_batch([*full.tensors(), full.dY], dist.get_world_size(), rank)
        leaves = [t.clone().requires_grad_(True) for t in mine[:5]]
        Y = v2x2ssd_cute(*leaves, chunk_size=16)
        grads = torch.autograd.grad(Y, leaves, mine[5])
        # whole-job bookkeeping: rank r pretends its step took (r + 1) ms
        units = mine[0].shape[0] * mine[0].shape[2]
        per_s, total_units, max_ms = shard.job_throughput(units, float(rank + 1))
        gathered = [None] * dist.get_world_size()
        dist.all_gather_object(gathered, [Y.detach().numpy()] + [g.numpy() for g in grads])
        if rank == 0:
            n = lambda t: t.double().numpy()
            want = scan_np.v2x2ssd(*[n(t) for t in full.tensors()], chunk_size=16)
            wg = scan_np.v2x2ssd_bwd(*[n(t) for t in full.tensors()], n(full.dY))
            got = [np.concatenate([g[i] for g in gathered], axis=0) for i in range(6)]
            errs = [_rel(got[0], want[0])] + [_rel(got[1 + i], wg[k]) for i, k in enumerate("UMKBC")]
            np.savez(out_path, errs=np.array(errs), per_s=per_s, total_units=total_units, max_ms=max_ms)
    finally:
        dist.destroy_process_group()


def test_two_ranks_own_disjoint_scan_shards_and_need_no_collective(tmp_path):
    store, out = tmp_path / "store", tmp_path / "out.npz"
    mp.spawn(_scan_worker, args=(str(store), str(out)), nprocs=WORLD, join=True)
    r = np.load(out)
    assert r["errs"].max() <= 1e-5, r["errs"]                  # float32 casts of a float64 oracle
    assert int(r["total_units"]) == 4 * 40                       # SUM over ranks of batch x T
    assert float(r["max_ms"]) == 2.0                             # MAX over ranks
    assert abs(float(r["per_s"]) - 160 / 2e-3) < 1e-6


# ---------------------------------------------------------------------------------------
def _mixer_worker(rank, store_path, out_path):
    _init(rank, store_path)
    import slinoss_b200 as sb
    try:
        torch.manual_seed(11)
        mixer = sb.SLinOSSMixer(16, d_state=8, expand=2, d_head=8, d_conv=4, chunk_size=8)
        x = torch.randn(4, 12, 16)
        w = torch.randn(4, 12, 16)

        def grads_of(xb, wb):
            mixer.zero_grad(set_to_none=True)
            (mixer(xb) * wb).mean().backward()
            return [p.grad.clone() for p in mixer.parameters()]

        full = grads_of(x, w)                                    # single-process answer
        xs, ws = shard.shard_batch([x, w], dist.get_world_size(), rank)
        local = grads_of(xs, ws)
        shard.allreduce_mean_(local)
        errs = [_rel(a.numpy(), b.numpy()) for a, b in zip(local, full)]
        if rank == 0:
            np.savez(out_path, errs=np.array(errs))
    finally:
        dist.destroy_process_group()


def test_two_ranks_average_the_mixer_weight_gradients(tmp_path):
    store, out = tmp_path / "store", tmp_path / "out.npz"
    mp.spawn(_mixer_worker, args=(str(store), str(out)), nprocs=WORLD, join=True)
    assert np.load(out)["errs"].max() <= 2e-5


# ---------------------------------------------------------------------------------------
def _lm_worker(rank, store_path, out_path):
    """The stacked-LM step on two ranks: bucketed, hook-driven gradient averaging must give the
    single-process full-batch gradients, and the same as the flat one-bucket averaging."""
    _init(rank, store_path)
    from slinoss_b200.lm import SLinOSSLM, lm_stack_config
    try:
        torch.manual_seed(5)
        model = SLinOSSLM(50, lm_stack_config(d_model=16, n_layers=2, d_state=4, d_head=8, ffn_expand=2.0))
        model.extra_unused = torch.nn.Parameter(torch.ones(3))     # never gets a gradient
        ids = torch.randint(0, 50, (4, 12))

        def grads_of(batch, reducer=None):
            model.zero_grad(set_to_none=True)
            model.loss(batch).backward()
            if reducer is not None:
                reducer.finish()
            return [None if p.grad is None else p.grad.clone() for p in model.parameters()]

        full = grads_of(ids)                                   # single-process answer
        (mine,) = shard.shard_batch([ids], dist.get_world_size(), rank)
        flat = grads_of(mine)
        shard.allreduce_mean_(flat)
        # buckets of 2 KB: the 2-block model spreads over dozens of them
        reducer = shard.GradBucketReducer(model.parameters(), bucket_bytes=2048)
        bucketed = grads_of(mine, reducer)
        again = grads_of(mine, reducer)                        # the reducer is reusable step after step
        # the averaged gradients are left as views of the buckets (no copy back)
        b0 = reducer.buckets[0]
        lo, hi = b0["flat"].data_ptr(), b0["flat"].data_ptr() + b0["flat"].numel() * b0["flat"].element_size()
        views = all(lo <= q.grad.data_ptr() < hi for q in b0["params"] if q.grad is not None)
        reducer.remove()
        wide = shard.GradBucketReducer(model.parameters(), bucket_bytes=4096, reduce_dtype=torch.float64)
        in_double = grads_of(mine, wide)                       # summed in another type: copied back instead
        wide.remove()
        errs_wide = [_rel(a.numpy(), b.numpy()) for a, b in zip(in_double, flat) if b is not None]
        pairs = [(a, b, c, d) for a, b, c, d in zip(bucketed, flat, full, again) if c is not None]
        errs_flat = [_rel(a.numpy(), b.numpy()) for a, b, _, _ in pairs]
        errs_full = [_rel(a.numpy(), c.numpy()) for a, _, c, _ in pairs]
        errs_again = [_rel(a.numpy(), d.numpy()) for a, _, _, d in pairs]
        if rank == 0:
            np.savez(out_path, errs_flat=np.array(errs_flat), errs_full=np.array(errs_full),
                     errs_again=np.array(errs_again), n_buckets=len(reducer.buckets), views=views,
                     errs_wide=np.array(errs_wide))
    finally:
        dist.destroy_process_group()


def test_bucketed_gradient_allreduce_equals_flat_averaging_and_the_full_batch(tmp_path):
    store, out = tmp_path / "store", tmp_path / "out.npz"
    mp.spawn(_lm_worker, args=(str(store), str(out)), nprocs=WORLD, join=True)
    r = np.load(out)
    assert int(r["n_buckets"]) > 10
    assert r["errs_flat"].max() <= 1e-6, r["errs_flat"]       # same sums, same order of ranks
    assert r["errs_again"].max() == 0.0
    assert bool(r["views"]) and r["errs_wide"].max() <= 1e-6
    # equal shards: the mean of the ranks' mean-losses is the full-batch mean-loss
    assert r["errs_full"].max() <= 2e-5, r["errs_full"]


# ---------------------------------------------------------------------------------------
def test_shard_bounds_cover_the_units_once():
    for n in (0, 1, 7, 8, 33):
        for world in (1, 2, 3, 8):
            spans = [shard.shard_bounds(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard.shard_bounds(4, 2, 2)


def test_single_process_meaning_without_a_group():
    assert shard.world_size() == 1 and shard.rank() == 0
    assert shard.reduce_step_ms(3.5) == 3.5
    assert shard.job_throughput(100, 2.0) == (100 / 2e-3, 100, 2.0)
    g = [torch.ones(3), None]
    shard.allreduce_mean_(g)
    assert torch.equal(g[0], torch.ones(3))
    assert shard.rank_seed(5, 0) != shard.rank_seed(5, 1)


# ---------------------------------------------------------------------------------------
def _seqpar_worker(rank, store_path, out_path):
    _init(rank, store_path)
    from oracle import scan_np
    from slinoss_b200.ops.v2x2ssd import v2x2ssd_sequence_parallel
    from slinoss_b200.synthetic import make_scan_case
    try:
        full = make_scan_case(2, 4, 56, 4, 4, groups=2, seed=5, with_init=True, streaming=True)
        cut = [0, 24, 56]                                           # ragged: 24 tokens on rank 0, 32 on rank 1
        sl = slice(cut[rank], cut[rank + 1])
        leaves = [t[:, :, sl].clone().requires_grad_(True) for t in full.tensors()]
        extra = [t.clone().requires_grad_(True) for t in (full.initial_states, full.B_prev, full.U_prev)]
        Y, end, b_last, u_last = v2x2ssd_sequence_parallel(
            *leaves, chunk_size=16, initial_states=extra[0], B_prev=extra[1], U_prev=extra[2])
        gen = torch.Generator().manual_seed(9)
        d_end = torch.randn(end.shape, generator=gen)
        loss = (Y * full.dY[:, :, sl]).sum()
        if rank == WORLD - 1:
            loss = loss + (end * d_end).sum()                        # gradient of the whole sequence's end state
        grads = torch.autograd.grad(loss, leaves + extra, allow_unused=True)   # every rank: the exchange's backward is a collective
        gathered = [None] * WORLD
        dist.all_gather_object(gathered, [Y.detach().numpy(), end.detach().numpy()]
                               + [None if g is None else g.numpy() for g in grads])
        if rank == 0:
            n = lambda t: t.double().numpy()
            ins = [n(t) for t in full.tensors()]
            kw = dict(initial_states=n(full.initial_states), B_prev=n(full.B_prev), U_prev=n(full.U_prev))
            wY, wfin, _, _ = scan_np.v2x2ssm(*ins, **kw)
            wg = scan_np.v2x2ssd_bwd(*ins, n(full.dY), d_final_state=n(d_end), **kw)
            errs = [_rel(np.concatenate([g[0] for g in gathered], axis=2), wY), _rel(gathered[1][1], wfin)]
            for i, k in enumerate("UMKBC"):
                errs.append(_rel(np.concatenate([g[2 + i] for g in gathered], axis=2), wg[k]))
            for i, k in enumerate(("initial_states", "B_prev", "U_prev")):
                errs.append(_rel(gathered[0][7 + i], wg[k]))        # what precedes the sequence lives on rank 0
            np.savez(out_path, errs=np.array(errs))
    finally:
        dist.destroy_process_group()


def test_sequence_sharded_over_two_ranks_equals_the_whole_sequence(tmp_path):
    store, out = tmp_path / "store", tmp_path / "out.npz"
    mp.spawn(_seqpar_worker, args=(str(store), str(out)), nprocs=WORLD, join=True)
    errs = np.load(out)["errs"]
    assert errs.max() <= 2e-5, errs


# ---------------------------------------------------------------------------------------
def _mixer_seqpar_worker(rank, store_path, out_path):
    """A two-block stack on a sequence sharded in time: every mixer's conv takes its left context from the
    previous rank, its scan the start state and taps; outputs and gradients must equal the single-process full
    sequence."""
    _init(rank, store_path)
    import slinoss_b200 as sb
    try:
        torch.manual_seed(13)
        blk = sb.SLinOSSBlockConfig(d_model=16, mixer=sb.SLinOSSMixerConfig(d_state=8, expand=2.0, d_head=8,
                                                                            chunk_size=8),
                                    ffn=sb.SLinOSSMLPConfig(kind="gelu", expand=2.0, multiple_of=8))
        mixer = sb.SLinOSSStack(sb.SLinOSSStackConfig.uniform(blk, n_layers=2))    # two blocks: two exchanges deep
        x = torch.randn(2, 40, 16)
        w = torch.randn(2, 40, 16)
        cut = [0, 17, 40]                                        # ragged slices

        mixer.zero_grad(set_to_none=True)
        xf = x.clone().requires_grad_(True)
        out_full = mixer(xf)
        (out_full * w).sum().backward()
        full = [p.grad.clone() for p in mixer.parameters()]
        gx_full = xf.grad.clone()

        mixer.zero_grad(set_to_none=True)
        sl = slice(cut[rank], cut[rank + 1])
        xs = x[:, sl].clone().requires_grad_(True)
        out = mixer(xs, sequence_group=dist.group.WORLD)
        (out * w[:, sl]).sum().backward()                        # every rank: the exchanges' backward is collective
        local = [p.grad.clone() for p in mixer.parameters()]
        for g in local:                                          # every rank saw only its tokens: SUM over ranks
            dist.all_reduce(g, op=dist.ReduceOp.SUM)
        errs = [_rel(out.detach().numpy(), out_full[:, sl].detach().numpy()),
                _rel(xs.grad.numpy(), gx_full[:, sl].numpy())]
        errs += [_rel(a.numpy(), b.numpy()) for a, b in zip(local, full)]
        gathered = [None] * WORLD
        dist.all_gather_object(gathered, errs)
        if rank == 0:
            np.savez(out_path, errs=np.array(gathered))
    finally:
        dist.destroy_process_group()


def test_stack_on_a_time_sharded_sequence_equals_the_whole_sequence(tmp_path):
    store, out = tmp_path / "store", tmp_path / "out.npz"
    mp.spawn(_mixer_seqpar_worker, args=(str(store), str(out)), nprocs=WORLD, join=True)
    errs = np.load(out)["errs"]
    assert errs.max() <= 5e-5, errs


# ---------------------------------------------------------------------------------------
def _lm_seqpar_worker(rank, store_path, out_path):
    """The LM loss on token ids sharded in time: the shares add up to the single-process loss, their
    gradients (summed over ranks) to its gradient."""
    _init(rank, store_path)
    from slinoss_b200.lm import SLinOSSLM, lm_stack_config
    try:
        torch.manual_seed(7)
        model = SLinOSSLM(50, lm_stack_config(d_model=16, n_layers=2, d_state=4, d_head=8, ffn_expand=2.0))
        ids = torch.randint(0, 50, (3, 30))
        model.zero_grad(set_to_none=True)
        full = model.loss(ids)
        full.backward()
        want = [p.grad.clone() for p in model.parameters()]
        cut = [0, 13, 30]
        model.zero_grad(set_to_none=True)
        share = model.loss(ids[:, cut[rank]:cut[rank + 1]], sequence_group=dist.group.WORLD)
        share.backward()
        got = [p.grad.clone() for p in model.parameters()]
        total = share.detach().clone()
        dist.all_reduce(total)
        for g in got:
            dist.all_reduce(g)
        if rank == 0:
            errs = [abs(float(total) - float(full)) / abs(float(full))]
            errs += [_rel(a.numpy(), b.numpy()) for a, b in zip(got, want)]
            np.savez(out_path, errs=np.array(errs))
    finally:
        dist.destroy_process_group()


def test_lm_loss_on_time_sharded_ids_adds_up_to_the_whole_sequence(tmp_path):
    store, out = tmp_path / "store", tmp_path / "out.npz"
    mp.spawn(_lm_seqpar_worker, args=(str(store), str(out)), nprocs=WORLD, join=True)
    errs = np.load(out)["errs"]
    assert errs.max() <= 5e-5, errs
