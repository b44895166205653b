"""The allocation-free scan backward (``sl_v2x2ssd_bwd_static``).

Some users of the library cannot give it scratch memory because they cannot call
``cudaMalloc`` at that point (the GPU is fully owned by their own pool, or their
serving loop forbids allocator calls).  For them the library carries a fixed
scratch array; this test calls that entry point through the C ABI, twice in a row
on different problems (the second call sees the first call's leftovers in the
shared array), and checks every gradient against the regular entry point, which
takes a caller-allocated workspace.  It also checks that an oversized problem is
refused instead of overrunning the array.

This file sorts last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import pytest
import torch

from slinoss_b200 import _C
from slinoss_b200.synthetic import make_scan_case
from tests.util import rel

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _both(case, dtype):
    c = case.to(DEV)
    args = (c.U, c.M, c.K, c.B, c.C, c.initial_states, c.B_prev, c.U_prev)
    d_final = torch.randn(c.initial_states.shape, device=DEV) if c.initial_states is not None else None
    want = _C.scan_bwd(*args, c.dY, d_final, chunk_size=64, path="simt")
    outs = tuple(None if w is None else torch.full_like(w, float("nan")) for w in want)
    got = _C.scan_bwd_static(*args, c.dY, d_final, outs)
    torch.cuda.synchronize()
    return got, want


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_backward_matches_regular_entry_point(dtype):
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    names = ("dU", "dM", "dK", "dB", "dC", "d_initial", "dB_prev", "dU_prev")
    # two different problems back to back: the second one runs over the first one's leftovers;
    # the second has P > 64, i.e. the variant that accumulates into (self-cleared) scratch
    cases = [make_scan_case(2, 4, 300, 64, 64, groups=2, dtype=dtype, seed=11, streaming=True,
                            with_init=True),
             make_scan_case(1, 2, 90, 96, 16, dtype=dtype, seed=12, streaming=True, with_init=True)]
    for case in cases:
        got, want = _both(case, dtype)
        for name, g, w in zip(names, got, want):
            assert torch.isfinite(g).all(), name
            assert rel(g, w) <= tol, (name, rel(g, w))


def test_static_scratch_refuses_oversized_problems():
    limit = int(_C.lib().sl_static_scratch_bytes())
    assert limit == 64 << 20
    # batch*heads*T*(24*N+8) bytes of scratch: 8*16*4096*(24*64+8) is far above 64 MiB
    case = make_scan_case(1, 1, 8, 64, 64, dtype=torch.bfloat16).to(DEV)
    p = case.U.data_ptr()
    status = _C.lib().sl_v2x2ssd_bwd_static(p, p, p, p, p, None, None, None, p, None, p, p, p, p, p,
                                            None, None, None, 8, 16, 16, 4096, 64, 64, _C.SL_BF16,
                                            _C.SL_BF16, None)
    assert status == 8
    assert b"static" in _C.lib().sl_status_string(status)
