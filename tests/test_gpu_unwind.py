"""The bounded waits of the tensor-core scan kernels: an expired wait makes the kernel unwind
(drain what it has in flight, free its TMEM, return), the host sees it through
``sl_device_status`` and the next launch works normally.

The wait is made to expire without anything being wrong: ``SLINOSS_B200_WAIT_CLOCKS=1`` sets the
limit of the main loops' waits to one clock, so the very first wait for data that is still on its
way gives up.  The waits of the unwind path itself keep their long limit, so everything in flight
has landed before shared memory and TMEM are released.  One CTA; two chunks for the forward, sixteen
for the backward (with two, every one of its waits happened to find its data already there).
"""

import pytest
import torch

from oracle import scan_np
from slinoss_b200 import _C
from slinoss_b200.synthetic import make_scan_case
from tests.util import n64, rel

pytestmark = pytest.mark.gpu
DEV = "cuda"
SL_ERR_DEVICE_TIMEOUT = 7


def _forward(c):
    return _C.scan_fwd(c.U, c.M, c.K, c.B, c.C, None, None, None, chunk_size=64,
                       y_dtype=torch.bfloat16, want_final=True, path="tc", save_states=True)


def _backward(c, saved):
    return _C.scan_bwd(c.U, c.M, c.K, c.B, c.C, None, None, None, c.dY, None, chunk_size=64,
                       path="tc", saved=saved)


@pytest.mark.parametrize("which", ["forward", "backward"])
def test_expired_wait_unwinds_and_the_status_can_be_cleared(which, monkeypatch):
    case = make_scan_case(1, 1, 128 if which == "forward" else 1024, 64, 64, dtype=torch.bfloat16, seed=4)
    c = case.to(DEV)
    torch.cuda.synchronize()
    _C.device_status_reset()
    assert _C.device_status() == 0
    Y, fin, states = _forward(c)                      # a good forward: its states feed the backward
    torch.cuda.synchronize()
    assert _C.device_status() == 0

    monkeypatch.setenv("SLINOSS_B200_WAIT_CLOCKS", "1")
    if which == "forward":
        _forward(c)                                   # returns SL_OK: the launch itself is fine
    else:
        _backward(c, (states, fin))
    torch.cuda.synchronize()                          # the kernel has returned: no hang
    monkeypatch.delenv("SLINOSS_B200_WAIT_CLOCKS")
    assert _C.device_status() == SL_ERR_DEVICE_TIMEOUT
    site = _C.device_status_reset()
    assert site != 0
    assert _C.device_status() == 0 and _C.device_status_reset() == 0

    # the context is intact: the same calls with the normal limit give the right answers
    args = [n64(t) for t in case.tensors()]
    Y2, fin2, states2 = _forward(c)
    grads = _backward(c, (states2, fin2))
    torch.cuda.synchronize()
    assert _C.device_status() == 0
    assert rel(Y2, scan_np.v2x2ssm(*args)[0]) <= 2e-2
    want = scan_np.v2x2ssd_bwd(*args, n64(case.dY))
    for name, g in zip("UMKBC", grads[:5]):
        assert rel(g, want[name]) <= 2e-2, name
