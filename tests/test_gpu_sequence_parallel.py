"""The sequence-parallel scan on one GPU: a process group of ONE rank with the two passes and the exchange
forced, against the plain op (the multi-rank arithmetic is covered by the two-rank gloo test on CPU and was run
on 2 and 8 GPUs with the torchrun harness)."""

import pytest
import torch
import torch.distributed as dist

from slinoss_b200 import _C
from slinoss_b200.ops.v2x2ssd import v2x2ssd_cute, v2x2ssd_sequence_parallel
from slinoss_b200.synthetic import make_scan_case
from tests.util import rel

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture()
def one_rank_group(tmp_path):
    dist.init_process_group("nccl", init_method=f"file://{tmp_path / 'store'}", rank=0, world_size=1,
                            device_id=torch.device("cuda", torch.cuda.current_device()))
    yield
    dist.destroy_process_group()


def test_two_passes_and_exchange_on_one_rank_equal_the_plain_op(one_rank_group):
    case = make_scan_case(2, 4, 300, 64, 64, groups=2, dtype=torch.bfloat16, seed=4, with_init=True,
                          streaming=True).to(DEV)
    extra = dict(initial_states=case.initial_states, B_prev=case.B_prev, U_prev=case.U_prev)

    def run(sharded):
        lv = [t.clone().requires_grad_(True) for t in case.tensors()]
        if sharded:
            Y, end, _, _ = v2x2ssd_sequence_parallel(*lv, chunk_size=64, single_rank_exchange=True, **extra)
        else:
            Y, end, _, _ = v2x2ssd_cute(*lv, chunk_size=64, return_state=True, output_dtype=torch.float32, **extra)
        return Y, end, torch.autograd.grad(Y.float(), lv, case.dY.float())

    n0 = _C.kernel_launches()
    Ys, ends, gs = run(True)
    launched = _C.kernel_launches() - n0
    Yp, endp, gp = run(False)
    assert _C.device_status() == 0
    assert launched <= 12          # two forward launches, two tensor-core backward launch groups: no float32 sweeps
    assert rel(Ys, Yp) <= 1e-2 and rel(ends, endp) <= 1e-2
    for name, a, b in zip("UMKBC", gs, gp):
        assert rel(a, b) <= 2e-2, (name, rel(a, b))
