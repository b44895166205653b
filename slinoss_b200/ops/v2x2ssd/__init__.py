"""v2x2ssd scan operator on sm_100a CUDA kernels.

Drop-in surface of ``slinoss.ops.v2x2ssd`` for CUDA tensors:

``v2x2ssd``        same signature and 4-tuple result as the reference's ``v2x2ssd``
                   (slinoss/ops/v2x2ssd/reference.py:1267-1347)
``v2x2ssd_cute``   same signature as the reference's GPU entry point, with
                   ``return_state`` (slinoss/ops/v2x2ssd/cute/api.py:53-200)
``v2x2ssd_decode`` one-token update of ``(state, b_prev, u_prev)``
``v2x2ssd_sequence_parallel``  the same scan with the time axis sharded over the ranks of a process
                   group (one exchange of state-sized tensors between two local passes)

All of them are differentiable through ``torch.autograd`` (decode excepted) and
run only on CUDA tensors: there is no CPU path in this package.
"""

from .api import assert_nonzero_transitions, v2x2ssd, v2x2ssd_cute, v2x2ssd_decode
from .sequence_parallel import v2x2ssd_sequence_parallel

__all__ = ["assert_nonzero_transitions", "v2x2ssd", "v2x2ssd_cute", "v2x2ssd_decode", "v2x2ssd_sequence_parallel"]
