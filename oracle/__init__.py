"""CPU oracle for the v2x2ssd scan and its mixer hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is used by ``tests/``, by ``__graft_entry__.smoke()`` and by the
CPU-baseline leg of ``bench.py`` as the checker, never as the computing path.

Contents
--------
``scan_np``      numpy restatement of the sequential scan, the reference's
                 three-stage chunked scan and the analytic backward pass.
``mixer_torch``  torch (CPU, autograd) restatement of scan preparation, the
                 causal depthwise convolution and the gated RMSNorm tail.
``csrc``         C/OpenMP port of the scan forward+backward used to time the
                 CPU path on the host cores of the GPU box.

Parity status: PINNED.  Every function is checked in ``tests/`` against golden
vectors produced by importing the reference implementation itself
(``tests/golden/make_golden.py`` holds the generating script).
"""
