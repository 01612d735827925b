"""Failure detection of the tensor-core kernels: every wait inside them is bounded, and a wait that
runs out must surface on the host as an error instead of silently wrong numbers.  The failure is
produced without faulting or hanging anything: the library's self-test hook points one kernel's
first consumer wait at a barrier that nothing arrives at (limit: a few hundred polls), the kernel
leaves through its normal abort path (stops issuing, waits for what it has in flight, frees its
tensor memory) and sets the status word that the Python layer registered."""
import math

import pytest
import torch

from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu

KERN_FWD, KERN_DQ, KERN_DKDV = 1, 3, 4


def _inputs(N=400, d=64):
    B, H, cq, ck = 1, 2, 6, 11
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=4, dtype=torch.bfloat16)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    return (Q, K, V, dO, theta), (q, k, v, do, theta.cuda()), 1.0 / math.sqrt(d), cq, ck


def test_status_is_zero_after_normal_calls():
    import fmta_b200 as F
    _, (q, k, v, do, th), scale, cq, ck = _inputs()
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=1)
    D = F.rowdot(do, O)
    F.backward(q, k, v, do, D, LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=1)
    F.check_device_status()       # synchronises; raises on a non-zero word


@pytest.mark.parametrize("d,stream_pdc", [(64, True), (64, False), (128, None)])
@pytest.mark.parametrize("kernel", [KERN_FWD, KERN_DQ, KERN_DKDV])
def test_expired_wait_is_reported_and_the_next_call_is_clean(kernel, d, stream_pdc):
    """Every tensor-core kernel family: head dim 64 (recomputing and streaming dK/dV) and head dim 128."""
    import fmta_b200 as F
    from fmta_b200._lib import lib
    (Q, K, V, dO, theta), (q, k, v, do, th), scale, cq, ck = _inputs(d=d)
    F.check_device_status()
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=1)
    D = F.rowdot(do, O)
    assert lib.fmta_selftest_expire_next(kernel) == 0
    if kernel == KERN_FWD:
        F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=1)
    else:
        F.backward(q, k, v, do, D, LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=1, stream_pdc=stream_pdc)
    with pytest.raises(RuntimeError, match="bounded wait"):
        F.check_device_status()
    # the hook is one-shot and the context is intact: the same calls now give the right numbers
    O2, M2, L2, LSE2 = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=1)
    dQ, dK, dV, dTh = F.backward(q, k, v, do, F.rowdot(do, O2), LSE2, th, scale, cq - 1, (ck - 1) // 2, True, path=1)
    F.check_device_status()
    Or, _, _ = orc.conv_attn_fwd(Q, K, V, theta, scale, True)
    rq, rk, rv, rt = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, True)
    for got, ref in ((O2, Or), (dQ, rq), (dK, rk), (dV, rv)):
        assert float((got.float().cpu() - ref).abs().max()) <= 2e-2


def test_selftest_hook_rejects_other_kernels():
    from fmta_b200._lib import lib
    assert lib.fmta_selftest_expire_next(7) == -3
    assert lib.fmta_selftest_expire_next(0) == 0
