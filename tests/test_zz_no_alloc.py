"""fmta_bwd_dq_dw_static: the backward entry point for callers that cannot allocate device
memory (frozen memory pools, frameworks that own the GPU, bindings without an allocator).  It
must give the same dQ / dTheta as fmta_bwd_dq_dw, call after call, although its scratch is one
array inside the library that every call reuses.  Called through the C ABI with ctypes."""
import ctypes
import math

import pytest
import torch

from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_static_scratch_matches_workspace_variant_twice():
    import fmta_b200 as F
    from fmta_b200._lib import lib, FMTA_OP_BWD_DQ
    B, H, N, d, cq, ck = 2, 4, 300, 64, 6, 11
    scale = 1.0 / math.sqrt(d)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):           # two calls in a row: the second one sees the first one's leftovers
        Q, K, V, dO, th = orc.make_inputs(B, H, N, d, cq, ck, seed=11 + call, dtype=torch.bfloat16)
        q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
        th = th.cuda()
        O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True)
        D = F.rowdot(do, O)
        nbytes = lib.fmta_workspace_bytes(FMTA_OP_BWD_DQ, B, H, N, d, cq, ck, 1)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        dQ_a = torch.empty(B, H, N, d, device="cuda"); dT_a = torch.empty(H, cq, ck, device="cuda")
        dQ_b = torch.full_like(dQ_a, float("nan")); dT_b = torch.full_like(dT_a, float("nan"))
        rc = lib.fmta_bwd_dq_dw(_p(q), _p(k), _p(v), _p(do), _p(D), _p(LSE), _p(th), None, _p(dQ_a), _p(dT_a), None,
                                B, H, N, d, cq, ck, 1, scale, 1, _p(ws), nbytes, st)
        assert rc == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.fmta_bwd_dq_dw_static(_p(q), _p(k), _p(v), _p(do), _p(D), _p(LSE), _p(th), None, _p(dQ_b), _p(dT_b),
                                       None, B, H, N, d, cq, ck, 1, scale, 1, st)
        assert rc == 0, lib.fmta_strerror(rc)
        torch.cuda.synchronize()
        if call == 1:   # once the first call has looked up the array's address, a call leaves the device's free memory as it was
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernels, same summation order: identical results (the suite's tolerance is 2e-2)
        assert torch.equal(dQ_a, dQ_b)
        assert torch.equal(dT_a, dT_b)
        # and both agree with the oracle
        ref = orc.conv_attn_bwd_autograd(Q, K, V, th.cpu(), dO, scale, True)
        assert float((dQ_b.cpu() - ref[0]).abs().max()) <= 2e-2


def test_static_scratch_rejects_oversized_problems():
    from fmta_b200._lib import lib
    good = ctypes.c_void_p(0x1000)
    # B * ceil(N/64) * H*cq*ck * 4 bytes = 64 * 64 * 32*66 * 4 = 34.6 MB > 4 MiB: refused on the host
    rc = lib.fmta_bwd_dq_dw_static(good, good, good, good, good, good, good, None, good, good, None,
                                   64, 32, 4096, 64, 6, 11, 1, 0.125, 1, None)
    assert rc == -7
    assert b"4 MiB" in lib.fmta_strerror(rc)
    # without a filter or a mixing matrix there are no partial sums: no size limit applies, and the
    # filter-shape arguments are ignored as fmta_bwd_dq_dw ignores them (the NULL dQ is what is refused)
    rc = lib.fmta_bwd_dq_dw_static(good, good, good, good, good, good, None, None, None, None, None,
                                   64, 32, 4096, 64, 0, 0, 0, 0.125, 1, None)
    assert rc == -1
