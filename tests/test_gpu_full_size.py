"""Parity at the sequence lengths of the benchmark configurations (the oracle is O(N^2), so it
is run on a slice: a few heads of the training shape, row blocks of the long one, one (batch, head)
pair of the decode cache) plus size-independent properties on the full training shape."""
import math

import pytest
import torch

from helpers import TOL_BF16, maxabs, check_outputs, dtheta_tol
from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu


def _slice_fwd_bwd(B, H, N, d, cq, ck, seed, label):
    import fmta_b200 as F
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=seed, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    Or, Mr, Lr = orc.conv_attn_fwd(Q, K, V, theta, scale, True)
    rq, rk, rv, rt = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, True)
    ref = dict(O=Or, M=Mr, LSE=Mr + torch.log(Lr), dQ=rq, dK=rk, dV=rv, dTheta=rt)
    for path in (1, 0):
        O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=path)
        Dv = F.rowdot(do, O)
        dQ, dK, dV, dTh = F.backward(q, k, v, do, Dv, LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=path)
        torch.cuda.synchronize()
        check_outputs(dict(O=O, M=M, LSE=LSE, dQ=dQ, dK=dK, dV=dV, dTheta=dTh), ref, "%s path %d" % (label, path))


def test_training_shape_slice_N4096():
    """All four batch entries of ONE head of the bf16 training configuration (N=4096, d=64, theta (6,11)), so
    that dTheta carries the full batch sum: forward and fused backward on the tensor-core + band path and on
    the exact path against the dense oracle."""
    _slice_fwd_bwd(4, 1, 4096, 64, 6, 11, 4096, "config 1 slice (B=4, one head, N=4096, d=64)")


def test_sweep_shape_slice_N4096_d128():
    """One (batch, head) pair of the d = 128 sweep configuration at N=4096, theta (6,11), both paths."""
    _slice_fwd_bwd(1, 1, 4096, 128, 6, 11, 4128, "config 4 slice (one (b,h), N=4096, d=128)")


def test_sweep_shape_N65536_d128_row_blocks():
    """One (batch, head) pair of the sweep configuration at its longest sequence, N=65536, d=128: the forward
    is checked on row blocks with the O(rows x N) oracle; the backward (tensor-core path) must be finite,
    and dV / dTheta linear in dO."""
    import fmta_b200 as F
    B, H, N, d, cq, ck = 1, 1, 65536, 128, 6, 11
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=65536, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True)
    torch.cuda.synchronize()
    for i0, i1 in ((0, 24), (32760, 32776), (50001, 50017), (65520, 65536)):
        Or, Mr, Lr = orc.conv_attn_fwd_rowblock(Q, K, V, theta, i0, i1, scale, True)
        check_outputs(dict(O=O[:, :, i0:i1], M=M[:, :, i0:i1], LSE=LSE[:, :, i0:i1]),
                      dict(O=Or, M=Mr, LSE=Mr + torch.log(Lr)), "config 4 N=65536 rows %d-%d" % (i0, i1))
    g1 = F.backward(q, k, v, do, F.rowdot(do, O), LSE, th, scale, cq - 1, (ck - 1) // 2, True)
    do2 = (do.float() * 0.5).to(torch.bfloat16)
    g2 = F.backward(q, k, v, do2, F.rowdot(do2, O), LSE, th, scale, cq - 1, (ck - 1) // 2, True)
    torch.cuda.synchronize()
    for t in g1:
        assert torch.isfinite(t).all()
    assert float((g2[2] - 0.5 * g1[2]).abs().max()) <= 1e-2
    assert float((g2[3] - 0.5 * g1[3]).abs().max()) <= 5e-3 * float(g1[3].abs().max())


def test_long_sequence_row_blocks_N16384_d128():
    """d=128 sweep shape at N=16384: forward checked on row blocks with the O(rows x N) oracle."""
    import fmta_b200 as F
    B, H, N, d, cq, ck = 1, 1, 16384, 128, 6, 11
    Q, K, V, _, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=16384, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V))
    O, M, L = F.forward(q, k, v, theta.cuda(), scale, cq - 1, (ck - 1) // 2, True)
    torch.cuda.synchronize()
    for i0, i1 in ((0, 40), (8000, 8040), (12281, 12300), (16320, 16384)):
        Or, Mr, Lr = orc.conv_attn_fwd_rowblock(Q, K, V, theta, i0, i1, scale, True)
        assert maxabs(O[:, :, i0:i1], Or) <= TOL_BF16
        assert maxabs(M[:, :, i0:i1], Mr) <= TOL_BF16
        assert maxabs((M + torch.log(L))[:, :, i0:i1], Mr + torch.log(Lr)) <= TOL_BF16


def test_full_training_shape_properties():
    """Whole bf16 training configuration (B=4,H=16,N=4096,d=64): properties that need no oracle.
    O is linear in V; rows of P sum to one (O == 1 for V == 1); dV is linear in dO."""
    import fmta_b200 as F
    B, H, N, d, cq, ck = 4, 16, 4096, 64, 6, 11
    g = torch.Generator(device="cuda").manual_seed(1)
    q, k, v1, v2, do = (torch.randn(B, H, N, d, device="cuda", generator=g).to(torch.bfloat16) for _ in range(5))
    th = torch.randn(H, cq, ck, device="cuda", generator=g) * 0.02
    th[:, cq - 1, ck // 2] += 1.0
    scale = 1.0 / math.sqrt(d)
    f = lambda v: F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True)
    O1, M1, L1, LSE = f(v1)
    O2 = f(v2)[0]
    O12 = f((v1.float() + v2.float()).to(torch.bfloat16))[0]
    # v1+v2 is rounded to bf16 once more: allow that rounding (2^-8 relative on |v| <~ 6)
    assert float((O12 - (O1 + O2)).abs().max()) <= 4e-2
    ones = torch.ones_like(v1)
    Oone = f(ones)[0]
    assert float((Oone - 1.0).abs().max()) <= 1e-2
    assert torch.isfinite(M1).all() and torch.isfinite(L1).all() and float(L1.min()) >= 1.0 - 1e-3
    D1 = F.rowdot(do, O1)
    g1 = F.backward(q, k, v1, do, D1, LSE, th, scale, cq - 1, (ck - 1) // 2, True)
    for t in g1:
        assert torch.isfinite(t).all()
    # the gradient w.r.t. V does not depend on D and is linear in dO
    do2 = (do.float() * 0.5).to(torch.bfloat16)
    g2 = F.backward(q, k, v1, do2, F.rowdot(do2, O1), LSE, th, scale, cq - 1, (ck - 1) // 2, True)
    assert float((g2[2] - 0.5 * g1[2]).abs().max()) <= 1e-2
    assert float((g2[0] - 0.5 * g1[0]).abs().max()) <= 1e-2      # dQ, dK, dTheta are linear in dO too
    assert float((g2[3] - 0.5 * g1[3]).abs().max()) <= 5e-3 * float(g1[3].abs().max())


def test_decode_full_cache_length():
    """One (batch, head) pair of the decode configuration: Nk=32768, d=128, q_len=6, theta (6,11)."""
    import fmta_b200 as F
    B, H, Nk, d, cq, ck, q_len = 1, 2, 32768, 128, 6, 11, 6
    Q, K, V, _, theta = orc.make_inputs(B, H, 0, d, cq, ck, seed=32768, dtype=torch.bfloat16, Nk=Nk, q_len=q_len)
    scale = 1.0 / math.sqrt(d)
    Or, Mr, Lr = orc.decode_last_row_streaming(Q, K, V, theta, scale, chunk=4096)
    qb, kb, vb = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V))
    for ks in (1, 4):
        O, M, L = F.fwd_conv_attn_inference(qb, kb, vb, theta.cuda(), ks, scale, cq - 1, (ck - 1) // 2, False)
        assert maxabs(O, Or) <= TOL_BF16
        assert maxabs(M, Mr) <= TOL_BF16
        assert maxabs(M + torch.log(L), Mr + torch.log(Lr)) <= TOL_BF16


def _mix_inputs(B, H, N, d, cq, ck, G, seed):
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=seed, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(seed + 1)
    w = torch.eye(G).repeat(H // G, 1, 1) + 0.02 * torch.randn(H // G, G, G, generator=g)   # identity + N(0, 0.02)
    return Q, K, V, dO, theta, w.contiguous()


def test_head_mix_configuration_N8192_d128_forward_row_blocks():
    """Head-mixing configuration at its full sequence length (N=8192, d=128, theta (6,11), groups of 4, mixing
    matrices identity + N(0, 0.02)) on one group: the forward against the composed oracle on row blocks."""
    import fmta_b200 as F
    B, H, N, d, cq, ck, G = 1, 4, 8192, 128, 6, 11, 4
    Q, K, V, dO, theta, w = _mix_inputs(B, H, N, d, cq, ck, G, 8192)
    scale = 1.0 / math.sqrt(d)
    q, k, v = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V))
    o, l, m, lse = F.conv_headmix_forward(q, k, v, w.cuda(), theta.cuda(), scale, True, out_dtype=torch.float32)
    torch.cuda.synchronize()
    wd = orc.block_diag_mix(w)
    for i0, i1 in ((0, 24), (4090, 4106), (8176, 8192)):
        Or, Mr, Lr = orc.conv_headmix_fwd_rowblock(Q, K, V, theta, wd, i0, i1, scale, True)
        check_outputs(dict(O=o[:, :, i0:i1], M=m[:, :, i0:i1], LSE=lse[:, :, i0:i1]),
                      dict(O=Or, M=Mr, LSE=Mr + torch.log(Lr)), "config 3 N=8192 rows %d-%d" % (i0, i1))


def test_head_mix_configuration_N2048_d128_backward_dense_oracle():
    """The same operator at N=2048 (the dense composed oracle fits): forward and all five gradients
    (dQ, dK, dV, dTheta, dW) with non-trivial mixing matrices."""
    import fmta_b200 as F
    B, H, N, d, cq, ck, G = 1, 4, 2048, 128, 6, 11, 4
    Q, K, V, dO, theta, w = _mix_inputs(B, H, N, d, cq, ck, G, 2048)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th, wg = theta.cuda(), w.cuda()
    wd = orc.block_diag_mix(w)
    Or, Mr, Lr = orc.conv_headmix_fwd(Q, K, V, theta, wd, scale, True)
    rq, rk, rv, rt, rw = orc.conv_headmix_bwd_autograd(Q, K, V, theta, wd, dO, scale, True)
    rwg = torch.stack([rw[i * G:(i + 1) * G, i * G:(i + 1) * G] for i in range(H // G)])
    o, l, m, lse = F.conv_headmix_forward(q, k, v, wg, th, scale, True, out_dtype=torch.float32)
    dq, dw, dth = F.conv_headmix_bwd_dq_dw(q, k, v, wg, o, do, l, m, th, True, scale)
    dk, dv = F.conv_headmix_bwd_dkdv(q, k, v, wg, o, do, l, m, th, True, scale)
    torch.cuda.synchronize()
    check_outputs(dict(O=o, M=m, LSE=lse, dQ=dq, dK=dk, dV=dv, dTheta=dth, dW=dw),
                  dict(O=Or, M=Mr, LSE=Mr + torch.log(Lr), dQ=rq, dK=rk, dV=rv, dTheta=rt, dW=rwg),
                  "config 3 slice (one group of 4 heads, N=2048, d=128)")


def test_long_sequence_tensor_core_path_agrees_with_exact_path_N16384():
    """N = 16384 (d = 64): too long for the O(N^2) oracle, so the tensor-core + band path is held against
    the exact tile kernels (which the oracle pins at the lengths it reaches) on the same inputs, forward
    and backward; plus 256 (batch, head) pairs at N = 1024 to cover large leading dimensions."""
    import fmta_b200 as F
    for (B, H, N) in ((1, 2, 16384), (8, 32, 1024)):
        d, cq, ck = 64, 6, 11
        g = torch.Generator(device="cuda").manual_seed(N)
        q, k, v, do = (torch.randn(B, H, N, d, device="cuda", generator=g).to(torch.bfloat16) for _ in range(4))
        th = torch.randn(H, cq, ck, device="cuda", generator=g) * 0.02
        th[:, cq - 1, ck // 2] += 1.0
        scale = 1.0 / math.sqrt(d)
        res = []
        for path in (0, 1):
            O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=path)
            D = F.rowdot(do, O)
            res.append((O, LSE) + tuple(F.backward(q, k, v, do, D, LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=path)))
        names = ("O", "LSE", "dQ", "dK", "dV")
        for n, a, b in zip(names, res[0], res[1]):
            assert maxabs(a, b) <= TOL_BF16, (n, B, H, N)
        assert maxabs(res[0][5], res[1][5]) <= dtheta_tol(res[0][5])
