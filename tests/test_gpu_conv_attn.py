"""GPU parity of the conv-attention forward/backward kernels (through the C ABI) against the
CPU oracle and the golden fixtures produced by the reference's own PyTorch code."""
import math

import pytest
import torch

from helpers import TOL_BF16, load_golden, maxabs, bf16_round, check_outputs, dtheta_tol
from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu


def _run_fwd_bwd(Q, K, V, dO, theta, scale, causal):
    import fmta_b200 as F
    dev = "cuda"
    Qb, Kb, Vb, dOb = (t.to(dev).to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.to(dev)
    cq, ck = theta.shape[1:]
    O, M, L, LSE = F.forward(Qb, Kb, Vb, th, scale, cq - 1, (ck - 1) // 2, causal, return_lse=True)
    D = F.rowdot(dOb, O)
    dQ, dTh = F.dq_backward(Qb, Kb, Vb, dOb, D, LSE, th, scale, cq - 1, (ck - 1) // 2, causal)
    dK, dV = F.dkdv_backward(Qb, Kb, Vb, dOb, D, LSE, th, scale, cq - 1, (ck - 1) // 2, causal)
    torch.cuda.synchronize()
    return dict(O=O, M=M, L=L, LSE=LSE, dQ=dQ, dK=dK, dV=dV, dTheta=dTh)


def _check(got, ref, label):
    """O, M, LSE, dQ, dK, dV within 2e-2 of the oracle; dTheta within the one bound every path is held to
    (helpers.dtheta_tol).  L is compared through LSE (it scales with exp(-M))."""
    r = dict(O=ref["O"], M=ref["M"], LSE=ref["M"] + torch.log(ref["L"]), dQ=ref["dQ"], dK=ref["dK"], dV=ref["dV"],
             dTheta=ref["dTheta"])
    check_outputs(got, r, label)


@pytest.mark.parametrize("name", ["conv_ref_script_3x3", "conv_c0_3x5", "conv_6x11_ragged",
                                  "conv_5x5_noncausal", "conv_7x7_d128"])
def test_golden(name):
    """Reference-generated fixtures.  Inputs are rounded to bf16 for the kernel; the fixture
    (fp32 reference on fp32/bf16-exact inputs) is the target, tolerance 2e-2."""
    z = load_golden(name)
    scale, causal = float(z["scale"]), bool(z["causal"])
    # kernels see bf16 inputs: compare against the oracle on the same rounded inputs when the
    # fixture's inputs are not bf16-exact (conv_c0_3x5 is fp32), and against the fixture otherwise
    Q, K, V, dO = (bf16_round(z[k]) for k in ("Q", "K", "V", "dO"))
    exact = all(torch.equal(a, z[k]) for a, k in zip((Q, K, V, dO), ("Q", "K", "V", "dO")))
    if exact:
        ref = z
    else:
        O, M, L = orc.conv_attn_fwd(Q, K, V, z["theta"], scale, causal)
        dQ, dK, dV, dTh = orc.conv_attn_bwd_autograd(Q, K, V, z["theta"], dO, scale, causal)
        ref = dict(O=O, M=M, L=L, dQ=dQ, dK=dK, dV=dV, dTheta=dTh)
    got = _run_fwd_bwd(Q, K, V, dO, z["theta"], scale, causal)
    _check(got, ref, "golden %s" % name)


@pytest.mark.parametrize("B,H,N,d,cq,ck,causal", [
    (1, 1, 1, 64, 3, 3, True),        # single token
    (1, 2, 7, 32, 6, 11, True),       # N < filter
    (2, 2, 129, 64, 6, 11, True),     # one past a tile boundary
    (1, 2, 200, 128, 6, 11, True),
    (1, 2, 191, 64, 11, 11, True),    # widest square filter of the reference dispatch
    (1, 1, 130, 64, 1, 1, True),      # no conv at all
    (1, 2, 150, 64, 3, 5, False),
    (1, 1, 96, 64, 16, 17, True),     # largest supported filter (run-time path)
    (1, 2, 320, 64, 6, 11, False),
])
def test_oracle_shapes(B, H, N, d, cq, ck, causal):
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=N + cq, theta_std=0.05, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    O, M, L = orc.conv_attn_fwd(Q, K, V, theta, scale, causal)
    dQ, dK, dV, dTh = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, causal)
    got = _run_fwd_bwd(Q, K, V, dO, theta, scale, causal)
    _check(got, dict(O=O, M=M, L=L, dQ=dQ, dK=dK, dV=dV, dTheta=dTh), "B%d H%d N%d d%d theta(%d,%d) causal=%d separate calls" % (B, H, N, d, cq, ck, causal))


def test_module_autograd_matches_oracle():
    """The nn.Module / autograd.Function drop-in path end to end."""
    import fmta_b200 as F
    B, H, N, d, cq, ck = 2, 4, 100, 64, 6, 11
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=3, dtype=torch.bfloat16)
    mod = F.ConvAttentionCUDA(H, cq, ck, init_random=False).cuda()
    assert mod.conv_weight.shape == (H, cq, ck)
    with torch.no_grad():
        mod.conv_weight.copy_(theta.cuda())
    q, k, v = (t.cuda().to(torch.bfloat16).requires_grad_(True) for t in (Q, K, V))
    O = mod(q, k, v, causal=True)
    O.backward(dO.cuda())
    Or, Mr, Lr = orc.conv_attn_fwd(Q, K, V, theta, None, True)
    dQ, dK, dV, dTh = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, None, True)
    assert maxabs(O, Or) <= TOL_BF16
    assert maxabs(q.grad, dQ) <= TOL_BF16 and q.grad.dtype == torch.bfloat16
    assert maxabs(k.grad, dK) <= TOL_BF16
    assert maxabs(v.grad, dV) <= TOL_BF16
    assert maxabs(mod.conv_weight.grad, dTh) <= dtheta_tol(dTh)


def test_backward_is_deterministic():
    import fmta_b200 as F
    Q, K, V, dO, theta = orc.make_inputs(2, 2, 300, 64, 6, 11, seed=9, dtype=torch.bfloat16)
    a = _run_fwd_bwd(Q, K, V, dO, theta, 0.125, True)
    b = _run_fwd_bwd(Q, K, V, dO, theta, 0.125, True)
    for k in a:
        assert torch.equal(a[k], b[k]), k


def test_rejects_bad_inputs():
    import fmta_b200 as F
    Q = torch.zeros(1, 2, 16, 64, device="cuda", dtype=torch.bfloat16)
    th = torch.zeros(2, 3, 3, device="cuda")
    with pytest.raises(RuntimeError):
        F.forward(Q.float(), Q, Q, th, 1.0, 2, 1, True)            # not bf16
    with pytest.raises(RuntimeError):
        F.forward(Q.cpu(), Q, Q, th, 1.0, 2, 1, True)              # not CUDA
    with pytest.raises(RuntimeError):
        F.forward(Q, Q, Q, torch.zeros(2, 3, 4, device="cuda"), 1.0, 2, 1, True)   # even c_k
    with pytest.raises(RuntimeError):
        Q48 = torch.zeros(1, 2, 16, 48, device="cuda", dtype=torch.bfloat16)
        F.forward(Q48, Q48, Q48, th, 1.0, 2, 1, True)              # unsupported head dim
    with pytest.raises(RuntimeError):
        F.forward(Q, Q, Q, th, 1.0, 1, 1, True)                    # pads inconsistent with the filter


@pytest.mark.parametrize("path", [0, 1, 2])
@pytest.mark.parametrize("B,H,N,d,cq,ck,causal", [
    (1, 2, 520, 64, 6, 11, True),     # several 246-row dQ blocks (laid out from the last row) and 128-key dK tiles, ragged N
    (2, 1, 300, 64, 3, 5, False),     # no causal band: everything on the tensor-core kernels
    (1, 1, 100, 64, 6, 11, True),     # shorter than one tile
    (1, 2, 400, 64, 6, 17, True),     # wide key filter (W = 21): three key tiles per row tile, FMA output phase
    (1, 2, 700, 64, 3, 5, True),      # run-time filter shape in the band kernels, mma output phase
    (1, 1, 611, 64, 6, 13, True),     # W = 17: widest filter on the two-key-tile / mma output path
    (1, 1, 389, 64, 6, 15, True),     # W = 19: three key tiles, FMA output phase
    (1, 2, 257, 64, 1, 3, True),      # single query tap: band of 1
    (1, 1, 450, 64, 4, 7, True),
    (2, 1, 200, 64, 5, 9, True),
    (1, 2, 900, 64, 7, 7, True),      # seven query taps: two launches of the dK/dV kernel (the reference's 7x7 filter)
    (1, 1, 300, 64, 7, 17, True),     # largest filter of the tensor-core backward
    (2, 1, 260, 64, 7, 11, False),
    (1, 1, 77, 64, 6, 11, True),      # exactly one band CTA
    (1, 1, 78, 64, 6, 11, True),      # one position into the second band CTA
    (1, 1, 333, 64, 2, 3, True),      # tiny filter, band of 2
    (1, 1, 1500, 64, 6, 11, True),    # many key blocks per tile
    (1, 1, 63, 64, 6, 11, True),      # one key short of the 64-key tile of the dK~ adjoint kernel
    (1, 1, 64, 64, 6, 11, True),      # exactly one tile
    (1, 2, 65, 64, 6, 11, True),      # one key into the second tile: its halo rows are mostly past the end
    (1, 2, 129, 64, 7, 17, True),     # the same with the widest filter (halo of 8 rows fully used)
    (1, 1, 130, 64, 1, 3, False),     # one tap, no band
    # head dim 128: dQ tile of 128 - pad_q owned rows, 64-key dK/dV CTAs with 128-row query blocks
    (1, 2, 520, 128, 6, 11, True),
    (2, 1, 300, 128, 3, 5, False),    # no causal band: everything on the tensor-core kernels
    (1, 1, 100, 128, 6, 11, True),    # shorter than one tile
    (1, 1, 123, 128, 6, 11, True),    # exactly the rows one dQ tile owns
    (1, 1, 124, 128, 6, 11, True),    # one row into the second dQ tile
    (1, 1, 246, 64, 6, 11, True),     # exactly one dQ block of two tiles
    (1, 1, 247, 64, 6, 11, True),     # one row more: the first block holds that row only
    (1, 2, 257, 128, 1, 3, True),     # single query tap
    (1, 1, 450, 128, 4, 7, True),
    (1, 1, 611, 128, 6, 13, True),    # W = 17
    (1, 1, 389, 128, 6, 15, True),    # W = 19: FMA output phase of the band kernel
    (1, 1, 1500, 128, 6, 11, True),   # many key blocks per dQ tile, many row blocks per key tile
    (1, 2, 65, 128, 6, 11, True),     # one key into the second 64-key tile
    (2, 2, 333, 128, 5, 9, True),
])
def test_fused_backward_paths(path, B, H, N, d, cq, ck, causal):
    """fmta_bwd with the exact kernels (path 0) and with the stacked-GEMM tensor-core kernels plus
    the band kernel (path 1: the dQ kernel keeps P and dC and the dK/dV kernel streams them, head dim 64;
    "path 2": the dK/dV kernel recomputes them) against the oracle; forward run on both paths as well."""
    import fmta_b200 as F
    stream_pdc = (True if d == 64 and path == 1 else None) if path != 2 else False   # streaming is opt-in
    if path == 2:
        if d != 64:
            pytest.skip("the streaming dK/dV kernel exists for head dim 64 only: nothing to switch off")
        path = 1
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=17 + N, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, causal, return_lse=True, path=path)
    Dv = F.rowdot(do, O)
    dQ, dK, dV, dTh = F.backward(q, k, v, do, Dv, LSE, th, scale, cq - 1, (ck - 1) // 2, causal, path=path,
                                 stream_pdc=stream_pdc)
    torch.cuda.synchronize()
    Or, Mr, Lr = orc.conv_attn_fwd(Q, K, V, theta, scale, causal)
    rq, rk, rv, rt = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, causal)
    _check(dict(O=O, M=M, L=L, LSE=LSE, dQ=dQ, dK=dK, dV=dV, dTheta=dTh),
           dict(O=Or, M=Mr, L=Lr, dQ=rq, dK=rk, dV=rv, dTheta=rt),
           "B%d H%d N%d d%d theta(%d,%d) causal=%d path %d%s" % (B, H, N, d, cq, ck, causal, path,
                                                              " (recomputing dK/dV)" if stream_pdc is False else ""))


@pytest.mark.parametrize("B,H,N,cq,ck,causal", [(1, 2, 520, 6, 11, True), (2, 1, 300, 3, 5, False), (1, 2, 83, 6, 11, True)])
def test_head_dim_32_default_path(B, H, N, cq, ck, causal):
    """Head dim 32 with the library's default path: the head-dim-64 tensor-core kernels on zero-padded
    operands (the Python layer pads and slices); same bound as every other path."""
    import fmta_b200 as F
    d = 32
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=5 + N, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, causal, return_lse=True)
    assert O.shape == q.shape
    Dv = F.rowdot(do, O)
    dQ, dK, dV, dTh = F.backward(q, k, v, do, Dv, LSE, th, scale, cq - 1, (ck - 1) // 2, causal)
    torch.cuda.synchronize()
    Or, Mr, Lr = orc.conv_attn_fwd(Q, K, V, theta, scale, causal)
    rq, rk, rv, rt = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, causal)
    _check(dict(O=O, M=M, L=L, LSE=LSE, dQ=dQ, dK=dK, dV=dV, dTheta=dTh),
           dict(O=Or, M=Mr, L=Lr, dQ=rq, dK=rk, dV=rv, dTheta=rt),
           "B%d H%d N%d d32 (padded to 64) theta(%d,%d) causal=%d default path" % (B, H, N, cq, ck, causal))
    # the exact kernels (path 0) take head dim 32 as it is and agree
    O0, _, _ = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, causal, path=0)
    assert float((O0 - O).abs().max()) <= 2e-2


@pytest.mark.parametrize("B,H,N,d,cq,ck,causal,stream_pdc", [
    (2, 2, 640, 64, 6, 11, True, False), (2, 2, 640, 64, 6, 11, True, True), (1, 2, 333, 64, 7, 5, True, False),
    (1, 3, 512, 64, 3, 5, False, None), (1, 2, 512, 128, 6, 11, True, None), (1, 1, 200, 128, 2, 3, True, None)])
def test_forward_hands_stacked_keys_to_backward(B, H, N, d, cq, ck, causal, stream_pdc):
    """`forward(..., ktilde=buf)` leaves the stacked key operand in the caller's buffer and `backward(..., ktilde=buf)`
    skips its own pre-pass: every output is bit-identical to the pair of calls that each build the operand."""
    import fmta_b200 as F
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=77 + N, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    pq, pk = cq - 1, (ck - 1) // 2
    O0, M0, L0, LSE0 = F.forward(q, k, v, th, scale, pq, pk, causal, return_lse=True, path=1)
    Dv = F.rowdot(do, O0)
    ref = F.backward(q, k, v, do, Dv, LSE0, th, scale, pq, pk, causal, path=1, stream_pdc=stream_pdc)
    kt = F.ktilde_buffer(q, th)
    assert kt is not None and kt.shape == (B, H, cq, N, d)
    kt.fill_(float("nan"))
    O1, M1, L1, LSE1 = F.forward(q, k, v, th, scale, pq, pk, causal, return_lse=True, ktilde=kt)
    assert bool(torch.isfinite(kt.float()).all())
    got = F.backward(q, k, v, do, Dv, LSE1, th, scale, pq, pk, causal, stream_pdc=stream_pdc, ktilde=kt)
    torch.cuda.synchronize()
    for a, b, n in ((O0, O1, "O"), (M0, M1, "M"), (L0, L1, "L"), (LSE0, LSE1, "LSE")):
        assert torch.equal(a, b), n
    for a, b, n in zip(ref, got, ("dQ", "dK", "dV", "dTheta")):
        assert torch.equal(a, b), n
    # a stale buffer is the caller's responsibility, and it shows: with the operand zeroed the backward changes
    if N >= 512:
        kt.zero_()
        stale = F.backward(q, k, v, do, Dv, LSE1, th, scale, pq, pk, causal, stream_pdc=stream_pdc, ktilde=kt)
        assert not torch.equal(stale[0], ref[0])
    # rejected: the exact path, a buffer of the wrong shape
    with pytest.raises(RuntimeError):
        F.forward(q, k, v, th, scale, pq, pk, causal, path=0, ktilde=kt)
    with pytest.raises(RuntimeError):
        F.backward(q, k, v, do, Dv, LSE1, th, scale, pq, pk, causal, ktilde=kt[:, :, :1].contiguous())


def test_autograd_function_keeps_stacked_keys_when_asked(monkeypatch):
    """FMTA_KEEP_KTILDE (here: the module switch it sets) makes the autograd Function carry the operand from its
    forward to its backward; gradients are bit-identical to the default."""
    import fmta_b200 as F
    from fmta_b200 import conv_attn
    B, H, N, d, cq, ck = 1, 2, 384, 64, 6, 11
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=9, dtype=torch.bfloat16)
    grads = []
    for keep in (False, True):
        monkeypatch.setattr(conv_attn, "KEEP_KTILDE", keep)
        q, k, v = (t.cuda().to(torch.bfloat16).requires_grad_() for t in (Q, K, V))
        th = theta.cuda().requires_grad_()
        O = F.FlashConvAttentionCUDAFunction.apply(q, k, v, th, 1.0 / math.sqrt(d), cq - 1, (ck - 1) // 2, True)
        O.backward(dO.cuda().to(O.dtype))
        grads.append([t.grad.clone() for t in (q, k, v, th)] + [O.detach()])
    for a, b in zip(*grads):
        assert torch.equal(a, b)


def test_fp32_configuration_N256_theta_3x5_both_paths():
    """The fp32 CPU-path configuration of the benchmark (B=1, H=4, N=256, d=64, theta (3,5), N(0,0.05)
    filter) run through the bf16 kernels on both paths, against the oracle on the same bf16-rounded inputs."""
    import fmta_b200 as F
    B, H, N, d, cq, ck = 1, 4, 256, 64, 3, 5
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=0, theta_std=0.05, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    Or, Mr, Lr = orc.conv_attn_fwd(Q, K, V, theta, scale, True)
    rq, rk, rv, rt = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, True)
    for path in (0, 1):
        O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=path)
        dQ, dK, dV, dTh = F.backward(q, k, v, do, F.rowdot(do, O), LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=path)
        _check(dict(O=O, M=M, L=L, LSE=LSE, dQ=dQ, dK=dK, dV=dV, dTheta=dTh),
               dict(O=Or, M=Mr, L=Lr, dQ=rq, dK=rk, dV=rv, dTheta=rt), "config 0 (N=256, theta (3,5)) path %d" % path)


def test_tensor_core_path_rejected_when_unsupported():
    import fmta_b200 as F
    LSE = torch.zeros(1, 1, 64, device="cuda")
    Q = torch.zeros(1, 1, 64, 32, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):   # the tensor-core backward exists for d = 64 and d = 128
        F.backward(Q, Q, Q, Q, LSE, LSE, torch.zeros(1, 6, 11, device="cuda"), 1.0, 5, 5, True, path=1)
    Q = torch.zeros(1, 1, 64, 128, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):   # ... with up to six query taps at d = 128
        F.backward(Q, Q, Q, Q, LSE, LSE, torch.zeros(1, 7, 7, device="cuda"), 1.0, 6, 3, True, path=1)
