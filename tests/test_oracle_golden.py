"""Pins the CPU oracle to fixtures produced by the reference's own PyTorch functions
(tests/golden/make_golden.py).  fp32 against fp32: tolerance 1e-3 max-abs (the fp32 bound of the
benchmark contract); most quantities agree to ~1e-6."""
import glob
import os

import pytest
import torch

from helpers import GOLDEN, TOL_FP32, load_golden, maxabs
from oracle import conv_attn_oracle as orc

CONV = sorted(os.path.basename(f)[:-4] for f in glob.glob(os.path.join(GOLDEN, "conv_*.npz")))
DEC = sorted(os.path.basename(f)[:-4] for f in glob.glob(os.path.join(GOLDEN, "decode_*.npz")))
HEAD = sorted(os.path.basename(f)[:-4] for f in glob.glob(os.path.join(GOLDEN, "head_*.npz")))


def test_fixture_inventory():
    assert len(CONV) >= 5 and len(DEC) >= 3 and len(HEAD) >= 3


@pytest.mark.parametrize("name", CONV)
def test_conv_forward_and_backward(name):
    z = load_golden(name)
    s, c = float(z["scale"]), bool(z["causal"])
    for shift in (False, True):
        O, M, L = orc.conv_attn_fwd(z["Q"], z["K"], z["V"], z["theta"], s, c, shift_form=shift)
        assert maxabs(O, z["O"]) <= TOL_FP32
        assert maxabs(M, z["M"]) <= TOL_FP32
        assert maxabs(orc.lse_of(M, L), orc.lse_of(z["M"], z["L"])) <= TOL_FP32
    g_auto = orc.conv_attn_bwd_autograd(z["Q"], z["K"], z["V"], z["theta"], z["dO"], s, c)
    g_expl = orc.conv_attn_bwd_explicit(*(z[k].double() for k in ("Q", "K", "V", "theta", "dO")), s, c)
    for got in (g_auto, g_expl):
        for a, k in zip(got, ("dQ", "dK", "dV", "dTheta")):
            assert maxabs(a, z[k]) <= TOL_FP32, k


@pytest.mark.parametrize("name", CONV)
def test_rowblock_form(name):
    z = load_golden(name)
    s, c = float(z["scale"]), bool(z["causal"])
    N = z["Q"].shape[2]
    for i0, i1 in ((0, min(N, 5)), (N // 3, min(N, N // 3 + 17)), (max(0, N - 9), N)):
        O, M, L = orc.conv_attn_fwd_rowblock(z["Q"], z["K"], z["V"], z["theta"], i0, i1, s, c)
        assert maxabs(O, z["O"][:, :, i0:i1]) <= TOL_FP32
        assert maxabs(M, z["M"][:, :, i0:i1]) <= TOL_FP32


@pytest.mark.parametrize("name", DEC)
def test_decode(name):
    z = load_golden(name)
    s = float(z["scale"])
    for got in (orc.decode_last_row(z["Q"], z["K"], z["V"], z["theta"], s),
                orc.decode_last_row_streaming(z["Q"], z["K"], z["V"], z["theta"], s, chunk=50)):
        assert got[0].shape == z["O"].shape
        assert maxabs(got[0], z["O"]) <= TOL_FP32
        assert maxabs(got[1], z["M"]) <= TOL_FP32
        assert maxabs(orc.lse_of(got[1], got[2]), orc.lse_of(z["M"], z["L"])) <= TOL_FP32


def test_decode_front_padding_is_a_no_op():
    """The reference pads Q at the front with zero rows up to 16 (flash_conv_attention_inference.py:58-65)."""
    z = load_golden("decode_6x11_qlen6")
    Qp = torch.zeros(z["Q"].shape[0], z["Q"].shape[1], 16, z["Q"].shape[3])
    Qp[:, :, -z["Q"].shape[2]:] = z["Q"]
    a = orc.decode_last_row(Qp, z["K"], z["V"], z["theta"], float(z["scale"]))
    assert maxabs(a[0], z["O"]) <= 1e-6 and maxabs(a[1], z["M"]) <= 1e-6


def test_split_merge():
    z = load_golden("decode_6x11_qlen6")
    s = float(z["scale"])
    Nk = z["K"].shape[2]
    # un-normalised partials of 3 key ranges, computed with the full conv (halo included) then cut
    S = orc.masked_scores(z["Q"], z["K"], s, False)
    C = orc.conv_scores_dense(S, z["theta"])[:, :, -1, :]
    Os, Ms, Ls = [], [], []
    for lo, hi in ((0, 100), (100, 250), (250, Nk)):
        c = C[..., lo:hi]
        m = c.max(-1).values
        e = torch.exp(c - m[..., None])
        Os.append(torch.einsum("bhj,bhjd->bhd", e, z["V"][:, :, lo:hi]))
        Ms.append(m)
        Ls.append(e.sum(-1))
    O, M, L = orc.combine_splits(torch.stack(Os, 2), torch.stack(Ms, 2), torch.stack(Ls, 2))
    assert maxabs(O.unsqueeze(2), z["O"]) <= 1e-5
    assert maxabs(M.unsqueeze(2), z["M"]) <= 1e-6


@pytest.mark.parametrize("name", HEAD)
def test_head_conv(name):
    z = load_golden(name)
    s, c = float(z["scale"]), bool(z["causal"])
    O, L, M = orc.head_conv_fwd(z["q"], z["k"], z["v"], z["w"], s, c)
    assert maxabs(O, z["O"]) <= TOL_FP32 and maxabs(M, z["M"]) <= TOL_FP32
    assert maxabs(orc.lse_of(M, L), orc.lse_of(z["M"], z["L"])) <= TOL_FP32
    O2, M2, L2 = orc.conv_headmix_fwd(z["q"], z["k"], z["v"], None, z["w"], s, c)
    assert maxabs(O2, z["O"]) <= TOL_FP32
    dq, dk, dv, _, dw = orc.conv_headmix_bwd_autograd(z["q"], z["k"], z["v"], None, z["w"], z["dO"], s, c)
    for a, k in ((dq, "dq"), (dk, "dk"), (dv, "dv"), (dw, "dw")):
        assert maxabs(a, z[k]) <= TOL_FP32, k


def test_composed_reduces_to_conv_attn_with_identity_mix():
    z = load_golden("conv_6x11_ragged")
    H = z["Q"].shape[1]
    O, M, L = orc.conv_headmix_fwd(z["Q"], z["K"], z["V"], z["theta"], torch.eye(H), float(z["scale"]), True)
    assert maxabs(O, z["O"]) <= 1e-5 and maxabs(M, z["M"]) <= 1e-5


def test_adjoint_identity():
    """<conv(S), dC> == <S, conv^T(dC)> for the shift-and-add pair used by the explicit backward."""
    g = torch.Generator().manual_seed(0)
    S = torch.randn(1, 2, 23, 31, generator=g, dtype=torch.float64)
    dC = torch.randn(1, 2, 23, 31, generator=g, dtype=torch.float64)
    th = torch.randn(2, 6, 11, generator=g, dtype=torch.float64)
    lhs = (orc.conv_scores_shift(S, th) * dC).sum()
    rhs = (S * orc.conv_scores_transposed(dC, th)).sum()
    assert abs(float(lhs - rhs)) < 1e-9


def test_offset_causal_decode_is_last_row_of_causal_forward():
    """The offset-causal decode oracle has no reference counterpart; it is pinned by composition with
    the (pinned) training forward: same sequence, last row."""
    torch.manual_seed(3)
    for (N, cq, ck, q_len) in [(50, 6, 11, 6), (40, 3, 5, 8), (33, 2, 3, 2), (5, 6, 11, 5), (64, 6, 11, 16)]:
        B, H, d = 1, 2, 16
        Q, K, V = (torch.randn(B, H, N, d) for _ in range(3))
        th = torch.randn(H, cq, ck) * 0.1
        th[:, cq - 1, ck // 2] += 1
        O, M, L = orc.conv_attn_fwd(Q, K, V, th, None, True)
        Od, Md, Ld = orc.decode_last_row_offset_causal(Q[:, :, N - q_len:], K, V, th)
        assert maxabs(O[:, :, -1:], Od) <= 1e-5
        assert maxabs(M[:, :, -1:], Md) <= 1e-5
        assert maxabs(L[:, :, -1:], Ld) <= 1e-4
