"""GPU parity of the decode kernel (C ABI) against the reference-generated fixtures and the
streaming oracle."""
import math

import pytest
import torch

from helpers import TOL_BF16, load_golden, maxabs
from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu


def _run(Q, K, V, theta, scale, k_splits):
    import fmta_b200 as F
    cq, ck = theta.shape[1:]
    Qb, Kb, Vb = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V))
    O, M, L = F.fwd_conv_attn_inference(Qb, Kb, Vb, theta.cuda(), k_splits, scale, cq - 1, (ck - 1) // 2, False)
    torch.cuda.synchronize()
    return O, M, L


@pytest.mark.parametrize("name,k_splits", [("decode_ref_script_5x5", 4), ("decode_ref_script_5x5", 1),
                                           ("decode_6x11_qlen6", 3), ("decode_6x11_qlen6", 1),
                                           ("decode_3x3_qlen2", 2), ("decode_3x3_qlen2", 7)])
def test_golden(name, k_splits):
    z = load_golden(name)
    O, M, L = _run(z["Q"], z["K"], z["V"], z["theta"], float(z["scale"]), k_splits)
    assert O.shape == z["O"].shape and M.shape == z["M"].shape
    assert maxabs(O, z["O"]) <= TOL_BF16
    assert maxabs(M, z["M"]) <= TOL_BF16
    assert maxabs(M + torch.log(L), z["M"] + torch.log(z["L"])) <= TOL_BF16


@pytest.mark.parametrize("B,H,q_len,Nk,d,cq,ck,k_splits", [
    (2, 2, 6, 1000, 128, 6, 11, 4),
    (1, 3, 16, 513, 64, 6, 11, 5),     # 16 query rows but only 6 taps see them
    (1, 2, 12, 777, 64, 11, 11, 2),    # more than 8 live rows -> 16-row fragments
    (1, 1, 1, 65, 32, 3, 3, 1),        # a single query row
    (2, 1, 6, 17, 128, 6, 11, 1),      # cache shorter than a warp's step
    (1, 2, 6, 4096, 128, 6, 11, 16),
])
def test_oracle_shapes(B, H, q_len, Nk, d, cq, ck, k_splits):
    Q, K, V, _, theta = orc.make_inputs(B, H, 0, d, cq, ck, seed=Nk, dtype=torch.bfloat16, Nk=Nk, q_len=q_len)
    scale = 1.0 / math.sqrt(d)
    Or, Mr, Lr = orc.decode_last_row_streaming(Q, K, V, theta, scale, chunk=512)
    O, M, L = _run(Q, K, V, theta, scale, k_splits)
    assert maxabs(O, Or) <= TOL_BF16
    assert maxabs(M, Mr) <= TOL_BF16
    assert maxabs(M + torch.log(L), Mr + torch.log(Lr)) <= TOL_BF16


def test_split_invariance_and_split0_convention():
    import fmta_b200 as F
    Q, K, V, _, theta = orc.make_inputs(1, 2, 0, 64, 6, 11, seed=1, dtype=torch.bfloat16, Nk=2000, q_len=6)
    outs = [_run(Q, K, V, theta, 0.125, s) for s in (1, 2, 8, 31)]
    for O, M, L in outs[1:]:
        assert maxabs(O, outs[0][0]) <= 1e-4
        assert maxabs(M, outs[0][1]) <= 1e-5
    Qb, Kb, Vb = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V))
    Os, Ms, Ls = F.forward_inference(Qb, Kb, Vb, theta.cuda(), 8, 0.125, 5, 5, False, 0)
    assert Os.shape == (1, 2, 8, 64) and Ms.shape == (1, 2, 8)


def test_rejects_bad_inputs():
    import fmta_b200 as F
    Q = torch.zeros(1, 1, 17, 64, device="cuda", dtype=torch.bfloat16)
    K = torch.zeros(1, 1, 64, 64, device="cuda", dtype=torch.bfloat16)
    th = torch.zeros(1, 3, 3, device="cuda")
    with pytest.raises(ValueError):
        F.fwd_conv_attn_inference(Q, K, K, th, 1, 1.0, 2, 1, False)       # q_len > 16
    with pytest.raises(RuntimeError):
        F.fwd_conv_attn_inference(Q[:, :, :4], K, K, th, 65, 1.0, 2, 1, False)   # k_splits > Nk
    with pytest.raises(RuntimeError):
        F.fwd_conv_attn_inference(Q[:, :, :4], K, K, th, 0, 1.0, 2, 1, False)


@pytest.mark.parametrize("B,H,q_len,Nk,d,cq,ck,k_splits", [
    (1, 2, 6, 300, 64, 6, 11, 1),
    (2, 2, 6, 1000, 128, 6, 11, 4),
    (1, 1, 16, 257, 64, 6, 11, 3),     # more rows than filter taps
    (1, 2, 3, 129, 32, 3, 5, 2),
    (1, 1, 4, 4, 64, 6, 11, 1),        # cache shorter than the filter
])
def test_offset_causal_matches_oracle_and_training_forward(B, H, q_len, Nk, d, cq, ck, k_splits):
    """Decode with the training forward's mask: against its own oracle, and (the property it exists for)
    against row Nk-1 of the causal training forward run by the library over the same sequence."""
    import fmta_b200 as F
    Q, K, V, _, theta = orc.make_inputs(B, H, 0, d, cq, ck, seed=5 + Nk, dtype=torch.bfloat16, Nk=Nk, q_len=Nk)
    scale = 1.0 / math.sqrt(d)
    Qr = Q[:, :, Nk - q_len:, :].contiguous()
    Or, Mr, Lr = orc.decode_last_row_offset_causal(Qr, K, V, theta, scale)
    qb, kb, vb = (t.cuda().to(torch.bfloat16).contiguous() for t in (Qr, K, V))
    O, M, L = F.fwd_conv_attn_inference(qb, kb, vb, theta.cuda(), k_splits, scale, cq - 1, (ck - 1) // 2, True,
                                        offset_causal=True)
    assert maxabs(O, Or) <= TOL_BF16
    assert maxabs(M, Mr) <= TOL_BF16
    assert maxabs(M + torch.log(L), Mr + torch.log(Lr)) <= TOL_BF16
    Of, Mf, Lf = F.forward(Q.cuda().to(torch.bfloat16).contiguous(), kb, vb, theta.cuda(), scale, cq - 1, (ck - 1) // 2, True)
    assert maxabs(O[:, :, 0], Of[:, :, -1]) <= TOL_BF16
    assert maxabs((M + torch.log(L))[:, :, 0], (Mf + torch.log(Lf))[:, :, -1]) <= TOL_BF16
    # the mask matters: without it the last keys' scores differ
    O0, _, _ = F.fwd_conv_attn_inference(qb, kb, vb, theta.cuda(), k_splits, scale, cq - 1, (ck - 1) // 2, False)
    if Nk > 16 and cq > 1:
        assert maxabs(O0, O) > 0


def _paged_from_contiguous(K, V, page_size, n_extra_pages=3, seed=0):
    """Scatter contiguous caches [B,H,Nk,d] into pools [n_pages,H,page_size,d] through a random page
    permutation; returns (K_pool, V_pool, block_table)."""
    B, H, Nk, d = K.shape
    ppb = (Nk + page_size - 1) // page_size
    n_pages = B * ppb + n_extra_pages
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(n_pages, generator=g)[: B * ppb].view(B, ppb)
    Kp = torch.randn(n_pages, H, page_size, d, generator=g).to(torch.bfloat16)      # junk in unused slots
    Vp = torch.randn(n_pages, H, page_size, d, generator=g).to(torch.bfloat16)
    for b in range(B):
        for pgi in range(ppb):
            lo, hi = pgi * page_size, min(Nk, (pgi + 1) * page_size)
            Kp[perm[b, pgi], :, : hi - lo] = K[b, :, lo:hi].to(torch.bfloat16)
            Vp[perm[b, pgi], :, : hi - lo] = V[b, :, lo:hi].to(torch.bfloat16)
    return Kp.cuda(), Vp.cuda(), perm.to(torch.int32).cuda()


@pytest.mark.parametrize("B,H,q_len,Nk,d,cq,ck,k_splits,page", [
    (2, 2, 6, 1000, 128, 6, 11, 4, 64),
    (1, 3, 6, 333, 64, 6, 11, 1, 16),
    (2, 1, 4, 2048, 64, 3, 5, 3, 256),
])
def test_paged_cache_equals_contiguous(B, H, q_len, Nk, d, cq, ck, k_splits, page):
    """Same keys through a paged pool with a shuffled block table: bit-identical to the contiguous
    kernel (same arithmetic order), within tolerance of the oracle; with and without the causal mask."""
    import fmta_b200 as F
    Q, K, V, _, theta = orc.make_inputs(B, H, 0, d, cq, ck, seed=11 + Nk, dtype=torch.bfloat16, Nk=Nk, q_len=q_len)
    scale = 1.0 / math.sqrt(d)
    qb, kb, vb = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V))
    Kp, Vp, table = _paged_from_contiguous(K, V, page)
    th = theta.cuda()
    for oc in (False, True):
        Oc, Mc, Lc = F.forward_inference(qb, kb, vb, th, k_splits, scale, cq - 1, (ck - 1) // 2, False, offset_causal=oc)
        Op, Mp, Lp = F.forward_inference_paged(qb, Kp, Vp, table, th, k_splits, scale, cq - 1, (ck - 1) // 2,
                                               max_seq_len=Nk, offset_causal=oc)
        assert torch.equal(Oc[:, :, 0], Op[:, :, 0]) and torch.equal(Mc[:, :, 0], Mp[:, :, 0]) and torch.equal(Lc[:, :, 0], Lp[:, :, 0])
    Or, Mr, Lr = orc.decode_last_row(Q, K, V, theta, scale)
    Op, Mp, Lp = F.forward_inference_paged(qb, Kp, Vp, table, th, k_splits, scale, cq - 1, (ck - 1) // 2, max_seq_len=Nk)
    assert maxabs(Op[:, :, 0:1], Or) <= TOL_BF16


def test_paged_cache_ragged_lengths_and_append():
    """Sequences of different length in one call (seq_lens), and rows appended with kv_append_paged:
    each sequence must equal the contiguous decode of its own prefix."""
    import fmta_b200 as F
    B, H, q_len, d, cq, ck, page, Nmax = 3, 2, 6, 64, 6, 11, 32, 500
    Q, K, V, _, theta = orc.make_inputs(B, H, 0, d, cq, ck, seed=77, dtype=torch.bfloat16, Nk=Nmax, q_len=q_len)
    scale = 1.0 / math.sqrt(d)
    lens = [500, 123, 257]
    n_new = 5
    Kp, Vp, table = _paged_from_contiguous(K, V, page)
    th = theta.cuda()
    qb = Q.cuda().to(torch.bfloat16).contiguous()
    # start 5 rows short, then append the missing rows
    start = torch.tensor([l - n_new for l in lens], dtype=torch.int32).cuda()
    Knew = torch.stack([K[b, :, lens[b] - n_new:lens[b]] for b in range(B)]).to(torch.bfloat16).cuda().contiguous()
    Vnew = torch.stack([V[b, :, lens[b] - n_new:lens[b]] for b in range(B)]).to(torch.bfloat16).cuda().contiguous()
    # overwrite the rows to be appended with junk first, so that the append is what makes them right
    for b in range(B):
        for pos in range(lens[b] - n_new, lens[b]):
            Kp[table[b, pos // page].item(), :, pos % page] = 7.0
            Vp[table[b, pos // page].item(), :, pos % page] = -7.0
    F.kv_append_paged(Kp, Vp, table, start, Knew, Vnew)
    seq = torch.tensor(lens, dtype=torch.int32).cuda()
    for ks in (1, 4):
        Op, Mp, Lp = F.forward_inference_paged(qb, Kp, Vp, table, th, ks, scale, cq - 1, (ck - 1) // 2,
                                               seq_lens=seq, max_seq_len=Nmax, offset_causal=True)
        for b in range(B):
            kb = K[b:b + 1, :, :lens[b]].cuda().to(torch.bfloat16).contiguous()
            vb = V[b:b + 1, :, :lens[b]].cuda().to(torch.bfloat16).contiguous()
            Oc, Mc, Lc = F.forward_inference(qb[b:b + 1], kb, vb, th, 1, scale, cq - 1, (ck - 1) // 2, False, offset_causal=True)
            assert maxabs(Op[b:b + 1, :, 0], Oc[:, :, 0]) <= 1e-5
            assert maxabs((Mp + torch.log(Lp))[b:b + 1, :, 0], (Mc + torch.log(Lc))[:, :, 0]) <= 1e-5


def test_paged_lengths_beyond_the_table_are_clamped_not_followed():
    """A stale or oversized seq_lens entry must not walk the kernels off the block table: the decode
    treats it as max_seq_len, and the append drops rows whose page index lies past the table."""
    import fmta_b200 as F
    B, H, q_len, d, cq, ck, page, Nmax = 2, 2, 6, 64, 6, 11, 32, 160
    Q, K, V, _, theta = orc.make_inputs(B, H, 0, d, cq, ck, seed=5, dtype=torch.bfloat16, Nk=Nmax, q_len=q_len)
    scale = 1.0 / math.sqrt(d)
    Kp, Vp, table = _paged_from_contiguous(K, V, page)
    th = theta.cuda()
    qb = Q.cuda().to(torch.bfloat16).contiguous()
    full = torch.tensor([Nmax, Nmax], dtype=torch.int32).cuda()
    wild = torch.tensor([Nmax + 100000, 2 ** 30], dtype=torch.int32).cuda()
    zero = torch.tensor([0, -7], dtype=torch.int32).cuda()
    ref = F.forward_inference_paged(qb, Kp, Vp, table, th, 2, scale, cq - 1, (ck - 1) // 2, seq_lens=full, max_seq_len=Nmax)
    got = F.forward_inference_paged(qb, Kp, Vp, table, th, 2, scale, cq - 1, (ck - 1) // 2, seq_lens=wild, max_seq_len=Nmax)
    torch.cuda.synchronize()
    for a, b in zip(ref, got):
        assert torch.equal(a[:, :, 0], b[:, :, 0])
    one = F.forward_inference_paged(qb, Kp, Vp, table, th, 1, scale, cq - 1, (ck - 1) // 2, seq_lens=zero, max_seq_len=Nmax)
    torch.cuda.synchronize()
    assert torch.isfinite(one[0][:, :, 0]).all()          # lengths below 1 are read as 1
    # append: positions past max_pages * page_size are dropped, the pools stay as they were
    Kp0, Vp0 = Kp.clone(), Vp.clone()
    Knew = torch.ones(B, H, 3, d, dtype=torch.bfloat16, device="cuda")
    F.kv_append_paged(Kp, Vp, table, wild, Knew, Knew)
    torch.cuda.synchronize()
    assert torch.equal(Kp, Kp0) and torch.equal(Vp, Vp0)
