"""Context parallelism: windows of sequence positions computed by `fmta_fwd_window` / `fmta_bwd_window`
against the whole-sequence calls and the oracle, the autograd Function on one rank, and two NCCL ranks that
each hold a zigzag share of one sequence (skipped on a box with a single GPU)."""
import math
import os
import subprocess
import sys

import pytest
import torch

from helpers import check_outputs
from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _inputs(B, H, N, d, cq, ck, seed):
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=seed, dtype=torch.bfloat16)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    return (Q, K, V, dO, theta), (q, k, v, do, theta.cuda())


@pytest.mark.parametrize("B,H,N,d,cq,ck,causal,windows", [
    (1, 2, 1024, 64, 6, 11, True, [(0, 512), (512, 1024)]),
    (2, 2, 1500, 64, 6, 11, True, [(0, 256), (256, 1024), (1024, 1500)]),       # ragged end, unequal windows
    (1, 2, 1024, 64, 7, 5, True, [(0, 768), (768, 1024)]),                      # seven taps: two dK/dV passes per segment
    (1, 2, 1024, 64, 3, 5, False, [(0, 512), (512, 1024)]),                     # no causal mask
    (1, 2, 1100, 128, 6, 11, True, [(0, 512), (512, 768), (768, 1100)]),
    (1, 1, 768, 128, 2, 3, False, [(0, 256), (256, 768)])])
def test_windows_reproduce_the_whole_sequence(B, H, N, d, cq, ck, causal, windows):
    """Disjoint windows that cover the sequence, computed one after the other (backward in reverse order) into
    buffers pre-filled with NaN: the forward is bit-identical to the whole-sequence call, the backward equal to
    rounding (row tiles of dQ and of the band start at the window), the dTheta shares add up, and the oracle
    bound holds."""
    import fmta_b200 as F
    (Q, K, V, dO, theta), (q, k, v, do, th) = _inputs(B, H, N, d, cq, ck, 11 + N)
    scale = 1.0 / math.sqrt(d)
    pq, pk = cq - 1, (ck - 1) // 2
    O, M, L, LSE = F.forward(q, k, v, th, scale, pq, pk, causal, return_lse=True, path=1)
    Dv = F.rowdot(do, O)
    ref = F.backward(q, k, v, do, Dv, LSE, th, scale, pq, pk, causal, path=1, stream_pdc=False)
    nan = float("nan")
    out = (torch.full_like(O, nan),) + tuple(torch.full_like(M, nan) for _ in range(3))
    from fmta_b200 import context_parallel as cp
    kt = cp.stacked_keys(k, th, scale) if N % 256 == 0 else None    # shared operand on some cases, per-call pre-pass on the others
    for lo, hi in windows:
        F.forward_window(q, k, v, th, scale, pq, pk, causal, lo, hi, out=out, ktilde=kt)
        # nothing outside the windows done so far has been touched
        assert bool(torch.isnan(out[0][:, :, hi:]).all()) and bool(torch.isfinite(out[0][:, :, :hi]).all())
    for a, b, n in zip((O, M, L, LSE), out, ("O", "M", "L", "LSE")):
        assert torch.equal(a, b), n
    g = tuple(torch.full_like(ref[0], nan) for _ in range(3))
    dth = torch.zeros_like(ref[3])
    for lo, hi in reversed(windows):
        res = F.backward_window(q, k, v, do, Dv, LSE, th, scale, pq, pk, causal, lo, hi, out=g, ktilde=kt)
        dth += res[3]
        for t in g:
            assert bool(torch.isnan(t[:, :, :lo]).all()) and bool(torch.isfinite(t[:, :, lo:]).all())
    torch.cuda.synchronize()
    F.check_device_status()
    for a, b, n in zip(ref[:3], g, ("dQ", "dK", "dV")):
        assert float((a - b).abs().max()) <= 1e-6 * max(1.0, float(a.abs().max())), n
    assert float((dth - ref[3]).abs().max()) <= 1e-5 * max(1.0, float(ref[3].abs().max()))
    Or, Mr, Lr = orc.conv_attn_fwd(Q, K, V, theta, scale, causal)
    rq, rk, rv, rt = orc.conv_attn_bwd_autograd(Q, K, V, theta, dO, scale, causal)
    # L is compared through LSE (it scales with exp(-M))
    check_outputs(dict(O=out[0], M=out[1], LSE=out[3], dQ=g[0], dK=g[1], dV=g[2], dTheta=dth),
                  dict(O=Or, M=Mr, LSE=Mr + torch.log(Lr), dQ=rq, dK=rk, dV=rv, dTheta=rt),
                  "windows %s of B%d H%d N%d d%d theta(%d,%d) causal=%d" % (windows, B, H, N, d, cq, ck, causal))


def test_window_arguments_are_checked():
    import fmta_b200 as F
    (_, _, _, _, _), (q, k, v, do, th) = _inputs(1, 1, 1024, 64, 3, 3, 1)
    for lo, hi in ((128, 512), (0, 500), (512, 512), (0, 2048), (-256, 256)):
        with pytest.raises(RuntimeError):
            F.forward_window(q, k, v, th, 0.125, 2, 1, True, lo, hi)
    with pytest.raises(RuntimeError):      # head dim 32 has no tensor-core kernels, so no windows
        F.forward_window(q[..., :32].contiguous(), k[..., :32].contiguous(), v[..., :32].contiguous(), th, 0.125, 2, 1, True, 0, 512)


@pytest.mark.parametrize("layout", ["zigzag", "contiguous"])
def test_autograd_function_on_one_rank_equals_the_plain_function(layout):
    """Without a process group the Function computes the single window [0, N): same numbers as
    FlashConvAttentionCUDAFunction."""
    import fmta_b200 as F
    B, H, N, d, cq, ck = 1, 2, 512, 64, 6, 11
    (Q, K, V, dO, theta), _ = _inputs(B, H, N, d, cq, ck, 5)
    res = []
    for fn in (lambda *a: F.context_parallel_conv_attention(*a, True, None, layout),
               lambda *a: F.FlashConvAttentionCUDAFunction.apply(*a, True)):
        q, k, v = (t.cuda().float().requires_grad_() for t in (Q, K, V))     # fp32 leaves: gradients come back in fp32
        th = theta.cuda().requires_grad_()
        O = fn(q, k, v, th, 1.0 / math.sqrt(d), cq - 1, (ck - 1) // 2)
        O.backward(dO.cuda().to(O.dtype))
        res.append([O.detach()] + [t.grad for t in (q, k, v, th)])
    for a, b, n in zip(res[0], res[1], ("O", "dQ", "dK", "dV", "dTheta")):
        assert float((a.float() - b.float()).abs().max()) <= 1e-5 * max(1.0, float(b.float().abs().max())), n


_WORKER = r'''
import math, os, sys, datetime, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import fmta_b200 as F
from fmta_b200 import context_parallel as cp
from oracle import conv_attn_oracle as orc
rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=dev, timeout=datetime.timedelta(seconds=120))
for (B, H, N, d, cq, ck, layout) in ((1, 2, 2048, 64, 6, 11, "zigzag"), (1, 1, 1024, 128, 6, 11, "contiguous")):
    Q, K, V, dO, th = orc.make_inputs(B, H, N, d, cq, ck, seed=3 + N, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    dv = lambda t: t.to(dev).float().contiguous()      # bf16-representable values in fp32 leaves: gradients come back in fp32
    # the whole sequence on this GPU
    q, k, v = (dv(t).requires_grad_() for t in (Q, K, V)); t0 = th.to(dev).requires_grad_()
    O = F.FlashConvAttentionCUDAFunction.apply(q, k, v, t0, scale, cq - 1, (ck - 1) // 2, True)
    O.backward(dv(dO).to(O.dtype))
    # this rank's share of the sequence
    wins = cp.windows_for_rank(N, ws, rank, layout)
    loc = lambda t: cp.take_local(dv(t), wins)
    ql, kl, vl = (loc(t).requires_grad_() for t in (Q, K, V)); t1 = th.to(dev).requires_grad_()
    Ol = F.context_parallel_conv_attention(ql, kl, vl, t1, scale, cq - 1, (ck - 1) // 2, True, None, layout)
    Ol.backward(loc(dO).to(Ol.dtype))
    torch.cuda.synchronize()
    F.check_device_status(dev)
    assert torch.equal(Ol.detach(), cp.take_local(O.detach(), wins))
    for a, b, n in ((ql.grad, q.grad, "dQ"), (kl.grad, k.grad, "dK"), (vl.grad, v.grad, "dV")):
        e = float((a - cp.take_local(b, wins)).abs().max())
        assert e <= 1e-5 * max(1.0, float(b.abs().max())), (n, e)
    e = float((t1.grad - t0.grad).abs().max())
    assert e <= 1e-4 * max(1.0, float(t0.grad.abs().max())), ("dTheta", e)
dist.destroy_process_group()
print("OK", rank)
'''


def test_two_ranks_share_one_sequence_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    pkg = os.path.join(ROOT, "flash-multi-token-attention_b200")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29551", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), pkg, ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all("OK" in o for o in outs)


def test_windows_of_one_rank_at_N65536_d128():
    """The share of rank 0 of 8 (zigzag: the first and the last 4096 positions) of one (batch, head) pair at
    N = 65536, d = 128: 16 forward CTAs of one row tile each, up to 1020 key blocks long.  The window calls
    reproduce the whole-sequence forward bit for bit and the whole-sequence backward to rounding on their rows,
    and the forward meets the oracle bound on row blocks."""
    import fmta_b200 as F
    from fmta_b200 import context_parallel as cp
    B, H, N, d, cq, ck = 1, 1, 65536, 128, 6, 11
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=65536, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    pq, pk = cq - 1, (ck - 1) // 2
    O, M, L, LSE = F.forward(q, k, v, th, scale, pq, pk, True, return_lse=True)
    Dv = F.rowdot(do, O)
    ref = F.backward(q, k, v, do, Dv, LSE, th, scale, pq, pk, True)
    wins = cp.windows_for_rank(N, 8, 0, "zigzag")
    assert wins == [(0, 4096), (61440, 65536)]
    kt = cp.stacked_keys(k, th, scale)
    nan = float("nan")
    out = (torch.full_like(O, nan),) + tuple(torch.full_like(M, nan) for _ in range(3))
    g = tuple(torch.full_like(ref[0], nan) for _ in range(3))
    for lo, hi in wins:
        F.forward_window(q, k, v, th, scale, pq, pk, True, lo, hi, out=out, ktilde=kt)
        F.backward_window(q, k, v, do, Dv, LSE, th, scale, pq, pk, True, lo, hi, out=g, ktilde=kt)
    torch.cuda.synchronize()
    F.check_device_status()
    for lo, hi in wins:
        assert torch.equal(out[0][:, :, lo:hi], O[:, :, lo:hi]) and torch.equal(out[3][:, :, lo:hi], LSE[:, :, lo:hi])
        for a, b, n in zip(ref[:3], g, ("dQ", "dK", "dV")):
            e = float((a[:, :, lo:hi] - b[:, :, lo:hi]).abs().max())
            assert e <= 1e-6 * max(1.0, float(a.abs().max())), (n, lo, e)
    assert bool(torch.isnan(out[0][:, :, 4096:61440]).all()) and bool(torch.isnan(g[1][:, :, 4096:61440]).all())
    for i0, i1 in ((4080, 4096), (61440, 61456), (65520, 65536)):
        Or, Mr, Lr = orc.conv_attn_fwd_rowblock(Q, K, V, theta, i0, i1, scale, True)
        check_outputs(dict(O=out[0][:, :, i0:i1], M=out[1][:, :, i0:i1], LSE=out[3][:, :, i0:i1]),
                      dict(O=Or, M=Mr, LSE=Mr + torch.log(Lr)), "window rows %d-%d of N=65536, d=128" % (i0, i1))
