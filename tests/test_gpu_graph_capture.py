"""The training calls are stream-ordered and make no host synchronisation or device allocation of their own,
so a forward + D + backward step can be captured into a CUDA graph and replayed: the replay must give exactly
the numbers of the eager calls, also after the contents of the (static) input tensors changed.  Covers the
tensor-core kernels at both head dims, the exact kernels and decode."""
import math

import pytest
import torch

from oracle import conv_attn_oracle as orc

pytestmark = pytest.mark.gpu


def _step(F, q, k, v, do, th, scale, cq, ck, path):
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=path)
    D = F.rowdot(do, O)
    dQ, dK, dV, dTh = F.backward(q, k, v, do, D, LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=path)
    return O, LSE, dQ, dK, dV, dTh


@pytest.mark.parametrize("d,path", [(64, 1), (128, 1), (64, 0)])
def test_training_step_replays_from_a_cuda_graph(d, path):
    import fmta_b200 as F
    B, H, N, cq, ck = 1, 2, 600, 6, 11
    scale = 1.0 / math.sqrt(d)
    sets = []
    for seed in (11, 12):
        Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=seed, dtype=torch.bfloat16)
        sets.append([t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO)] + [theta.cuda()])
    static = [t.clone() for t in sets[0]]

    # warm-up on a side stream (first-call attribute setting, allocator pools), as graph capture requires
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            _step(F, *static, scale, cq, ck, path)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()

    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = _step(F, *static, scale, cq, ck, path)
    for inputs in (sets[1], sets[0]):
        for dst, src in zip(static, inputs):
            dst.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        got = [o.clone() for o in outs]
        ref = _step(F, *inputs, scale, cq, ck, path)
        torch.cuda.synchronize()
        for name, g, r in zip(("O", "LSE", "dQ", "dK", "dV", "dTheta"), got, ref):
            assert torch.equal(g, r), name
    F.check_device_status()


def test_decode_replays_from_a_cuda_graph():
    import fmta_b200 as F
    B, H, d, Nk, q_len, cq, ck = 2, 4, 128, 3000, 6, 6, 11
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, H, q_len, d, generator=g).cuda().to(torch.bfloat16)
    ks = [torch.randn(B, H, Nk, d, generator=g).cuda().to(torch.bfloat16) for _ in range(2)]
    v = torch.randn(B, H, Nk, d, generator=g).cuda().to(torch.bfloat16)
    th = (torch.randn(H, cq, ck, generator=g) * 0.02).cuda()
    th[:, cq - 1, ck // 2] += 1.0
    scale = 1.0 / math.sqrt(d)
    k = ks[0].clone()

    def run(kk):
        return F.fwd_conv_attn_inference(q, kk, v, th, 4, scale, cq - 1, (ck - 1) // 2, False)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        run(k)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        outs = run(k)
    for src in (ks[1], ks[0]):
        k.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        ref = run(src)
        torch.cuda.synchronize()
        for g_, r_ in zip(outs, ref):
            assert torch.equal(g_, r_)


_PLAIN_ORDER_WORKER = r'''
import math, sys, torch
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import fmta_b200 as F
from oracle import conv_attn_oracle as orc
out = {}
for d in (64, 128):
    B, H, N, cq, ck = 2, 2, 700, 6, 11
    Q, K, V, dO, theta = orc.make_inputs(B, H, N, d, cq, ck, seed=21 + d, dtype=torch.bfloat16)
    q, k, v, do = (t.cuda().to(torch.bfloat16).contiguous() for t in (Q, K, V, dO))
    th = theta.cuda()
    scale = 1.0 / math.sqrt(d)
    for rep in range(3):          # back to back: the launches of one step follow those of the step before
        O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True, path=1)
        g = F.backward(q, k, v, do, F.rowdot(do, O), LSE, th, scale, cq - 1, (ck - 1) // 2, True, path=1)
    torch.cuda.synchronize()
    F.check_device_status()
    out[d] = [t.cpu() for t in (O, LSE) + tuple(g)]
torch.save(out, sys.argv[3])
print("OK")
'''


def test_plain_stream_order_gives_the_same_bits(tmp_path):
    """FMTA_NO_PDL=1 (every kernel launched in plain stream order) against the default, programmatic dependent
    launch: the same step in two processes, bit-identical outputs -- the early-started kernels read nothing before
    their predecessors have completed."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "flash-multi-token-attention_b200")
    script = tmp_path / "worker.py"
    script.write_text(_PLAIN_ORDER_WORKER)
    res = []
    for flag in ("0", "1"):
        dst = tmp_path / ("out%s.pt" % flag)
        r = subprocess.run([sys.executable, str(script), pkg, root, str(dst)], env=dict(os.environ, FMTA_NO_PDL=flag),
                           stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
        assert r.returncode == 0 and "OK" in r.stdout, r.stdout
        res.append(torch.load(dst))
    for d in (64, 128):
        for a, b, n in zip(res[0][d], res[1][d], ("O", "LSE", "dQ", "dK", "dV", "dTheta")):
            assert torch.equal(a, b), (d, n)
