"""CPU-side checks: the C-ABI library loads and exports every symbol declared in
include/fmta_b200.h, host-side validation rejects bad arguments without touching a GPU, and the
batch x head sharding logic (including a world_size-2 gloo all-reduce of the filter gradient)."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

from helpers import ROOT


def _declared_symbols():
    txt = open(os.path.join(ROOT, "include", "fmta_b200.h")).read()
    return sorted(set(re.findall(r"\b(fmta_[a-z_A-Z0-9]+)\s*\(", txt)))


def test_library_exports_every_declared_symbol():
    import fmta_b200
    from fmta_b200 import _lib
    names = _declared_symbols()
    assert len(names) >= 9
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), n
    assert set(_lib.EXPORTS) <= set(names)
    assert _lib.lib.fmta_version() >= 100


def test_status_strings():
    from fmta_b200._lib import lib
    seen = {lib.fmta_strerror(s).decode() for s in range(0, -8, -1)}
    assert len(seen) == 8 and "ok" in seen


def test_host_validation_needs_no_gpu():
    """Every rejection below happens before any CUDA call."""
    from fmta_b200._lib import lib
    P = ctypes.c_void_p
    good = P(0x1000)
    def fwd(Q=good, O=good, N=16, d=64, cq=3, ck=3, theta=good, G=1, w=None, H=2):
        return lib.fmta_fwd(Q, good, good, theta, w, O, None, None, None, 1, H, N, d, cq, ck, G, 1.0, 1, 0, 0,
                            None, 0, None)
    assert fwd(Q=None) == -1
    assert fwd(N=0) == -2
    assert fwd(d=48) == -3
    assert fwd(ck=4) == -3
    assert fwd(cq=17) == -3
    assert fwd(Q=P(0x1004)) == -4
    assert fwd(G=3, w=good, H=6) == -3
    assert fwd(G=4, w=good, H=6) == -2
    # the pair that shares the stacked key operand: the buffer is required and must be aligned; shapes without
    # tensor-core kernels are refused rather than served by the exact kernels
    keep = lambda kt=good, d=64, th=good: lib.fmta_fwd_keep_ktilde(good, good, good, th, good, None, None, None, 1, 2, 16, d,
                                                                   3, 3, 1.0, 1, 0, None, 0, kt, None)
    assert keep(kt=None) == -1 and keep(th=None) == -1 and keep(kt=P(0x1008)) == -4 and keep(d=32) == -3
    use = lambda kt=good, d=64: lib.fmta_bwd_with_ktilde(good, good, good, good, good, good, good, good, good, good, good,
                                                         1, 2, 16, d, 3, 3, 1.0, 1, None, 0, kt, None)
    assert use(kt=None) == -1 and use(kt=P(0x1008)) == -4 and use(d=32) == -3
    dec = lambda q_len=6, ks=1, Nk=64: lib.fmta_decode(good, good, good, good, good, good, good, 1, 1, q_len, Nk,
                                                        64, 3, 3, ks, 1.0, None)
    assert dec(q_len=17) == -2 and dec(ks=0) == -2 and dec(ks=65) == -2
    assert lib.fmta_decode_offset_causal(good, good, good, good, good, good, good, 1, 1, 17, 64, 64, 3, 3, 1, 1.0,
                                         None) == -2
    pag = lambda table=good, page=64, max_pages=4, Nk=200: lib.fmta_decode_paged(
        good, good, good, table, None, good, good, good, good, 1, 1, 6, Nk, 64, 3, 3, 1, 1.0, page, max_pages, 0, None)
    assert pag(table=None) == -1
    assert pag(page=48) == -2 and pag(page=8) == -2          # power of two, at least one 16-key step
    assert pag(max_pages=3) == -2                            # 200 keys need 4 pages of 64
    assert pag(max_pages=4096, Nk=64) == -2                  # block-table row longer than the kernel stages
    app = lambda kp=good, page=64, n_new=1: lib.fmta_kv_append_paged(kp, good, good, good, good, good, 1, 1, n_new,
                                                                     64, page, 4, None)
    assert app(kp=None) == -1 and app(page=24) == -2 and app(n_new=0) == -2
    assert lib.fmta_bwd_dq_dw(good, good, good, good, good, good, good, None, good, good, None, 1, 2, 64, 64, 3, 3,
                              1, 1.0, 1, None, 0, None) == -5     # workspace missing
    assert lib.fmta_workspace_bytes(1, 4, 16, 4096, 64, 6, 11, 1) == 4 * 64 * 16 * 66 * 4
    # head mix: one dW partial per CTA of the finest kernel that may run (16-row tiles from 16 heads per group on)
    assert lib.fmta_workspace_bytes(1, 2, 16, 1000, 64, 1, 1, 16) == (2 * 63) * (16 * 1 + 1 * 16 * 16) * 4
    assert lib.fmta_workspace_bytes(1, 2, 8, 1000, 64, 1, 1, 4) == (2 * 16) * (8 * 1 + 2 * 4 * 4) * 4
    # optional exchange scratch of conv + mix: two sets of two 80 x 84 fp32 tiles per CTA; none without a mix
    assert lib.fmta_workspace_bytes(5, 2, 32, 8192, 128, 6, 11, 4) == 2 * 2 * 32 * 128 * 2 * 80 * 84 * 4
    assert lib.fmta_workspace_bytes(5, 2, 32, 8192, 128, 6, 11, 1) == 0
    # 32 mixed heads: accepted without a conv up to head dim 64 (the missing workspace is what is reported), refused otherwise
    mix = lambda d, theta: lib.fmta_bwd_dq_dw(good, good, good, good, good, good, theta, good, good, good if theta else None, good,
                                              1, 32, 64, d, 3, 3, 32, 1.0, 1, None, 0, None)
    assert mix(64, None) == -5 and mix(128, None) == -3 and mix(64, good) == -3


def test_ops_refuse_cpu_tensors():
    import fmta_b200 as F
    Q = torch.zeros(1, 2, 16, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        F.forward(Q, Q, Q, torch.zeros(2, 3, 3), 1.0, 2, 1, True)
    with pytest.raises(RuntimeError):
        F.fwd_conv_attn_inference(Q, Q, Q, torch.zeros(2, 3, 3), 1, 1.0, 2, 1, False)


def test_module_state_dict_names():
    import fmta_b200 as F
    m = F.ConvAttentionCUDA(4, 6, 11, init_random=False)
    assert list(m.state_dict().keys()) == ["conv_weight"]
    assert m.conv_weight.shape == (4, 6, 11) and float(m.conv_weight[0, 5, 5]) == 1.0
    assert float(m.conv_weight.sum()) == 4.0
    m2 = F.ConvAttentionCUDA(2, 3, 3, init_random=False, init_first=True)
    assert float(m2.conv_weight[1, 0, 0]) == 1.0
    h = F.HeadConvAttention(8)
    assert list(h.state_dict().keys()) == ["head_conv_weights"] and h.head_conv_weights.dtype == torch.float16


def test_unit_partition_covers_everything():
    from fmta_b200 import sharding as sh
    for n in (1, 7, 16, 64, 1024):
        for ws in (1, 2, 4, 8):
            rs = [sh.unit_range(n, ws, r) for r in range(ws)]
            assert rs[0][0] == 0 and rs[-1][1] == n
            assert all(rs[i][1] == rs[i + 1][0] for i in range(ws - 1))
            assert max(b - a for a, b in rs) - min(b - a for a, b in rs) <= 1
    # head-mix groups stay whole; plan kinds
    assert sh.shard_plan(2, 32, 4, 8, 3)["mode"] == "head"
    assert sh.shard_plan(2, 32, 4, 8, 3)["h_lo"] == 12
    assert sh.shard_plan(8, 12, 4, 8, 0)["mode"] == "batch"
    p = sh.shard_plan(3, 12, 4, 2, 1)
    assert p["mode"] == "unit"
    pieces = sh.unit_slices(sh.shard_plan(3, 12, 4, 2, 0)) + sh.unit_slices(p)
    covered = sorted((b, h) for b, h0, h1 in pieces for h in range(h0, h1))
    assert covered == [(b, h) for b in range(3) for h in range(12)]
    assert all(h0 % 4 == 0 and h1 % 4 == 0 for _, h0, h1 in pieces)


_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
from fmta_b200 import sharding as sh
from oracle import conv_attn_oracle as orc
dist.init_process_group("gloo", rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, ws = dist.get_rank(), dist.get_world_size()
B, H, N, d, cq, ck = 2, 4, 24, 16, 3, 5
Q, K, V, dO, th = orc.make_inputs(B, H, N, d, cq, ck, seed=7)
full = orc.conv_attn_bwd_autograd(Q, K, V, th, dO, None, True)
for mode_B, mode_H in ((B, H), (B, 3)):       # head split, then (H=3 -> not divisible) batch split
    Hh = mode_H
    plan = sh.shard_plan(B, Hh, 1, ws, rank)
    sl = lambda t: sh.local_slice(t[:, :Hh], plan)
    th_l = th[plan["h_lo"]:plan["h_hi"]]
    g = orc.conv_attn_bwd_autograd(sl(Q), sl(K), sl(V), th_l, sl(dO), None, True)
    dth = sh.allreduce_param_grad(g[3], plan)
    ref = orc.conv_attn_bwd_autograd(Q[:, :Hh], K[:, :Hh], V[:, :Hh], th[:Hh], dO[:, :Hh], None, True)
    assert dth.shape == ref[3].shape, (dth.shape, ref[3].shape, plan)
    assert float((dth - ref[3]).abs().max()) < 1e-4, plan
    assert float((g[0] - ref[0][plan["b_lo"]:plan["b_hi"], plan["h_lo"]:plan["h_hi"]]).abs().max()) < 1e-5
dist.destroy_process_group()
print("OK", rank)
'''


def test_sharded_backward_matches_unsharded_gloo_world2(tmp_path):
    """Two CPU ranks: each runs the (oracle) backward on its batch x head slice, the filter
    gradient is all-reduced; the result must equal the unsharded one."""
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    pkg = os.path.join(ROOT, "flash-multi-token-attention_b200")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533", WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script), pkg, ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all("OK" in o for o in outs)


def test_context_parallel_windows_partition_the_sequence():
    from fmta_b200 import context_parallel as cp
    for N, W, layout in ((4096, 1, "zigzag"), (4096, 2, "zigzag"), (65536, 8, "zigzag"), (8192, 4, "contiguous")):
        plan = [cp.windows_for_rank(N, W, r, layout) for r in range(W)]
        seen = torch.zeros(N, dtype=torch.int32)
        for wins in plan:
            assert sum(hi - lo for lo, hi in wins) == N // W
            for lo, hi in wins:
                assert lo % cp.ALIGN == 0 and hi % cp.ALIGN == 0
                seen[lo:hi] += 1
        assert bool((seen == 1).all())
        if layout == "zigzag" and W > 1:
            # a causal forward costs about (rows x mean key count); the zigzag shares are equal to one chunk's worth
            cost = [sum((hi - lo) * (lo + hi) / 2 for lo, hi in wins) for wins in plan]
            assert max(cost) - min(cost) <= 1e-9 * max(cost)
        # gather_sequence / take_local are inverse to each other (one rank: no process group needed)
        full = torch.arange(N, dtype=torch.float32).view(1, 1, N, 1).expand(1, 2, N, 3).contiguous()
        for r in range(W):
            loc = cp.take_local(full, plan[r])
            at = 0
            for lo, hi in plan[r]:
                assert torch.equal(loc[:, :, at:at + hi - lo], full[:, :, lo:hi])
                at += hi - lo
    for bad in ((1000, 2, "zigzag"), (4096, 3, "contiguous"), (4096, 2, "ring")):
        with pytest.raises(ValueError):
            cp.windows_for_rank(*bad[:2], 0, bad[2])


def test_window_entry_points_validate_on_the_host():
    from fmta_b200._lib import lib
    P = ctypes.c_void_p
    good = P(0x1000)
    fw = lambda lo, hi, N=1024, d=64: lib.fmta_fwd_window(good, good, good, good, good, None, None, None, 1, 1, N, d, 3, 3,
                                                          1.0, 1, 0, lo, hi, None, None, 0, None)
    bw = lambda lo, hi, N=1024, d=64: lib.fmta_bwd_window(good, good, good, good, good, good, good, good, good, good, good,
                                                          1, 1, N, d, 3, 3, 1.0, 1, lo, hi, None, None, 0, None)
    for f in (fw, bw):
        assert f(0, 0) == -2                       # a window is required
        assert f(0, 512, d=32) == -3               # tensor-core shapes only
    assert lib.fmta_fwd_window(good, good, good, None, good, None, None, None, 1, 1, 1024, 64, 3, 3, 1.0, 1, 0, 0, 512,
                               None, None, 0, None) == -1
    sk = lambda K=good, kt=good, d=64: lib.fmta_stacked_keys(K, good, kt, 1, 1, 1024, d, 3, 3, 1.0, None)
    assert sk(K=None) == -1 and sk(kt=None) == -1 and sk(d=32) == -3 and sk(kt=P(0x1004)) == -4


_CP_WORKER = r'''
import math, os, sys, datetime, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
from fmta_b200 import context_parallel as cp
from oracle import conv_attn_oracle as orc
rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=ws, timeout=datetime.timedelta(seconds=120))

# the oracle stands in for the CUDA window calls, so that the gathers, the window bookkeeping and the all-reduce
# of the filter gradient run on CPU ranks
def fwd_window(Q, K, V, th, scale, pq, pk, causal, lo, hi, out=None, ktilde=None):
    O, M, L = orc.conv_attn_fwd(Q.float(), K.float(), V.float(), th, scale, causal)
    if out is None:
        out = (torch.full_like(O, float("nan")),) + tuple(torch.full_like(M, float("nan")) for _ in range(3))
    for dst, src in zip(out, (O, M, L, M + torch.log(L))):
        dst[:, :, lo:hi] = src[:, :, lo:hi]
    return out
def bwd_window(Q, K, V, dO, D, L, th, scale, pq, pk, causal, lo, hi, out=None, ktilde=None):
    with torch.enable_grad():                      # called from inside an autograd backward
        g = orc.conv_attn_bwd_autograd(Q.float(), K.float(), V.float(), th.detach(), dO.float(), scale, causal)
    if out is None:
        out = tuple(torch.full_like(g[0], float("nan")) for _ in range(3))
    for dst, src in zip(out, g[:3]):
        dst[:, :, lo:hi] = src[:, :, lo:hi]
    return out + (g[3] * ((hi - lo) / Q.shape[2]),)       # shares that add up to the whole gradient
cp.forward_window, cp.backward_window = fwd_window, bwd_window
cp.stacked_keys = lambda K, th, scale: None
cp._rowdot = lambda dO, O: (dO.float() * O.float()).sum(-1)

B, H, N, d, cq, ck = 1, 2, 1024, 16, 3, 5
Q, K, V, dO, th = orc.make_inputs(B, H, N, d, cq, ck, seed=4, dtype=torch.bfloat16)
scale = 1.0 / math.sqrt(d)
Or, _, _ = orc.conv_attn_fwd(Q, K, V, th, scale, True)
gr = orc.conv_attn_bwd_autograd(Q, K, V, th, dO, scale, True)
for layout in ("zigzag", "contiguous"):
    wins = cp.windows_for_rank(N, ws, rank, layout)
    ql, kl, vl = (cp.take_local(t, wins).requires_grad_() for t in (Q, K, V))
    t1 = th.clone().requires_grad_()
    Ol = cp.context_parallel_conv_attention(ql, kl, vl, t1, scale, cq - 1, (ck - 1) // 2, True, None, layout)
    Ol.backward(cp.take_local(dO, wins))
    assert float((Ol.detach() - cp.take_local(Or, wins)).abs().max()) <= 1e-5
    for a, b in ((ql.grad, gr[0]), (kl.grad, gr[1]), (vl.grad, gr[2])):
        assert float((a - cp.take_local(b, wins)).abs().max()) <= 1e-4
    assert float((t1.grad - gr[3]).abs().max()) <= 1e-3 * float(gr[3].abs().max())
dist.destroy_process_group()
print("OK", rank)
'''


def test_context_parallel_plumbing_gloo_world2(tmp_path):
    """Two CPU ranks hold zigzag / contiguous shares of one sequence; the gathers, the window bookkeeping and the
    all-reduce of the filter gradient run for real, the window computation is the oracle."""
    script = tmp_path / "cp_worker.py"
    script.write_text(_CP_WORKER)
    pkg = os.path.join(ROOT, "flash-multi-token-attention_b200")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29537", WORLD_SIZE="2", OMP_NUM_THREADS="2")
    procs = [subprocess.Popen([sys.executable, str(script), pkg, ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all("OK" in o for o in outs)
