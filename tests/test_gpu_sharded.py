"""Two GPU ranks (one process per GPU, NCCL): every rank runs the CUDA forward + backward on its
(batch, head) slice of one problem, the filter gradient goes through sharding.allreduce_param_grad;
the result must equal the one-GPU run of the whole problem.  Skipped on a box with a single GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r'''
import math, os, sys, datetime, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import fmta_b200 as F
from fmta_b200 import sharding as sh
from oracle import conv_attn_oracle as orc
rank, ws = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", rank=rank, world_size=ws, device_id=dev, timeout=datetime.timedelta(seconds=120))

def run(q, k, v, do, th, scale, cq, ck):
    O, M, L, LSE = F.forward(q, k, v, th, scale, cq - 1, (ck - 1) // 2, True, return_lse=True)
    return F.backward(q, k, v, do, F.rowdot(do, O), LSE, th, scale, cq - 1, (ck - 1) // 2, True)

for (B, H, N, d, cq, ck) in ((2, 4, 300, 128, 6, 11), (2, 3, 260, 64, 6, 11)):   # head split; H=3: batch split
    Q, K, V, dO, th = orc.make_inputs(B, H, N, d, cq, ck, seed=7 + H, dtype=torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    dv = lambda t: t.to(dev).to(torch.bfloat16).contiguous()
    full = run(dv(Q), dv(K), dv(V), dv(dO), th.to(dev), scale, cq, ck)            # the whole problem on this GPU
    plan = sh.shard_plan(B, H, 1, ws, rank)
    sl = lambda t: sh.local_slice(dv(t), plan)
    th_l = th[plan["h_lo"]:plan["h_hi"]].contiguous().to(dev)
    g = run(sl(Q), sl(K), sl(V), sl(dO), th_l, scale, cq, ck)
    dth = sh.allreduce_param_grad(g[3], plan)
    torch.cuda.synchronize()
    F.check_device_status(dev)
    assert dth.shape == full[3].shape, (dth.shape, full[3].shape, plan)
    # same kernels, same per-head summation order for a head split; a batch split changes the order of the
    # batch sum (fp32 rounding only)
    tol = 0.0 if plan["mode"] == "head" else 1e-3
    assert float((dth - full[3]).abs().max()) <= tol, (plan, float((dth - full[3]).abs().max()))
    assert torch.equal(g[0], full[0][plan["b_lo"]:plan["b_hi"], plan["h_lo"]:plan["h_hi"]])
dist.destroy_process_group()
print("OK", rank)
'''


def test_sharded_backward_matches_one_gpu_nccl_world2(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "worker.py"
    script.write_text(_WORKER)
    pkg = os.path.join(ROOT, "flash-multi-token-attention_b200")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29547", WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script), pkg, ROOT], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all("OK" in o for o in outs)
