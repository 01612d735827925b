"""Shared helpers of the parity tests."""
import os

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(ROOT, "tests", "golden")

# Tolerances stated by the benchmark contract: max abs error against an fp32 reference.
TOL_FP32 = 1e-3   # fp32 paths (oracle restatement vs the reference's outputs)
TOL_BF16 = 2e-2   # bf16 kernels vs the fp32 oracle fed the same bf16-rounded inputs


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(np.asarray(z[k])) for k in z.files}


def maxabs(a, b):
    return float((a.detach().float().cpu() - b.detach().float().cpu()).abs().max())


def bf16_round(t):
    return t.to(torch.bfloat16).to(torch.float32)
