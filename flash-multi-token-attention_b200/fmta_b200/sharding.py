"""Batch x head sharding across the GPUs of one box (one process per GPU).

Every (batch, head) pair of conv attention is independent in forward and backward except for
the filter gradient, which sums over the batch; head-mixing groups (G consecutive heads) must
stay whole on one GPU.  So work units are (batch, head-group) pairs, block-partitioned over the
ranks, and the only collective is one all-reduce of the small fp32 gradient (dTheta [H,c_q,c_k],
dW [H/G,G,G]) on the compute stream.  No kernel reads another GPU's memory.
"""
from typing import List, Tuple

import torch
import torch.distributed as dist


def unit_range(n_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous block partition: ranks [0, n_units % world) get one extra unit."""
    base, rem = divmod(n_units, world_size)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def shard_plan(B: int, H: int, G: int, world_size: int, rank: int):
    """How a rank's slice of a [B, H, ...] problem looks.

    Returns dict(mode, b_lo, b_hi, h_lo, h_hi): ``mode == "head"`` when the head groups divide
    evenly over the ranks (every head's filter gradient is then wholly local and the all-reduce
    only gathers), else ``"batch"`` (split the batch axis; gradients need a true sum), else
    ``"unit"`` (flattened (batch, group) units; the slice is a list of per-batch head ranges).
    """
    groups = H // G
    if groups % world_size == 0:
        per = groups // world_size
        return dict(mode="head", b_lo=0, b_hi=B, h_lo=rank * per * G, h_hi=(rank + 1) * per * G)
    if B % world_size == 0:
        per = B // world_size
        return dict(mode="batch", b_lo=rank * per, b_hi=(rank + 1) * per, h_lo=0, h_hi=H)
    lo, hi = unit_range(B * groups, world_size, rank)
    return dict(mode="unit", u_lo=lo, u_hi=hi, groups=groups, G=G)


def unit_slices(plan) -> List[Tuple[int, int, int]]:
    """(b, h_lo, h_hi) pieces of a ``"unit"`` plan, merged per batch element."""
    out = []
    groups, G = plan["groups"], plan["G"]
    u = plan["u_lo"]
    while u < plan["u_hi"]:
        b, g0 = divmod(u, groups)
        g1 = min(groups, g0 + (plan["u_hi"] - u))
        out.append((b, g0 * G, g1 * G))
        u += g1 - g0
    return out


def local_slice(t: torch.Tensor, plan) -> torch.Tensor:
    """Slice a [B, H, ...] tensor for a "head" or "batch" plan (contiguous copy)."""
    return t[plan["b_lo"]:plan["b_hi"], plan["h_lo"]:plan["h_hi"]].contiguous()


def allreduce_param_grad(local_grad: torch.Tensor, plan, group=None) -> torch.Tensor:
    """Sum the per-rank filter / mixing gradient into the full tensor.

    ``local_grad`` is indexed by the heads (or head groups) of this rank's slice.  For a "head"
    plan it is placed into a zero tensor covering all ranks' heads and all-reduced (SUM), which
    amounts to a gather; for a "batch" plan it already covers every head and the all-reduce is
    a true sum.  One small collective on the current stream.
    """
    on = dist.is_available() and dist.is_initialized()
    ws = dist.get_world_size(group) if on else 1
    rk = dist.get_rank(group) if on else 0
    if plan["mode"] == "head":
        n_local = local_grad.shape[0]
        full = torch.zeros((n_local * ws,) + tuple(local_grad.shape[1:]), dtype=local_grad.dtype,
                           device=local_grad.device)
        full[rk * n_local:(rk + 1) * n_local] = local_grad
    else:
        full = local_grad.clone()
    if ws > 1:
        dist.all_reduce(full, op=dist.ReduceOp.SUM, group=group)
    return full
