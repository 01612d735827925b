"""Context (sequence) parallelism for conv attention on the GPUs of one box, one process per GPU.

Used when (batch, head) pairs run out before GPUs do -- one long sequence, few heads.  Every rank holds a
share of the sequence positions of Q, K, V.  The score map couples every query row with every earlier key, and
the key-query convolution couples neighbouring rows and keys across any cut, so the ranks first gather the
whole Q, K, V (bf16, NVLink; a few hundred MB at N = 65536) and then each computes only its own windows of
sequence positions with `fmta_fwd_window` / `fmta_bwd_window`:

  forward   O, LSE of the query rows in the rank's windows (all keys they see);
  backward  dQ of those query rows, dK and dV of the KEYS in the same windows (from all query rows that see
            them -- so dO, D and LSE are gathered too), and the windows' share of the filter gradient.

Nothing but the small filter gradient is summed across ranks (one all-reduce); no rank reads another rank's
memory from a kernel.  Under a causal mask a window late in the sequence costs more in the forward and the dQ
kernel and less in the dK/dV kernel; the ``"zigzag"`` layout gives rank r the chunks r and 2W-1-r of 2W equal
chunks, which evens out all three.  The reference has no sequence parallelism (its kernels take one whole
sequence per (batch, head)).
"""
from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib
from ._lib import lib, ptr, stream_ptr, check, as_f32, require_cuda_bf16, require_on, arm_status

ALIGN = 256      # a window starts on a multiple of this many positions (fmta_fwd_window)

Window = Tuple[int, int]


def windows_for_rank(N: int, world_size: int, rank: int, layout: str = "zigzag") -> List[Window]:
    """The windows [lo, hi) of sequence positions that ``rank`` computes and holds, in the order in which its
    local tensors store them.  ``"zigzag"``: chunks r and 2W-1-r of 2W equal chunks (N a multiple of
    2 * W * ALIGN); ``"contiguous"``: one block of N / W positions (N a multiple of W * ALIGN)."""
    if not 0 <= rank < world_size:
        raise ValueError("rank %d outside a world of %d" % (rank, world_size))
    if layout not in ("zigzag", "contiguous"):
        raise ValueError("layout must be 'zigzag' or 'contiguous'")
    if world_size == 1:
        return [(0, N)]                      # one rank: the whole sequence, any length
    if layout == "zigzag":
        if N % (2 * world_size * ALIGN) != 0:
            raise ValueError("zigzag layout: the sequence length must be a multiple of %d" % (2 * world_size * ALIGN))
        c = N // (2 * world_size)
        return [(rank * c, (rank + 1) * c), ((2 * world_size - 1 - rank) * c, (2 * world_size - rank) * c)]
    if N % (world_size * ALIGN) != 0:
        raise ValueError("contiguous layout: the sequence length must be a multiple of %d" % (world_size * ALIGN))
    c = N // world_size
    return [(rank * c, (rank + 1) * c)]


def take_local(full: torch.Tensor, windows: Sequence[Window]) -> torch.Tensor:
    """The rows of ``full`` ([B, H, N, ...]) that lie in ``windows``, concatenated in that order."""
    return torch.cat([full[:, :, lo:hi] for lo, hi in windows], dim=2).contiguous()


def gather_sequence(local: torch.Tensor, plan: Sequence[Sequence[Window]], group=None) -> torch.Tensor:
    """All-gather the ranks' local [B, H, n_local, ...] tensors into the whole [B, H, N, ...] tensor, every
    window at its place in the sequence.  ``plan[r]`` = ``windows_for_rank(N, W, r, layout)``."""
    world = len(plan)
    local = local.contiguous()
    if world == 1:
        parts = [local]
    else:
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local, group=group)
    N = sum(hi - lo for wins in plan for lo, hi in wins)
    full = local.new_empty(local.shape[:2] + (N,) + local.shape[3:])
    for part, wins in zip(parts, plan):
        at = 0
        for lo, hi in wins:
            full[:, :, lo:hi] = part[:, :, at:at + hi - lo]
            at += hi - lo
    return full


def _dims(Q, conv_kernel, pad_q, pad_k):
    B, H, N, d = Q.shape
    if conv_kernel.dim() != 3 or conv_kernel.shape[0] != H:
        raise RuntimeError("conv_kernel must be [heads, kx, ky]")
    cq, ck = int(conv_kernel.shape[1]), int(conv_kernel.shape[2])
    if pad_q != cq - 1 or pad_k != (ck - 1) // 2:
        raise RuntimeError("pad_q/pad_k must be (kx-1, (ky-1)//2) for a [heads,kx,ky] kernel")
    return B, H, N, d, cq, ck


def stacked_keys(K, conv_kernel, scale):
    """`fmta_stacked_keys`: the stacked key operand (bf16 [B, H, c_q, N, d]) that the tensor-core kernels read the
    keys through, made once for all the window calls of a step (``ktilde`` of `forward_window` / `backward_window`)."""
    require_cuda_bf16(K, "K")
    require_on(K, conv_kernel, "conv_kernel")
    B, H, N, d = K.shape
    cq, ck = int(conv_kernel.shape[1]), int(conv_kernel.shape[2])
    kt = torch.empty((B, H, cq, N, d), dtype=torch.bfloat16, device=K.device)
    st = lib.fmta_stacked_keys(ptr(K), ptr(as_f32(conv_kernel)), ptr(kt), B, H, N, d, cq, ck, float(scale), stream_ptr())
    check(st, "fmta_stacked_keys")
    return kt


def _check_kt(ktilde, Q, cq):
    if ktilde is None:
        return
    B, H, N, d = Q.shape
    require_on(Q, ktilde, "ktilde", (B, H, cq, N, d))
    if ktilde.dtype != torch.bfloat16 or not ktilde.is_contiguous():
        raise RuntimeError("ktilde must be a contiguous bf16 tensor (see stacked_keys)")


def forward_window(Q, K, V, conv_kernel, scale, pad_q, pad_k, causal, row_lo, row_hi, out=None, ktilde=None):
    """`fmta_fwd_window`: O (fp32), M, L, LSE of the query rows [row_lo, row_hi) of the WHOLE tensors Q, K, V
    ([B, H, N, d] bf16).  ``out`` = (O, M, L, LSE) whole-size buffers to write the window into (allocated
    uninitialised when None); rows outside the window are left as they are.  ``ktilde``: `stacked_keys` of the
    same K, conv_kernel and scale (None: the call makes its own).  Returns ``out``."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        require_cuda_bf16(t, n)
    B, H, N, d, cq, ck = _dims(Q, conv_kernel, pad_q, pad_k)
    require_on(Q, K, "K", Q.shape); require_on(Q, V, "V", Q.shape); require_on(Q, conv_kernel, "conv_kernel")
    arm_status(Q.device)
    theta = as_f32(conv_kernel)
    if out is None:
        out = (torch.empty((B, H, N, d), dtype=torch.float32, device=Q.device),) + tuple(
            torch.empty((B, H, N), dtype=torch.float32, device=Q.device) for _ in range(3))
    O, M, L, LSE = out
    require_on(Q, O, "O", Q.shape)
    for t, n in ((M, "M"), (L, "L"), (LSE, "LSE")):
        require_on(Q, t, n, Q.shape[:-1])
    _check_kt(ktilde, Q, cq)
    ws_bytes = lib.fmta_workspace_bytes(_lib.FMTA_OP_FWD_TC, B, H, N, d, cq, ck, 1)
    ws = torch.empty(max(int(ws_bytes), 16), dtype=torch.uint8, device=Q.device)
    st = lib.fmta_fwd_window(ptr(Q), ptr(K), ptr(V), ptr(theta), ptr(O), ptr(M), ptr(L), ptr(LSE), B, H, N, d, cq, ck,
                             float(scale), int(bool(causal)), _lib.FMTA_DTYPE_BF16 if O.dtype == torch.bfloat16 else _lib.FMTA_DTYPE_F32,
                             int(row_lo), int(row_hi), ptr(ktilde), ptr(ws), ws_bytes, stream_ptr())
    check(st, "fmta_fwd_window")
    return out


def backward_window(Q, K, V, dO, D, L, conv_kernel, scale, pad_q, pad_k, causal, row_lo, row_hi, out=None, ktilde=None):
    """`fmta_bwd_window` on the WHOLE tensors (Q, K, V, dO bf16 [B, H, N, d]; D and the log-sum-exp ``L`` fp32
    [B, H, N], complete): dQ of the query rows and dK, dV of the keys in [row_lo, row_hi) are written into
    ``out`` = (dQ, dK, dV) (fp32, whole size; allocated uninitialised when None), other rows are left alone.
    Returns (dQ, dK, dV, dconv_kernel share of the window)."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (dO, "dO")):
        require_cuda_bf16(t, n)
    B, H, N, d, cq, ck = _dims(Q, conv_kernel, pad_q, pad_k)
    for t, n in ((K, "K"), (V, "V"), (dO, "dO")):
        require_on(Q, t, n, Q.shape)
    require_on(Q, D, "D", Q.shape[:-1]); require_on(Q, L, "L (log-sum-exp)", Q.shape[:-1])
    require_on(Q, conv_kernel, "conv_kernel")
    arm_status(Q.device)
    theta, Dv, LSE = as_f32(conv_kernel), as_f32(D), as_f32(L)
    if out is None:
        out = tuple(torch.empty((B, H, N, d), dtype=torch.float32, device=Q.device) for _ in range(3))
    dQ, dK, dV = out
    for t, n in ((dQ, "dQ"), (dK, "dK"), (dV, "dV")):
        require_on(Q, t, n, Q.shape)
        if t.dtype != torch.float32 or not t.is_contiguous():
            raise RuntimeError("%s must be a contiguous fp32 tensor" % n)
    dTheta = torch.empty((H, cq, ck), dtype=torch.float32, device=Q.device)
    _check_kt(ktilde, Q, cq)
    ws_bytes = lib.fmta_workspace_bytes(_lib.FMTA_OP_BWD_TC, B, H, N, d, cq, ck, 1)
    ws = torch.empty(max(int(ws_bytes), 16), dtype=torch.uint8, device=Q.device)
    st = lib.fmta_bwd_window(ptr(Q), ptr(K), ptr(V), ptr(dO), ptr(Dv), ptr(LSE), ptr(theta), ptr(dQ), ptr(dK), ptr(dV),
                             ptr(dTheta), B, H, N, d, cq, ck, float(scale), int(bool(causal)), int(row_lo), int(row_hi),
                             ptr(ktilde), ptr(ws), ws_bytes, stream_ptr())
    check(st, "fmta_bwd_window")
    return dQ, dK, dV, dTheta


_SIDE_STREAMS = {}


def _side_stream(device, i):
    key = (device.index if device.index is not None else torch.cuda.current_device(), i)
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return _SIDE_STREAMS[key]


def _on_streams(windows, fn, device):
    """``fn(i, lo, hi)`` for every window; on a GPU the second window runs on a side stream, so that its CTAs fill
    the SMs the first window's last wave leaves idle (the windows write disjoint rows and have their own workspaces).
    Returns the results in window order."""
    if len(windows) < 2 or device.type != "cuda":
        return [fn(i, lo, hi) for i, (lo, hi) in enumerate(windows)]
    main = torch.cuda.current_stream(device)
    res = [None] * len(windows)
    sides = []
    for i, (lo, hi) in enumerate(windows):
        if i == 0:
            continue
        side = _side_stream(device, i)
        side.wait_stream(main)
        with torch.cuda.stream(side):
            res[i] = fn(i, lo, hi)
        sides.append(side)
    res[0] = fn(0, *windows[0])
    for side in sides:
        main.wait_stream(side)
    return res


def _rowdot(dO, O):
    from .conv_attn import rowdot
    return rowdot(dO, O)


class ContextParallelConvAttentionFunction(torch.autograd.Function):
    """Conv attention over a sequence that is sharded across the ranks of ``group``.

    ``apply(q, k, v, conv_kernel, scale, pad_q, pad_k, causal, group, layout)``: q, k, v are the rank's LOCAL
    [B, H, N / W, d] positions (the windows of `windows_for_rank`, concatenated); returns the local rows of O
    (fp32).  The gradients of q, k, v are local as well; the gradient of conv_kernel is complete on every rank
    (all-reduced)."""

    @staticmethod
    def forward(ctx, q, k, v, conv_kernel, scale, pad_q, pad_k, causal, group=None, layout="zigzag"):
        world = dist.get_world_size(group) if dist.is_initialized() else 1
        rank = dist.get_rank(group) if dist.is_initialized() else 0
        N = q.shape[2] * world
        plan = [windows_for_rank(N, world, r, layout) for r in range(world)]
        Qf, Kf, Vf = (gather_sequence(t.to(torch.bfloat16), plan, group) for t in (q, k, v))
        B, H, _, d = Qf.shape
        out = (torch.empty((B, H, N, d), dtype=torch.float32, device=Qf.device),) + tuple(
            torch.empty((B, H, N), dtype=torch.float32, device=Qf.device) for _ in range(3))
        kt = stacked_keys(Kf, conv_kernel, scale)      # once per step: both windows, forward and backward, read it
        _on_streams(plan[rank], lambda i, lo, hi: forward_window(Qf, Kf, Vf, conv_kernel, scale, pad_q, pad_k, causal,
                                                                 lo, hi, out=out, ktilde=kt), Qf.device)
        o_loc, lse_loc = take_local(out[0], plan[rank]), take_local(out[3], plan[rank])
        ctx.save_for_backward(Qf, Kf, Vf, conv_kernel, o_loc, lse_loc)
        ctx.kt = kt
        ctx.args = (scale, pad_q, pad_k, causal, group, plan, rank)
        ctx.in_dtypes = (q.dtype, k.dtype, v.dtype)
        return o_loc

    @staticmethod
    def backward(ctx, do_loc):
        Qf, Kf, Vf, conv_kernel, o_loc, lse_loc = ctx.saved_tensors
        scale, pad_q, pad_k, causal, group, plan, rank = ctx.args
        do_b = do_loc.to(torch.bfloat16).contiguous()
        d_loc = _rowdot(do_b, o_loc)                                  # D of the local rows
        dOf = gather_sequence(do_b, plan, group)
        Df, LSEf = gather_sequence(d_loc, plan, group), gather_sequence(lse_loc, plan, group)
        out = tuple(torch.empty(Qf.shape, dtype=torch.float32, device=Qf.device) for _ in range(3))
        kt, ctx.kt = ctx.kt, None
        res = _on_streams(plan[rank], lambda i, lo, hi: backward_window(Qf, Kf, Vf, dOf, Df, LSEf, conv_kernel, scale, pad_q,
                                                                        pad_k, causal, lo, hi, out=out, ktilde=kt), Qf.device)
        dth = res[0][3]
        for r in res[1:]:
            dth = dth + r[3]
        if len(plan) > 1:
            dist.all_reduce(dth, group=group)
        tq, tk, tv = ctx.in_dtypes
        dq, dk, dv = (take_local(t, plan[rank]) for t in out)
        return dq.to(tq), dk.to(tk), dv.to(tv), dth.to(conv_kernel.dtype), None, None, None, None, None, None


def context_parallel_conv_attention(q, k, v, conv_kernel, scale, pad_q, pad_k, causal=True, group=None,
                                    layout="zigzag"):
    """Functional form of `ContextParallelConvAttentionFunction`."""
    return ContextParallelConvAttentionFunction.apply(q, k, v, conv_kernel, scale, pad_q, pad_k, causal, group, layout)
