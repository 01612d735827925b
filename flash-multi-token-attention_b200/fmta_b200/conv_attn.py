"""Conv-attention operator API, mirroring the reference's ``conv_attn`` package:

* extension-level functions ``forward`` / ``dq_backward`` / ``dkdv_backward`` with the pybind
  signatures of ``conv_attn/bindings.cpp:43-57``;
* ``FlashConvAttentionCUDAFunction`` and ``ConvAttentionCUDA`` as in
  ``conv_attn/conv_attention_cuda.py:8-163``.

Differences from the reference, all towards the PyTorch oracle it is judged against: theta,
LSE and D stay fp32 (the reference rounds them to bf16, conv_attention_cuda.py:77,115,144),
rectangular filters (c_q != c_k) are supported, launches go to torch's current stream.
"""
import math
import os

import torch
import torch.nn as nn

from . import _lib
from ._lib import lib, check, ptr, stream_ptr, require_cuda_bf16, as_f32, require_on, arm_status


def _dims(Q, conv_kernel, pad_q, pad_k):
    B, H, N, d = Q.shape
    if conv_kernel.dim() != 3 or conv_kernel.shape[0] != H:
        raise RuntimeError("conv_kernel must have shape [heads, kx, ky]")
    cq, ck = int(conv_kernel.shape[1]), int(conv_kernel.shape[2])
    if pad_q != cq - 1 or pad_k != (ck - 1) // 2:
        raise RuntimeError("pad_q/pad_k must be (kx-1, (ky-1)//2) for a [heads,kx,ky] kernel")
    return B, H, N, d, cq, ck


def _workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


# Head dim 32 has no tensor-core kernels of its own (their operand tiles are 128-byte rows = 64 bf16).  With
# the library's default path it runs on the head-dim-64 tensor-core kernels with the head dim zero-padded: the
# scores, the softmax and the first 32 output / gradient columns are unchanged, at twice the tensor work of a
# native kernel and still several times faster than the exact kernels.  FMTA_PAD_D32=0 turns it off.
PAD_D32 = os.environ.get("FMTA_PAD_D32", "1") != "0"


def _pads_to_64(d, cq, path):
    """True when a head-dim-32 call with the default path goes to the padded head-dim-64 tensor-core kernels."""
    return PAD_D32 and d == 32 and path == -1 and cq <= 7 and lib.fmta_set_path(99) != 0


def _pad64(t):
    return torch.nn.functional.pad(t, (0, 32)).contiguous()


# The tensor-core kernels read the keys through a stacked operand (c_q filtered copies of K, bf16) that a pre-pass
# writes; forward and backward each run it.  A training step can keep the forward's copy for the backward
# (c_q times the size of K for as long as the graph lives; about 2 % of a step at B=4, H=16, N=4096, d=64):
# `ktilde_buffer` + the ``ktilde`` argument of `forward` / `backward`, or FMTA_KEEP_KTILDE=1 for the autograd Function.
KEEP_KTILDE = os.environ.get("FMTA_KEEP_KTILDE", "0") != "0"


def ktilde_buffer(Q, conv_kernel):
    """An uninitialised bf16 [B, H, c_q, N, d] buffer for the ``ktilde`` argument of `forward` and `backward`, or
    None where the stacked operand cannot be shared (shapes without tensor-core backward kernels, or the exact
    kernels selected process-wide)."""
    B, H, N, d = Q.shape
    cq = conv_kernel.shape[1]
    if not ((d == 64 and cq <= 7) or (d == 128 and cq <= 6)) or lib.fmta_set_path(99) == 0:
        return None
    return torch.empty((B, H, cq, N, d), dtype=torch.bfloat16, device=Q.device)


def _check_ktilde(ktilde, Q, cq, path):
    B, H, N, d = Q.shape
    require_on(Q, ktilde, "ktilde", (B, H, cq, N, d))
    if ktilde.dtype != torch.bfloat16 or not ktilde.is_contiguous():
        raise RuntimeError("ktilde must be a contiguous bf16 tensor (see ktilde_buffer)")
    if path == 0:
        raise RuntimeError("ktilde belongs to the tensor-core path; path=0 selects the exact kernels")


def forward(Q, K, V, conv_kernel, scale, pad_q, pad_k, causal, out_dtype=torch.float32, return_lse=False,
            path=-1, ktilde=None):
    """(O, M, L) -- `forward` of conv_attn/bindings.cpp:46-48.  O is fp32 as in
    fwd_wrapper.cu:44-46 unless ``out_dtype=torch.bfloat16``; ``return_lse`` appends M+log L.
    ``ktilde`` (from `ktilde_buffer`): the stacked key operand is left there for `backward`."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        require_cuda_bf16(t, n)
    B, H, N, d, cq, ck = _dims(Q, conv_kernel, pad_q, pad_k)
    if K.shape != Q.shape or V.shape != Q.shape:
        raise RuntimeError("Q, K, V must have the same shape [batch, heads, seq, d_head]")
    if ktilde is not None:
        _check_ktilde(ktilde, Q, cq, path)
    elif _pads_to_64(d, cq, path):
        out = forward(_pad64(Q), _pad64(K), _pad64(V), conv_kernel, scale, pad_q, pad_k, causal, out_dtype, return_lse, path)
        return (out[0][..., :32].contiguous(),) + tuple(out[1:])
    require_on(Q, K, "K"); require_on(Q, V, "V"); require_on(Q, conv_kernel, "conv_kernel")
    arm_status(Q.device)
    theta = as_f32(conv_kernel)
    O = torch.empty((B, H, N, d), dtype=out_dtype, device=Q.device)
    M = torch.empty((B, H, N), dtype=torch.float32, device=Q.device)
    L = torch.empty_like(M)
    LSE = torch.empty_like(M) if return_lse else None
    ws_bytes = lib.fmta_workspace_bytes(_lib.FMTA_OP_FWD_TC, B, H, N, d, cq, ck, 1) if path != 0 else 0
    ws = _workspace(ws_bytes, Q.device) if ws_bytes else None
    odt = _lib.FMTA_DTYPE_BF16 if out_dtype == torch.bfloat16 else _lib.FMTA_DTYPE_F32
    if ktilde is not None:
        st = lib.fmta_fwd_keep_ktilde(ptr(Q), ptr(K), ptr(V), ptr(theta), ptr(O), ptr(M), ptr(L), ptr(LSE), B, H, N, d,
                                      cq, ck, float(scale), int(bool(causal)), odt, ptr(ws), ws_bytes, ptr(ktilde),
                                      stream_ptr())
        check(st, "fmta_fwd_keep_ktilde")
        return (O, M, L, LSE) if return_lse else (O, M, L)
    st = lib.fmta_fwd(ptr(Q), ptr(K), ptr(V), ptr(theta), None, ptr(O), ptr(M), ptr(L), ptr(LSE), B, H, N, d,
                      cq, ck, 1, float(scale), int(bool(causal)),
                      _lib.FMTA_DTYPE_BF16 if out_dtype == torch.bfloat16 else _lib.FMTA_DTYPE_F32,
                      int(path), ptr(ws), ws_bytes, stream_ptr())
    check(st, "fmta_fwd")
    return (O, M, L, LSE) if return_lse else (O, M, L)


def rowdot(dO, O):
    """D = rowsum(dO * O) in fp32 (conv_attention_cuda.py:144 without the bf16 rounding)."""
    require_cuda_bf16(dO, "dO")
    if O.dtype not in (torch.float32, torch.bfloat16) or not O.is_contiguous():
        raise RuntimeError("O must be contiguous fp32 or bf16")
    require_on(dO, O, "O", dO.shape)
    D = torch.empty(dO.shape[:-1], dtype=torch.float32, device=dO.device)
    st = lib.fmta_bwd_prep_D(ptr(dO), ptr(O), 1 if O.dtype == torch.bfloat16 else 0, ptr(D),
                             D.numel(), dO.shape[-1], stream_ptr())
    check(st, "fmta_bwd_prep_D")
    return D


def _check_bwd_args(Q, K, V, dO, D, L, conv_kernel):
    """Same device and the expected shape for every tensor whose address goes to the backward kernels."""
    for t, n in ((K, "K"), (V, "V"), (dO, "dO")):
        require_on(Q, t, n, Q.shape)
    require_on(Q, D, "D", Q.shape[:-1])
    require_on(Q, L, "L (log-sum-exp)", Q.shape[:-1])
    require_on(Q, conv_kernel, "conv_kernel")
    arm_status(Q.device)


def dq_backward(Q, K, V, dO, D, L, conv_kernel, scale, pad_q, pad_k, causal):
    """(dQ fp32, dconv_kernel fp32 [H,kx,ky]) -- `dq_backward` of conv_attn/bindings.cpp:50-52.
    ``L`` is the log-sum-exp M + log L, as in the reference (conv_attention_cuda.py:130)."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (dO, "dO")):
        require_cuda_bf16(t, n)
    B, H, N, d, cq, ck = _dims(Q, conv_kernel, pad_q, pad_k)
    _check_bwd_args(Q, K, V, dO, D, L, conv_kernel)
    theta, Dv, LSE = as_f32(conv_kernel), as_f32(D), as_f32(L)
    dQ = torch.empty((B, H, N, d), dtype=torch.float32, device=Q.device)
    dTheta = torch.empty((H, cq, ck), dtype=torch.float32, device=Q.device)
    ws_bytes = lib.fmta_workspace_bytes(_lib.FMTA_OP_BWD_DQ, B, H, N, d, cq, ck, 1)
    ws = _workspace(ws_bytes, Q.device)
    st = lib.fmta_bwd_dq_dw(ptr(Q), ptr(K), ptr(V), ptr(dO), ptr(Dv), ptr(LSE), ptr(theta), None, ptr(dQ),
                            ptr(dTheta), None, B, H, N, d, cq, ck, 1, float(scale), int(bool(causal)),
                            ptr(ws), ws_bytes, stream_ptr())
    check(st, "fmta_bwd_dq_dw")
    return dQ, dTheta


def dkdv_backward(Q, K, V, dO, D, L, conv_kernel, scale, pad_q, pad_k, causal):
    """(dK fp32, dV fp32) -- `dkdv_backward` of conv_attn/bindings.cpp:54-56."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (dO, "dO")):
        require_cuda_bf16(t, n)
    B, H, N, d, cq, ck = _dims(Q, conv_kernel, pad_q, pad_k)
    _check_bwd_args(Q, K, V, dO, D, L, conv_kernel)
    theta, Dv, LSE = as_f32(conv_kernel), as_f32(D), as_f32(L)
    dK = torch.empty((B, H, N, d), dtype=torch.float32, device=Q.device)
    dV = torch.empty_like(dK)
    st = lib.fmta_bwd_dkdv(ptr(Q), ptr(K), ptr(V), ptr(dO), ptr(Dv), ptr(LSE), ptr(theta), None, ptr(dK), ptr(dV),
                           B, H, N, d, cq, ck, 1, float(scale), int(bool(causal)), stream_ptr())
    check(st, "fmta_bwd_dkdv")
    return dK, dV


# The streaming dK/dV kernel (head dim 64) needs 4 * B*H*N*roundup(N,128) bytes for P and dC; it is used when
# that is at most this many bytes (the recomputing kernel otherwise).  Off by default (0): since the recomputing pair
# got its current block order and row-block layout it is the faster one at every size measured on B200 (backward at
# N = 4096: 8 (batch, head) pairs 0.406 against 0.461 ms streaming, 16 pairs 0.588 against 0.601; N = 1024 and 2048
# likewise by 4-8 %); ``stream_pdc=True`` or FMTA_STREAM_LIMIT_GB select the streaming pair.
STREAM_LIMIT_BYTES = int(float(os.environ.get("FMTA_STREAM_LIMIT_GB", "0")) * (1 << 30))


def backward(Q, K, V, dO, D, L, conv_kernel, scale, pad_q, pad_k, causal, path=-1, stream_pdc=None, ktilde=None):
    """(dQ, dK, dV, dconv_kernel), all fp32, in one call (`fmta_bwd`): what the reference obtains
    from `dq_backward` + `dkdv_backward` (conv_attention_cuda.py:147-152).  ``path`` as in the C ABI:
    0 exact kernels, 1 tensor-core kernels + band kernel, -1 library default.  ``stream_pdc``: let the dQ
    kernel keep P and dC for a streaming dK/dV kernel (None: whenever they fit STREAM_LIMIT_BYTES).
    ``ktilde``: the buffer `forward` filled for the same K, conv_kernel and scale; its pre-pass is then skipped."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V"), (dO, "dO")):
        require_cuda_bf16(t, n)
    B, H, N, d, cq, ck = _dims(Q, conv_kernel, pad_q, pad_k)
    _check_bwd_args(Q, K, V, dO, D, L, conv_kernel)
    if ktilde is not None:
        _check_ktilde(ktilde, Q, cq, path)
    elif _pads_to_64(d, cq, path):
        dQ, dK, dV, dTheta = backward(_pad64(Q), _pad64(K), _pad64(V), _pad64(dO), D, L, conv_kernel, scale, pad_q, pad_k,
                                      causal, path, stream_pdc)
        return dQ[..., :32].contiguous(), dK[..., :32].contiguous(), dV[..., :32].contiguous(), dTheta
    theta, Dv, LSE = as_f32(conv_kernel), as_f32(D), as_f32(L)
    dQ = torch.empty((B, H, N, d), dtype=torch.float32, device=Q.device)
    dK = torch.empty_like(dQ)
    dV = torch.empty_like(dQ)
    dTheta = torch.empty((H, cq, ck), dtype=torch.float32, device=Q.device)
    op = _lib.FMTA_OP_BWD_DQ if path == 0 else _lib.FMTA_OP_BWD_TC
    if path != 0 and d == 64 and stream_pdc is not False:
        big = lib.fmta_workspace_bytes(_lib.FMTA_OP_BWD_TC_STREAM, B, H, N, d, cq, ck, 1)
        base = lib.fmta_workspace_bytes(_lib.FMTA_OP_BWD_TC, B, H, N, d, cq, ck, 1)
        if stream_pdc or big - base <= STREAM_LIMIT_BYTES:
            op = _lib.FMTA_OP_BWD_TC_STREAM
    ws_bytes = lib.fmta_workspace_bytes(op, B, H, N, d, cq, ck, 1)
    ws = _workspace(ws_bytes, Q.device)
    if ktilde is not None:
        st = lib.fmta_bwd_with_ktilde(ptr(Q), ptr(K), ptr(V), ptr(dO), ptr(Dv), ptr(LSE), ptr(theta), ptr(dQ), ptr(dK),
                                      ptr(dV), ptr(dTheta), B, H, N, d, cq, ck, float(scale), int(bool(causal)), ptr(ws),
                                      ws_bytes, ptr(ktilde), stream_ptr())
        check(st, "fmta_bwd_with_ktilde")
        return dQ, dK, dV, dTheta
    st = lib.fmta_bwd(ptr(Q), ptr(K), ptr(V), ptr(dO), ptr(Dv), ptr(LSE), ptr(theta), None, ptr(dQ), ptr(dK), ptr(dV),
                      ptr(dTheta), None, B, H, N, d, cq, ck, 1, float(scale), int(bool(causal)), int(path), ptr(ws),
                      ws_bytes, stream_ptr())
    check(st, "fmta_bwd")
    return dQ, dK, dV, dTheta


class FlashConvAttentionCUDAFunction(torch.autograd.Function):
    """autograd.Function with the argument list of conv_attention_cuda.py:96-163."""

    @staticmethod
    def forward(ctx, Q, K, V, conv_kernel, scale, pad_q, pad_k, causal):
        Qb, Kb, Vb = (t.to(torch.bfloat16).contiguous() for t in (Q, K, V))
        needs_grad = any(t.requires_grad for t in (Q, K, V, conv_kernel))
        ctx.ktilde = ktilde_buffer(Qb, conv_kernel) if (KEEP_KTILDE and needs_grad) else None
        O, M, L, LSE = forward(Qb, Kb, Vb, conv_kernel, scale, pad_q, pad_k, causal, return_lse=True, ktilde=ctx.ktilde)
        ctx.save_for_backward(Qb, Kb, Vb, conv_kernel, LSE, O)
        ctx.scale, ctx.pad_q, ctx.pad_k, ctx.causal = scale, pad_q, pad_k, causal
        ctx.in_dtypes = (Q.dtype, K.dtype, V.dtype)
        return O

    @staticmethod
    def backward(ctx, dO):
        Q, K, V, conv_kernel, LSE, O = ctx.saved_tensors
        dOb = dO.to(torch.bfloat16).contiguous()
        D = rowdot(dOb, O)
        dQ, dK, dV, dTheta = backward(Q, K, V, dOb, D, LSE, conv_kernel, ctx.scale, ctx.pad_q, ctx.pad_k, ctx.causal,
                                      ktilde=ctx.ktilde)
        ctx.ktilde = None
        tq, tk, tv = ctx.in_dtypes
        return dQ.to(tq), dK.to(tk), dV.to(tv), dTheta.to(conv_kernel.dtype), None, None, None, None


class ConvAttentionCUDA(nn.Module):
    """Drop-in for ``ConvAttentionCUDA`` (conv_attention_cuda.py:8-93): same constructor,
    parameter name (``conv_weight`` [n_heads, kernel_size_q, kernel_size_k]) and init rules, so
    state_dicts interchange.  ``forward`` returns O (fp32)."""

    def __init__(self, n_heads, kernel_size_q=3, kernel_size_k=3, init_random=True, init_first=False):
        super().__init__()
        self.n_heads = n_heads
        self.kernel_size_q = kernel_size_q
        self.kernel_size_k = kernel_size_k
        self.init_random = init_random
        self.init_first = init_first
        self.conv_weight = nn.Parameter(torch.empty(n_heads, kernel_size_q, kernel_size_k))
        self._init_parameters()

    def _init_parameters(self):
        with torch.no_grad():
            if self.init_random:
                nn.init.normal_(self.conv_weight, mean=0.0, std=0.2)
            else:
                self.conv_weight.zero_()
                if self.init_first:
                    self.conv_weight[:, 0, 0] = 1.0
                else:  # identity: last query tap, centre key tap
                    self.conv_weight[:, self.kernel_size_q - 1, self.kernel_size_k // 2] = 1.0

    def forward(self, Q, K, V, causal=True, softmax_scale=None):
        if softmax_scale is None:
            softmax_scale = 1.0 / math.sqrt(Q.shape[-1])
        pad_k = (self.kernel_size_k - 1) // 2
        pad_q = self.kernel_size_q - 1
        return FlashConvAttentionCUDAFunction.apply(Q, K, V, self.conv_weight, softmax_scale, pad_q, pad_k, causal)
