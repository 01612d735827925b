"""Head-mixing attention API, mirroring the reference's ``head_conv_attn`` package
(``head_conv_attn.py:11-116`` and the host functions of ``fwd_kernel.py:282``,
``bwd_dq_dw.py:373``, ``bwd_dk_dv.py:407``), plus the composed "key-query conv then grouped
head mix" operator of the head-mixing training configuration.

Without a key-query conv (the reference's operator) all G heads of a mixing group are handled by
one CTA (G in {2,4,8,16,32}; 32 up to head dim 64).  A mix that follows a key-query conv runs inside
a thread-block cluster: the G <= 16 heads of a group live in G CTAs that exchange their score tiles
through distributed shared memory.  A dense [H,H] matrix is the single-group case G = H; grouped
mixing takes ``w`` as [H/G, G, G].
"""
import math
import os

import torch
import torch.nn as nn

from . import _lib
from ._lib import lib, check, ptr, stream_ptr, as_f32, require_on


def _bf16c(t):
    return t.to(torch.bfloat16).contiguous()


def _group_of(w, H, d=0, has_conv=False):
    """(G, w as fp32 [H/G, G, G]) from a dense [H,H] or grouped [H/G,G,G] matrix."""
    if w.dim() == 2:
        if w.shape[0] != H or w.shape[1] != H:
            raise RuntimeError("w must be [heads, heads] or [heads/G, G, G]")
        G = H
        wg = as_f32(w).reshape(1, H, H)
    elif w.dim() == 3:
        G = int(w.shape[1])
        if w.shape[2] != G or w.shape[0] * G != H:
            raise RuntimeError("grouped w must be [heads/G, G, G]")
        wg = as_f32(w)
    else:
        raise RuntimeError("w must be [heads, heads] or [heads/G, G, G]")
    if G == 32 and (has_conv or d > 64):
        raise NotImplementedError("32 mixed heads are supported without a key-query conv and up to head dim 64")
    if G not in (2, 4, 8, 16, 32):
        raise NotImplementedError("head mixing supports group sizes 2, 4, 8, 16, 32 (got %d)" % G)
    return G, wg


# A mix that follows a key-query conv exchanges the heads' score tiles between the CTAs of a cluster; with this
# optional scratch (two fp32 tiles per CTA) the exchange goes through global memory, which is faster.  Above the
# limit the calls run without it.
MIX_EXCHANGE_LIMIT_BYTES = int(float(os.environ.get("FMTA_MIX_EXCHANGE_LIMIT_GB", "4")) * (1 << 30))


def _exchange_bytes(th, B, H, N, d, cq, ck, G):
    if th is None or G <= 1:
        return 0
    n = int(lib.fmta_workspace_bytes(_lib.FMTA_OP_MIX_EXCHANGE, B, H, N, d, cq, ck, G))
    return n if n <= MIX_EXCHANGE_LIMIT_BYTES else 0


def _theta_args(conv_kernel):
    if conv_kernel is None:
        return None, 1, 1
    th = as_f32(conv_kernel)
    return th, int(th.shape[1]), int(th.shape[2])


def conv_headmix_forward(q, k, v, w, conv_kernel=None, scale=1.0, causal=False, out_dtype=None):
    """(o, l, m, lse): o in ``out_dtype`` (default: dtype of q), l = sum exp, m = max, fp32 [B,H,N]."""
    qb, kb, vb = _bf16c(q), _bf16c(k), _bf16c(v)
    if not qb.is_cuda:
        raise RuntimeError("q must be a CUDA tensor")
    require_on(qb, kb, "k", qb.shape); require_on(qb, vb, "v", qb.shape); require_on(qb, w, "w")
    if conv_kernel is not None:
        require_on(qb, conv_kernel, "conv_kernel")
    B, H, N, d = qb.shape
    G, wg = _group_of(w, H, d, conv_kernel is not None)
    th, cq, ck = _theta_args(conv_kernel)
    odt = out_dtype or (q.dtype if q.dtype in (torch.float32, torch.bfloat16) else torch.float32)
    O = torch.empty((B, H, N, d), dtype=odt, device=q.device)
    M = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    L = torch.empty_like(M)
    LSE = torch.empty_like(M)
    xb = _exchange_bytes(th, B, H, N, d, cq, ck, G)
    ws = torch.empty(xb, dtype=torch.uint8, device=q.device) if xb else None
    st = lib.fmta_fwd(ptr(qb), ptr(kb), ptr(vb), ptr(th), ptr(wg), ptr(O), ptr(M), ptr(L), ptr(LSE), B, H, N, d,
                      cq, ck, G, float(scale), int(bool(causal)),
                      _lib.FMTA_DTYPE_BF16 if odt == torch.bfloat16 else _lib.FMTA_DTYPE_F32, 0, ptr(ws), xb,
                      stream_ptr())
    check(st, "fmta_fwd(head mix)")
    if odt != q.dtype and out_dtype is None:
        O = O.to(q.dtype)
    return O, L, M, LSE


def head_conv_attention_forward(q, k, v, w, scale=1.0, causal=False):
    """(o, l, m) -- fwd_kernel.py:282-364."""
    o, l, m, _ = conv_headmix_forward(q, k, v, w, None, scale, causal)
    return o, l, m


def _bwd_common(q, k, v, w, o, do, l, m, conv_kernel, causal, scale, lse=None):
    qb, kb, vb, dob = _bf16c(q), _bf16c(k), _bf16c(v), _bf16c(do)
    if not qb.is_cuda:
        raise RuntimeError("q must be a CUDA tensor")
    B, H, N, d = qb.shape
    for t, n in ((kb, "k"), (vb, "v"), (dob, "do"), (o, "o")):
        require_on(qb, t, n, qb.shape)
    for t, n in ((l, "l"), (m, "m")):
        require_on(qb, t, n, (B, H, N))
    require_on(qb, w, "w")
    if conv_kernel is not None:
        require_on(qb, conv_kernel, "conv_kernel")
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    G, wg = _group_of(w, H, d, conv_kernel is not None)
    th, cq, ck = _theta_args(conv_kernel)
    if lse is None:
        lse = m.float() + torch.log(l.float())
    lse = as_f32(lse)
    oc = o.contiguous() if o.dtype in (torch.float32, torch.bfloat16) else o.float().contiguous()
    D = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    st = lib.fmta_bwd_prep_D(ptr(dob), ptr(oc), 1 if oc.dtype == torch.bfloat16 else 0, ptr(D), D.numel(), d,
                             stream_ptr())
    check(st, "fmta_bwd_prep_D")
    return qb, kb, vb, dob, B, H, N, d, G, wg, th, cq, ck, lse, D, float(scale)


def conv_headmix_bwd_dq_dw(q, k, v, w, o, do, l, m, conv_kernel=None, causal=False, scale=None):
    """(dq fp32, dw fp32 shaped like w, dtheta fp32 or None)."""
    qb, kb, vb, dob, B, H, N, d, G, wg, th, cq, ck, lse, D, scale = _bwd_common(q, k, v, w, o, do, l, m, conv_kernel, causal, scale)
    dQ = torch.empty((B, H, N, d), dtype=torch.float32, device=q.device)
    dW = torch.empty((H // G, G, G), dtype=torch.float32, device=q.device)
    dTh = torch.empty((H, cq, ck), dtype=torch.float32, device=q.device) if th is not None else None
    ws_bytes = int(lib.fmta_workspace_bytes(_lib.FMTA_OP_BWD_DQ, B, H, N, d, cq, ck, G))
    xb = _exchange_bytes(th, B, H, N, d, cq, ck, G)
    if xb:
        ws_bytes = (ws_bytes + 255) // 256 * 256 + xb
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    st = lib.fmta_bwd_dq_dw(ptr(qb), ptr(kb), ptr(vb), ptr(dob), ptr(D), ptr(lse), ptr(th), ptr(wg), ptr(dQ),
                            ptr(dTh), ptr(dW), B, H, N, d, cq, ck, G, scale, int(bool(causal)), ptr(ws), ws_bytes,
                            stream_ptr())
    check(st, "fmta_bwd_dq_dw(head mix)")
    return dQ, dW.reshape(w.shape), dTh


def conv_headmix_bwd_dkdv(q, k, v, w, o, do, l, m, conv_kernel=None, causal=False, scale=None):
    """(dk fp32, dv fp32)."""
    qb, kb, vb, dob, B, H, N, d, G, wg, th, cq, ck, lse, D, scale = _bwd_common(q, k, v, w, o, do, l, m, conv_kernel, causal, scale)
    dK = torch.empty((B, H, N, d), dtype=torch.float32, device=q.device)
    dV = torch.empty_like(dK)
    st = lib.fmta_bwd_dkdv(ptr(qb), ptr(kb), ptr(vb), ptr(dob), ptr(D), ptr(lse), ptr(th), ptr(wg), ptr(dK), ptr(dV),
                           B, H, N, d, cq, ck, G, scale, int(bool(causal)), stream_ptr())
    check(st, "fmta_bwd_dkdv(head mix)")
    return dK, dV


def conv_headmix_backward(q, k, v, w, o, do, l, m, conv_kernel=None, causal=False, scale=None, lse=None):
    """(dq, dk, dv, dw shaped like w, dtheta or None), all fp32, from ONE call of the fused backward entry
    point: D = rowsum(dO * O) and the log-sum-exp are prepared once for both halves (the two host functions
    above, which mirror the reference's pair of calls, each prepare them again)."""
    qb, kb, vb, dob, B, H, N, d, G, wg, th, cq, ck, lse, D, scale = _bwd_common(q, k, v, w, o, do, l, m, conv_kernel,
                                                                                causal, scale, lse)
    dQ = torch.empty((B, H, N, d), dtype=torch.float32, device=q.device)
    dK = torch.empty_like(dQ)
    dV = torch.empty_like(dQ)
    dW = torch.empty((H // G, G, G), dtype=torch.float32, device=q.device)
    dTh = torch.empty((H, cq, ck), dtype=torch.float32, device=q.device) if th is not None else None
    ws_bytes = int(lib.fmta_workspace_bytes(_lib.FMTA_OP_BWD_DQ, B, H, N, d, cq, ck, G))
    xb = _exchange_bytes(th, B, H, N, d, cq, ck, G)
    if xb:
        ws_bytes = (ws_bytes + 255) // 256 * 256 + xb
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=q.device)
    st = lib.fmta_bwd(ptr(qb), ptr(kb), ptr(vb), ptr(dob), ptr(D), ptr(lse), ptr(th), ptr(wg), ptr(dQ), ptr(dK), ptr(dV),
                      ptr(dTh), ptr(dW), B, H, N, d, cq, ck, G, scale, int(bool(causal)), 0, ptr(ws), ws_bytes,
                      stream_ptr())
    check(st, "fmta_bwd(head mix)")
    return dQ, dK, dV, dW.reshape(w.shape), dTh


def head_conv_attention_bwd_dq_dw(q, k, v, w, o, do, l, m, causal=False, scale=None):
    """(dq in q's dtype, dw) -- bwd_dq_dw.py:373-460."""
    dq, dw, _ = conv_headmix_bwd_dq_dw(q, k, v, w, o, do, l, m, None, causal, scale)
    return dq.to(q.dtype), dw.to(w.dtype)


def head_conv_attention_bwd_dkdv(q, k, v, w, o, do, l, m, causal=False, scale=None):
    """(dk, dv) in the input dtypes -- bwd_dk_dv.py:407-485."""
    dk, dv = conv_headmix_bwd_dkdv(q, k, v, w, o, do, l, m, None, causal, scale)
    return dk.to(k.dtype), dv.to(v.dtype)


class HeadConvAttentionFunction(torch.autograd.Function):
    """Same argument list as head_conv_attn.py:11-63."""

    @staticmethod
    def forward(ctx, q, k, v, w, causal=False, scale=None):
        if scale is None:
            scale = 1.0 / math.sqrt(q.shape[-1])
        output, l, m = head_conv_attention_forward(q, k, v, w, scale=scale, causal=causal)
        ctx.save_for_backward(q, k, v, w, output, l, m)
        ctx.causal, ctx.scale = causal, scale
        return output

    @staticmethod
    def backward(ctx, grad_output):
        q, k, v, w, output, l, m = ctx.saved_tensors
        grad_q = grad_k = grad_v = grad_w = None
        need_qw = ctx.needs_input_grad[0] or ctx.needs_input_grad[3]
        need_kv = ctx.needs_input_grad[1] or ctx.needs_input_grad[2]
        if need_qw and need_kv:     # the usual case: one fused call, D and the log-sum-exp prepared once
            dq, dk, dv, dw, _ = conv_headmix_backward(q, k, v, w, output, grad_output, l, m, None, ctx.causal, ctx.scale)
            return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dw.to(w.dtype), None, None
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[3]:
            grad_q, grad_w = head_conv_attention_bwd_dq_dw(q, k, v, w, output, grad_output, l, m,
                                                           causal=ctx.causal, scale=ctx.scale)
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            grad_k, grad_v = head_conv_attention_bwd_dkdv(q, k, v, w, output, grad_output, l, m,
                                                          causal=ctx.causal, scale=ctx.scale)
        return grad_q, grad_k, grad_v, grad_w, None, None


class HeadConvAttention(nn.Module):
    """Drop-in for head_conv_attn.py:66-98 (parameter ``head_conv_weights`` [H,H])."""

    def __init__(self, n_heads, dtype=torch.float16):
        super().__init__()
        self.n_heads = n_heads
        self.dtype = dtype
        self.head_conv_weights = nn.Parameter(torch.randn(n_heads, n_heads, dtype=dtype) / math.sqrt(n_heads))

    def forward(self, q, k, v, causal=False, scale=None):
        return HeadConvAttentionFunction.apply(q, k, v, self.head_conv_weights, causal, scale)


def head_conv_attention(q, k, v, w, causal=False, scale=None):
    """Functional form (head_conv_attn.py:101-116)."""
    return HeadConvAttentionFunction.apply(q, k, v, w, causal, scale)


class ConvHeadMixFunction(torch.autograd.Function):
    """Key-query conv followed by a grouped head mix (w [H/G,G,G]), then softmax and PV."""

    @staticmethod
    def forward(ctx, q, k, v, conv_kernel, w, causal, scale):
        o, l, m, lse = conv_headmix_forward(q, k, v, w, conv_kernel, scale, causal, out_dtype=torch.float32)
        ctx.save_for_backward(q, k, v, conv_kernel, w, o, l, m, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, conv_kernel, w, o, l, m, lse = ctx.saved_tensors
        dq, dk, dv, dw, dth = conv_headmix_backward(q, k, v, w, o, do, l, m, conv_kernel, ctx.causal, ctx.scale, lse=lse)
        return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dth.to(conv_kernel.dtype), dw.to(w.dtype), None, None


def conv_headmix_attention(q, k, v, conv_kernel, w, causal=True, scale=None):
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return ConvHeadMixFunction.apply(q, k, v, conv_kernel, w, causal, scale)
