"""Generate the golden fixtures in this folder from the REFERENCE's own PyTorch code.

Run where the reference checkout is available:

    python tests/golden/make_golden.py --reference /path/to/flash-multi-token-attention

The two reference files are loaded by file path (importing the reference package
triggers a JIT CUDA build and then fails on a module that is missing from it):
``flash_multi_token_attention/conv_attn/conv_attention_pytorch.py`` (``ConvAttention``)
and ``flash_multi_token_attention/head_conv_attn/head_conv_fn_pytorch.py``
(``pytorch_reference_head_conv_attention``).  Gradients are taken with autograd
through those functions, exactly as ``scripts/test_conv_attn.py:115-126`` does.

Every fixture stores its inputs too, so checking it needs neither the reference
nor a particular random-number generator.  Shapes follow the reference's own
comparison scripts (``scripts/test_conv_attn.py:37-61``,
``scripts/test_fwd_inference_conv_attn.py:31-56``, ``fwd_kernel.py:381-396``) plus
the fp32 CPU configuration of the benchmark (B=1,H=4,N=256,d=64, theta (3,5)).
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _randn(g, *shape):
    return torch.randn(*shape, generator=g, dtype=torch.float32)


def conv_case(ref, name, B, H, N, d, c_q, c_k, causal, seed, theta_std, identity, dtype_round=None):
    if ONLY is not None and name != ONLY:
        return
    g = torch.Generator().manual_seed(seed)
    Q, K, V, dO = (_randn(g, B, H, N, d) for _ in range(4))
    theta = _randn(g, H, c_q, c_k) * theta_std
    if identity:
        theta[:, c_q - 1, c_k // 2] += 1.0
    if dtype_round is not None:
        Q, K, V, dO = (t.to(dtype_round).float() for t in (Q, K, V, dO))
    scale = 1.0 / d ** 0.5
    mod = ref.ConvAttention(H, c_q, c_k, init_random=True)
    mod.conv_weight.data = theta.clone()
    q, k, v = (t.clone().requires_grad_(True) for t in (Q, K, V))
    O, M, L = mod(q, k, v, causal=causal, softmax_scale=scale)
    O.backward(dO)
    out = dict(Q=Q, K=K, V=V, dO=dO, theta=theta, O=O.detach(), M=M.detach(), L=L.detach(),
               dQ=q.grad, dK=k.grad, dV=v.grad, dTheta=mod.conv_weight.grad,
               scale=np.float32(scale), causal=np.int32(causal))
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        **{k_: (v_.numpy() if torch.is_tensor(v_) else v_) for k_, v_ in out.items()})
    print(name, "O", tuple(O.shape))


def decode_case(ref, name, B, H, q_len, Nk, d, c_q, c_k, seed, theta_std, identity):
    if ONLY is not None and name != ONLY:
        return
    g = torch.Generator().manual_seed(seed)
    Q = _randn(g, B, H, q_len, d).to(torch.bfloat16).float()
    K = _randn(g, B, H, Nk, d).to(torch.bfloat16).float()
    V = _randn(g, B, H, Nk, d).to(torch.bfloat16).float()
    theta = _randn(g, H, c_q, c_k) * theta_std
    if identity:
        theta[:, c_q - 1, c_k // 2] += 1.0
    scale = 1.0 / d ** 0.5
    mod = ref.ConvAttention(H, c_q, c_k, init_random=True)
    mod.conv_weight.data = theta.clone()
    with torch.no_grad():
        O, M, L = mod(Q, K, V, causal=False, softmax_scale=scale)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), Q=Q.numpy(), K=K.numpy(), V=V.numpy(),
                        theta=theta.numpy(), O=O[:, :, -1:, :].numpy(), M=M[:, :, -1:].numpy(),
                        L=L[:, :, -1:].numpy(), scale=np.float32(scale))
    print(name, "O", tuple(O[:, :, -1:, :].shape))


def head_case(refh, name, B, H, N, d, causal, seed, w_kind):
    if ONLY is not None and name != ONLY:
        return
    g = torch.Generator().manual_seed(seed)
    q, k, v, dO = (_randn(g, B, H, N, d) for _ in range(4))
    if w_kind == "dense":
        w = _randn(g, H, H) / 2
    else:  # block-diagonal groups of 4: identity + N(0, 0.02)
        w = torch.block_diag(*[torch.eye(4) + 0.02 * _randn(g, 4, 4) for _ in range(H // 4)])
    scale = 1.0 / d ** 0.5
    qq, kk, vv, ww = (t.clone().requires_grad_(True) for t in (q, k, v, w))
    O, L, M = refh.pytorch_reference_head_conv_attention(qq, kk, vv, ww, scale=scale, causal=causal)
    O.backward(dO)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), q=q.numpy(), k=k.numpy(), v=v.numpy(),
                        dO=dO.numpy(), w=w.numpy(), O=O.detach().numpy(), L=L.detach().numpy(),
                        M=M.detach().numpy(), dq=qq.grad.numpy(), dk=kk.grad.numpy(),
                        dv=vv.grad.numpy(), dw=ww.grad.numpy(), scale=np.float32(scale),
                        causal=np.int32(causal))
    print(name, "O", tuple(O.shape))


ONLY = None


def main():
    global ONLY
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    ap.add_argument("--only", default=None, help="write only the fixture of this name (default: all)")
    a = ap.parse_args()
    ONLY = a.only
    base = os.path.join(a.reference, "flash_multi_token_attention")
    ref = _load(os.path.join(base, "conv_attn", "conv_attention_pytorch.py"), "ref_conv_attention_pytorch")
    refh = _load(os.path.join(base, "head_conv_attn", "head_conv_fn_pytorch.py"), "ref_head_conv_fn_pytorch")
    torch.set_grad_enabled(True)
    # the reference's own fwd+bwd comparison shape (scripts/test_conv_attn.py:37-61)
    conv_case(ref, "conv_ref_script_3x3", 2, 4, 16, 64, 3, 3, True, 42, 0.2, False, torch.bfloat16)
    # benchmark configuration 0 (fp32 CPU path)
    conv_case(ref, "conv_c0_3x5", 1, 4, 256, 64, 3, 5, True, 0, 0.05, True)
    # rectangular (6,11) filter of the training configurations, ragged N
    conv_case(ref, "conv_6x11_ragged", 1, 2, 83, 32, 6, 11, True, 1, 0.02, True, torch.bfloat16)
    conv_case(ref, "conv_5x5_noncausal", 1, 2, 48, 32, 5, 5, False, 2, 0.1, False, torch.bfloat16)
    conv_case(ref, "conv_7x7_d128", 1, 1, 70, 128, 7, 7, True, 3, 0.05, True, torch.bfloat16)
    # decode: the reference's own script shape, and the (6,11) / q_len=6 serving shape
    decode_case(ref, "decode_ref_script_5x5", 1, 1, 16, 240, 32, 5, 5, 42, 0.02, False)
    decode_case(ref, "decode_6x11_qlen6", 1, 2, 6, 333, 128, 6, 11, 5, 0.02, True)
    decode_case(ref, "decode_3x3_qlen2", 1, 2, 2, 97, 64, 3, 3, 6, 0.2, False)
    # head-conv (fwd_kernel.py:381-396 uses B=2,H=16,N=201,d=32, w = randn/2, seed 34)
    head_case(refh, "head_dense16_noncausal", 1, 16, 45, 32, False, 34, "dense")
    head_case(refh, "head_dense16_causal", 1, 16, 40, 32, True, 35, "dense")
    head_case(refh, "head_group4_causal", 2, 8, 50, 32, True, 36, "group4")
    # 32 heads, the other head count the reference accepts (fwd_kernel.py:300)
    head_case(refh, "head_dense32_causal", 1, 32, 24, 32, True, 37, "dense")


if __name__ == "__main__":
    sys.exit(main())
