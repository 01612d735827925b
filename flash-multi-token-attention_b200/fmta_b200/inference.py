"""Decode API, mirroring ``conv_attn/flash_conv_attention_inference.py``:
``forward_inference`` (the pybind function of fwd_inference_bindings.cpp:20-23) and
``fwd_conv_attn_inference`` (the Python wrapper at :33-93)."""
import torch

from ._lib import lib, check, ptr, stream_ptr, require_cuda_bf16, as_f32


def _split_outputs(B, H, k_splits, d, device):
    """O_splits [B,H,k_splits,d], M_splits, L_splits [B,H,k_splits] carved out of one allocation."""
    n = B * H * k_splits
    buf = torch.empty(n * (d + 2), dtype=torch.float32, device=device)
    return (buf[: n * d].view(B, H, k_splits, d), buf[n * d: n * (d + 1)].view(B, H, k_splits),
            buf[n * (d + 1):].view(B, H, k_splits))


def forward_inference(Q, K, V, conv_kernel, k_splits, scale, pad_q, pad_k, causal, num_k_blocks=None,
                      offset_causal=False):
    """(O_splits [B,H,k_splits,d], M_splits, L_splits [B,H,k_splits]) fp32 with the merged,
    normalised result in split 0 (fwd_inference.cu:359-368).  ``causal`` is accepted and has no
    effect, exactly as in the reference kernel (fwd_inference.cu:36 is never read);
    ``num_k_blocks`` is accepted for signature compatibility and ignored.  ``offset_causal=True``
    (an addition) applies the training forward's mask with query row r placed at position
    Nk - rows + r, so that the result equals the last row of the causal training forward."""
    for t, n in ((Q, "Q"), (K, "K"), (V, "V")):
        require_cuda_bf16(t, n)
    B, H, q_len, d = Q.shape
    if q_len > 16 or q_len < 1:
        raise RuntimeError("Q sequence length must be between 1 and 16 for inference")
    if K.shape[0] != B or K.shape[1] != H or K.shape[3] != d or V.shape != K.shape:
        raise RuntimeError("K/V must be [batch, heads, seq_len, d_head] matching Q")
    Nk = K.shape[2]
    cq, ck = int(conv_kernel.shape[1]), int(conv_kernel.shape[2])
    if pad_q != cq - 1 or pad_k != (ck - 1) // 2:
        raise RuntimeError("pad_q/pad_k must be (kx-1, (ky-1)//2)")
    if k_splits <= 0:
        raise RuntimeError("k_splits must be positive")
    if k_splits > Nk:
        raise RuntimeError("k_splits cannot be larger than seq_len_k")
    theta = as_f32(conv_kernel)
    O, M, L = _split_outputs(B, H, k_splits, d, Q.device)
    fn = lib.fmta_decode_offset_causal if offset_causal else lib.fmta_decode
    st = fn(ptr(Q), ptr(K), ptr(V), ptr(theta), ptr(O), ptr(M), ptr(L), B, H, q_len, Nk, d, cq, ck,
            int(k_splits), float(scale), stream_ptr())
    check(st, "fmta_decode")
    return O, M, L


def fwd_conv_attn_inference(Q, K, V, conv_kernel, k_splits, scale, pad_q, pad_k, causal, offset_causal=False):
    """(O [B,H,1,d], M [B,H,1], L [B,H,1]) for the last query row
    (flash_conv_attention_inference.py:33-93).  The reference front-pads Q to 16 rows with
    zeros; zero rows contribute nothing, so Q is passed as is."""
    if Q.shape[2] > 16:
        raise ValueError(f"Q sequence length must be <= 16 for inference, got {Q.shape[2]}")
    O, M, L = forward_inference(Q, K, V, conv_kernel, k_splits, scale, pad_q, pad_k, causal,
                                offset_causal=offset_causal)
    return O[:, :, 0:1, :], M[:, :, 0:1], L[:, :, 0:1]


def forward_inference_paged(Q, K_pool, V_pool, block_table, conv_kernel, k_splits, scale, pad_q, pad_k,
                            seq_lens=None, max_seq_len=None, offset_causal=False):
    """Decode over a paged key/value cache (an addition: the reference cache is contiguous).
    ``K_pool``/``V_pool`` bf16 [n_pages, H, page_size, d]; ``block_table`` int32 [B, max_pages] maps
    page p of sequence b to a pool page; ``seq_lens`` int32 [B] (optional) gives each sequence's
    cache length, bounded by ``max_seq_len`` (default: max_pages * page_size).  Returns
    (O_splits, M_splits, L_splits) as ``forward_inference``; equals ``forward_inference`` on the
    gathered cache."""
    for t, n in ((Q, "Q"), (K_pool, "K_pool"), (V_pool, "V_pool")):
        require_cuda_bf16(t, n)
    B, H, q_len, d = Q.shape
    if q_len > 16 or q_len < 1:
        raise RuntimeError("Q sequence length must be between 1 and 16 for inference")
    if K_pool.dim() != 4 or K_pool.shape[1] != H or K_pool.shape[3] != d or V_pool.shape != K_pool.shape:
        raise RuntimeError("K_pool/V_pool must be [n_pages, heads, page_size, d_head] matching Q")
    page_size = int(K_pool.shape[2])
    if block_table.dtype != torch.int32 or not block_table.is_cuda or not block_table.is_contiguous() \
            or block_table.dim() != 2 or block_table.shape[0] != B:
        raise RuntimeError("block_table must be a contiguous CUDA int32 tensor [batch, max_pages]")
    max_pages = int(block_table.shape[1])
    if seq_lens is not None and (seq_lens.dtype != torch.int32 or not seq_lens.is_cuda or seq_lens.numel() != B):
        raise RuntimeError("seq_lens must be a CUDA int32 tensor [batch]")
    Nk = int(max_seq_len) if max_seq_len is not None else max_pages * page_size
    cq, ck = int(conv_kernel.shape[1]), int(conv_kernel.shape[2])
    if pad_q != cq - 1 or pad_k != (ck - 1) // 2:
        raise RuntimeError("pad_q/pad_k must be (kx-1, (ky-1)//2)")
    theta = as_f32(conv_kernel)
    O, M, L = _split_outputs(B, H, k_splits, d, Q.device)
    st = lib.fmta_decode_paged(ptr(Q), ptr(K_pool), ptr(V_pool), ptr(block_table), ptr(seq_lens), ptr(theta), ptr(O),
                               ptr(M), ptr(L), B, H, q_len, Nk, d, cq, ck, int(k_splits), float(scale), page_size,
                               max_pages, int(bool(offset_causal)), stream_ptr())
    check(st, "fmta_decode_paged")
    return O, M, L


def kv_append_paged(K_pool, V_pool, block_table, seq_lens, K_new, V_new):
    """Write ``K_new``/``V_new`` (bf16 [B,H,n_new,d]) at positions seq_lens[b] .. seq_lens[b]+n_new-1 of
    each sequence of a paged cache.  ``seq_lens`` is read, not advanced; the pages must already be in
    ``block_table``."""
    for t, n in ((K_pool, "K_pool"), (V_pool, "V_pool"), (K_new, "K_new"), (V_new, "V_new")):
        require_cuda_bf16(t, n)
    B, H, n_new, d = K_new.shape
    st = lib.fmta_kv_append_paged(ptr(K_pool), ptr(V_pool), ptr(block_table), ptr(seq_lens), ptr(K_new), ptr(V_new),
                                  B, H, n_new, d, int(K_pool.shape[2]), int(block_table.shape[1]), stream_ptr())
    check(st, "fmta_kv_append_paged")
