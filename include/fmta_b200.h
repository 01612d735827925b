/*
 * fmta_b200 - C ABI of the B200-native fused multi-token (conv) attention hot path.
 *
 * One shared library (libfmta_b200.so), plain pointers and sizes, no torch types.  Each entry
 * point is what a binding of the reference package would call in place of one of its pybind11
 * functions; the reference interface it replaces is cited beside it (paths are relative to the
 * reference checkout).
 *
 * Conventions
 *   - every tensor pointer is DEVICE memory, contiguous, row-major in the stated shape;
 *     Q/K/V/dO are bf16 (the reference contract, fwd_wrapper.cu:30-33), theta / W / LSE / D
 *     are fp32 (the reference rounds them to bf16, conv_attention_cuda.py:77,115,144; this
 *     library does not);
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing
 *     synchronises the device (the reference launches on the legacy default stream and
 *     device-synchronises in decode, fwd_inference.cu:425);
 *   - return value 0 = enqueued; negative = rejected on the host, nothing was launched
 *     (see fmta_strerror).  Launch errors reported by the CUDA runtime map to FMTA_ERR_CUDA;
 *   - the callee allocates nothing unless stated; workspaces are caller-owned and sized by
 *     fmta_workspace_bytes;
 *   - supported head dims: 32, 64, 128.  Filter shapes: any c_q in [1,16], odd c_k in [1,17]
 *     (c_k must be odd: the reference's own PyTorch path fails for even c_k);
 *   - head mixing: G consecutive heads form a group mixed by a G x G matrix
 *     (W layout [H/G, G, G], row = output head); G in {1,2,4,8,16}, H % G == 0; G = 32 as well when
 *     theta is NULL and d <= 64 (the reference's head-conv operator accepts 16 or 32 heads,
 *     head_conv_attn/fwd_kernel.py:300).
 */
#ifndef FMTA_B200_H_
#define FMTA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FMTA_OK 0
#define FMTA_ERR_NULL (-1)        /* a required pointer is NULL */
#define FMTA_ERR_SHAPE (-2)       /* a dimension is out of range or inconsistent */
#define FMTA_ERR_UNSUPPORTED (-3) /* head dim / filter shape / group size not supported */
#define FMTA_ERR_ALIGN (-4)       /* a pointer is not 16-byte aligned */
#define FMTA_ERR_WORKSPACE (-5)   /* workspace missing or too small */
#define FMTA_ERR_CUDA (-6)        /* the CUDA runtime rejected a launch (see fmta_last_cuda_error) */
#define FMTA_ERR_SCRATCH_LIMIT (-7) /* problem needs more than FMTA_STATIC_SCRATCH_BYTES of built-in scratch */
#define FMTA_ERR_DEVICE_WAIT (-8) /* a bounded wait inside a kernel ran out (status word, see fmta_set_status_word) */

/* Size of the library's built-in scratch array used by fmta_bwd_dq_dw_static (4 MiB per GPU). */
#define FMTA_STATIC_SCRATCH_BYTES ((size_t)4 << 20)

#define FMTA_DTYPE_F32 0
#define FMTA_DTYPE_BF16 1

#define FMTA_OP_BWD_DQ 1 /* for fmta_workspace_bytes */
#define FMTA_OP_FWD_TC 2
#define FMTA_OP_BWD_TC 3
#define FMTA_OP_BWD_TC_STREAM 4 /* FMTA_OP_BWD_TC plus room for P and dC (bf16, 4 * B*H*N*roundup(N,128) bytes) */
/* OPTIONAL scratch of a head mix that follows a key-query conv (theta and wmix both given): with it the heads
 * of a group exchange their score tiles through global memory (L2), about 1.5x faster than through distributed
 * shared memory.  fmta_fwd: a workspace of this size; fmta_bwd_dq_dw and fmta_bwd (path 0): this size behind the
 * FMTA_OP_BWD_DQ bytes rounded up to 256.  A smaller workspace is not an error. */
#define FMTA_OP_MIX_EXCHANGE 5

/* Library version (major*10000 + minor*100 + patch). */
int fmta_version(void);

/* Text for a status code returned by any entry point. */
const char* fmta_strerror(int status);

/*
 * Process-wide kernel selection for the entry points that have no `path` argument:
 * -1 = library default, 0 = exact tile kernels only, 1 = tensor-core kernels off the causal band
 * plus exact kernels on it.  Returns the previous value.
 */
int fmta_set_path(int path);

/*
 * Failure detection.  Every wait inside the tensor-core kernels (on an mbarrier fed by TMA, by the
 * tensor cores or by other warps) is bounded; a kernel whose wait runs out stops issuing work, waits
 * (bounded) for what it has in flight, frees its tensor memory and sets a status word, and the
 * outputs of that call are invalid.  The reference has no counterpart (its forward only prints a
 * launch error, conv_attn/kernels/fwd.cu:306-309; its backward throws on one, dq_bwd.cu:585-586).
 * fmta_set_status_word registers, for the CURRENT device, a caller-owned int32 in device memory
 * (zeroed by the caller); from then on the tensor-core kernels of every entry point set that word
 * themselves when a wait of theirs runs out.  The caller reads the word after a synchronisation it does
 * anyway: non-zero = FMTA_ERR_DEVICE_WAIT.  NULL unregisters.  Process-wide per device, not thread-safe.
 */
int fmta_set_status_word(int* device_word);

/*
 * Self-test of the above: the next launch of the named tensor-core kernel (ids as in
 * fmta_profile_kernel: 1 forward, 3 dQ, 4 dK/dV; 0 cancels) points its first consumer wait at a
 * barrier that nothing arrives at, with a limit of a few hundred polls, so that the wait runs out
 * and the kernel takes its abort path.  Nothing faults or spins without bound; the call's outputs
 * are garbage and the status word reads non-zero.
 */
int fmta_selftest_expire_next(int kernel_id);

/*
 * Timing hook for benchmarks: while armed, every launch of the chosen kernel is bracketed by
 * cudaEventRecord(start) / cudaEventRecord(stop) on the launch stream, so a caller can time one
 * kernel inside a multi-kernel entry point.  kernel_id: 1 fwd tensor-core, 2 fwd exact, 3 dQ
 * tensor-core, 4 dK/dV tensor-core, 5 dQ exact, 6 dK/dV exact, 7 decode, 8 backward band,
 * 9 stacked-key pre-pass (last launch of the call), 10 its adjoint;
 * 0 disarms.  The events
 * are cudaEvent_t handles owned by the caller.  Not thread-safe; meant for single-threaded benches.
 */
int fmta_profile_kernel(int kernel_id, void* start_event, void* stop_event);

/* cudaError_t value of the last launch failure seen by this thread (0 if none). */
int fmta_last_cuda_error(void);

/*
 * Forward.  Replaces `forward(Q,K,V,conv_kernel,scale,pad_q,pad_k,causal) -> (O,M,L)`
 * (conv_attn/bindings.cpp:46-48, kernels/fwd_wrapper.cu:15-100) and, with `wmix`,
 * `head_conv_attention_forward(q,k,v,w,scale,causal) -> (o,l,m)` (head_conv_attn/fwd_kernel.py:282).
 *   Q,K,V  bf16 [B,H,N,d]      theta fp32 [H,cq,ck] or NULL (no key-query conv)
 *   wmix   fp32 [H/G,G,G] or NULL     O [B,H,N,d] fp32 or bf16 (o_dtype)
 *   M,L    fp32 [B,H,N] row max / row sum of exp(C-M), either may be NULL
 *   LSE    fp32 [B,H,N] = M + log L, may be NULL
 * path: 0 = exact tile kernel everywhere; 1 = stacked-GEMM tensor-core kernel off the causal
 * band plus the band kernel on it (needs workspace, see FMTA_OP_FWD_TC); -1 = library default.
 */
int fmta_fwd(const void* Q, const void* K, const void* V, const float* theta, const float* wmix,
             void* O, float* M, float* L, float* LSE, int B, int H, int N, int d, int cq, int ck,
             int G, float scale, int causal, int o_dtype, int path, void* workspace,
             size_t workspace_bytes, void* stream);

/*
 * D[b,h,i] = sum_d dO[b,h,i,:] * O[b,h,i,:], kept in fp32.  Replaces the torch expression at
 * conv_attention_cuda.py:144 (which rounds D to bf16).  rows = B*H*N.
 */
int fmta_bwd_prep_D(const void* dO, const void* O, int o_dtype, float* D, size_t rows, int d,
                    void* stream);

/*
 * dQ and the filter / mixing gradients.  Replaces `dq_backward(Q,K,V,dO,D,L,conv_kernel,...) ->
 * (dQ, dconv_kernel)` (conv_attn/bindings.cpp:50-52, kernels/dq_bwd_wrapper.cu:11-93; its `L`
 * argument is LSE) and `head_conv_attention_bwd_dq_dw` (head_conv_attn/bwd_dq_dw.py:373).
 *   dQ fp32 [B,H,N,d]   dTheta fp32 [H,cq,ck] (NULL when theta is NULL)
 *   dW fp32 [H/G,G,G] (NULL when wmix is NULL)
 * dTheta and dW are summed over the batch in a fixed order (per-CTA partials in `workspace`,
 * then one reduction), so repeated calls give bit-identical results.
 */
int fmta_bwd_dq_dw(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                   const float* LSE, const float* theta, const float* wmix, float* dQ,
                   float* dTheta, float* dW, int B, int H, int N, int d, int cq, int ck, int G,
                   float scale, int causal, void* workspace, size_t workspace_bytes, void* stream);

/*
 * dK and dV.  Replaces `dkdv_backward(...) -> (dK, dV)` (conv_attn/bindings.cpp:54-56,
 * kernels/dkdv_wrapper.cu:12-89) and `head_conv_attention_bwd_dkdv` (head_conv_attn/bwd_dk_dv.py:407).
 */
int fmta_bwd_dkdv(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                  const float* LSE, const float* theta, const float* wmix, float* dK, float* dV,
                  int B, int H, int N, int d, int cq, int ck, int G, float scale, int causal,
                  void* stream);

/*
 * Whole backward in one call: dQ, dK, dV, dTheta (and dW).  Replaces the pair of calls made by
 * `FlashConvAttentionCUDAFunction.backward` (conv_attn/conv_attention_cuda.py:147-152).
 * path: 0 = exact tile kernels; 1 = stacked-GEMM tensor-core kernels for the entries off the
 * causal band + the band kernel (accumulating) on the band -- needs d = 64 with c_q <= 7 or d = 128 with c_q <= 6, no head
 * mixing, and a workspace of fmta_workspace_bytes(FMTA_OP_BWD_TC, ...); -1 = the process-wide
 * default (fmta_set_path), which picks 1 whenever it is available and the workspace suffices.
 * With path 0 the workspace need is that of FMTA_OP_BWD_DQ.
 * Head dim 64 with a workspace of fmta_workspace_bytes(FMTA_OP_BWD_TC_STREAM, ...) or more: the dQ kernel
 * leaves the probabilities P and dC = P (dP - D) of every entry off the causal band in the workspace (bf16),
 * and the dK/dV kernel streams them through two accumulating GEMMs instead of recomputing scores and
 * exponentials (4*B*H*N^2 bytes: 1 GiB per 16 (batch, head) pairs at N = 4096) -- an option: on B200 the
 * recomputing pair is as fast or faster at every size measured, so pass the plain FMTA_OP_BWD_TC size unless
 * measurement says otherwise; same numbers as the recomputing kernel (it rounds P and dC to bf16 too).
 */
int fmta_bwd(const void* Q, const void* K, const void* V, const void* dO, const float* D,
             const float* LSE, const float* theta, const float* wmix, float* dQ, float* dK, float* dV,
             float* dTheta, float* dW, int B, int H, int N, int d, int cq, int ck, int G, float scale,
             int causal, int path, void* workspace, size_t workspace_bytes, void* stream);

/*
 * Forward / backward pair that shares the stacked key operand (no counterpart in the reference, whose
 * backward recomputes everything from Q, K, V).  The tensor-core kernels read keys through
 * Ktilde[b,h,t,j,:] = scale * log2(e) * sum_u theta[h,t,u] * K[b,h,j-u,:] (bf16 [B,H,cq,N,d], written by a
 * pre-pass).  fmta_fwd and fmta_bwd each run that pre-pass into their own workspace; a training step that calls
 * fmta_fwd_keep_ktilde instead leaves the operand in the caller's buffer `ktilde` (B*H*cq*N*d*2 bytes, 16-byte
 * aligned), and fmta_bwd_with_ktilde reads it back and skips the second pre-pass.  The caller guarantees that K,
 * theta and scale are unchanged in between; the results are bit-identical to fmta_fwd / fmta_bwd with path 1.
 * Tensor-core path only: the shapes fmta_fwd / fmta_bwd accept with path = 1 (theta given, no head mixing) and
 * the same workspace sizes (FMTA_OP_FWD_TC / FMTA_OP_BWD_TC or FMTA_OP_BWD_TC_STREAM); anything else returns
 * FMTA_ERR_UNSUPPORTED or FMTA_ERR_WORKSPACE.
 */
int fmta_fwd_keep_ktilde(const void* Q, const void* K, const void* V, const float* theta, void* O, float* M, float* L,
                         float* LSE, int B, int H, int N, int d, int cq, int ck, float scale, int causal, int o_dtype,
                         void* workspace, size_t workspace_bytes, void* ktilde, void* stream);
int fmta_bwd_with_ktilde(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                         const float* LSE, const float* theta, float* dQ, float* dK, float* dV, float* dTheta,
                         int B, int H, int N, int d, int cq, int ck, float scale, int causal, void* workspace,
                         size_t workspace_bytes, const void* ktilde, void* stream);

/*
 * One window of sequence positions of a forward / backward (no counterpart in the reference, which has no
 * sequence parallelism): the building block of context-parallel training and prefill, where every GPU holds the
 * whole Q, K, V (dO, D, LSE) of its (batch, head) pairs -- gathered over NVLink -- and computes one or two
 * windows of the sequence.  [row_lo, row_hi) starts on a multiple of 256 and ends on one or at N.
 *   fmta_fwd_window: writes O, M, L, LSE of the query rows in the window and touches no other row.  Reads Q from
 *     row_lo - pad_q on and, with a causal mask, K and V up to row_hi + pad_k.
 *   fmta_bwd_window: writes dQ of the query rows in the window, dK and dV of the KEYS in the window (each from all
 *     the query rows that see them, so D and LSE must be complete), and in dTheta the window's share: the shares of
 *     disjoint windows that cover [0, N) add up to the dTheta of fmta_bwd.  No other row of dQ, dK, dV is touched.
 * Tensor-core path only (theta given, the shapes of fmta_fwd / fmta_bwd with path = 1), with the workspace of the
 * whole problem (FMTA_OP_FWD_TC / FMTA_OP_BWD_TC).  ktilde: NULL, or the stacked key operand of the whole sequence
 * (bf16 [B,H,cq,N,d]) made once by fmta_stacked_keys for these K, theta and scale -- every window call otherwise
 * repeats that O(N) pre-pass.  The windows of one sequence computed one after the other into the
 * same buffers give the results of fmta_fwd / fmta_bwd (dQ to rounding: its row tiles start at the window).
 */
int fmta_stacked_keys(const void* K, const float* theta, void* ktilde, int B, int H, int N, int d, int cq, int ck,
                      float scale, void* stream);
int fmta_fwd_window(const void* Q, const void* K, const void* V, const float* theta, void* O, float* M, float* L,
                    float* LSE, int B, int H, int N, int d, int cq, int ck, float scale, int causal, int o_dtype,
                    int row_lo, int row_hi, const void* ktilde, void* workspace, size_t workspace_bytes, void* stream);
int fmta_bwd_window(const void* Q, const void* K, const void* V, const void* dO, const float* D, const float* LSE,
                    const float* theta, float* dQ, float* dK, float* dV, float* dTheta, int B, int H, int N, int d,
                    int cq, int ck, float scale, int causal, int row_lo, int row_hi, const void* ktilde, void* workspace,
                    size_t workspace_bytes, void* stream);

/*
 * Decode: last query row over a KV cache with split-K.  Replaces
 * `forward_inference(Q,K,V,conv_kernel,k_splits,scale,pad_q,pad_k,causal,num_k_blocks) ->
 * (O_splits,M_splits,L_splits)` (conv_attn/fwd_inference_bindings.cpp:20-23,
 * kernels/fwd_inference_wrapper.cu:13-120).  As there, scores are rectangular (q_len recent
 * query rows x Nk keys), no causal mask is applied, and the merged, normalised result is left in
 * split 0; the other splits hold un-normalised partials.
 *   Q bf16 [B,H,q_len,d] (1 <= q_len <= 16; no padding to 16 rows is needed)
 *   K,V bf16 [B,H,Nk,d]   theta fp32 [H,cq,ck]
 *   O_splits fp32 [B,H,k_splits,d]   M_splits, L_splits fp32 [B,H,k_splits]
 */
int fmta_decode(const void* Q, const void* K, const void* V, const float* theta, float* O_splits,
                float* M_splits, float* L_splits, int B, int H, int q_len, int Nk, int d, int cq,
                int ck, int k_splits, float scale, void* stream);

/*
 * Decode with the causal mask of the training forward ("offset-causal").  No counterpart in the
 * reference, whose decode kernel accepts `causal` and never reads it (kernels/fwd_inference.cu:36).
 * Query row r of the `rows = min(q_len, c_q)` most recent rows sits at sequence position
 * Nk - rows + r; the score of a key later than that position is set to zero before the conv,
 * exactly as the training forward zeroes future scores.  With q_len >= min(c_q, Nk) the merged
 * result in split 0 equals row Nk-1 of `fmta_fwd` (causal) over the same Nk-long sequence.
 * Arguments and outputs as `fmta_decode`.
 */
int fmta_decode_offset_causal(const void* Q, const void* K, const void* V, const float* theta, float* O_splits,
                              float* M_splits, float* L_splits, int B, int H, int q_len, int Nk, int d, int cq,
                              int ck, int k_splits, float scale, void* stream);

/*
 * Decode over a PAGED key/value cache (no counterpart in the reference, whose cache is one
 * contiguous [B,H,Nk,d] tensor).  K_pool / V_pool are bf16 [n_pages, H, page_size, d]; page p of
 * sequence b is pool page block_table[b * max_pages + p] (int32).  page_size is a power of two
 * >= 16, max_pages <= 2048.  seq_lens (int32 [B], device memory, may be NULL) gives the cache
 * length of each sequence (>= 1); without it every sequence has Nk_max keys.  Nk_max bounds the
 * lengths (max_pages * page_size >= Nk_max).  offset_causal as in fmta_decode_offset_causal.
 * Outputs as `fmta_decode`.  The result is that of `fmta_decode` on the gathered cache.
 */
int fmta_decode_paged(const void* Q, const void* K_pool, const void* V_pool, const int* block_table,
                      const int* seq_lens, const float* theta, float* O_splits, float* M_splits,
                      float* L_splits, int B, int H, int q_len, int Nk_max, int d, int cq, int ck,
                      int k_splits, float scale, int page_size, int max_pages, int offset_causal,
                      void* stream);

/*
 * Incremental append to a paged cache (no reference counterpart): rows K_new / V_new, bf16
 * [B,H,n_new,d], go to positions seq_lens[b] .. seq_lens[b] + n_new - 1 of sequence b; the pages
 * they land on must already be listed in block_table.  seq_lens is read, not advanced.
 */
int fmta_kv_append_paged(void* K_pool, void* V_pool, const int* block_table, const int* seq_lens,
                         const void* K_new, const void* V_new, int B, int H, int n_new, int d,
                         int page_size, int max_pages, void* stream);

/*
 * Allocation-free variant of fmta_bwd_dq_dw (no counterpart in the reference, whose wrappers
 * always allocate with torch).  Same arguments without the workspace: the per-CTA partial sums
 * of dTheta / dW go to a 4 MiB array that lives inside the library's device image.  Meant for
 * callers that cannot allocate device memory at the call site -- a serving loop whose memory
 * pool is frozen, a host framework that owns the whole GPU, a foreign-language binding with no
 * allocator to hand -- and so cannot provide the workspace of fmta_bwd_dq_dw.  The function
 * itself calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - limit: fmta_workspace_bytes(FMTA_OP_BWD_DQ, ...) must not exceed
 *     FMTA_STATIC_SCRATCH_BYTES, i.e. B * ceil(N/64) * (H*cq*ck + H*G) * 4 <= 4 MiB (the bf16
 *     training shape B=4,H=16,N=4096,(6,11) needs 1.03 MiB); larger problems return
 *     FMTA_ERR_SCRATCH_LIMIT and launch nothing;
 *   - the first call on each device looks up the array's device address (one
 *     cudaGetSymbolAddress with that device current); make that first call outside any
 *     stream capture;
 *   - all calls on a device share the one array.  It keeps the previous call's contents, which
 *     is harmless because every slot is rewritten before it is read, but two calls whose kernels
 *     overlap on the GPU (different streams, or different host threads) race on it: serialise
 *     them.  The array occupies 4 MiB on every GPU that loads the library, until the process ends.
 */
int fmta_bwd_dq_dw_static(const void* Q, const void* K, const void* V, const void* dO,
                          const float* D, const float* LSE, const float* theta, const float* wmix,
                          float* dQ, float* dTheta, float* dW, int B, int H, int N, int d, int cq,
                          int ck, int G, float scale, int causal, void* stream);

/* Bytes of caller-owned workspace an op needs for the given problem (0 if none). */
size_t fmta_workspace_bytes(int op, int B, int H, int N, int d, int cq, int ck, int G);

#ifdef __cplusplus
}
#endif
#endif /* FMTA_B200_H_ */
