// Instantiations and launcher of the decode kernel and the split combine.
#include "decode.cuh"
#include "launch_util.cuh"

namespace fmta {

cudaError_t launch_decode(const DecodeParams& p, cudaStream_t stream) {
  dim3 grid(p.k_splits, p.H, p.B), block(kDecWarps * 32);
  ScopedKernelTimer* timer_ = new ScopedKernelTimer(kKernDecode, stream);
  const int rows = p.q_len < p.cq ? p.q_len : p.cq;
  const bool r16 = rows > 8;
  const bool paged = p.block_table != nullptr;
#define FMTA_DEC(DD)                                                                 \
  if (p.d == DD) {                                                                   \
    if (paged) {                                                                     \
      if (r16) decode_kernel<DD, true, true><<<grid, block, 0, stream>>>(p);         \
      else decode_kernel<DD, false, true><<<grid, block, 0, stream>>>(p);            \
    } else {                                                                         \
      if (r16) decode_kernel<DD, true, false><<<grid, block, 0, stream>>>(p);        \
      else decode_kernel<DD, false, false><<<grid, block, 0, stream>>>(p);           \
    }                                                                                \
  }
  FMTA_DEC(32) else FMTA_DEC(64) else FMTA_DEC(128) else return cudaErrorInvalidValue;
#undef FMTA_DEC
  cudaError_t e = cudaGetLastError();
  delete timer_;   // stop event right after the decode kernel, before the combine
  if (e != cudaSuccess) return e;
  combine_splits_kernel<<<p.B * p.H, 128, 0, stream>>>(p.O_splits, p.M_splits, p.L_splits, p.k_splits, p.d);
  return cudaGetLastError();
}

cudaError_t launch_kv_append_paged(void* Kpool, void* Vpool, const int* block_table, const int* seq_lens,
                                   const void* Knew, const void* Vnew, int B, int H, int n_new, int d, int page_size,
                                   int page_shift, int max_pages, cudaStream_t stream) {
  const int chunks = n_new * (d / 8);
  dim3 grid((chunks + 127) / 128, H, B), block(128);
  bf16* kp = reinterpret_cast<bf16*>(Kpool); bf16* vp = reinterpret_cast<bf16*>(Vpool);
  const bf16* kn = reinterpret_cast<const bf16*>(Knew); const bf16* vn = reinterpret_cast<const bf16*>(Vnew);
  if (d == 32) kv_append_paged_kernel<32><<<grid, block, 0, stream>>>(kp, vp, block_table, seq_lens, kn, vn, H, n_new, page_size, page_shift, max_pages);
  else if (d == 64) kv_append_paged_kernel<64><<<grid, block, 0, stream>>>(kp, vp, block_table, seq_lens, kn, vn, H, n_new, page_size, page_shift, max_pages);
  else if (d == 128) kv_append_paged_kernel<128><<<grid, block, 0, stream>>>(kp, vp, block_table, seq_lens, kn, vn, H, n_new, page_size, page_shift, max_pages);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

}  // namespace fmta
