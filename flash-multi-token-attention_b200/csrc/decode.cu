// Instantiations and launcher of the decode kernel and the split combine.
#include "decode.cuh"
#include "launch_util.cuh"

namespace fmta {

cudaError_t launch_decode(const DecodeParams& p, cudaStream_t stream) {
  dim3 grid(p.k_splits, p.H, p.B), block(kDecWarps * 32);
  ScopedKernelTimer* timer_ = new ScopedKernelTimer(kKernDecode, stream);
  const int rows = p.q_len < p.cq ? p.q_len : p.cq;
  const bool r16 = rows > 8;
#define FMTA_DEC(DD)                                                      \
  if (p.d == DD) {                                                        \
    if (r16) decode_kernel<DD, true><<<grid, block, 0, stream>>>(p);      \
    else decode_kernel<DD, false><<<grid, block, 0, stream>>>(p);         \
  }
  FMTA_DEC(32) else FMTA_DEC(64) else FMTA_DEC(128) else return cudaErrorInvalidValue;
#undef FMTA_DEC
  cudaError_t e = cudaGetLastError();
  delete timer_;   // stop event right after the decode kernel, before the combine
  if (e != cudaSuccess) return e;
  combine_splits_kernel<<<p.B * p.H, 128, 0, stream>>>(p.O_splits, p.M_splits, p.L_splits, p.k_splits, p.d);
  return cudaGetLastError();
}

}  // namespace fmta
