// Instantiations and launcher of the exact dQ / dTheta / dW backward kernel, plus the small
// helper kernels of the backward (partial reduction, D = rowsum(dO*O)).
#include "bwd_exact.cuh"
#include "launch_util.cuh"

namespace fmta {

// Sum per-slot partials: out[i] = sum_s part[s * n + i].  32 outputs per CTA, 8 threads per output;
// thread k adds the slots s = k, k+8, ... in order, then the 8 sub-sums are added in order of k:
// a fixed summation tree, so the result is bit-reproducible.
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ part, float* __restrict__ out,
                                                              int n_slots, int n) {
  __shared__ float sSub[8][33];
  const int col = threadIdx.x & 31, k = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + col;
  float t = 0.f;
  pdl_wait();                                          // launched with programmatic stream serialization
  if (i < n)
    for (int s = k; s < n_slots; s += 8) t += part[(size_t)s * n + i];
  sSub[k][col] = t;
  __syncthreads();
  if (k == 0 && i < n) {
    float r = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q) r += sSub[q][col];
    out[i] = r;
  }
}

// D[row] = sum_d dO[row,d] * O[row,d]; one warp per row.  O may be fp32 or bf16.
template <bool O_BF16>
__global__ void rowdot_kernel(const bf16* __restrict__ dO, const void* __restrict__ O, float* __restrict__ Dv, size_t rows, int d) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  float t = 0.f;
  for (int c = lane * 2; c < d; c += 64) {
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dO + row * d + c);
    float o0, o1;
    if (O_BF16) {
      const __nv_bfloat162 o = *reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const bf16*>(O) + row * d + c);
      o0 = __low2float(o); o1 = __high2float(o);
    } else {
      const float2 o = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(O) + row * d + c);
      o0 = o.x; o1 = o.y;
    }
    t = fmaf(__low2float(g), o0, t);
    t = fmaf(__high2float(g), o1, t);
  }
  t = warp_sum(t);
  if (lane == 0) Dv[row] = t;
}

// The same with TPR = d / 8 threads per row, 16 bytes of dO (and 16 or 32 of O) per thread: one load
// instruction per operand and thread, 256 / TPR rows per block.
template <bool O_BF16, int TPR>
__global__ void __launch_bounds__(256) rowdot_vec_kernel(const bf16* __restrict__ dO, const void* __restrict__ O,
                                                         float* __restrict__ Dv, size_t rows) {
  constexpr int D = TPR * 8;
  const size_t row = (size_t)blockIdx.x * (256 / TPR) + threadIdx.x / TPR;
  const int c = (threadIdx.x % TPR) * 8;
  float t = 0.f;
  pdl_trigger();
  pdl_wait();                                          // launched with programmatic stream serialization
  if (row < rows) {
    const uint4 g = *reinterpret_cast<const uint4*>(dO + row * D + c);
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
    float o[8];
    if (O_BF16) {
      const uint4 ov = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(O) + row * D + c);
      const uint32_t ow[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { o[2 * e] = __uint_as_float(ow[e] << 16); o[2 * e + 1] = __uint_as_float(ow[e] & 0xffff0000u); }
    } else {
      const float4 o0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(O) + row * D + c);
      const float4 o1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(O) + row * D + c + 4);
      o[0] = o0.x; o[1] = o0.y; o[2] = o0.z; o[3] = o0.w; o[4] = o1.x; o[5] = o1.y; o[6] = o1.z; o[7] = o1.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      t = fmaf(__uint_as_float(gw[e] << 16), o[2 * e], t);
      t = fmaf(__uint_as_float(gw[e] & 0xffff0000u), o[2 * e + 1], t);
    }
  }
#pragma unroll
  for (int off = TPR / 2; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
  if (row < rows && c == 0) Dv[row] = t;
}

template <int D, int CQ, int CK>
static cudaError_t launch_bwd_dq_t(const TrainParams& p, cudaStream_t stream) {
  const int own = 64;
  const int nQB = (p.N + own - 1) / own;
  dim3 grid(nQB, p.H, p.B), block(256);
  const bool mix = (p.Wmix != nullptr) && p.G > 1;
  if (mix) {
    if constexpr (CQ == 3) {
      return cudaErrorInvalidValue;
    } else {
      using Cfg = BwdExactCfg<D, CQ, CK, true>;
      return launch_kernel<TrainParams>(bwd_dq_kernel<D, CQ, CK, true>, grid, block, Cfg::kSmemBytes, stream, p.G, p);
    }
  }
  using Cfg = BwdExactCfg<D, CQ, CK, false>;
  return launch_kernel<TrainParams>(bwd_dq_kernel<D, CQ, CK, false>, grid, block, Cfg::kSmemBytes, stream, 1, p);
}

cudaError_t launch_bwd_dq(const TrainParams& p, cudaStream_t stream) {
  ScopedKernelTimer timer_(kKernBwdDqExact, stream);
  if (hm_dense_supported(p)) return launch_hm_bwd_dq(p, stream);   // head mix without a conv: all heads of a group in one CTA
  const bool mix = (p.Wmix != nullptr) && p.G > 1;
  int cq = p.cq, ck = p.ck;
  const bool has_theta = p.theta != nullptr;
  if (mix && cq == 3 && ck == 5) { cq = -1; }
  FMTA_DISPATCH_D(p.d, FMTA_DISPATCH_CONV(cq, ck, has_theta, return launch_bwd_dq_t<D_, CQ_, CK_>(p, stream);););
  return cudaErrorInvalidValue;
}

cudaError_t launch_reduce_partials(const float* part, float* out, int n_slots, int n, cudaStream_t stream) {
  return launch_pdl(reduce_partials_kernel, dim3((n + 31) / 32), dim3(256), 0, stream, part, out, n_slots, n);
}

cudaError_t launch_rowdot(const void* dO, const void* O, int o_bf16, float* Dv, size_t rows, int d, cudaStream_t stream) {
  const bf16* g = reinterpret_cast<const bf16*>(dO);
#define FMTA_ROWDOT(TPR)                                                                                   \
  { const unsigned nb = (unsigned)((rows + 256 / TPR - 1) / (256 / TPR));                                  \
    if (o_bf16) return launch_pdl(rowdot_vec_kernel<true, TPR>, dim3(nb), dim3(256), 0, stream, g, O, Dv, rows);      \
    return launch_pdl(rowdot_vec_kernel<false, TPR>, dim3(nb), dim3(256), 0, stream, g, O, Dv, rows); }
  const bool al = (reinterpret_cast<uintptr_t>(dO) % 16 == 0) && (reinterpret_cast<uintptr_t>(O) % 16 == 0);
  if (al && d == 64) FMTA_ROWDOT(8)
  if (al && d == 128) FMTA_ROWDOT(16)
  if (al && d == 32) FMTA_ROWDOT(4)
#undef FMTA_ROWDOT
  const unsigned blocks = (unsigned)((rows + 7) / 8);
  if (o_bf16) rowdot_kernel<true><<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(dO), O, Dv, rows, d);
  else rowdot_kernel<false><<<blocks, 256, 0, stream>>>(reinterpret_cast<const bf16*>(dO), O, Dv, rows, d);
  return cudaGetLastError();
}

}  // namespace fmta
