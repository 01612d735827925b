// Instantiations and launcher of the exact dK / dV backward kernel.
#include "bwd_exact.cuh"
#include "launch_util.cuh"

namespace fmta {

template <int D, int CQ, int CK>
static cudaError_t launch_bwd_dkdv_t(const TrainParams& p, cudaStream_t stream) {
  const int own = 64;
  const int nKB = (p.N + own - 1) / own;
  dim3 grid(nKB, p.H, p.B), block(256);
  const bool mix = (p.Wmix != nullptr) && p.G > 1;
  if (mix) {
    if constexpr (CQ == 3) {
      return cudaErrorInvalidValue;
    } else {
      using Cfg = BwdExactCfg<D, CQ, CK, true>;
      return launch_kernel<TrainParams>(bwd_dkdv_kernel<D, CQ, CK, true>, grid, block, Cfg::kSmemBytes, stream, p.G, p);
    }
  }
  using Cfg = BwdExactCfg<D, CQ, CK, false>;
  return launch_kernel<TrainParams>(bwd_dkdv_kernel<D, CQ, CK, false>, grid, block, Cfg::kSmemBytes, stream, 1, p);
}

cudaError_t launch_bwd_dkdv(const TrainParams& p, cudaStream_t stream) {
  ScopedKernelTimer timer_(kKernBwdDkdvExact, stream);
  if (hm_dense_supported(p)) return launch_hm_bwd_dkdv(p, stream);   // head mix without a conv: all heads of a group in one CTA
  const bool mix = (p.Wmix != nullptr) && p.G > 1;
  int cq = p.cq, ck = p.ck;
  const bool has_theta = p.theta != nullptr;
  if (mix && cq == 3 && ck == 5) { cq = -1; }
  FMTA_DISPATCH_D(p.d, FMTA_DISPATCH_CONV(cq, ck, has_theta, return launch_bwd_dkdv_t<D_, CQ_, CK_>(p, stream);););
  return cudaErrorInvalidValue;
}

}  // namespace fmta
