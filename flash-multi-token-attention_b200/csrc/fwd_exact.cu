// Instantiations and launcher of the exact forward tile kernel.
#include "fwd_exact.cuh"
#include "launch_util.cuh"

namespace fmta {

template <int D, int CQ, int CK>
static cudaError_t launch_fwd_exact_t(const TrainParams& p, cudaStream_t stream) {
  const int own = 64;
  const int nQB = (p.N + own - 1) / own;
  dim3 grid(nQB, p.H, p.B), block(256);
  const bool mix = (p.Wmix != nullptr) && p.G > 1;
  if (mix) {
    if constexpr (CQ == 3) {
      return cudaErrorInvalidValue;  // unreachable: the dispatcher routes mixed (3,5) to the run-time path
    } else {
      using Cfg = FwdExactCfg<D, CQ, CK, true>;
      return launch_kernel<TrainParams>(fwd_exact_kernel<D, CQ, CK, true>, grid, block, Cfg::kSmemBytes, stream, p.G, p);
    }
  }
  using Cfg = FwdExactCfg<D, CQ, CK, false>;
  return launch_kernel<TrainParams>(fwd_exact_kernel<D, CQ, CK, false>, grid, block, Cfg::kSmemBytes, stream, 1, p);
}

cudaError_t launch_fwd_exact(const TrainParams& p, cudaStream_t stream) {
  ScopedKernelTimer timer_(kKernFwdExact, stream);
  if (hm_dense_supported(p)) return launch_hm_fwd(p, stream);   // head mix without a conv: all heads of a group in one CTA
  const bool mix = (p.Wmix != nullptr) && p.G > 1;
  int cq = p.cq, ck = p.ck;
  const bool has_theta = p.theta != nullptr;
  if (mix && cq == 3 && ck == 5) { cq = -1; }  // force the run-time path
  FMTA_DISPATCH_D(p.d, FMTA_DISPATCH_CONV(cq, ck, has_theta, return launch_fwd_exact_t<D_, CQ_, CK_>(p, stream);););
  return cudaErrorInvalidValue;
}

}  // namespace fmta
