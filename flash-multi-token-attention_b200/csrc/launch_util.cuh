// Host-side launch helpers shared by the kernel translation units.
#pragma once
#include <cuda_runtime.h>

#include <cstdlib>

#include "fmta_params.h"

namespace fmta {

// FMTA_NO_PDL=1 in the environment launches every kernel with plain stream order (read once per process).
inline bool pdl_enabled() {
  static const bool on = [] { const char* e = getenv("FMTA_NO_PDL"); return !(e && e[0] == '1'); }();
  return on;
}

// Launch `kern` with dynamic shared memory and, when cluster_y > 1, a thread-block cluster of
// (1, cluster_y, 1) CTAs (the heads of one mixing group).  No TMA multicast is involved; the
// cluster only provides distributed shared memory and cluster barriers.
template <typename P>
inline cudaError_t launch_kernel(void (*kern)(const P), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, int cluster_y, const P& params) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (cluster_y > 1) {
    if (cluster_y > 8) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
      if (e != cudaSuccess) return e;
    }
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = cluster_y;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  } else if (cluster_y == -1 && pdl_enabled()) {   // no cluster; programmatic stream serialization (the kernel calls pdl_wait())
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, params);
}

// Launch with programmatic stream serialization: the kernel may be scheduled before the previous kernel of the
// stream has completed (it calls pdl_wait() before touching global memory).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (pdl_enabled()) { cfg.attrs = attr; cfg.numAttrs = 1; }
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Compile-time specialisations of the filter shape: (6,11) and (3,5) are unrolled, a NULL filter skips
// the conv (template value (1,1)), anything else takes the run-time path (CQ = CK = 0).
#define FMTA_DISPATCH_CONV(cq, ck, has_theta, ...)                           \
  do {                                                                        \
    if (!(has_theta)) { constexpr int CQ_ = 1, CK_ = 1; __VA_ARGS__ }                               \
    else if ((cq) == 6 && (ck) == 11) { constexpr int CQ_ = 6, CK_ = 11; __VA_ARGS__ }          \
    else if ((cq) == 3 && (ck) == 5) { constexpr int CQ_ = 3, CK_ = 5; __VA_ARGS__ }            \
    else { constexpr int CQ_ = 0, CK_ = 0; __VA_ARGS__ }                                        \
  } while (0)

#define FMTA_DISPATCH_D(d, ...)                                   \
  do {                                                            \
    if ((d) == 32) { constexpr int D_ = 32; __VA_ARGS__ }          \
    else if ((d) == 64) { constexpr int D_ = 64; __VA_ARGS__ }     \
    else if ((d) == 128) { constexpr int D_ = 128; __VA_ARGS__ }   \
    else return cudaErrorInvalidValue;                            \
  } while (0)

// Optional timing hook: when armed for a kernel id, the launcher of that kernel records the two
// events around the launch on the launch stream (see fmta_profile_kernel in the C ABI).
enum KernelId : int { kKernNone = 0, kKernFwdTc = 1, kKernFwdExact = 2, kKernBwdDqTc = 3, kKernBwdDkdvTc = 4,
                      kKernBwdDqExact = 5, kKernBwdDkdvExact = 6, kKernDecode = 7, kKernBwdBand = 8, kKernKtilde = 9, kKernDkPost = 10 };
struct ProfileHook { int id; cudaEvent_t start, stop; };
extern ProfileHook g_profile_hook;
struct ScopedKernelTimer {
  bool on; cudaStream_t st;
  ScopedKernelTimer(int id, cudaStream_t s) : on(g_profile_hook.id == id), st(s) { if (on) cudaEventRecord(g_profile_hook.start, st); }
  ~ScopedKernelTimer() { if (on) cudaEventRecord(g_profile_hook.stop, st); }
};

// Failure detection.  A tensor-core kernel whose bounded wait ran out sets a status word: the word the caller
// registered for the current device (fmta_set_status_word) -- the kernels write it directly, no extra launch --
// or, when none is registered, a word of the call's workspace.  status_word_of returns the registered word, or
// clears (on `stream`) and returns `ws_word`.  take_selftest_expire returns 1 once after
// fmta_selftest_expire_next(id) named this kernel: that launch runs with its first consumer wait pointed at a
// barrier nothing arrives at, so the wait runs out and the kernel leaves through its abort path.
cudaError_t status_word_of(int* ws_word, cudaStream_t stream, int** word);
int* registered_status_word();
int take_selftest_expire(int kernel_id);

cudaError_t launch_fwd_exact(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_bwd_dq(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_bwd_dkdv(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_reduce_partials(const float* part, float* out, int n_slots, int n, cudaStream_t stream);
cudaError_t launch_rowdot(const void* dO, const void* O, int o_bf16, float* Dv, size_t rows, int d, cudaStream_t stream);
cudaError_t launch_decode(const DecodeParams& p, cudaStream_t stream);
cudaError_t launch_kv_append_paged(void* Kpool, void* Vpool, const int* block_table, const int* seq_lens,
                                   const void* Knew, const void* Vnew, int B, int H, int n_new, int d, int page_size,
                                   int page_shift, int max_pages, cudaStream_t stream);
bool fwd_tc_supported(const TrainParams& p);
// pre-pass of the tensor-core kernels: Kt[b,h,t,j,:] = scale * log2(e) * sum_u theta[h,t,u] * K[b,h,j + pad_k - u,:]
cudaError_t launch_ktilde(const TrainParams& p, __nv_bfloat16* Kt, cudaStream_t stream);
size_t fwd_tc_workspace_bytes(int B, int H, int N, int d, int cq);
bool bwd_tc_supported(const TrainParams& p);
size_t bwd_tc_workspace_bytes(int B, int H, int N, int d, int cq);
// keep_pdc: the dQ kernel also writes P and dC (workspace of FMTA_OP_BWD_TC_STREAM) and the dK/dV kernel
// streams them instead of recomputing them (head dim 64)
// dense head mixing without a key-query conv: all heads of a group in one CTA (headmix_dense.cu)
bool hm_dense_supported(const TrainParams& p);
int hm_dq_slots(int B, int N, int G);
cudaError_t launch_hm_fwd(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_hm_bwd_dq(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_hm_bwd_dkdv(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_bwd_dq_tc(const TrainParams& p, void* workspace, bool keep_pdc, cudaStream_t stream);
cudaError_t launch_bwd_dkdv_tc(const TrainParams& p, void* workspace, float* dTheta_part_tc, bool keep_pdc, cudaStream_t stream);
size_t bwd_tc_stream_workspace_bytes(int B, int H, int N, int d, int cq);
int bwd_tc_theta_slots(int B, int N, int d);
int bwd_band_theta_slots(int B, int N, int cq, int ck);
cudaError_t launch_bwd_band(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_fwd_band(const TrainParams& p, cudaStream_t stream);
cudaError_t launch_fwd_tc(const TrainParams& p, void* workspace, const float** Opart, const float** Mpart,
                          const float** Lpart, cudaStream_t stream);

}  // namespace fmta
