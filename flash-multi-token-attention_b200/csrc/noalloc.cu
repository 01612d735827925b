// fmta_bwd_dq_dw_static: the dQ / dTheta / dW backward for callers that must not allocate.
//
// fmta_bwd_dq_dw needs a caller-owned workspace for its per-CTA partial sums.  Some hosts of
// this library cannot supply one: code running where device allocation is forbidden or would
// synchronise the device (inside a serving loop with a frozen memory pool, under a framework
// that owns every byte of the GPU, from a foreign-language binding that has no allocator handle
// at all).  For them this translation unit keeps the partials in a fixed file-scope device
// array.  The price is a hard size limit and no concurrency between calls (see the header).
#include <cuda_runtime.h>

#include <mutex>

#include "../../include/fmta_b200.h"
#include "fmta_params.h"
#include "launch_util.cuh"

using namespace fmta;

namespace {

// Per-CTA partials of dTheta (and dW): one slot per (batch, 64-row query block).
// 1 Mi floats = 4 MiB, resident on every GPU that loads the library until the process exits.
constexpr size_t kStaticScratchFloats = FMTA_STATIC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

constexpr int kMaxDevices = 64;
float* g_scratch_ptr[kMaxDevices] = {};   // device address of g_static_scratch, per device
std::mutex g_scratch_mutex;

// The array's name is only a host-side handle; the kernels need its device address, which is
// looked up once per device with that device current.
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FMTA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return FMTA_ERR_CUDA;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return FMTA_OK;
}

}  // namespace

extern "C" int fmta_bwd_dq_dw_static(const void* Q, const void* K, const void* V, const void* dO,
                                     const float* D, const float* LSE, const float* theta,
                                     const float* wmix, float* dQ, float* dTheta, float* dW, int B,
                                     int H, int N, int d, int cq, int ck, int G, float scale,
                                     int causal, void* stream) {
  // Range checks first (the same ones fmta_bwd_dq_dw applies), so that the size below is computed from
  // sane values; the filter shape and the group size only count when theta / wmix are given.
  if (B < 1 || H < 1 || N < 1 || B > 65535 || H > 65535) return FMTA_ERR_SHAPE;
  if (theta && (cq < 1 || ck < 1)) return FMTA_ERR_SHAPE;
  if (theta && (cq > 16 || ck > 17 || (ck % 2) == 0)) return FMTA_ERR_UNSUPPORTED;
  if (wmix) {
    if (G < 1) return FMTA_ERR_SHAPE;
    if (G == 32) { if (theta || d > 64) return FMTA_ERR_UNSUPPORTED; }
    else if (G != 2 && G != 4 && G != 8 && G != 16) return FMTA_ERR_UNSUPPORTED;
    if (H % G != 0) return FMTA_ERR_SHAPE;
  }
  // Scratch is needed only for the filter / mixing gradients; an over-limit problem is rejected before
  // anything touches the device.
  size_t need = 0;
  if (theta || wmix) {
    size_t slots = (size_t)B * (size_t)((N + 63) / 64);
    if (wmix && !theta) slots = (size_t)hm_dq_slots(B, N, G);   // the kernel of a mix without a conv: finer row tiles
    if (theta) need += slots * (size_t)H * (size_t)cq * (size_t)ck * sizeof(float);
    if (wmix) need += slots * (size_t)H * (size_t)G * sizeof(float);
  }
  if (need > FMTA_STATIC_SCRATCH_BYTES) return FMTA_ERR_SCRATCH_LIMIT;
  if (need == 0)   // no partial sums to keep: the plain entry point needs no workspace either
    return fmta_bwd_dq_dw(Q, K, V, dO, D, LSE, theta, wmix, dQ, dTheta, dW, B, H, N, d, cq, ck, G, scale, causal,
                          nullptr, 0, stream);
  float* scratch = nullptr;
  if (int s = scratch_for_current_device(&scratch)) return s;
  // Every partial slot is overwritten by the CTA that owns it before the reduction reads it, so
  // the array needs no clearing between calls even though it keeps the previous call's contents.
  return fmta_bwd_dq_dw(Q, K, V, dO, D, LSE, theta, wmix, dQ, dTheta, dW, B, H, N, d, cq, ck, G, scale,
                        causal, scratch, FMTA_STATIC_SCRATCH_BYTES, stream);
}
