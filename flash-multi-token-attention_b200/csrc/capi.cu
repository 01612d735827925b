// C-ABI entry points of libfmta_b200.so: argument validation, parameter blocks, launches.
// Declarations and the reference interfaces they stand in for are in include/fmta_b200.h.
#include <cuda_runtime.h>

#include "../../include/fmta_b200.h"
#include "fmta_params.h"
#include "launch_util.cuh"

using namespace fmta;

namespace {

thread_local int g_last_cuda_error = 0;
int g_path = -1;   // process-wide default: -1 auto, 0 exact kernels only, 1 tensor-core kernels + band kernel

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return FMTA_OK;
  g_last_cuda_error = (int)e;
  (void)cudaGetLastError();  // clear the sticky launch-configuration error, if any
  return FMTA_ERR_CUDA;
}

int check_train_dims(int B, int H, int N, int d, int cq, int ck, int G, bool has_theta, bool has_w) {
  if (B < 1 || H < 1 || N < 1 || B > 65535 || H > 65535) return FMTA_ERR_SHAPE;
  if (d != 32 && d != 64 && d != 128) return FMTA_ERR_UNSUPPORTED;
  if (has_theta) {
    if (cq < 1 || ck < 1) return FMTA_ERR_SHAPE;
    if (cq > 16 || ck > 17 || (ck % 2) == 0) return FMTA_ERR_UNSUPPORTED;
  }
  if (has_w) {
    // 32 heads per group: only without a key-query conv and up to head dim 64 (the kernels that keep all heads
    // of a group in one CTA); the cluster kernels behind conv + mix hold one head per CTA of a cluster of <= 16
    if (G == 32) { if (has_theta || d > 64) return FMTA_ERR_UNSUPPORTED; }
    else if (G != 1 && G != 2 && G != 4 && G != 8 && G != 16) return FMTA_ERR_UNSUPPORTED;
    if (H % G != 0) return FMTA_ERR_SHAPE;
  }
  return FMTA_OK;
}

}  // namespace

namespace {
constexpr int kMaxDevices = 64;
int* g_status_word[kMaxDevices] = {};   // caller-owned device word per device (fmta_set_status_word)
int g_selftest_kernel = 0;              // kernel id whose next launch runs the expiry self-test

}  // namespace

namespace fmta {
ProfileHook g_profile_hook = {0, nullptr, nullptr};

int* registered_status_word() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  return g_status_word[dev];
}

cudaError_t status_word_of(int* ws_word, cudaStream_t stream, int** word) {
  if (int* reg = registered_status_word()) { *word = reg; return cudaSuccess; }
  *word = ws_word;
  return cudaMemsetAsync(ws_word, 0, sizeof(int), stream);
}

int take_selftest_expire(int kernel_id) {
  if (g_selftest_kernel != kernel_id) return 0;
  g_selftest_kernel = 0;
  return 1;
}
}  // namespace fmta

extern "C" {

int fmta_version(void) { return 100; }

const char* fmta_strerror(int status) {
  switch (status) {
    case FMTA_OK: return "ok";
    case FMTA_ERR_NULL: return "a required pointer is NULL";
    case FMTA_ERR_SHAPE: return "a dimension is out of range or inconsistent";
    case FMTA_ERR_UNSUPPORTED: return "unsupported head dim, filter shape (c_q<=16, odd c_k<=17) or group size";
    case FMTA_ERR_ALIGN: return "a tensor pointer is not 16-byte aligned";
    case FMTA_ERR_WORKSPACE: return "workspace missing or too small (see fmta_workspace_bytes)";
    case FMTA_ERR_CUDA: return "the CUDA runtime rejected a launch (see fmta_last_cuda_error)";
    case FMTA_ERR_DEVICE_WAIT: return "a bounded wait inside a tensor-core kernel ran out (device status word set); the outputs of that call are invalid";
    case FMTA_ERR_SCRATCH_LIMIT: return "problem too large for the built-in 4 MiB scratch of fmta_bwd_dq_dw_static; use fmta_bwd_dq_dw with a workspace";
    default: return "unknown status";
  }
}

int fmta_last_cuda_error(void) { return g_last_cuda_error; }

int fmta_profile_kernel(int kernel_id, void* start_event, void* stop_event) {
  if (kernel_id < 0 || kernel_id > 10) return FMTA_ERR_SHAPE;
  if (kernel_id != 0 && (!start_event || !stop_event)) return FMTA_ERR_NULL;
  g_profile_hook.id = kernel_id;
  g_profile_hook.start = (cudaEvent_t)start_event;
  g_profile_hook.stop = (cudaEvent_t)stop_event;
  return FMTA_OK;
}

int fmta_set_path(int path) {
  const int old = g_path;
  if (path >= -1 && path <= 1) g_path = path;
  return old;
}

int fmta_set_status_word(int* device_word) {
  int dev = -1;
  if (int s = check_cuda(cudaGetDevice(&dev))) return s;
  if (dev < 0 || dev >= kMaxDevices) return FMTA_ERR_SHAPE;
  g_status_word[dev] = device_word;
  return FMTA_OK;
}

int fmta_selftest_expire_next(int kernel_id) {
  if (kernel_id != 0 && kernel_id != kKernFwdTc && kernel_id != kKernBwdDqTc && kernel_id != kKernBwdDkdvTc)
    return FMTA_ERR_UNSUPPORTED;
  g_selftest_kernel = kernel_id;
  return FMTA_OK;
}

size_t fmta_workspace_bytes(int op, int B, int H, int N, int d, int cq, int ck, int G) {
  (void)d;
  if (op == FMTA_OP_BWD_DQ) {
    // one partial per CTA: 64 query rows per CTA in the tile kernels; the all-heads-in-one-CTA kernels of a
    // head mix without a conv use 16 to 64 rows (the caller need not know which kernel runs: take the larger)
    size_t slots = (size_t)B * ((N + 63) / 64);
    if (G > 1 && (size_t)hm_dq_slots(B, N, G) > slots) slots = (size_t)hm_dq_slots(B, N, G);
    size_t n = slots * H * (size_t)(cq * ck);
    if (G > 1) n += slots * (size_t)(H / G) * G * G;
    return n * sizeof(float);
  }
  if (op == FMTA_OP_BWD_TC || op == FMTA_OP_BWD_TC_STREAM) {
    // dTheta partials of the band kernel and of the tensor-core post-pass (one contiguous slot
    // array, rounded up), followed by the tensor-core backward's buffers
    const size_t slots = (size_t)bwd_band_theta_slots(B, N, cq, ck) + (size_t)bwd_tc_theta_slots(B, N, d);
    const size_t part = (slots * H * (size_t)(cq * ck) * sizeof(float) + 1023) / 1024 * 1024;
    return part + (op == FMTA_OP_BWD_TC_STREAM && d == 64 ? bwd_tc_stream_workspace_bytes(B, H, N, d, cq)
                                                          : bwd_tc_workspace_bytes(B, H, N, d, cq));
  }
  if (op == FMTA_OP_MIX_EXCHANGE) {
    // optional scratch of the conv + mix cluster kernels: two sets (alternate tiles) of two fp32 tiles per CTA
    // (one CTA per 64 rows / keys and head)
    if (G <= 1) return 0;
    return (size_t)2 * B * H * ((N + 63) / 64) * 2 * kMixXchFloats * sizeof(float);
  }
  if (op == FMTA_OP_FWD_TC) {
    // the stacked key operand (c_q bf16 copies of K) + un-normalised partial O (fp32), M, L
    return fwd_tc_workspace_bytes(B, H, N, d, cq);
  }
  return 0;
}

// A window [lo, hi) of sequence positions: starts on a multiple of 256 (the rows of one CTA of the forward
// kernel, and a multiple of every other kernel's tile start) and ends on one or at N.
static int check_window(int lo, int hi, int N) {
  if (lo < 0 || hi <= lo || hi > N) return FMTA_ERR_SHAPE;
  if (lo % 256 != 0 || (hi % 256 != 0 && hi != N)) return FMTA_ERR_SHAPE;
  return FMTA_OK;
}

static int fwd_impl(const void* Q, const void* K, const void* V, const float* theta, const float* wmix,
                    void* O, float* M, float* L, float* LSE, int B, int H, int N, int d, int cq, int ck,
                    int G, float scale, int causal, int o_dtype, int path, void* workspace,
                    size_t workspace_bytes, void* stream, void* ktilde, int row_lo = 0, int row_hi = 0,
                    int ktilde_valid = 0) {
  if (!Q || !K || !V || !O) return FMTA_ERR_NULL;
  if (ktilde && !aligned16(ktilde)) return FMTA_ERR_ALIGN;
  if (int s = check_train_dims(B, H, N, d, cq, ck, G, theta != nullptr, wmix != nullptr)) return s;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(O)) return FMTA_ERR_ALIGN;
  if (o_dtype != FMTA_DTYPE_F32 && o_dtype != FMTA_DTYPE_BF16) return FMTA_ERR_UNSUPPORTED;
  TrainParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.theta = theta; p.Wmix = (wmix && G > 1) ? wmix : nullptr;
  p.O = O; p.M = M; p.L = L; p.LSEout = LSE;
  p.B = B; p.H = H; p.N = N; p.d = d;
  p.cq = theta ? cq : 1; p.ck = theta ? ck : 1; p.G = (wmix && G > 1) ? G : 1;
  p.scale = scale; p.causal = causal; p.o_bf16 = (o_dtype == FMTA_DTYPE_BF16);
  // a 1x1 mixing "group" is a per-head scalar; fold it away by treating it as no mix only
  // when W is absent -- with G == 1 and W given the scalar still applies:
  if (wmix && G == 1) return FMTA_ERR_UNSUPPORTED;
  if (path != 0 && path != 1 && path != -1) return FMTA_ERR_SHAPE;
  bool use_tc = (path != 0) && fwd_tc_supported(p);
  if (path == 1 && !use_tc) return FMTA_ERR_UNSUPPORTED;
  if (use_tc) {
    const size_t need = fwd_tc_workspace_bytes(B, H, N, d, p.cq);
    if (!workspace || workspace_bytes < need) {
      if (path == 1) return FMTA_ERR_WORKSPACE;
      use_tc = false;   // library default without a workspace: exact kernel everywhere
    }
  }
  if (ktilde && !use_tc) return FMTA_ERR_UNSUPPORTED;   // only the tensor-core path makes the stacked key operand
  p.Kt_ext = reinterpret_cast<__nv_bfloat16*>(ktilde);
  p.kt_valid = ktilde != nullptr && ktilde_valid;        // the caller's buffer already holds the operand: no pre-pass
  if (row_hi > 0) {                                      // a window of rows: tensor-core path only
    if (int s = check_window(row_lo, row_hi, N)) return s;
    if (!use_tc) return FMTA_ERR_UNSUPPORTED;
    p.row_lo = row_lo; p.row_hi = row_hi;
  }
  if (use_tc) {
    // stacked tensor-core kernel off the causal band, then the band kernel, which continues the
    // online softmax from the un-normalised partial and writes the final O, M, L
    if (int s = check_cuda(launch_fwd_tc(p, workspace, &p.Opart, &p.Mpart, &p.Lpart, (cudaStream_t)stream))) return s;
    return check_cuda(launch_fwd_band(p, (cudaStream_t)stream));
  }
  // conv + mix: with enough workspace the heads' tiles are exchanged through global memory (faster)
  if (p.Wmix && p.theta && workspace && aligned16(workspace) &&
      workspace_bytes >= fmta_workspace_bytes(FMTA_OP_MIX_EXCHANGE, B, H, N, d, p.cq, p.ck, p.G))
    p.xchg = reinterpret_cast<float*>(workspace);
  return check_cuda(launch_fwd_exact(p, (cudaStream_t)stream));
}

int fmta_fwd(const void* Q, const void* K, const void* V, const float* theta, const float* wmix,
             void* O, float* M, float* L, float* LSE, int B, int H, int N, int d, int cq, int ck,
             int G, float scale, int causal, int o_dtype, int path, void* workspace,
             size_t workspace_bytes, void* stream) {
  return fwd_impl(Q, K, V, theta, wmix, O, M, L, LSE, B, H, N, d, cq, ck, G, scale, causal, o_dtype, path, workspace,
                  workspace_bytes, stream, nullptr);
}

int fmta_fwd_keep_ktilde(const void* Q, const void* K, const void* V, const float* theta, void* O, float* M, float* L,
                         float* LSE, int B, int H, int N, int d, int cq, int ck, float scale, int causal, int o_dtype,
                         void* workspace, size_t workspace_bytes, void* ktilde, void* stream) {
  if (!ktilde || !theta) return FMTA_ERR_NULL;
  return fwd_impl(Q, K, V, theta, nullptr, O, M, L, LSE, B, H, N, d, cq, ck, 1, scale, causal, o_dtype, 1, workspace,
                  workspace_bytes, stream, ktilde);
}

int fmta_bwd_prep_D(const void* dO, const void* O, int o_dtype, float* D, size_t rows, int d,
                    void* stream) {
  if (!dO || !O || !D) return FMTA_ERR_NULL;
  if (rows == 0 || d < 2 || (d % 2) != 0) return FMTA_ERR_SHAPE;
  if (o_dtype != FMTA_DTYPE_F32 && o_dtype != FMTA_DTYPE_BF16) return FMTA_ERR_UNSUPPORTED;
  return check_cuda(launch_rowdot(dO, O, o_dtype == FMTA_DTYPE_BF16, D, rows, d, (cudaStream_t)stream));
}

// conv + mix backward: the exchange scratch, when the workspace has room for it behind the partial sums
// (`part_bytes`, rounded up to 256); nullptr = exchange through distributed shared memory
static float* mix_exchange_scratch(const TrainParams& p, void* workspace, size_t workspace_bytes, size_t part_bytes) {
  if (!p.Wmix || !p.theta || p.G <= 1 || !workspace) return nullptr;
  const size_t off = (part_bytes + 255) / 256 * 256;
  const size_t need = fmta_workspace_bytes(FMTA_OP_MIX_EXCHANGE, p.B, p.H, p.N, p.d, p.cq, p.ck, p.G);
  if (workspace_bytes < off + need || !aligned16(workspace)) return nullptr;
  return reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(workspace) + off);
}

static int fill_bwd(TrainParams& p, const void* Q, const void* K, const void* V, const void* dO,
                    const float* D, const float* LSE, const float* theta, const float* wmix, int B,
                    int H, int N, int d, int cq, int ck, int G, float scale, int causal) {
  if (!Q || !K || !V || !dO || !D || !LSE) return FMTA_ERR_NULL;
  if (int s = check_train_dims(B, H, N, d, cq, ck, G, theta != nullptr, wmix != nullptr)) return s;
  if (wmix && G == 1) return FMTA_ERR_UNSUPPORTED;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V) || !aligned16(dO)) return FMTA_ERR_ALIGN;
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.dO = (const __nv_bfloat16*)dO; p.Dvec = D; p.LSE = LSE;
  p.theta = theta; p.Wmix = wmix;
  p.B = B; p.H = H; p.N = N; p.d = d;
  p.cq = theta ? cq : 1; p.ck = theta ? ck : 1; p.G = wmix ? G : 1;
  p.scale = scale; p.causal = causal;
  return FMTA_OK;
}

int fmta_bwd_dq_dw(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                   const float* LSE, const float* theta, const float* wmix, float* dQ,
                   float* dTheta, float* dW, int B, int H, int N, int d, int cq, int ck, int G,
                   float scale, int causal, void* workspace, size_t workspace_bytes, void* stream) {
  TrainParams p = {};
  if (int s = fill_bwd(p, Q, K, V, dO, D, LSE, theta, wmix, B, H, N, d, cq, ck, G, scale, causal)) return s;
  if (!dQ || !aligned16(dQ)) return dQ ? FMTA_ERR_ALIGN : FMTA_ERR_NULL;
  if ((theta && !dTheta) || (wmix && !dW)) return FMTA_ERR_NULL;
  const size_t need = fmta_workspace_bytes(FMTA_OP_BWD_DQ, B, H, N, d, p.cq, p.ck, p.G);
  const bool want_part = (theta != nullptr) || (wmix != nullptr);
  if (want_part && (!workspace || workspace_bytes < need)) return FMTA_ERR_WORKSPACE;
  const int slots = hm_dense_supported(p) ? hm_dq_slots(B, N, p.G) : B * ((N + 63) / 64);   // one partial per CTA of the kernel that runs
  const size_t n_theta = (size_t)H * p.cq * p.ck;
  p.dQ = dQ;
  p.n_slots = slots;
  p.dTheta_part = theta ? reinterpret_cast<float*>(workspace) : nullptr;
  p.dW_part = wmix ? reinterpret_cast<float*>(workspace) + (theta ? (size_t)slots * n_theta : 0) : nullptr;
  p.xchg = mix_exchange_scratch(p, workspace, workspace_bytes, need);
  cudaStream_t st = (cudaStream_t)stream;
  if (int s = check_cuda(launch_bwd_dq(p, st))) return s;
  if (theta)
    if (int s = check_cuda(launch_reduce_partials(p.dTheta_part, dTheta, slots, (int)n_theta, st))) return s;
  if (wmix)
    if (int s = check_cuda(launch_reduce_partials(p.dW_part, dW, slots, H * G, st))) return s;
  return FMTA_OK;
}

int fmta_bwd_dkdv(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                  const float* LSE, const float* theta, const float* wmix, float* dK, float* dV,
                  int B, int H, int N, int d, int cq, int ck, int G, float scale, int causal,
                  void* stream) {
  TrainParams p = {};
  if (int s = fill_bwd(p, Q, K, V, dO, D, LSE, theta, wmix, B, H, N, d, cq, ck, G, scale, causal)) return s;
  if (!dK || !dV) return FMTA_ERR_NULL;
  if (!aligned16(dK) || !aligned16(dV)) return FMTA_ERR_ALIGN;
  p.dK = dK; p.dV = dV;
  return check_cuda(launch_bwd_dkdv(p, (cudaStream_t)stream));
}

static int bwd_impl(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                    const float* LSE, const float* theta, const float* wmix, float* dQ, float* dK, float* dV,
                    float* dTheta, float* dW, int B, int H, int N, int d, int cq, int ck, int G, float scale,
                    int causal, int path, void* workspace, size_t workspace_bytes, void* stream, const void* ktilde,
                    int row_lo = 0, int row_hi = 0) {
  TrainParams p = {};
  if (ktilde && !aligned16(ktilde)) return FMTA_ERR_ALIGN;
  if (int s = fill_bwd(p, Q, K, V, dO, D, LSE, theta, wmix, B, H, N, d, cq, ck, G, scale, causal)) return s;
  if (!dQ || !dK || !dV) return FMTA_ERR_NULL;
  if (!aligned16(dQ) || !aligned16(dK) || !aligned16(dV)) return FMTA_ERR_ALIGN;
  if ((theta && !dTheta) || (wmix && !dW)) return FMTA_ERR_NULL;
  if (path != 0 && path != 1 && path != -1) return FMTA_ERR_SHAPE;
  if (path == -1) path = g_path;
  cudaStream_t st = (cudaStream_t)stream;
  bool use_tc = (path != 0) && bwd_tc_supported(p);
  if (path == 1 && !use_tc) return FMTA_ERR_UNSUPPORTED;
  const size_t need_tc = fmta_workspace_bytes(FMTA_OP_BWD_TC, B, H, N, d, p.cq, p.ck, p.G);
  if (use_tc && (!workspace || workspace_bytes < need_tc)) {
    if (path == 1) return FMTA_ERR_WORKSPACE;
    use_tc = false;
  }
  p.dQ = dQ; p.dK = dK; p.dV = dV;
  int slots_ex = (!use_tc && hm_dense_supported(p)) ? hm_dq_slots(B, N, p.G) : B * ((N + 63) / 64);
  const size_t n_theta = (size_t)H * p.cq * p.ck;
  if (ktilde && !use_tc) return FMTA_ERR_UNSUPPORTED;   // only the tensor-core path uses the stacked key operand
  if (!use_tc) {
    const size_t need = fmta_workspace_bytes(FMTA_OP_BWD_DQ, B, H, N, d, p.cq, p.ck, p.G);
    const bool want_part = (theta != nullptr) || (wmix != nullptr);
    if (want_part && (!workspace || workspace_bytes < need)) return FMTA_ERR_WORKSPACE;
    p.n_slots = slots_ex;
    p.dTheta_part = theta ? reinterpret_cast<float*>(workspace) : nullptr;
    p.dW_part = wmix ? reinterpret_cast<float*>(workspace) + (theta ? (size_t)slots_ex * n_theta : 0) : nullptr;
    p.xchg = mix_exchange_scratch(p, workspace, workspace_bytes, need);
    if (int s = check_cuda(launch_bwd_dq(p, st))) return s;
    if (int s = check_cuda(launch_bwd_dkdv(p, st))) return s;
    if (theta)
      if (int s = check_cuda(launch_reduce_partials(p.dTheta_part, dTheta, slots_ex, (int)n_theta, st))) return s;
    if (wmix)
      if (int s = check_cuda(launch_reduce_partials(p.dW_part, dW, slots_ex, H * G, st))) return s;
    return FMTA_OK;
  }
  // tensor-core kernels for the entries off the causal band, then the band kernel adds its part
  p.Kt_ext = reinterpret_cast<__nv_bfloat16*>(const_cast<void*>(ktilde));   // the forward's stacked key operand, kept by the caller
  p.kt_valid = ktilde != nullptr;
  int Nw = N;                                                   // positions this call owns
  if (row_hi > 0) {
    if (int s = check_window(row_lo, row_hi, N)) return s;
    p.row_lo = row_lo; p.row_hi = row_hi; Nw = row_hi - row_lo;
  }
  slots_ex = bwd_band_theta_slots(B, Nw, p.cq, p.ck);           // one dTheta partial per band CTA
  const int slots_tc = bwd_tc_theta_slots(B, Nw, d);
  float* part = reinterpret_cast<float*>(workspace);
  const size_t part_bytes = ((size_t)(slots_ex + slots_tc) * n_theta * sizeof(float) + 1023) / 1024 * 1024;
  void* tcw = reinterpret_cast<unsigned char*>(workspace) + part_bytes;
  // with the larger workspace of FMTA_OP_BWD_TC_STREAM (head dim 64) the dQ kernel leaves P and dC in global
  // memory and the dK/dV kernel streams them instead of recomputing them
  const bool keep_pdc = (d == 64) && row_hi == 0 &&
      workspace_bytes >= fmta_workspace_bytes(FMTA_OP_BWD_TC_STREAM, B, H, N, d, p.cq, p.ck, p.G);
  if (int s = check_cuda(launch_bwd_dq_tc(p, tcw, keep_pdc, st))) return s;
  if (int s = check_cuda(launch_bwd_dkdv_tc(p, tcw, part + (size_t)slots_ex * n_theta, keep_pdc, st))) return s;
  p.n_slots = slots_ex;
  p.dTheta_part = part;
  if (causal) {
    if (int s = check_cuda(launch_bwd_band(p, st))) return s;
  } else {   // no causal mask: no band
    if (int s = check_cuda(cudaMemsetAsync(part, 0, (size_t)slots_ex * n_theta * sizeof(float), st))) return s;
  }
  return check_cuda(launch_reduce_partials(part, dTheta, slots_ex + slots_tc, (int)n_theta, st));
}

int fmta_bwd(const void* Q, const void* K, const void* V, const void* dO, const float* D,
             const float* LSE, const float* theta, const float* wmix, float* dQ, float* dK, float* dV,
             float* dTheta, float* dW, int B, int H, int N, int d, int cq, int ck, int G, float scale,
             int causal, int path, void* workspace, size_t workspace_bytes, void* stream) {
  return bwd_impl(Q, K, V, dO, D, LSE, theta, wmix, dQ, dK, dV, dTheta, dW, B, H, N, d, cq, ck, G, scale, causal, path,
                  workspace, workspace_bytes, stream, nullptr);
}

int fmta_bwd_with_ktilde(const void* Q, const void* K, const void* V, const void* dO, const float* D,
                         const float* LSE, const float* theta, float* dQ, float* dK, float* dV, float* dTheta,
                         int B, int H, int N, int d, int cq, int ck, float scale, int causal, void* workspace,
                         size_t workspace_bytes, const void* ktilde, void* stream) {
  if (!ktilde || !theta) return FMTA_ERR_NULL;
  return bwd_impl(Q, K, V, dO, D, LSE, theta, nullptr, dQ, dK, dV, dTheta, nullptr, B, H, N, d, cq, ck, 1, scale, causal, 1,
                  workspace, workspace_bytes, stream, ktilde);
}

int fmta_stacked_keys(const void* K, const float* theta, void* ktilde, int B, int H, int N, int d, int cq, int ck,
                      float scale, void* stream) {
  if (!K || !theta || !ktilde) return FMTA_ERR_NULL;
  if (int s = check_train_dims(B, H, N, d, cq, ck, 1, true, false)) return s;
  if (d != 64 && d != 128) return FMTA_ERR_UNSUPPORTED;      // the tensor-core kernels' head dims
  if (!aligned16(K) || !aligned16(ktilde)) return FMTA_ERR_ALIGN;
  TrainParams p = {};
  p.K = (const __nv_bfloat16*)K; p.theta = theta;
  p.B = B; p.H = H; p.N = N; p.d = d; p.cq = cq; p.ck = ck; p.G = 1; p.scale = scale;
  return check_cuda(launch_ktilde(p, reinterpret_cast<__nv_bfloat16*>(ktilde), (cudaStream_t)stream));
}

int fmta_fwd_window(const void* Q, const void* K, const void* V, const float* theta, void* O, float* M, float* L,
                    float* LSE, int B, int H, int N, int d, int cq, int ck, float scale, int causal, int o_dtype,
                    int row_lo, int row_hi, const void* ktilde, void* workspace, size_t workspace_bytes, void* stream) {
  if (!theta) return FMTA_ERR_NULL;
  if (row_hi <= 0) return FMTA_ERR_SHAPE;
  return fwd_impl(Q, K, V, theta, nullptr, O, M, L, LSE, B, H, N, d, cq, ck, 1, scale, causal, o_dtype, 1, workspace,
                  workspace_bytes, stream, const_cast<void*>(ktilde), row_lo, row_hi, 1);
}

int fmta_bwd_window(const void* Q, const void* K, const void* V, const void* dO, const float* D, const float* LSE,
                    const float* theta, float* dQ, float* dK, float* dV, float* dTheta, int B, int H, int N, int d,
                    int cq, int ck, float scale, int causal, int row_lo, int row_hi, const void* ktilde, void* workspace,
                    size_t workspace_bytes, void* stream) {
  if (!theta) return FMTA_ERR_NULL;
  if (row_hi <= 0) return FMTA_ERR_SHAPE;
  return bwd_impl(Q, K, V, dO, D, LSE, theta, nullptr, dQ, dK, dV, dTheta, nullptr, B, H, N, d, cq, ck, 1, scale, causal, 1,
                  workspace, workspace_bytes, stream, ktilde, row_lo, row_hi);
}

static int decode_impl(const void* Q, const void* K, const void* V, const float* theta, float* O_splits,
                       float* M_splits, float* L_splits, int B, int H, int q_len, int Nk, int d, int cq,
                       int ck, int k_splits, float scale, int offset_causal, void* stream,
                       const int* block_table = nullptr, const int* seq_lens = nullptr, int page_size = 0,
                       int max_pages = 0) {
  if (!Q || !K || !V || !theta || !O_splits || !M_splits || !L_splits) return FMTA_ERR_NULL;
  if (B < 1 || H < 1 || Nk < 1 || B > 65535 || H > 65535) return FMTA_ERR_SHAPE;
  if (q_len < 1 || q_len > 16) return FMTA_ERR_SHAPE;          // flash_conv_attention_inference.py:66-67
  if (k_splits < 1 || k_splits > Nk) return FMTA_ERR_SHAPE;     // fwd_inference_wrapper.cu:65-66
  if (d != 32 && d != 64 && d != 128) return FMTA_ERR_UNSUPPORTED;
  if (cq < 1 || ck < 1) return FMTA_ERR_SHAPE;
  if (cq > 16 || ck > 17 || (ck % 2) == 0) return FMTA_ERR_UNSUPPORTED;
  if (!aligned16(Q) || !aligned16(K) || !aligned16(V)) return FMTA_ERR_ALIGN;
  DecodeParams p = {};
  p.Q = (const __nv_bfloat16*)Q; p.K = (const __nv_bfloat16*)K; p.V = (const __nv_bfloat16*)V;
  p.theta = theta; p.O_splits = O_splits; p.M_splits = M_splits; p.L_splits = L_splits;
  p.B = B; p.H = H; p.q_len = q_len; p.Nk = Nk; p.d = d; p.cq = cq; p.ck = ck; p.k_splits = k_splits;
  p.scale = scale;
  p.offset_causal = offset_causal;
  if (block_table) {
    int shift = 0;
    while ((1 << shift) < page_size) ++shift;
    if (page_size < 16 || (1 << shift) != page_size) return FMTA_ERR_SHAPE;      // power of two, >= one 16-key step
    if (max_pages < (Nk + page_size - 1) / page_size || max_pages > 2048) return FMTA_ERR_SHAPE;
    p.block_table = block_table; p.seq_lens = seq_lens;
    p.page_size = page_size; p.page_shift = shift; p.max_pages = max_pages;
  }
  return check_cuda(launch_decode(p, (cudaStream_t)stream));
}

int fmta_decode(const void* Q, const void* K, const void* V, const float* theta, float* O_splits,
                float* M_splits, float* L_splits, int B, int H, int q_len, int Nk, int d, int cq,
                int ck, int k_splits, float scale, void* stream) {
  return decode_impl(Q, K, V, theta, O_splits, M_splits, L_splits, B, H, q_len, Nk, d, cq, ck, k_splits, scale, 0, stream);
}

int fmta_decode_offset_causal(const void* Q, const void* K, const void* V, const float* theta, float* O_splits,
                              float* M_splits, float* L_splits, int B, int H, int q_len, int Nk, int d, int cq,
                              int ck, int k_splits, float scale, void* stream) {
  return decode_impl(Q, K, V, theta, O_splits, M_splits, L_splits, B, H, q_len, Nk, d, cq, ck, k_splits, scale, 1, stream);
}

int fmta_decode_paged(const void* Q, const void* K_pool, const void* V_pool, const int* block_table,
                      const int* seq_lens, const float* theta, float* O_splits, float* M_splits, float* L_splits,
                      int B, int H, int q_len, int Nk_max, int d, int cq, int ck, int k_splits, float scale,
                      int page_size, int max_pages, int offset_causal, void* stream) {
  if (!block_table) return FMTA_ERR_NULL;
  return decode_impl(Q, K_pool, V_pool, theta, O_splits, M_splits, L_splits, B, H, q_len, Nk_max, d, cq, ck, k_splits,
                     scale, offset_causal ? 1 : 0, stream, block_table, seq_lens, page_size, max_pages);
}

int fmta_kv_append_paged(void* K_pool, void* V_pool, const int* block_table, const int* seq_lens, const void* K_new,
                         const void* V_new, int B, int H, int n_new, int d, int page_size, int max_pages,
                         void* stream) {
  if (!K_pool || !V_pool || !block_table || !seq_lens || !K_new || !V_new) return FMTA_ERR_NULL;
  if (B < 1 || H < 1 || n_new < 1 || B > 65535 || H > 65535 || max_pages < 1) return FMTA_ERR_SHAPE;
  if (d != 32 && d != 64 && d != 128) return FMTA_ERR_UNSUPPORTED;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  if (page_size < 16 || (1 << shift) != page_size) return FMTA_ERR_SHAPE;
  if (!aligned16(K_pool) || !aligned16(V_pool) || !aligned16(K_new) || !aligned16(V_new)) return FMTA_ERR_ALIGN;
  return check_cuda(launch_kv_append_paged(K_pool, V_pool, block_table, seq_lens, K_new, V_new, B, H, n_new, d,
                                           page_size, shift, max_pages, (cudaStream_t)stream));
}

}  // extern "C"
