// Stacked-GEMM conv-attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Off the causal band (query - key >= pad_q + pad_k) the conv'd logits are a plain GEMM with a
// stacked contraction:
//     C[i,j] = sum_a  q_{i-(pad_q-a)} . Kt_a[j],     Kt_a[j] = scale * sum_b theta[a,b] k_{j+b-pad_k}
// so those tiles are FlashAttention with c_q accumulating MMAs per score tile and no work on the
// FP32 pipe.  This file holds
//   ktilde_kernel : the memory-bound pre-pass that writes the c_q bf16 operands Kt_a;
//   fwd_tc_kernel : the warp-specialised main kernel (1 TMA warp, 1 MMA warp, 4 softmax warps);
//   launch_fwd_tc : tensor maps + launches.
// The kernel leaves an UN-normalised partial (O, m, l) per query row; the exact tile kernel then
// walks the remaining (band) key blocks starting from that state and writes the final O, M, L.
//
// Row-shifted A operands without copies: Q is staged in the no-swizzle K-major core-matrix
// layout [d/8][rows][8 elements]; the M-direction stride of that layout is 16 bytes, so the
// operand "Q shifted by s rows" is the same buffer with the descriptor start address advanced
// by 16*s bytes.  K-tilde / V tiles use the 128-byte swizzle that TMA writes natively.
//
// Every wait on an mbarrier is bounded (tc::mbar_wait); on expiry the CTA raises an abort flag,
// records it in the caller's status word, drains its outstanding copies, frees its TMEM and
// returns.  No TMA multicast, no cluster, cta_group::1 only.
#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "fmta_params.h"
#include "fmta_tc.cuh"
#include "launch_util.cuh"

namespace fmta {

// ------------------------------------------------------------------------------------------
// Kt[bh, a, j, :] = scale * sum_b theta[h, a, b] * K[bh, j + b - pad_k, :]   (bf16, zero beyond ends)
template <int D>
__global__ void __launch_bounds__(256) ktilde_kernel(const bf16* __restrict__ K, const float* __restrict__ theta,
                                                     bf16* __restrict__ Kt, int H, int N, int cq, int ck,
                                                     float scale) {
  constexpr int CPR = D / 8;          // 16-byte chunks per row
  constexpr int RPB = 256 / CPR;      // rows per block
  __shared__ float sTh[16 * 20];
  const int bh = blockIdx.y, h = bh % H;
  for (int i = threadIdx.x; i < cq * ck; i += 256) sTh[(i / ck) * 20 + (i % ck)] = theta[(size_t)h * cq * ck + i] * scale;
  __syncthreads();
  const int j = blockIdx.x * RPB + threadIdx.x / CPR, c = threadIdx.x % CPR;
  if (j >= N) return;
  const int pk = (ck - 1) / 2;
  const bf16* Kb = K + (size_t)bh * N * D;
  for (int a0 = 0; a0 < cq; a0 += 8) {
    float acc[8][8];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[a][e] = 0.f;
    for (int b = 0; b < ck; ++b) {
      const int jj = j + b - pk;
      if (jj < 0 || jj >= N) continue;
      const uint4 kv = *reinterpret_cast<const uint4*>(Kb + (size_t)jj * D + c * 8);
      const uint32_t w32[4] = {kv.x, kv.y, kv.z, kv.w};
      float kf[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) { kf[2 * e] = __uint_as_float(w32[e] << 16); kf[2 * e + 1] = __uint_as_float(w32[e] & 0xffff0000u); }
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        if (a0 + a < cq) {
          const float w = sTh[(a0 + a) * 20 + b];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[a][e] = fmaf(w, kf[e], acc[a][e]);
        }
      }
    }
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      if (a0 + a < cq) {
        uint4 o;
        o.x = pack_bf16(acc[a][0], acc[a][1]); o.y = pack_bf16(acc[a][2], acc[a][3]);
        o.z = pack_bf16(acc[a][4], acc[a][5]); o.w = pack_bf16(acc[a][6], acc[a][7]);
        *reinterpret_cast<uint4*>(Kt + (((size_t)bh * cq + a0 + a) * N + j) * D + c * 8) = o;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
struct TcParams {
  float* Opart;   // [B,H,N,D] un-normalised
  float* Mpart;   // [B,H,N]
  float* Lpart;
  int* status;    // device word: set non-zero when a bounded wait expired
  int H, N, cq, ck, causal;
};

template <int D, int BC>
struct TcCfg {
  static constexpr int BM = 128;               // query rows per CTA (= TMEM lanes)
  static constexpr int HALO = 16;              // rows staged above the block (pad_q <= 15)
  static constexpr int QR = BM + HALO;
  static constexpr int TILE_BYTES = BC * D * 2;
  static constexpr int NSLOT = (D == 64) ? 12 : 7;
  static constexpr int oQ = 0;
  static constexpr int oP = oQ + QR * D * 2;
  static constexpr int P_BYTES = BM * BC * 2;
  static constexpr int oRing = ((oP + 2 * P_BYTES + 1023) / 1024) * 1024;
  static constexpr int oBar = oRing + NSLOT * TILE_BYTES;
  static constexpr int kSmemBytes = oBar + 512 + 1024;   // + alignment slack
  static constexpr int kTmemCols = 256;        // S0 [0,BC) S1 [BC,2BC) O [2BC, 2BC+D)
  static_assert(2 * BC + D <= kTmemCols, "TMEM budget");
  static_assert(BC == 64, "softmax code assumes 64 keys per block");
};

template <int D, int BC>
__global__ void __launch_bounds__(192, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKt,
              const __grid_constant__ CUtensorMap tmV, const TcParams p) {
  using Cfg = TcCfg<D, BC>;
  constexpr int BM = Cfg::BM, HALO = Cfg::HALO, QR = Cfg::QR, NSLOT = Cfg::NSLOT;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem + Cfg::oQ;
  unsigned char* sP = smem + Cfg::oP;
  unsigned char* sRing = smem + Cfg::oRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* full = bars;                 // [NSLOT]
  uint64_t* empty = bars + NSLOT;        // [NSLOT]
  uint64_t* q_full = bars + 2 * NSLOT;
  uint64_t* s_full = q_full + 1;         // [2]
  uint64_t* p_full = s_full + 2;         // [2]
  uint64_t* o_full = p_full + 2;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(o_full + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_issued = s_abort + 1;
  volatile int* s_consumed = s_abort + 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int nQB = (N + BM - 1) / BM;
  const int qb = nQB - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int bh = b * p.H + h;
  const int i0 = qb * BM;
  int nkb;
  if (p.causal) {
    const int t = i0 - pq - pk + 1;
    nkb = t > 0 ? t / BC : 0;
  } else {
    nkb = (N + BC - 1) / BC;
  }

  if (tid == 0) {
    for (int i = 0; i < NSLOT; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 1); }
    tc::mbar_init(q_full, 1);
    tc::mbar_init(&s_full[0], 1); tc::mbar_init(&s_full[1], 1);
    tc::mbar_init(&p_full[0], BM); tc::mbar_init(&p_full[1], BM);
    tc::mbar_init(o_full, 1);
    *s_abort = 0; *s_issued = 0; *s_consumed = 0;
    tc::mbar_fence_init();
  }
  if (warp == 5) {
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tS[2] = {tmem, tmem + BC};
  const uint32_t tO = tmem + 2 * BC;

  if (warp == 4) {
    // ===================== TMA producer =====================
    if (lane == 0 && nkb > 0) {
      tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmKt); tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, QR * D * 2);
      for (int kc = 0; kc < D / 8; ++kc)   // one 16-byte-wide column slab per load -> [kc][row][8]
        tc::tma_load_3d(sQ + kc * (QR * 16), &tmQ, q_full, kc * 8, i0 - HALO, bh);
      int id = 0;
      bool ok = true;
      auto put = [&](bool isV, int kb, int a) {
        const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
        if (!tc::mbar_wait(&empty[slot], ph ^ 1, s_abort)) { ok = false; return; }
        tc::mbar_expect_tx(&full[slot], Cfg::TILE_BYTES);
        unsigned char* dst = sRing + slot * Cfg::TILE_BYTES;
#pragma unroll
        for (int s = 0; s < D / 64; ++s) {
          if (isV) tc::tma_load_3d(dst + s * (BC * 128), &tmV, &full[slot], s * 64, kb * BC, bh);
          else tc::tma_load_3d(dst + s * (BC * 128), &tmKt, &full[slot], s * 64, kb * BC, bh * cq + a);
        }
        ++id;
        *s_issued = id;
      };
      // same order as the MMA warp consumes: S(0); then S(kb+1), V(kb)
      for (int a = 0; a < cq && ok; ++a) put(false, 0, a);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        if (kb + 1 < nkb) for (int a = 0; a < cq && ok; ++a) put(false, kb + 1, a);
        if (ok) put(true, kb, 0);
      }
    }
  } else if (warp == 5) {
    // ===================== MMA issuer =====================
    if (lane == 0 && nkb > 0) {
      constexpr uint32_t idescS = tc::make_idesc(BM, BC, 0, 0);
      constexpr uint32_t idescPV = tc::make_idesc(BM, D, 0, 1);
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP), aRing = smem_u32(sRing);
      int id = 0;
      bool ok = tc::mbar_wait(q_full, 0, s_abort);
      auto issue_S = [&](int kb) {
        for (int a = 0; a < cq && ok; ++a) {
          const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
          if (!tc::mbar_wait(&full[slot], ph, s_abort)) { ok = false; return; }
          tc::tc_fence_after();
          const uint32_t aB = aRing + slot * Cfg::TILE_BYTES;
          const uint32_t aA = aQ + (HALO - pq + a) * 16;
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t ad = tc::make_sdesc(aA + (2 * k) * (QR * 16), QR * 16, 128, tc::kLayoutNone);
            const uint64_t bd = tc::make_sdesc(aB + (k / 4) * (BC * 128) + (k % 4) * 32, 16, 1024, tc::kLayoutSW128);
            tc::mma_ss(tS[kb & 1], ad, bd, idescS, (a | k) != 0);
          }
          tc::mma_commit(&empty[slot]);
          ++id;
          *s_consumed = id;
        }
        if (ok) tc::mma_commit(&s_full[kb & 1]);
      };
      auto issue_PV = [&](int kb) {
        const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
        if (!tc::mbar_wait(&full[slot], ph, s_abort)) { ok = false; return; }
        if (!tc::mbar_wait(&p_full[kb & 1], (kb >> 1) & 1, s_abort)) { ok = false; return; }
        tc::tc_fence_after();
        const uint32_t aB = aRing + slot * Cfg::TILE_BYTES;
        const uint32_t aA = aP + (kb & 1) * Cfg::P_BYTES;
#pragma unroll
        for (int k = 0; k < BC / 16; ++k) {
          const uint64_t ad = tc::make_sdesc(aA + (2 * k) * (BM * 16), BM * 16, 128, tc::kLayoutNone);
          const uint64_t bd = tc::make_sdesc(aB + k * 2048, BC * 128, 1024, tc::kLayoutSW128);
          tc::mma_ss(tO, ad, bd, idescPV, (kb | k) != 0);
        }
        tc::mma_commit(&empty[slot]);
        tc::mma_commit(o_full);
        ++id;
        *s_consumed = id;
      };
      if (ok) issue_S(0);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        if (kb + 1 < nkb) issue_S(kb + 1);
        if (ok) issue_PV(kb);
      }
    }
  } else {
    // ===================== softmax warps: one query row per thread =====================
    const int m = tid;                                  // row within the block = TMEM lane
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      ok = __all_sync(0xffffffffu, tc::mbar_wait(&s_full[kb & 1], (kb >> 1) & 1, s_abort));
      if (!ok) break;   // warp-uniform: the TMEM loads below are warp-collective
      tc::tc_fence_after();
      float s[BC];
      {
        float t0[32], t1[32];
        tc::tmem_ld32(tS[kb & 1] + lane_base, t0);
        tc::tmem_ld32(tS[kb & 1] + lane_base + 32, t1);
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = t0[i]; s[32 + i] = t1[i]; }
      }
      if (!p.causal) {
#pragma unroll
        for (int i = 0; i < BC; ++i) if (kb * BC + i >= N) s[i] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int i = 1; i < BC; ++i) mx = fmaxf(mx, s[i]);
      const float m_new = fmaxf(m_run, mx);             // finite: every block holds a valid key
      const float mb = m_new * kLog2e;
      float sum = 0.f;
      uint32_t pk32[BC / 2];
#pragma unroll
      for (int i = 0; i < BC; i += 2) {
        const float p0 = exp2f(fmaf(s[i], kLog2e, -mb)), p1 = exp2f(fmaf(s[i + 1], kLog2e, -mb));
        sum += p0 + p1;
        pk32[i / 2] = pack_bf16(p0, p1);
      }
      const float alpha = exp2f((m_run - m_new) * kLog2e);   // 0 on the first block
      l_run = l_run * alpha + sum;
      m_run = m_new;
      if (kb > 0) {
        // O *= alpha (needs PV(kb-1) complete; that also frees P buffer kb&1 used by PV(kb-2))
        ok = __all_sync(0xffffffffu, tc::mbar_wait(o_full, (kb - 1) & 1, s_abort));
        if (!ok) break;
        tc::tc_fence_after();
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tc::tmem_ld32(tO + lane_base + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tc::tmem_st32(tO + lane_base + c * 32, o);
        }
        tc::tmem_wait_st();
      }
      unsigned char* pb = sP + (kb & 1) * Cfg::P_BYTES + m * 16;
#pragma unroll
      for (int kc = 0; kc < BC / 8; ++kc)
        *reinterpret_cast<uint4*>(pb + kc * (BM * 16)) = make_uint4(pk32[4 * kc], pk32[4 * kc + 1], pk32[4 * kc + 2], pk32[4 * kc + 3]);
      tc::fence_proxy_async_smem();
      tc::tc_fence_before();
      tc::mbar_arrive(&p_full[kb & 1]);
    }
    // ---- epilogue: un-normalised partial row ----
    const int gi = i0 + m;
    if (nkb > 0 && ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(o_full, (nkb - 1) & 1, s_abort));
    tc::tc_fence_after();
    const bool have = (nkb > 0) && ok;                  // warp-uniform
    float* orow = p.Opart + ((size_t)bh * N + (gi < N ? gi : 0)) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      float o[32];
      if (have) {
        tc::tmem_ld32(tO + lane_base + c * 32, o);      // warp-collective: every lane takes part
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0.f;
      }
      if (gi < N) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(orow + c * 32 + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
      }
    }
    if (gi < N) {
      p.Mpart[(size_t)bh * N + gi] = have ? m_run : -INFINITY;
      p.Lpart[(size_t)bh * N + gi] = have ? l_run : 0.f;
    }
  }
  __syncwarp();

  // ===================== teardown =====================
  tc::tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicExch(p.status, 1);
    if (tid == 128) {   // drain copies that were issued but never consumed, with a bounded wait
      volatile int never = 0;
      for (int id = *s_consumed; id < *s_issued; ++id) tc::mbar_wait(&full[id % NSLOT], (id / NSLOT) & 1, &never);
    }
    __syncthreads();
  }
  if (warp == 5) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// bf16 tensor viewed as [outer][rows][D] (D contiguous); box = {box_x, box_rows, 1}
bool make_map(CUtensorMap* map, const void* base, int D, int rows, size_t outer, int box_x, int box_rows, bool sw128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)outer};
  cuuint64_t strides[2] = {(cuuint64_t)D * 2, (cuuint64_t)rows * D * 2};
  cuuint32_t box[3] = {(cuuint32_t)box_x, (cuuint32_t)box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D>
cudaError_t launch_tc_t(const TrainParams& p, bf16* Kt, float* Opart, float* Mpart, float* Lpart, int* status,
                        cudaStream_t stream) {
  constexpr int BC = 64;
  using Cfg = TcCfg<D, BC>;
  const size_t BH = (size_t)p.B * p.H;
  {
    constexpr int RPB = 256 / (D / 8);
    dim3 grid((p.N + RPB - 1) / RPB, (unsigned)BH);
    ktilde_kernel<D><<<grid, 256, 0, stream>>>(p.K, p.theta, Kt, p.H, p.N, p.cq, p.ck, p.scale);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  alignas(64) CUtensorMap tmQ, tmKt, tmV;
  if (!make_map(&tmQ, p.Q, D, p.N, BH, 8, Cfg::QR, false)) return cudaErrorInvalidValue;
  if (!make_map(&tmKt, Kt, D, p.N, BH * p.cq, 64, BC, true)) return cudaErrorInvalidValue;
  if (!make_map(&tmV, p.V, D, p.N, BH, 64, BC, true)) return cudaErrorInvalidValue;
  TcParams tp;
  tp.Opart = Opart; tp.Mpart = Mpart; tp.Lpart = Lpart; tp.status = status;
  tp.H = p.H; tp.N = p.N; tp.cq = p.cq; tp.ck = p.ck; tp.causal = p.causal;
  auto kern = fwd_tc_kernel<D, BC>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((p.N + Cfg::BM - 1) / Cfg::BM, p.H, p.B);
  kern<<<grid, 192, Cfg::kSmemBytes, stream>>>(tmQ, tmKt, tmV, tp);
  return cudaGetLastError();
}

}  // namespace

bool fwd_tc_supported(const TrainParams& p) {
  return p.theta != nullptr && p.Wmix == nullptr && (p.d == 64 || p.d == 128) && p.cq >= 1 && p.cq <= 16 &&
         get_encode_fn() != nullptr;
}

size_t fwd_tc_workspace_bytes(int B, int H, int N, int d, int cq) {
  const size_t rows = (size_t)B * H * N;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  return up(rows * cq * d * 2) + up(rows * d * 4) + 2 * up(rows * 4) + 1024;
}

// Runs the pre-pass and the stacked kernel; on return p_out describes where the exact band kernel
// must pick up (Opart / Mpart / Lpart).
cudaError_t launch_fwd_tc(const TrainParams& p, void* workspace, const float** Opart, const float** Mpart,
                          const float** Lpart, cudaStream_t stream) {
  const size_t rows = (size_t)p.B * p.H * p.N;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  unsigned char* w = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~uintptr_t(1023));
  bf16* Kt = reinterpret_cast<bf16*>(w); w += up(rows * p.cq * p.d * 2);
  float* Op = reinterpret_cast<float*>(w); w += up(rows * p.d * 4);
  float* Mp = reinterpret_cast<float*>(w); w += up(rows * 4);
  float* Lp = reinterpret_cast<float*>(w); w += up(rows * 4);
  int* status = reinterpret_cast<int*>(w);
  cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int), stream);
  if (e != cudaSuccess) return e;
  if (p.d == 64) e = launch_tc_t<64>(p, Kt, Op, Mp, Lp, status, stream);
  else e = launch_tc_t<128>(p, Kt, Op, Mp, Lp, status, stream);
  *Opart = Op; *Mpart = Mp; *Lpart = Lp;
  return e;
}

}  // namespace fmta
