// Exact conv-attention forward tile kernel (register-fragment tensor cores + FP32-pipe conv).
//
// One CTA owns 64 query rows of one (batch, head) and walks key blocks of 64 columns:
//   S_ext = scale * Q_ext K_ext^T   on rows [i0-16, i0+64) x keys [j0-8, j0+72)   (mma.sync)
//           with future entries (key > query) set to ZERO when causal
//   C     = conv(S_ext, theta)       on the 64 x 64 owned tile                      (FP32 pipe)
//   [mix] C'_g = sum_g' W[g,g'] C_g' across the G heads of a thread-block cluster   (DSMEM)
//   online softmax (key > query -> -inf), P -> bf16, O += P V                       (mma.sync)
// The halo rows/columns are recomputed per tile in shared memory, so O never makes a round
// trip through HBM inside the key loop.
//
// This kernel is exact for every tile, including the causal band where the stacked-GEMM
// formulation (fwd_tc.cu) does not apply.  It is the path for head mixing, d = 32, calls
// without a workspace and `path = 0`; the tensor-core path handles the band in fwd_band.cu.
#pragma once
#include <cooperative_groups.h>

#include "conv_tile.cuh"
#include "fmta_common.cuh"
#include "fmta_params.h"

namespace fmta {
namespace cg = cooperative_groups;

template <int D, int CQ, int CK, bool MIX>
struct FwdExactCfg {
  static constexpr bool kNoConv = (CQ == 1 && CK == 1);
  static constexpr int NT = 256;
  static constexpr int BR = 64, BC = 64;
  static constexpr int HR = kNoConv ? 0 : 16;
  static constexpr int HC = kNoConv ? 0 : 8;
  static constexpr int SR = BR + HR, SC = BC + 2 * HC;
  static constexpr int S_LD = SC + 4;
  static constexpr int C_LD = BC + 4;
  static constexpr int QK_LD = D + 8;
  static constexpr int P_LD = BC + 8;
  static constexpr bool kNeedC = !kNoConv || MIX;
  // byte offsets into dynamic shared memory
  static constexpr int oQ = 0;
  static constexpr int oK = oQ + SR * QK_LD * 2;
  static constexpr int oV = oK + SC * QK_LD * 2;
  static constexpr int oS = oV + BC * QK_LD * 2;
  static constexpr int oC = oS + SR * S_LD * 4;
  static constexpr int oP = oC + (kNeedC ? BR * C_LD * 4 : 0);
  static constexpr int oStat = oP + BR * P_LD * 2;
  static constexpr int oTheta = oStat + 3 * BR * 4;
  static constexpr int oW = oTheta + kMaxCQ * kThetaLd * 4;
  static constexpr int kSmemBytes = oW + 256 * 4;
};

template <int D, int CQ, int CK, bool MIX>
__global__ void __launch_bounds__(256, 1) fwd_exact_kernel(const TrainParams p) {
  using Cfg = FwdExactCfg<D, CQ, CK, MIX>;
  constexpr int BR = Cfg::BR, BC = Cfg::BC, HR = Cfg::HR, HC = Cfg::HC, SR = Cfg::SR, SC = Cfg::SC;
  constexpr int S_LD = Cfg::S_LD, C_LD = Cfg::C_LD, QK_LD = Cfg::QK_LD, P_LD = Cfg::P_LD;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + Cfg::oQ);
  bf16* sK = reinterpret_cast<bf16*>(smem + Cfg::oK);
  bf16* sV = reinterpret_cast<bf16*>(smem + Cfg::oV);
  float* sS = reinterpret_cast<float*>(smem + Cfg::oS);
  float* sC = reinterpret_cast<float*>(smem + Cfg::oC);
  bf16* sP = reinterpret_cast<bf16*>(smem + Cfg::oP);
  float* sM = reinterpret_cast<float*>(smem + Cfg::oStat);
  float* sL = sM + BR;
  float* sAlpha = sL + BR;
  float* sTheta = reinterpret_cast<float*>(smem + Cfg::oTheta);
  float* sW = reinterpret_cast<float*>(smem + Cfg::oW);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H;
  const int nQB = (N + BR - 1) / BR, nKB = (N + BC - 1) / BC;
  const int qb = nQB - 1 - (int)blockIdx.x;  // long (late) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int i0 = qb * BR;
  const int cq = (CQ > 0) ? CQ : p.cq, ck = (CQ > 0) ? CK : p.ck;
  const int pq = cq - 1, pk = (ck - 1) / 2;
  const bool causal = p.causal != 0;
  const size_t bh = (size_t)b * H + h;
  const bf16* Qg = p.Q + bh * (size_t)N * D;
  const bf16* Kg = p.K + bh * (size_t)N * D;
  const bf16* Vg = p.V + bh * (size_t)N * D;

  if constexpr (!Cfg::kNoConv) {
    for (int i = tid; i < cq * ck; i += Cfg::NT)
      sTheta[(i / ck) * kThetaLd + (i % ck)] = p.theta[((size_t)h * cq) * ck + i];
  }
  int G = 1, grank = 0;
  if constexpr (MIX) {
    G = p.G;
    grank = h % G;
    if (tid < G * G) sW[tid] = p.Wmix[(size_t)(h / G) * G * G + tid];
  }

  // head mix: the heads' tiles go through global memory (L2) when the caller gave the scratch, else through
  // distributed shared memory; a CTA's slot and the slots of its group (same row block, same batch entry)
  // (two sets of slots used by alternate key blocks: a CTA may publish its next tile while a slower head of the
  // group still reads the previous one, which saves the cluster barrier after the reads)
  const size_t xstride = (size_t)gridDim.x * 2 * kMixXchFloats;
  const size_t xset = (size_t)gridDim.x * gridDim.y * gridDim.z * 2 * kMixXchFloats;
  const float* xbase0 = (MIX && p.xchg) ? p.xchg + (((size_t)b * H + (h / G) * G) * gridDim.x + blockIdx.x) * 2 * kMixXchFloats : nullptr;
  float* xme0 = (MIX && p.xchg) ? p.xchg + (((size_t)b * H + h) * gridDim.x + blockIdx.x) * 2 * kMixXchFloats : nullptr;
  const int kb_begin = 0, kb_end = causal ? min(nKB - 1, (i0 + BR - 1) / BC) : nKB - 1;

  // running softmax state and output accumulators
  constexpr int ONT = D / 16;  // n8-tiles per warp (half of the head dim)
  float accO[ONT][4];
  const int mt = warp & 3, nh = warp >> 2;
  const int fr0 = mt * 16 + (lane >> 2), fr1 = fr0 + 8;
  if (tid < BR) { sM[tid] = -INFINITY; sL[tid] = 0.f; }
#pragma unroll
  for (int j = 0; j < ONT; ++j) { accO[j][0] = accO[j][1] = accO[j][2] = accO[j][3] = 0.f; }

  load_rows_async<D, Cfg::NT>(sQ, QK_LD, Qg, i0 - HR, SR, N, tid);
  cp_async_commit();

  for (int kb = kb_begin; kb <= kb_end; ++kb) {
    const int j0 = kb * BC;
    load_rows_async<D, Cfg::NT>(sK, QK_LD, Kg, j0 - HC, SC, N, tid);
    load_rows_async<D, Cfg::NT>(sV, QK_LD, Vg, j0, BC, N, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();

    // ---- S_ext = scale * Q_ext K_ext^T (future entries zeroed when causal) ----
    {
      constexpr int NU = (SR / 16) * (SC / 16);
      for (int u = warp; u < NU; u += Cfg::NT / 32) {
        const int um = u / (SC / 16), un = u % (SC / 16);
        float acc[2][4] = {};
        warp_gemm<2, false, false>(acc, sQ + um * 16 * QK_LD, QK_LD, sK + un * 16 * QK_LD, QK_LD, D, lane);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const int r = um * 16 + (lane >> 2) + hh * 8;
            const int c = un * 16 + j * 8 + (lane & 3) * 2;
            const int qi = i0 - HR + r, kj = j0 - HC + c;
            float v0 = acc[j][2 * hh] * p.scale, v1 = acc[j][2 * hh + 1] * p.scale;
            if (causal && !Cfg::kNoConv) {
              if (kj > qi) v0 = 0.f;
              if (kj + 1 > qi) v1 = 0.f;
            }
            *reinterpret_cast<float2*>(sS + r * S_LD + c) = make_float2(v0, v1);
          }
        }
      }
    }
    __syncthreads();

    // ---- key-query conv on the owned 64x64 tile ----
    float* cbuf = sS;  // tile that the softmax reads, row stride C_LD
    if constexpr (!Cfg::kNoConv) {
      const int r = tid & 63, s = tid >> 6;
      float acc[16];
      conv_strip<CQ, CK, HC - (CK - 1) / 2, false>(acc, sS, S_LD, r, s, HR - pq, sTheta, cq, ck, HC - pk);
      float4* o = reinterpret_cast<float4*>(sC + r * C_LD + s * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      cbuf = sC;
    }
    if constexpr (MIX) {
      // C'_g = sum_g' W[g,g'] C_g' : read the other heads' tiles through distributed shared memory
      cg::cluster_group cluster = cg::this_cluster();
      const int r = tid & 63, s = tid >> 6;
      const float* xbase = xbase0 ? xbase0 + (size_t)(kb & 1) * xset : nullptr;
      float* xme = xme0 ? xme0 + (size_t)(kb & 1) * xset : nullptr;
      if (xme != nullptr) {   // publish the own tile for the other heads of the group
        const float4* src = reinterpret_cast<const float4*>(cbuf + r * C_LD + s * 16);
        float4* dst = reinterpret_cast<float4*>(xme + r * C_LD + s * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = src[i];
        __threadfence();
      }
      cluster.sync();
      float* mixed = Cfg::kNoConv ? sC : sS;  // a buffer nobody reads remotely
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
      if (xme != nullptr) mix_global16(acc, xbase, xstride, r * C_LD + s * 16, sW + grank * G, 1, G, grank, cbuf);
      else mix_remote16(acc, cluster, cbuf, r * C_LD + s * 16, sW + grank * G, 1, G);
      float4* o = reinterpret_cast<float4*>(mixed + r * C_LD + s * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = make_float4(acc[4 * i], acc[4 * i + 1], acc[4 * i + 2], acc[4 * i + 3]);
      if (xme != nullptr) __syncthreads();   // `mixed` is visible CTA-wide (the other heads read this CTA's slot, not its shared memory)
      else cluster.sync();                   // all remote reads of cbuf are done; `mixed` is visible CTA-wide
      cbuf = mixed;
    } else {
      __syncthreads();
    }

    // ---- online softmax: one warp per 8 rows, 2 columns per lane ----
#pragma unroll 2
    for (int rr = 0; rr < 8; ++rr) {
      const int r = warp * 8 + rr;
      const int c = 2 * lane;
      float2 v = *reinterpret_cast<const float2*>(cbuf + r * C_LD + c);
      const int qi = i0 + r, kj = j0 + c;
      if (kj < 0 || kj >= N || (causal && kj > qi)) v.x = -INFINITY;
      if (kj + 1 < 0 || kj + 1 >= N || (causal && kj + 1 > qi)) v.y = -INFINITY;
      const float mx = warp_max(fmaxf(v.x, v.y));
      const float m_old = sM[r];
      const float m_new = fmaxf(m_old, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float p0 = exp2f((v.x - m_use) * kLog2e), p1 = exp2f((v.y - m_use) * kLog2e);
      const float sum = warp_sum(p0 + p1);
      *reinterpret_cast<uint32_t*>(sP + r * P_LD + c) = pack_bf16(p0, p1);
      if (lane == 0) {
        const float alpha = (m_old == -INFINITY) ? 0.f : exp2f((m_old - m_use) * kLog2e);
        sM[r] = m_new;
        sL[r] = sL[r] * alpha + sum;
        sAlpha[r] = alpha;
      }
    }
    __syncthreads();

    // ---- O = alpha * O + P V ----
    {
      const float a0 = sAlpha[fr0], a1 = sAlpha[fr1];
#pragma unroll
      for (int j = 0; j < ONT; ++j) {
        accO[j][0] *= a0; accO[j][1] *= a0; accO[j][2] *= a1; accO[j][3] *= a1;
      }
      warp_gemm<ONT, false, true>(accO, sP + mt * 16 * P_LD, P_LD, sV + nh * (D / 2), QK_LD, BC, lane);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- epilogue: normalise, write O, M, L (and LSE) ----
  {
    const float l0 = sL[fr0], l1 = sL[fr1];
    const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
#pragma unroll
    for (int j = 0; j < ONT; ++j) {
      const int col = nh * (D / 2) + j * 8 + (lane & 3) * 2;
      const float o00 = accO[j][0] * inv0, o01 = accO[j][1] * inv0, o10 = accO[j][2] * inv1, o11 = accO[j][3] * inv1;
      if (p.o_bf16) {
        bf16* O = reinterpret_cast<bf16*>(p.O);
        if (i0 + fr0 < N) *reinterpret_cast<uint32_t*>(O + (bh * N + i0 + fr0) * D + col) = pack_bf16(o00, o01);
        if (i0 + fr1 < N) *reinterpret_cast<uint32_t*>(O + (bh * N + i0 + fr1) * D + col) = pack_bf16(o10, o11);
      } else {
        float* O = reinterpret_cast<float*>(p.O);
        if (i0 + fr0 < N) *reinterpret_cast<float2*>(O + (bh * N + i0 + fr0) * D + col) = make_float2(o00, o01);
        if (i0 + fr1 < N) *reinterpret_cast<float2*>(O + (bh * N + i0 + fr1) * D + col) = make_float2(o10, o11);
      }
    }
    if (tid < BR && i0 + tid < N) {
      const float m = sM[tid], l = sL[tid];
      if (p.M) p.M[bh * N + i0 + tid] = m;
      if (p.L) p.L[bh * N + i0 + tid] = l;
      if (p.LSEout) p.LSEout[bh * N + i0 + tid] = m + logf(l);
    }
  }
}

}  // namespace fmta
