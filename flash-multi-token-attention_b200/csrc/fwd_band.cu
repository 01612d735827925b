// Forward over the causal band: the entries 0 <= i - j < pad_q + pad_k that the stacked-GEMM
// tensor-core kernel (fwd_tc.cu) leaves out, merged into that kernel's un-normalised partial
// (Opart, Mpart, Lpart) to give the final O, M, L (and LSE).
//
// As in the backward band kernel everything lives in (row, diagonal) coordinates:
//   Sb[i, e] = scale * q_i . k_{i-e},  e in [0, W),  W = pad_q + 2 pad_k                 (mma.sync)
//   Cb[i, d] = sum_{a,b} theta[a,b] Sb[i-pad_q+a, d+a-pad_q+pad_k-b],  d in [0, band)    (FP32 pipe)
//   m = max(Mpart_i, max_d Cb),  p_d = exp(Cb - m),  l = Lpart_i exp(Mpart_i - m) + sum_d p_d
//   O_i = (exp(Mpart_i - m) Opart_i + sum_d p_d v_{i-d}) / l                            (mma.sync)
// A CTA owns 64 query rows.  Without a causal mask there is no band and the kernel only
// normalises the partial.
#include "fmta_common.cuh"
#include "fmta_params.h"
#include "launch_util.cuh"

namespace fmta {

template <int D>
struct FwdBandCfg {
  static constexpr int NT = 256;
  static constexpr int R = 64;                        // query rows per CTA
  static constexpr int MAXBAND = 15 + 8, MAXW = MAXBAND + 8;   // c_q <= 16, c_k <= 17
  static constexpr int RS = R + 16;                   // Sb / Q rows (16 halo rows above)
  static constexpr int RK = R + 48;                   // K rows: start 48 rows earlier
  static constexpr int RV = R + 32;                   // V rows: start 32 rows earlier
  static constexpr int LD = D + 8;
  static constexpr int SB_LD = 55;                    // band + W <= 54 columns, odd
  static constexpr int C_LD = 25;                     // Cb row stride (odd)
  static constexpr int P_LD = 56;                     // P tile: up to 48 key columns + 8 (ldmatrix, conflict-free)
  static constexpr int kThLd = 20;
  static constexpr int oQ = 0;
  static constexpr int oK = oQ + RS * LD * 2;
  static constexpr int oV = oK + RK * LD * 2;
  static constexpr int oSb = oV + RV * LD * 2;
  static constexpr int oC = oSb + RS * SB_LD * 4;
  static constexpr int oP = oC + R * C_LD * 4;
  static constexpr int oStat = oP + R * P_LD * 2;     // alpha [R], 1/l [R]
  static constexpr int oTheta = oStat + 2 * R * 4;
  static constexpr int kSmemBytes = oTheta + 16 * kThLd * 4;
};

template <int D, int CQ, int CK>   // filter shape at compile time, or (0, 0): read from the parameters
__global__ void __launch_bounds__(FwdBandCfg<D>::NT, 2) fwd_band_kernel(const TrainParams p) {
  using Cfg = FwdBandCfg<D>;
  constexpr int NT = Cfg::NT, R = Cfg::R, RS = Cfg::RS, RK = Cfg::RK, RV = Cfg::RV, LD = Cfg::LD;
  constexpr int SB_LD = Cfg::SB_LD, C_LD = Cfg::C_LD, P_LD = Cfg::P_LD, kThLd = Cfg::kThLd;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + Cfg::oQ);
  bf16* sK = reinterpret_cast<bf16*>(smem + Cfg::oK);
  bf16* sV = reinterpret_cast<bf16*>(smem + Cfg::oV);
  float* sSb = reinterpret_cast<float*>(smem + Cfg::oSb);
  float* sC = reinterpret_cast<float*>(smem + Cfg::oC);
  bf16* sP = reinterpret_cast<bf16*>(smem + Cfg::oP);
  float* sAlpha = reinterpret_cast<float*>(smem + Cfg::oStat);
  float* sInvL = sAlpha + R;
  float* sTheta = reinterpret_cast<float*>(smem + Cfg::oTheta);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H, cq = (CQ > 0) ? CQ : p.cq, ck = (CQ > 0) ? CK : p.ck;
  const int pq = cq - 1, pk = (ck - 1) / 2;
  const int band = p.causal ? pq + pk : 0;            // no causal mask: no band, normalise only
  const int W = band > 0 ? band + pk : 0;
  const int h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * H + h;
  const int t0 = win_lo(p) + blockIdx.x * R;          // a window starts on a multiple of R
  const int koff = (band > 16) ? 32 : 16;             // the P tile of 16 rows starts koff keys before them
  pdl_trigger();
  pdl_wait();                                         // launched with programmatic stream serialization

  if (band > 0) {
    load_rows_async<D, NT>(sQ, LD, p.Q + bh * (size_t)N * D, t0 - 16, RS, N, tid);
    load_rows_async<D, NT>(sK, LD, p.K + bh * (size_t)N * D, t0 - 48, RK, N, tid);
    load_rows_async<D, NT>(sV, LD, p.V + bh * (size_t)N * D, t0 - 32, RV, N, tid);
    cp_async_commit();
    for (int i = tid; i < cq * ck; i += NT) sTheta[(i / ck) * kThLd + (i % ck)] = p.theta[((size_t)h * cq) * ck + i];
    for (int i = tid; i < RS * SB_LD; i += NT) sSb[i] = 0.f;
    for (int i = tid; i < R * P_LD / 2; i += NT) reinterpret_cast<uint32_t*>(sP)[i] = 0u;
    cp_async_wait<0>();
  }
  __syncthreads();

  if (band > 0) {
    // ---- Sb on 16 x 16 tiles along the diagonal ----
    const int nkt = (W > 17) ? 3 : 2;
    for (int job = warp; job < (RS / 16) * nkt; job += NT / 32) {
      const int m = job / nkt, kt = job % nkt;
      const int krow = 16 * m + 32 - 16 * (nkt - 1) + 16 * kt;
      float acc[2][4] = {};
      warp_gemm<2, false, false>(acc, sQ + 16 * m * LD, LD, sK + krow * LD, LD, D, lane);
      const int eoff = 16 * (nkt - 1 - kt);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int x = (lane >> 2) + 8 * hh, y = 8 * j + 2 * (lane & 3) + u;
            const int e = x - y + eoff;
            if (e >= 0 && e < W) sSb[(16 * m + x) * SB_LD + band + e] = acc[j][2 * hh + u] * p.scale;
          }
    }
    __syncthreads();

    // ---- conv ----
    if constexpr (CQ > 0) {
      // compile-time filter: a thread owns half of the diagonals of one row and keeps the score
      // segment each filter row needs in registers
      constexpr int PQ = CQ - 1, PK = (CK - 1) / 2, BAND = PQ + PK, HB = (BAND + 1) / 2, SEG = HB + CK - 1;
      if (tid < 2 * R) {
        const int x = tid >> 1, half = tid & 1;
        const int d0 = half * HB, cnt = half ? BAND - HB : HB;
        float c[HB];
#pragma unroll
        for (int i = 0; i < HB; ++i) c[i] = 0.f;
#pragma unroll
        for (int a = 0; a < CQ; ++a) {
          const float* row = sSb + (x + 16 - PQ + a) * SB_LD + BAND + d0 + a - PQ + PK - (CK - 1);
          float seg[SEG];
#pragma unroll
          for (int i = 0; i < SEG; ++i) seg[i] = row[i];
#pragma unroll
          for (int bb = 0; bb < CK; ++bb) {
            const float w = sTheta[a * kThLd + bb];
#pragma unroll
            for (int i = 0; i < HB; ++i) c[i] = fmaf(w, seg[i + (CK - 1 - bb)], c[i]);
          }
        }
#pragma unroll
        for (int i = 0; i < HB; ++i)
          if (i < cnt) sC[x * C_LD + d0 + i] = c[i];
      }
    } else {
    // run-time filter: (row, diagonal) pairs, KC per thread side by side
    constexpr int KC = (CQ > 0) ? (R * (CQ - 1 + (CK - 1) / 2) + NT - 1) / NT : (R * Cfg::MAXBAND + NT - 1) / NT;
    const int nout = R * band;
    float c[KC];
    const float* rp[KC];
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int o = min(tid + k * NT, nout - 1);
      const int x = o / band, dd = o - x * band;
      rp[k] = sSb + (x + 16 - pq) * SB_LD + band + dd - pq + pk;
      c[k] = 0.f;
    }
#pragma unroll
    for (int a = 0; a < cq; ++a) {
      const float* th = sTheta + a * kThLd;
#pragma unroll
      for (int bb = 0; bb < ck; ++bb) {
        const float w = th[bb];
#pragma unroll
        for (int k = 0; k < KC; ++k) c[k] = fmaf(w, rp[k][a * (SB_LD + 1) - bb], c[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int o = tid + k * NT;
      if (o < nout) { const int x = o / band; sC[x * C_LD + (o - x * band)] = c[k]; }
    }
    }
    __syncthreads();
  }

  // ---- merge with the partial softmax state: one thread per row ----
  if (tid < R) {
    const int gi = t0 + tid;
    if (gi < N) {
      const float m_old = p.Mpart[bh * N + gi], l_old = p.Lpart[bh * N + gi];
      float m_new = m_old;
      for (int dd = 0; dd < band; ++dd)
        if (gi - dd >= 0) m_new = fmaxf(m_new, sC[tid * C_LD + dd]);
      const float alpha = (m_old == -INFINITY) ? 0.f : exp2f((m_old - m_new) * kLog2e);
      float l = l_old * alpha;
      const int xin = tid & 15;
      bf16* prow = sP + tid * P_LD + xin + koff;     // column of key i - dd is xin + koff - dd
      for (int dd = 0; dd < band; ++dd) {
        if (gi - dd >= 0) {
          const float pr = exp2f((sC[tid * C_LD + dd] - m_new) * kLog2e);
          l += pr;
          prow[-dd] = __float2bfloat16(pr);
        }
      }
      sAlpha[tid] = alpha;
      sInvL[tid] = l > 0.f ? 1.f / l : 0.f;
      if (p.M) p.M[bh * N + gi] = m_new;
      if (p.L) p.L[bh * N + gi] = l;
      if (p.LSEout) p.LSEout[bh * N + gi] = m_new + logf(l);
    } else {
      sAlpha[tid] = 0.f;
      sInvL[tid] = 0.f;
    }
  }
  __syncthreads();

  // ---- O = (alpha * Opart + P V) / l on 16 x 32 output tiles ----
  constexpr int CT = D / 32;                          // column tiles of 32
  for (int job = warp; job < (R / 16) * CT; job += NT / 32) {
    const int m = job / CT, ctile = job % CT;
    const int x0 = 16 * m + (lane >> 2), x1 = x0 + 8;
    const int g0 = t0 + x0, g1 = t0 + x1;
    const float a0 = sAlpha[x0], a1 = sAlpha[x1];
    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = ctile * 32 + j * 8 + (lane & 3) * 2;
      float2 v0 = make_float2(0.f, 0.f), v1 = v0;
      if (g0 < N) v0 = *reinterpret_cast<const float2*>(p.Opart + (bh * N + g0) * D + col);
      if (g1 < N) v1 = *reinterpret_cast<const float2*>(p.Opart + (bh * N + g1) * D + col);
      acc[j][0] = v0.x * a0; acc[j][1] = v0.y * a0; acc[j][2] = v1.x * a1; acc[j][3] = v1.y * a1;
    }
    if (band > 0)
      warp_gemm<4, false, true>(acc, sP + 16 * m * P_LD, P_LD, sV + (16 * m + 32 - koff) * LD + ctile * 32, LD, koff + 16, lane);
    const float i0 = sInvL[x0], i1 = sInvL[x1];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int col = ctile * 32 + j * 8 + (lane & 3) * 2;
      const float o00 = acc[j][0] * i0, o01 = acc[j][1] * i0, o10 = acc[j][2] * i1, o11 = acc[j][3] * i1;
      if (p.o_bf16) {
        bf16* O = reinterpret_cast<bf16*>(p.O);
        if (g0 < N) *reinterpret_cast<uint32_t*>(O + (bh * N + g0) * D + col) = pack_bf16(o00, o01);
        if (g1 < N) *reinterpret_cast<uint32_t*>(O + (bh * N + g1) * D + col) = pack_bf16(o10, o11);
      } else {
        float* O = reinterpret_cast<float*>(p.O);
        if (g0 < N) *reinterpret_cast<float2*>(O + (bh * N + g0) * D + col) = make_float2(o00, o01);
        if (g1 < N) *reinterpret_cast<float2*>(O + (bh * N + g1) * D + col) = make_float2(o10, o11);
      }
    }
  }
}

template <int D>
static cudaError_t launch_fwd_band_t(const TrainParams& p, cudaStream_t stream) {
  using Cfg = FwdBandCfg<D>;
  dim3 grid((win_hi(p) - win_lo(p) + Cfg::R - 1) / Cfg::R, p.H, p.B);
  if (p.cq == 6 && p.ck == 11)
    return launch_kernel<TrainParams>(fwd_band_kernel<D, 6, 11>, grid, dim3(Cfg::NT), Cfg::kSmemBytes, stream, -1, p);
  if (p.cq == 7 && p.ck == 7)
    return launch_kernel<TrainParams>(fwd_band_kernel<D, 7, 7>, grid, dim3(Cfg::NT), Cfg::kSmemBytes, stream, -1, p);
  if (p.cq == 3 && p.ck == 5)
    return launch_kernel<TrainParams>(fwd_band_kernel<D, 3, 5>, grid, dim3(Cfg::NT), Cfg::kSmemBytes, stream, -1, p);
  return launch_kernel<TrainParams>(fwd_band_kernel<D, 0, 0>, grid, dim3(Cfg::NT), Cfg::kSmemBytes, stream, -1, p);
}

// Finishes the forward started by the stacked tensor-core kernel: band entries + normalisation.
cudaError_t launch_fwd_band(const TrainParams& p, cudaStream_t stream) {
  ScopedKernelTimer timer_(kKernFwdExact, stream);
  if (p.d == 64) return launch_fwd_band_t<64>(p, stream);
  return launch_fwd_band_t<128>(p, stream);
}

}  // namespace fmta
