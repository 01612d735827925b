// Backward of the causal band: the entries 0 <= i - j < pad_q + pad_k that the stacked-GEMM
// tensor-core kernels leave out (there the conv window reaches zero-masked future scores, so
// the "stacked GEMM" identity does not hold).
//
// The band is thin (pad_q + pad_k diagonals), so everything is kept in (row, diagonal)
// coordinates instead of 64 x 64 tiles:
//   Sb[i, e]  = scale * q_i . k_{i-e}            e in [0, W),  W = pad_q + 2 pad_k     (mma.sync)
//   dPb[i, d] = dO_i . v_{i-d}                   d in [0, band), band = pad_q + pad_k   (mma.sync)
//   Cb[i, d]  = sum_{a,b} theta[a,b] Sb[i-pad_q+a, d+a-pad_q+pad_k-b]   (Sb = 0 for e < 0: future)
//   P = exp(Cb - LSE_i),  dC = P (dPb - D_i)
//   dTheta[a,b] += sum_{i,d} dC[i,d] Sb[i-pad_q+a, d+a-pad_q+pad_k-b]
//   dSb[i, e] = scale * sum_{a,b} theta[a,b] dC[i+pad_q-a, e-a+pad_q-pad_k+b]
//   dQ_i += sum_e dSb[i,e] k_{i-e};  dK_j += sum_e dSb[j+e,e] q_{j+e};  dV_j += sum_d P[j+d,d] dO_{j+d}
// One CTA owns R consecutive positions (as query rows for dQ, as keys for dK/dV, as rows for
// dTheta) and recomputes the halo of dC rows above them, so that no two CTAs add into the same
// output element: the result is deterministic.  dQ/dK/dV are ADDED to what the tensor-core
// kernels wrote before.
#include "fmta_common.cuh"
#include "fmta_params.h"
#include "launch_util.cuh"

namespace fmta {

namespace bandcfg {
constexpr int kThetaLdBand = 20;                     // filter row stride in shared memory (c_k <= 17)
constexpr int NT = 256;
constexpr int MAXPQ = 6, MAXPK = 8;                 // c_q <= 7, c_k <= 17
constexpr int MAXBAND = MAXPQ + MAXPK;              // 14
constexpr int MAXW = MAXBAND + MAXPK;               // 22
constexpr int RC = 96;                              // dC rows computed per CTA (6 tiles of 16)
constexpr int RS = RC + 16;                         // Sb / Q rows: start 16 rows earlier
constexpr int RK = RC + 48;                         // K rows: start 48 rows earlier
constexpr int SB_LD = 37;                           // band (zero pad for e < 0) + W columns, odd
constexpr int DC_LD = 45;                           // pad_k + band + pad_q + 2 pad_k columns (<= 44), odd
constexpr int P_LD = 15;
constexpr int DS_LD = 23;
constexpr int A_LD = 40;                            // bf16 operand tiles of the output GEMMs: 32 columns + 8 (ldmatrix)
// shared-memory layout for head dim D
template <int D>
struct Layout {
  static constexpr int LD = D + 8;                  // bf16 row stride (ldmatrix without bank conflicts)
  static constexpr int oQ = 0;
  static constexpr int oK = oQ + RS * LD * 2;
  static constexpr int oV = oK + RK * LD * 2;       // V rows; later reused for the padded dC rows
  static constexpr int kVBytes = (RS * LD * 2 > RC * DC_LD * 4) ? RS * LD * 2 : RC * DC_LD * 4;
  static constexpr int odO = oV + kVBytes;
  static constexpr int oSb = odO + RC * LD * 2;
  static constexpr int oP = oSb + RS * SB_LD * 4;   // dPb, overwritten in place by P
  static constexpr int odS = oP + RC * P_LD * 4;
  static constexpr int oLD = odS + RC * DS_LD * 4;  // LSE*log2e [RC], D [RC]
  static constexpr int oTheta = oLD + 2 * RC * 4;
  static constexpr int oRed = oTheta + 7 * kThetaLdBand * 4;
  static constexpr int kSmemBytes = oRed + NT * 4;
  static constexpr int kCtasPerSm = (2 * kSmemBytes <= 225 * 1024) ? 2 : 1;
};
}  // namespace bandcfg

// positions owned per CTA for a filter shape
inline int bwd_band_positions(int cq, int ck) {
  const int pq = cq - 1, pk = (ck - 1) / 2;
  const int r = bandcfg::RC - (pq + 2 * pk - 1 + pq);
  return r < bandcfg::RC ? r : bandcfg::RC;
}


template <int D, int CQ, int CK>   // head dim; filter shape at compile time, or (0, 0): read from the parameters
__global__ void __launch_bounds__(bandcfg::NT, bandcfg::Layout<D>::kCtasPerSm) bwd_band_kernel(const TrainParams p) {
  using namespace bandcfg;
  using BL = Layout<D>;
  constexpr int LD = BL::LD, oQ = BL::oQ, oK = BL::oK, oV = BL::oV, odO = BL::odO, oSb = BL::oSb, oP = BL::oP;
  constexpr int odS = BL::odS, oLD = BL::oLD, oTheta = BL::oTheta, oRed = BL::oRed;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + oQ);
  bf16* sK = reinterpret_cast<bf16*>(smem + oK);
  bf16* sV = reinterpret_cast<bf16*>(smem + oV);
  float* sdC = reinterpret_cast<float*>(smem + oV);
  bf16* sdO = reinterpret_cast<bf16*>(smem + odO);
  float* sSb = reinterpret_cast<float*>(smem + oSb);
  float* sP = reinterpret_cast<float*>(smem + oP);
  float* sdS = reinterpret_cast<float*>(smem + odS);
  // with W <= 17 the output phase runs on mma.sync from dense bf16 tiles: P in the dS buffer's place,
  // dS (two arrangements) in the Sb buffer's place once dTheta no longer needs Sb
  bf16* sAV = reinterpret_cast<bf16*>(smem + odS);
  bf16* sAQ = reinterpret_cast<bf16*>(smem + oSb);
  bf16* sAK = sAQ + RC * A_LD;
  float* sLse = reinterpret_cast<float*>(smem + oLD);
  float* sDv = sLse + RC;
  float* sTheta = reinterpret_cast<float*>(smem + oTheta);
  float* sRed = reinterpret_cast<float*>(smem + oRed);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H, cq = (CQ > 0) ? CQ : p.cq, ck = (CQ > 0) ? CK : p.ck;
  const int pq = cq - 1, pk = (ck - 1) / 2, band = pq + pk, W = band + pk;
  const int Rt = min(RC, RC - (W - 1 + pq));           // positions per CTA
  const bool mma_out = (W <= 17);
  const int h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * H + h;
  const int t0 = win_lo(p) + blockIdx.x * Rt;
  const int R = p.row_hi > 0 ? min(Rt, p.row_hi - t0) : Rt;   // a call with a window owns no position past its end
  pdl_trigger();
  pdl_wait();                                          // launched with programmatic stream serialization
  const bf16* Qg = p.Q + bh * (size_t)N * D;
  const bf16* Kg = p.K + bh * (size_t)N * D;
  const bf16* Vg = p.V + bh * (size_t)N * D;
  const bf16* dOg = p.dO + bh * (size_t)N * D;

  load_rows_async<D, NT>(sQ, LD, Qg, t0 - 16, RS, N, tid);
  load_rows_async<D, NT>(sK, LD, Kg, t0 - 48, RK, N, tid);
  load_rows_async<D, NT>(sV, LD, Vg, t0 - 16, RS, N, tid);
  load_rows_async<D, NT>(sdO, LD, dOg, t0, RC, N, tid);
  cp_async_commit();
  for (int i = tid; i < cq * ck; i += NT) sTheta[(i / ck) * kThetaLdBand + (i % ck)] = p.theta[((size_t)h * cq) * ck + i];
  for (int i = tid; i < RS * SB_LD; i += NT) sSb[i] = 0.f;
  if (mma_out) for (int i = tid; i < RC * A_LD / 2; i += NT) reinterpret_cast<uint32_t*>(sAV)[i] = 0u;
  if (tid < RC) {
    const int gi = t0 + tid;
    sLse[tid] = gi < N ? p.LSE[bh * N + gi] * kLog2e : 0.f;
    sDv[tid] = gi < N ? p.Dvec[bh * N + gi] : 0.f;
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- Sb and dPb on 16 x 16 tiles along the diagonal ----
  {
    const int nkt = (W > 17) ? 3 : 2;
    const int nS = (RS / 16) * nkt, nP = (RC / 16) * 2;
    for (int job = warp; job < nS + nP; job += NT / 32) {
      float acc[2][4] = {};
      if (job < nS) {
        const int m = job / nkt, kt = job % nkt;
        const int krow = 16 * m + 32 - 16 * (nkt - 1) + 16 * kt;
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
      } else {
        const int jj = job - nS, m = jj >> 1, kt = jj & 1;
        warp_gemm<2, false, false>(acc, sdO + 16 * m * LD, LD, sV + (16 * m + 16 * kt) * LD, LD, D, lane);
        const int doff = 16 * (1 - kt);
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const int x = (lane >> 2) + 8 * hh, y = 8 * j + 2 * (lane & 3) + u;
              const int dd = x - y + doff;
              if (dd >= 0 && dd < band) sP[(16 * m + x) * P_LD + dd] = acc[j][2 * hh + u];
            }
      }
    }
  }
  __syncthreads();

  // ---- the padded dC rows take over the V buffer ----
  for (int i = tid; i < RC * DC_LD; i += NT) sdC[i] = 0.f;
  __syncthreads();

  // ---- conv, P and dC ----
  if constexpr (CQ > 0) {
    // compile-time filter: a thread owns half of the diagonals of one row and keeps the score
    // segment each filter row needs in registers (one shared-memory load per ~5 FMAs)
    constexpr int PQ = CQ - 1, PK = (CK - 1) / 2, BAND = PQ + PK, HB = (BAND + 1) / 2, SEG = HB + CK - 1;
    if (tid < 2 * RC) {
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
          const float w = sTheta[a * kThetaLdBand + bb];
#pragma unroll
          for (int i = 0; i < HB; ++i) c[i] = fmaf(w, seg[i + (CK - 1 - bb)], c[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < HB; ++i) {
        if (i < cnt) {
          const int dd = d0 + i;
          const float cval = c[i];
      const int gi = t0 + x;
          const bool live = (gi < N) && (gi - dd >= 0);
          const float pr = live ? exp2f(cval * kLog2e - sLse[x]) : 0.f;
          const float dp = sP[x * P_LD + dd];
          sdC[x * DC_LD + pk + dd] = pr * (dp - sDv[x]);
          if (mma_out) {            // P^T operand of dV: row = key position x - dd, column = x relative to that key's tile
            const int j = x - dd;
            if (j >= 0) sAV[j * A_LD + x - (j & ~15)] = __float2bfloat16(pr);
          } else {
            sP[x * P_LD + dd] = pr;
          }
        }
      }
    }
  } else
  if (band > 0) {   // run-time filter: (row, diagonal) pairs, KC per thread side by side for ILP
    constexpr int KC = (CQ > 0) ? (RC * (CQ - 1 + (CK - 1) / 2) + NT - 1) / NT : (RC * MAXBAND + NT - 1) / NT;
    const int nout = RC * band;
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
      const float* th = sTheta + a * kThetaLdBand;
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
      if (o < nout) {
        const int x = o / band, dd = o - x * band;
        const int gi = t0 + x;
        const bool live = (gi < N) && (gi - dd >= 0);
        const float pr = live ? exp2f(c[k] * kLog2e - sLse[x]) : 0.f;
        const float dp = sP[x * P_LD + dd];
        sdC[x * DC_LD + pk + dd] = pr * (dp - sDv[x]);
        if (mma_out) {            // P^T operand of dV: row = key position x - dd, column = x relative to that key's tile
          const int j = x - dd;
          if (j >= 0) sAV[j * A_LD + x - (j & ~15)] = __float2bfloat16(pr);
        } else {
          sP[x * P_LD + dd] = pr;
        }
      }
    }
  }
  __syncthreads();

  // ---- dTheta ----
  if constexpr (CQ > 0) {
    // one warp per filter row a, lanes over the owned rows; the dC row and the score segment live in registers
    constexpr int PQ = CQ - 1, PK = (CK - 1) / 2, BAND = PQ + PK, SEG = BAND + CK - 1;
    if (warp < CQ) {
      const int a = warp;
      float t[CK];
#pragma unroll
      for (int bb = 0; bb < CK; ++bb) t[bb] = 0.f;
      for (int x = lane; x < R; x += 32) {
        float dc[BAND], seg[SEG];
        const float* rc = sdC + x * DC_LD + PK;
        const float* row = sSb + (x + 16 - PQ + a) * SB_LD + BAND + a - PQ + PK - (CK - 1);
#pragma unroll
        for (int i = 0; i < BAND; ++i) dc[i] = rc[i];
#pragma unroll
        for (int i = 0; i < SEG; ++i) seg[i] = row[i];
#pragma unroll
        for (int bb = 0; bb < CK; ++bb)
#pragma unroll
          for (int i = 0; i < BAND; ++i) t[bb] = fmaf(dc[i], seg[i + (CK - 1 - bb)], t[bb]);
      }
#pragma unroll
      for (int bb = 0; bb < CK; ++bb) {
        const float v = warp_sum(t[bb]);
        if (lane == 0) sRed[a * CK + bb] = v;
      }
    }
  } else
  {   // run-time filter: one thread per tap, row groups in parallel; the columns past the band are zero
    const int ntaps = cq * ck;
    const int ngroups = NT / ntaps;
    const int g = tid / ntaps, tap = tid - g * ntaps;
    float t0s = 0.f, t1s = 0.f;
    if (g < ngroups) {
      const int a = tap / ck, bb = tap - a * ck;
      const float* rs = sSb + (16 - pq + a) * SB_LD + band + a - pq + pk - bb;
      const float* rc = sdC + pk;
      constexpr int NB = (CQ > 0) ? (CQ - 1 + (CK - 1) / 2) : MAXBAND;
      int x = g;
      for (; x + ngroups < R; x += 2 * ngroups) {
        const float* rs0 = rs + x * SB_LD; const float* rc0 = rc + x * DC_LD;
        const float* rs1 = rs0 + ngroups * SB_LD; const float* rc1 = rc0 + ngroups * DC_LD;
#pragma unroll
        for (int dd = 0; dd < NB; ++dd) { t0s = fmaf(rc0[dd], rs0[dd], t0s); t1s = fmaf(rc1[dd], rs1[dd], t1s); }
      }
      if (x < R) {
        const float* rs0 = rs + x * SB_LD; const float* rc0 = rc + x * DC_LD;
#pragma unroll
        for (int dd = 0; dd < NB; ++dd) t0s = fmaf(rc0[dd], rs0[dd], t0s);
      }
    }
    sRed[tid] = t0s + t1s;
  }
  if (mma_out) {      // Sb is dead now: its place takes the two dense arrangements of dS
    __syncthreads();
    for (int i = tid; i < 2 * RC * A_LD / 2; i += NT) reinterpret_cast<uint32_t*>(sAQ)[i] = 0u;
    __syncthreads();
  }
  // ---- adjoint conv: dSb[i', e] for the rows that feed the owned positions ----
  if constexpr (CQ > 0) {
    // a thread owns half of the diagonals e of one row; the dC segment of each filter row in registers
    constexpr int PQ = CQ - 1, PK = (CK - 1) / 2, WW = PQ + 2 * PK, HW = (WW + 1) / 2, SEG = HW + CK - 1;
    if (tid < 2 * (R + WW - 1)) {
      const int xr = tid >> 1, half = tid & 1;
      const int e0 = half * HW, cnt = half ? WW - HW : HW;
      float sa[HW];
#pragma unroll
      for (int i = 0; i < HW; ++i) sa[i] = 0.f;
#pragma unroll
      for (int a = 0; a < CQ; ++a) {
        const float* row = sdC + (xr + PQ - a) * DC_LD + e0 - a + PQ;   // column pk + (e - a + pq - pk + b)
        float seg[SEG];
#pragma unroll
        for (int i = 0; i < SEG; ++i) seg[i] = row[i];
#pragma unroll
        for (int bb = 0; bb < CK; ++bb) {
          const float w = sTheta[a * kThetaLdBand + bb];
#pragma unroll
          for (int i = 0; i < HW; ++i) sa[i] = fmaf(w, seg[i + bb], sa[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < HW; ++i) {
        if (i < cnt) {
          const int e = e0 + i;
          const float sval = sa[i];
        const float v = sval * p.scale;
          if (mma_out) {
            const bf16 vb = __float2bfloat16(v);
            sAQ[xr * A_LD + (xr & 15) - e + 16] = vb;            // dQ: row = query position, column = key relative to (tile start - 16)
            const int j = xr - e;
            if (j >= 0) sAK[j * A_LD + xr - (j & ~15)] = vb;     // dK: row = key position, column = query relative to the key's tile
          } else {
            sdS[xr * DS_LD + e] = v;
          }
        }
      }
    }
  } else
  if (W > 0) {   // run-time filter
    constexpr int KA = (CQ > 0) ? ((RC - (CQ - 1)) * (CQ - 1 + CK - 1) + NT - 1) / NT : (RC * MAXW + NT - 1) / NT;
    const int nout = (R + W - 1) * W;
    float sacc[KA];
    const float* rp[KA];
#pragma unroll
    for (int k = 0; k < KA; ++k) {
      const int o = min(tid + k * NT, nout - 1);
      const int xr = o / W, e = o - xr * W;
      rp[k] = sdC + (xr + pq) * DC_LD + e + pq;   // tap (a, b) reads column pk + (e - a + pq - pk + b) of row xr + pq - a
      sacc[k] = 0.f;
    }
#pragma unroll
    for (int a = 0; a < cq; ++a) {
      const float* th = sTheta + a * kThetaLdBand;
#pragma unroll
      for (int bb = 0; bb < ck; ++bb) {
        const float w = th[bb];
#pragma unroll
        for (int k = 0; k < KA; ++k) sacc[k] = fmaf(w, rp[k][bb - a * (DC_LD + 1)], sacc[k]);
      }
    }
#pragma unroll
    for (int k = 0; k < KA; ++k) {
      const int o = tid + k * NT;
      if (o < nout) {
        const int xr = o / W, e = o - xr * W;
        const float v = sacc[k] * p.scale;
        if (mma_out) {
          const bf16 vb = __float2bfloat16(v);
          sAQ[xr * A_LD + (xr & 15) - e + 16] = vb;            // dQ: row = query position, column = key relative to (tile start - 16)
          const int j = xr - e;
          if (j >= 0) sAK[j * A_LD + xr - (j & ~15)] = vb;     // dK: row = key position, column = query relative to the key's tile
        } else {
          sdS[xr * DS_LD + e] = v;
        }
      }
    }
  }
  __syncthreads();
  {
    const int ntaps = cq * ck;
    if (tid < ntaps) {
      const int ngroups = (CQ > 0) ? 1 : NT / ntaps;
      float t = 0.f;
      for (int g = 0; g < ngroups; ++g) t += sRed[g * ntaps + tid];
      const int slot = b * gridDim.x + blockIdx.x;
      p.dTheta_part[((size_t)slot * H + h) * ntaps + tid] = t;
    }
  }

  if (mma_out) {
    // ---- dQ, dK, dV on mma.sync: 16 positions x 32 head dims per job, accumulating onto the values in memory ----
    const int ntile = (R + 15) / 16;
    constexpr int NCH = D / 32;                                          // 32-column chunks of the head dim
    for (int job = warp; job < ntile * 3 * NCH; job += NT / 32) {
      const int m = job / (3 * NCH), which = (job % (3 * NCH)) / NCH, ch = job % NCH;      // which: 0 dQ, 1 dK, 2 dV
      const int x0 = 16 * m + (lane >> 2), x1 = x0 + 8;
      const bool ok0 = (x0 < R) && (t0 + x0 < N), ok1 = (x1 < R) && (t0 + x1 < N);
      float* gout = (which == 0) ? p.dQ : (which == 1) ? p.dK : p.dV;
      float* g0 = gout + (bh * N + t0 + x0) * D + ch * 32 + (lane & 3) * 2;
      float* g1 = gout + (bh * N + t0 + x1) * D + ch * 32 + (lane & 3) * 2;
      float acc[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 v0 = make_float2(0.f, 0.f), v1 = v0;
        if (ok0) v0 = *reinterpret_cast<const float2*>(g0 + j * 8);
        if (ok1) v1 = *reinterpret_cast<const float2*>(g1 + j * 8);
        acc[j][0] = v0.x; acc[j][1] = v0.y; acc[j][2] = v1.x; acc[j][3] = v1.y;
      }
      const int kd = (m == RC / 16 - 1 && which != 0) ? 16 : 32;        // the last tile must not read past the Q / dO rows
      const bf16* A = (which == 0) ? sAQ : (which == 1) ? sAK : sAV;
      const bf16* Bm = (which == 0) ? sK + (16 * m + 32) * LD : (which == 1) ? sQ + (16 * m + 16) * LD : sdO + (16 * m) * LD;
      warp_gemm<4, false, true>(acc, A + 16 * m * A_LD, A_LD, Bm + ch * 32, LD, kd, lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (ok0) *reinterpret_cast<float2*>(g0 + j * 8) = make_float2(acc[j][0], acc[j][1]);
        if (ok1) *reinterpret_cast<float2*>(g1 + j * 8) = make_float2(acc[j][2], acc[j][3]);
      }
    }
  } else {
  // ---- dQ, dK, dV of the owned positions: one warp per position (two at a time), two head dims per lane ----
    for (int xr0 = warp; xr0 < R; xr0 += 2 * (NT / 32)) {
      const int xr1 = xr0 + NT / 32;
      const int ta = t0 + xr0, tb = t0 + xr1;
      if (ta >= N) break;
      const bool two = (xr1 < R) && (tb < N);
      const int xb = two ? xr1 : xr0;                       // second position (a repeat of the first when absent)
     for (int c0 = 0; c0 < D; c0 += 64) {                   // 64 head dims per pass of the warp
      const int col = c0 + 2 * lane;
      float* ga = p.dQ + (bh * N + ta) * D + col;
      float* gb = p.dQ + (bh * N + t0 + xb) * D + col;
      const ptrdiff_t kofs = p.dK - p.dQ, vofs = p.dV - p.dQ;  // element offsets between the three outputs
      float2 aq0 = *reinterpret_cast<const float2*>(ga), ak0 = *reinterpret_cast<const float2*>(ga + kofs), av0 = *reinterpret_cast<const float2*>(ga + vofs);
      float2 aq1 = *reinterpret_cast<const float2*>(gb), ak1 = *reinterpret_cast<const float2*>(gb + kofs), av1 = *reinterpret_cast<const float2*>(gb + vofs);
#pragma unroll 3
      for (int e = 0; e < W; ++e) {
        const float s10 = sdS[xr0 * DS_LD + e], s11 = sdS[xb * DS_LD + e];
        const float s20 = sdS[(xr0 + e) * DS_LD + e], s21 = sdS[(xb + e) * DS_LD + e];
        const __nv_bfloat162 k0 = *reinterpret_cast<const __nv_bfloat162*>(sK + (xr0 + 48 - e) * LD + col);
        const __nv_bfloat162 k1 = *reinterpret_cast<const __nv_bfloat162*>(sK + (xb + 48 - e) * LD + col);
        const __nv_bfloat162 q0 = *reinterpret_cast<const __nv_bfloat162*>(sQ + (xr0 + 16 + e) * LD + col);
        const __nv_bfloat162 q1 = *reinterpret_cast<const __nv_bfloat162*>(sQ + (xb + 16 + e) * LD + col);
        aq0.x = fmaf(s10, __low2float(k0), aq0.x); aq0.y = fmaf(s10, __high2float(k0), aq0.y);
        aq1.x = fmaf(s11, __low2float(k1), aq1.x); aq1.y = fmaf(s11, __high2float(k1), aq1.y);
        ak0.x = fmaf(s20, __low2float(q0), ak0.x); ak0.y = fmaf(s20, __high2float(q0), ak0.y);
        ak1.x = fmaf(s21, __low2float(q1), ak1.x); ak1.y = fmaf(s21, __high2float(q1), ak1.y);
      }
#pragma unroll 2
      for (int dd = 0; dd < band; ++dd) {
        const float p0 = sP[(xr0 + dd) * P_LD + dd], p1 = sP[(xb + dd) * P_LD + dd];
        const __nv_bfloat162 o0 = *reinterpret_cast<const __nv_bfloat162*>(sdO + (xr0 + dd) * LD + col);
        const __nv_bfloat162 o1 = *reinterpret_cast<const __nv_bfloat162*>(sdO + (xb + dd) * LD + col);
        av0.x = fmaf(p0, __low2float(o0), av0.x); av0.y = fmaf(p0, __high2float(o0), av0.y);
        av1.x = fmaf(p1, __low2float(o1), av1.x); av1.y = fmaf(p1, __high2float(o1), av1.y);
      }
      *reinterpret_cast<float2*>(ga) = aq0; *reinterpret_cast<float2*>(ga + kofs) = ak0; *reinterpret_cast<float2*>(ga + vofs) = av0;
      if (two) { *reinterpret_cast<float2*>(gb) = aq1; *reinterpret_cast<float2*>(gb + kofs) = ak1; *reinterpret_cast<float2*>(gb + vofs) = av1; }
     }
    }
  }
}


int bwd_band_theta_slots(int B, int N, int cq, int ck) {
  const int R = bwd_band_positions(cq, ck);
  return B * ((N + R - 1) / R);
}

// Adds the band part of dQ/dK/dV and writes one dTheta partial per CTA into p.dTheta_part
// ([slots][H][cq*ck]).  Nothing to do when the filter has no band (pad_q + pad_k == 0).
template <int D>
static cudaError_t launch_bwd_band_d(const TrainParams& p, dim3 grid, cudaStream_t stream) {
  constexpr int smem = bandcfg::Layout<D>::kSmemBytes;
  if (p.cq == 6 && p.ck == 11)
    return launch_kernel<TrainParams>(bwd_band_kernel<D, 6, 11>, grid, dim3(bandcfg::NT), smem, stream, -1, p);
  if (p.cq == 7 && p.ck == 7 && D == 64)
    return launch_kernel<TrainParams>(bwd_band_kernel<D, 7, 7>, grid, dim3(bandcfg::NT), smem, stream, -1, p);
  if (p.cq == 3 && p.ck == 5)
    return launch_kernel<TrainParams>(bwd_band_kernel<D, 3, 5>, grid, dim3(bandcfg::NT), smem, stream, -1, p);
  return launch_kernel<TrainParams>(bwd_band_kernel<D, 0, 0>, grid, dim3(bandcfg::NT), smem, stream, -1, p);
}

cudaError_t launch_bwd_band(const TrainParams& p, cudaStream_t stream) {
  const int R = bwd_band_positions(p.cq, p.ck);
  dim3 grid((win_hi(p) - win_lo(p) + R - 1) / R, p.H, p.B);
  ScopedKernelTimer timer_(kKernBwdBand, stream);
  if (p.d == 128) return launch_bwd_band_d<128>(p, grid, stream);
  return launch_bwd_band_d<64>(p, grid, stream);
}

}  // namespace fmta
