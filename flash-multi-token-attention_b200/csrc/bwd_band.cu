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
constexpr int D = 64;
constexpr int NT = 256;
constexpr int MAXPQ = 5, MAXPK = 8;                 // c_q <= 6, c_k <= 17
constexpr int MAXBAND = MAXPQ + MAXPK;              // 13
constexpr int MAXW = MAXBAND + MAXPK;               // 21
constexpr int RC = 96;                              // dC rows computed per CTA (6 tiles of 16)
constexpr int RS = RC + 16;                         // Sb / Q rows: start 16 rows earlier
constexpr int RK = RC + 48;                         // K rows: start 48 rows earlier
constexpr int LD = D + 8;                           // bf16 row stride (ldmatrix without bank conflicts)
constexpr int SB_LD = 37;                           // band (zero pad for e < 0) + W columns, odd
constexpr int DC_LD = 43;                           // pad_k + band + pad_q + 2 pad_k columns, odd
constexpr int P_LD = 13;
constexpr int DS_LD = 21;
constexpr int oQ = 0;
constexpr int oK = oQ + RS * LD * 2;
constexpr int oV = oK + RK * LD * 2;                // V rows; later reused for the padded dC rows
constexpr int kVBytes = (RS * LD * 2 > RC * DC_LD * 4) ? RS * LD * 2 : RC * DC_LD * 4;
constexpr int odO = oV + kVBytes;
constexpr int oSb = odO + RC * LD * 2;
constexpr int oP = oSb + RS * SB_LD * 4;            // dPb, overwritten in place by P
constexpr int odS = oP + RC * P_LD * 4;
constexpr int oLD = odS + RC * DS_LD * 4;           // LSE*log2e [RC], D [RC]
constexpr int oTheta = oLD + 2 * RC * 4;
constexpr int oRed = oTheta + 6 * kThetaLdBand * 4;
constexpr int kSmemBytes = oRed + NT * 4;
}  // namespace bandcfg

// positions owned per CTA for a filter shape
inline int bwd_band_positions(int cq, int ck) {
  const int pq = cq - 1, pk = (ck - 1) / 2;
  const int r = bandcfg::RC - (pq + 2 * pk - 1 + pq);
  return r < bandcfg::RC ? r : bandcfg::RC;
}

__global__ void __launch_bounds__(bandcfg::NT, 2) bwd_band_kernel(const TrainParams p) {
  using namespace bandcfg;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + oQ);
  bf16* sK = reinterpret_cast<bf16*>(smem + oK);
  bf16* sV = reinterpret_cast<bf16*>(smem + oV);
  float* sdC = reinterpret_cast<float*>(smem + oV);
  bf16* sdO = reinterpret_cast<bf16*>(smem + odO);
  float* sSb = reinterpret_cast<float*>(smem + oSb);
  float* sP = reinterpret_cast<float*>(smem + oP);
  float* sdS = reinterpret_cast<float*>(smem + odS);
  float* sLse = reinterpret_cast<float*>(smem + oLD);
  float* sDv = sLse + RC;
  float* sTheta = reinterpret_cast<float*>(smem + oTheta);
  float* sRed = reinterpret_cast<float*>(smem + oRed);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H, cq = p.cq, ck = p.ck;
  const int pq = cq - 1, pk = (ck - 1) / 2, band = pq + pk, W = band + pk;
  const int R = min(RC, RC - (W - 1 + pq));
  const int h = blockIdx.y, b = blockIdx.z;
  const size_t bh = (size_t)b * H + h;
  const int t0 = blockIdx.x * R;
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

  // ---- conv, P and dC: one (row, diagonal) pair at a time ----
  for (int o = tid; o < RC * band; o += NT) {
    const int x = o / band, dd = o - x * band;
    const int gi = t0 + x;
    float c = 0.f;
    for (int a = 0; a < cq; ++a) {
      const float* row = sSb + (x + 16 - pq + a) * SB_LD + band + dd + a - pq + pk;
      const float* th = sTheta + a * kThetaLdBand;
      for (int bb = 0; bb < ck; ++bb) c = fmaf(th[bb], row[-bb], c);
    }
    const bool live = (gi < N) && (gi - dd >= 0);
    const float pr = live ? exp2f(c * kLog2e - sLse[x]) : 0.f;
    const float dp = sP[x * P_LD + dd];
    sP[x * P_LD + dd] = pr;
    sdC[x * DC_LD + pk + dd] = pr * (dp - sDv[x]);
  }
  __syncthreads();

  // ---- dTheta: one thread per tap, row groups in parallel ----
  {
    const int ntaps = cq * ck;
    const int ngroups = NT / ntaps;
    const int g = tid / ntaps, tap = tid - g * ntaps;
    float t = 0.f;
    if (g < ngroups) {
      const int a = tap / ck, bb = tap - a * ck;
      for (int x = g; x < R; x += ngroups) {
        const float* rs = sSb + (x + 16 - pq + a) * SB_LD + band + a - pq + pk - bb;
        const float* rc = sdC + x * DC_LD + pk;
        for (int dd = 0; dd < band; ++dd) t = fmaf(rc[dd], rs[dd], t);
      }
    }
    sRed[tid] = t;
  }
  // ---- adjoint conv: dSb[i', e] for the rows that feed the owned positions ----
  {
    const int nrows = R + W - 1;
    for (int o = tid; o < nrows * W; o += NT) {
      const int xr = o / W, e = o - xr * W;
      float s = 0.f;
      for (int a = 0; a < cq; ++a) {
        const float* row = sdC + (xr + pq - a) * DC_LD + e - a + pq;   // column pk + (e - a + pq - pk + b)
        const float* th = sTheta + a * kThetaLdBand;
        for (int bb = 0; bb < ck; ++bb) s = fmaf(th[bb], row[bb], s);
      }
      sdS[xr * DS_LD + e] = s * p.scale;
    }
  }
  __syncthreads();
  {
    const int ntaps = cq * ck;
    if (tid < ntaps) {
      const int ngroups = NT / ntaps;
      float t = 0.f;
      for (int g = 0; g < ngroups; ++g) t += sRed[g * ntaps + tid];
      const int slot = b * gridDim.x + blockIdx.x;
      p.dTheta_part[((size_t)slot * H + h) * ntaps + tid] = t;
    }
  }

  // ---- dQ, dK, dV of the owned positions: one warp per position, two head dims per lane ----
  for (int xr = warp; xr < R; xr += NT / 32) {
    const int t = t0 + xr;
    if (t >= N) break;
    float* gq = p.dQ + (bh * N + t) * D + 2 * lane;
    float* gk = p.dK + (bh * N + t) * D + 2 * lane;
    float* gv = p.dV + (bh * N + t) * D + 2 * lane;
    float2 aq = *reinterpret_cast<const float2*>(gq);
    float2 ak = *reinterpret_cast<const float2*>(gk);
    float2 av = *reinterpret_cast<const float2*>(gv);
    for (int e = 0; e < W; ++e) {
      const float s1 = sdS[xr * DS_LD + e];
      const __nv_bfloat162 kk = *reinterpret_cast<const __nv_bfloat162*>(sK + (xr + 48 - e) * LD + 2 * lane);
      aq.x = fmaf(s1, __low2float(kk), aq.x); aq.y = fmaf(s1, __high2float(kk), aq.y);
      const float s2 = sdS[(xr + e) * DS_LD + e];
      const __nv_bfloat162 qq = *reinterpret_cast<const __nv_bfloat162*>(sQ + (xr + 16 + e) * LD + 2 * lane);
      ak.x = fmaf(s2, __low2float(qq), ak.x); ak.y = fmaf(s2, __high2float(qq), ak.y);
    }
    for (int dd = 0; dd < band; ++dd) {
      const float pr = sP[(xr + dd) * P_LD + dd];
      const __nv_bfloat162 oo = *reinterpret_cast<const __nv_bfloat162*>(sdO + (xr + dd) * LD + 2 * lane);
      av.x = fmaf(pr, __low2float(oo), av.x); av.y = fmaf(pr, __high2float(oo), av.y);
    }
    *reinterpret_cast<float2*>(gq) = aq;
    *reinterpret_cast<float2*>(gk) = ak;
    *reinterpret_cast<float2*>(gv) = av;
  }
}

bool bwd_band_supported(const TrainParams& p) {
  const int pq = p.cq - 1, pk = (p.ck - 1) / 2;
  return p.theta != nullptr && p.Wmix == nullptr && p.d == bandcfg::D && pq <= bandcfg::MAXPQ && pk <= bandcfg::MAXPK;
}

int bwd_band_theta_slots(int B, int N, int cq, int ck) {
  const int R = bwd_band_positions(cq, ck);
  return B * ((N + R - 1) / R);
}

// Adds the band part of dQ/dK/dV and writes one dTheta partial per CTA into p.dTheta_part
// ([slots][H][cq*ck]).  Nothing to do when the filter has no band (pad_q + pad_k == 0).
cudaError_t launch_bwd_band(const TrainParams& p, cudaStream_t stream) {
  const int R = bwd_band_positions(p.cq, p.ck);
  dim3 grid((p.N + R - 1) / R, p.H, p.B);
  ScopedKernelTimer timer_(kKernBwdBand, stream);
  return launch_kernel<TrainParams>(bwd_band_kernel, grid, dim3(bandcfg::NT), bandcfg::kSmemBytes, stream, 1, p);
}

}  // namespace fmta
