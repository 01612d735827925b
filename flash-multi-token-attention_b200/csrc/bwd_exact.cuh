// Exact conv-attention backward tile kernels.
//
// For a 64x64 (query block, key block) tile both kernels recompute, in shared memory,
//   S   on rows [i0-16, i0+80) x keys [j0-16, j0+80)   (zero-masked, scaled)          mma.sync
//   C   = conv(S) and P = exp(C - LSE) on rows [i0, i0+80) x keys [j0-8, j0+72)       FP32 pipe
//   dP  = dO V^T on the same region, dC = P * (dP - D)                                mma.sync
//   [mix] C'_g = sum W[g,g'] C_g' before P;  dW[g,g'] += sum dC'_g C_g';  dC_g' = sum_g W[g,g'] dC'_g
//         across the G heads of a thread-block cluster through distributed shared memory
//   dTheta[a,b] += sum_{owned} dC[i,j] S[i+a-pad_q, j+b-pad_k]                          FP32 pipe
//   dS  = adjoint conv(dC) on the owned 64x64 tile, zeroed where key > query          FP32 pipe
// The extended regions are what the conv and its adjoint need so that the owned tile is exact;
// they are recomputed per tile instead of read-modify-writing dQ/dK/dV in HBM.
//
//   bwd_dq_kernel  : one CTA per query block, loops key blocks;   dQ = scale * sum dS K, dTheta, dW
//   bwd_dkdv_kernel: one CTA per key block,   loops query blocks; dK = scale * sum dS^T Q, dV = sum P^T dO
// dTheta / dW leave the kernel as one partial per CTA slot (summed in a fixed order by
// reduce_partials_kernel) so the result does not depend on scheduling.
#pragma once
#include <cooperative_groups.h>

#include "conv_tile.cuh"
#include "fmta_common.cuh"
#include "fmta_params.h"

namespace fmta {
namespace cg = cooperative_groups;

template <int D, int CQ, int CK, bool MIX>
struct BwdExactCfg {
  static constexpr bool kNoConv = (CQ == 1 && CK == 1);
  static constexpr int NT = 256;
  static constexpr int BR = 64, BC = 64;
  static constexpr int H1 = kNoConv ? 0 : 16;  // halo rows after the block (dC region) / before (S region)
  static constexpr int HC = kNoConv ? 0 : 8;   // halo columns per side of the dC region
  static constexpr int ER = BR + H1, EC = BC + 2 * HC;       // region of C, P, dP, dC
  static constexpr int SR = BR + 2 * H1, SC = BC + 4 * HC;   // region of S
  static constexpr int S_LD = SC + 4, E_LD = EC + 4;
  static constexpr int QK_LD = D + 8;
  static constexpr int B_LD = BC + 8;  // bf16 P / dS tiles
  static constexpr int oQ = 0;
  static constexpr int oK = oQ + SR * QK_LD * 2;
  static constexpr int odO = oK + SR * QK_LD * 2;
  static constexpr int oV = odO + ER * QK_LD * 2;
  static constexpr int oS = oV + ER * QK_LD * 2;
  static constexpr int oE = oS + SR * S_LD * 4;
  static constexpr int oX = oE + ER * E_LD * 4;               // MIX only: own C, later final dC
  static constexpr int oPb = oX + (MIX ? ER * E_LD * 4 : 0);
  static constexpr int oDS = oPb + BR * B_LD * 2;
  static constexpr int oLSE = oDS + BR * B_LD * 2;
  static constexpr int oTheta = oLSE + 2 * ER * 4;
  static constexpr int oW = oTheta + kMaxCQ * kThetaLd * 4;
  static constexpr int oDTh = oW + 256 * 4;                  // [8 warps][kMaxCQ*kThetaLd]
  static constexpr int oDW = oDTh + 8 * kMaxCQ * kThetaLd * 4;  // [8 warps][64]
  static constexpr int kSmemBytes = oDW + 8 * 64 * 4;
};

// Sum 16 per-lane values across the warp with a reduce-scatter butterfly (16 shuffles instead
// of 80).  On return lanes with (lane & 1) == 0 hold in `out` the warp total of value index
// idx = 8*bit4 + 4*bit3 + 2*bit2 + bit1 of their lane id.
FMTA_DEVINL float reduce_scatter16(float (&v)[16], int lane, int& idx) {
  const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4, b1 = lane & 2;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float send = b4 ? v[k] : v[k + 8], keep = b4 ? v[k + 8] : v[k];
    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float send = b3 ? v[k] : v[k + 4], keep = b3 ? v[k + 4] : v[k];
    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
  }
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    const float send = b2 ? v[k] : v[k + 2], keep = b2 ? v[k + 2] : v[k];
    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
  }
  {
    const float send = b1 ? v[0] : v[1], keep = b1 ? v[1] : v[0];
    v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  v[0] += __shfl_xor_sync(0xffffffffu, v[0], 1);
  idx = (b4 ? 8 : 0) + (b3 ? 4 : 0) + (b2 ? 2 : 0) + (b1 ? 1 : 0);
  return v[0];
}

template <int D, int CQ, int CK, bool MIX>
struct BwdSmem {
  using Cfg = BwdExactCfg<D, CQ, CK, MIX>;
  bf16 *sQ, *sK, *sdO, *sV, *sPb, *sDS;
  float *sS, *sE, *sX, *sLSE, *sDv, *sTheta, *sW, *sDTh, *sDW;
  __device__ explicit BwdSmem(unsigned char* base) {
    sQ = reinterpret_cast<bf16*>(base + Cfg::oQ);
    sK = reinterpret_cast<bf16*>(base + Cfg::oK);
    sdO = reinterpret_cast<bf16*>(base + Cfg::odO);
    sV = reinterpret_cast<bf16*>(base + Cfg::oV);
    sS = reinterpret_cast<float*>(base + Cfg::oS);
    sE = reinterpret_cast<float*>(base + Cfg::oE);
    sX = reinterpret_cast<float*>(base + Cfg::oX);
    sPb = reinterpret_cast<bf16*>(base + Cfg::oPb);
    sDS = reinterpret_cast<bf16*>(base + Cfg::oDS);
    sLSE = reinterpret_cast<float*>(base + Cfg::oLSE);
    sDv = sLSE + Cfg::ER;
    sTheta = reinterpret_cast<float*>(base + Cfg::oTheta);
    sW = reinterpret_cast<float*>(base + Cfg::oW);
    sDTh = reinterpret_cast<float*>(base + Cfg::oDTh);
    sDW = reinterpret_cast<float*>(base + Cfg::oDW);
  }
};

// Steps shared by both kernels for one (i0, j0) tile.  Expects sQ (rows i0-H1..), sK (keys
// j0-2HC..), sdO (rows i0..), sV (keys j0-HC..), sLSE/sDv (rows i0..) to be loaded and visible.
// Leaves bf16 P (owned tile) in sPb and bf16 dS (owned tile) in sDS, visible CTA-wide.
template <int D, int CQ, int CK, bool MIX, bool WANT_DTHETA>
FMTA_DEVINL void bwd_tile(const BwdSmem<D, CQ, CK, MIX>& sm, const TrainParams& p, int i0, int j0,
                          int cq, int ck, int G, int grank, int tid, const float* xbase = nullptr, size_t xstride = 0,
                          float* xme = nullptr) {
  // head mix: xme != nullptr -> the heads' tiles are exchanged through global memory (slot A: own C, slot B:
  // dC'; xbase = slot pair of head 0 of the group, xstride floats between heads), else through distributed
  // shared memory
  using Cfg = BwdExactCfg<D, CQ, CK, MIX>;
  constexpr int BR = Cfg::BR, H1 = Cfg::H1, HC = Cfg::HC, ER = Cfg::ER, EC = Cfg::EC;
  constexpr int SR = Cfg::SR, SC = Cfg::SC, S_LD = Cfg::S_LD, E_LD = Cfg::E_LD, QK_LD = Cfg::QK_LD;
  constexpr int B_LD = Cfg::B_LD;
  const int lane = tid & 31, warp = tid >> 5;
  const int N = p.N;
  const bool causal = p.causal != 0;
  const int pq = cq - 1, pk = (ck - 1) / 2;
  // the adjoint conv of the owned rows reads dC rows up to pad_q below them: the rows of the E region beyond
  // that (it is laid out for pad_q = 15) are neither computed nor exchanged
  const int er_eff = Cfg::kNoConv ? ER : min(ER, BR + pq);
  // band mode: entries with query - key >= pad_q + pad_k belong to the stacked tensor-core kernels

  // ---- 1. S on the large region ----
  {
    constexpr int NU = (SR / 16) * (SC / 16);
    for (int u = warp; u < NU; u += Cfg::NT / 32) {
      const int um = u / (SC / 16), un = u % (SC / 16);
      float acc[2][4] = {};
      warp_gemm<2, false, false>(acc, sm.sQ + um * 16 * QK_LD, QK_LD, sm.sK + un * 16 * QK_LD, QK_LD, D, lane);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = um * 16 + (lane >> 2) + hh * 8;
          const int c = un * 16 + j * 8 + (lane & 3) * 2;
          const int qi = i0 - H1 + r, kj = j0 - 2 * HC + c;
          float v0 = acc[j][2 * hh] * p.scale, v1 = acc[j][2 * hh + 1] * p.scale;
          if (causal && !Cfg::kNoConv) {
            if (kj > qi) v0 = 0.f;
            if (kj + 1 > qi) v1 = 0.f;
          }
          *reinterpret_cast<float2*>(sm.sS + r * S_LD + c) = make_float2(v0, v1);
        }
    }
  }
  __syncthreads();

  // ---- 2. C = conv(S) on the E region -> (mix) -> P = exp(C - LSE), masked ----
  float* cown = MIX ? sm.sX : sm.sE;  // where this head's own conv output goes
  for (int t = tid; t < er_eff * (EC / 16); t += Cfg::NT) {
    const int r = t % er_eff, s = t / er_eff;
    float acc[16];
    if constexpr (!Cfg::kNoConv) {
      conv_strip<CQ, CK, HC - (CK - 1) / 2, false>(acc, sm.sS, S_LD, r, s, H1 - pq, sm.sTheta, cq, ck, HC - pk);
    } else {
      const float4* src = reinterpret_cast<const float4*>(sm.sS + r * S_LD + s * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) { float4 v = src[i]; acc[4*i] = v.x; acc[4*i+1] = v.y; acc[4*i+2] = v.z; acc[4*i+3] = v.w; }
    }
    if constexpr (!MIX) {
      const int qi = i0 + r;
      const float lse = sm.sLSE[r];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kj = j0 - HC + s * 16 + i;
        const bool ok = (qi < N) && (kj >= 0) && (kj < N) && !(causal && kj > qi);
        acc[i] = ok ? exp2f((acc[i] - lse) * kLog2e) : 0.f;
      }
    }
    float4* o = reinterpret_cast<float4*>(cown + r * E_LD + s * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = make_float4(acc[4*i], acc[4*i+1], acc[4*i+2], acc[4*i+3]);
    if constexpr (MIX) {
      if (xme != nullptr) {
        float4* og = reinterpret_cast<float4*>(xme + r * E_LD + s * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) og[i] = make_float4(acc[4*i], acc[4*i+1], acc[4*i+2], acc[4*i+3]);
      }
    }
  }
  if constexpr (MIX) {
    cg::cluster_group cluster = cg::this_cluster();
    if (xme != nullptr) __threadfence();
    cluster.sync();  // every head's conv output is in its sX (and in its global slot)
    for (int t = tid; t < er_eff * (EC / 16); t += Cfg::NT) {
      const int r = t % er_eff, s = t / er_eff;
      float acc[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
      if (xme != nullptr) mix_global16(acc, xbase, xstride, r * E_LD + s * 16, sm.sW + grank * G, 1, G, grank, sm.sX);
      else mix_remote16(acc, cluster, sm.sX, r * E_LD + s * 16, sm.sW + grank * G, 1, G);
      const int qi = i0 + r;
      const float lse = sm.sLSE[r];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int kj = j0 - HC + s * 16 + i;
        const bool ok = (qi < N) && (kj >= 0) && (kj < N) && !(causal && kj > qi);
        acc[i] = ok ? exp2f((acc[i] - lse) * kLog2e) : 0.f;
      }
      float4* o = reinterpret_cast<float4*>(sm.sE + r * E_LD + s * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = make_float4(acc[4*i], acc[4*i+1], acc[4*i+2], acc[4*i+3]);
    }
  }
  __syncthreads();

  // ---- 3. dP = dO V^T on the E region; dC = P * (dP - D) in place; bf16 P of the owned tile ----
  {
    constexpr int NU = (ER / 16) * (EC / 16);
    for (int u = warp; u < NU; u += Cfg::NT / 32) {
      const int um = u / (EC / 16), un = u % (EC / 16);
      if (um * 16 >= er_eff) continue;
      float acc[2][4] = {};
      warp_gemm<2, false, false>(acc, sm.sdO + um * 16 * QK_LD, QK_LD, sm.sV + un * 16 * QK_LD, QK_LD, D, lane);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = um * 16 + (lane >> 2) + hh * 8;
          const int c = un * 16 + j * 8 + (lane & 3) * 2;
          float2* pe = reinterpret_cast<float2*>(sm.sE + r * E_LD + c);
          const float2 pv = *pe;
          const float dv = sm.sDv[r];
          if (r < BR && c >= HC && c < HC + Cfg::BC)
            *reinterpret_cast<uint32_t*>(sm.sPb + r * B_LD + (c - HC)) = pack_bf16(pv.x, pv.y);
          *pe = make_float2(pv.x * (acc[j][2 * hh] - dv), pv.y * (acc[j][2 * hh + 1] - dv));
        }
    }
  }
  float* dcfin = sm.sE;  // final per-head dC (after the transposed mix)
  if constexpr (MIX) {
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();
    if (xme != nullptr) {   // publish dC' (slot B)
      for (int t = tid; t < er_eff * (EC / 16); t += Cfg::NT) {
        const int r = t % er_eff, s = t / er_eff;
        const float4* src = reinterpret_cast<const float4*>(sm.sE + r * E_LD + s * 16);
        float4* og = reinterpret_cast<float4*>(xme + kMixXchFloats + r * E_LD + s * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) og[i] = src[i];
      }
      __threadfence();
    }
    cluster.sync();  // all dC' tiles complete, all remote reads of sX (own C) done
    // Transposed mix dC_own = sum_g W[g, own] dC'_g, and (dQ kernel) column `own` of dW on the way:
    // dW[g, own] += sum over the owned tile of dC'_g * C_own -- the dC' strips of all heads pass through this
    // CTA's registers here anyway, and C_own is the strip of sX that the result is about to replace.
    const int nstrips = er_eff * (EC / 16);
    for (int t0 = 0; t0 < nstrips; t0 += Cfg::NT) {        // warp-uniform trip count (the dW sums use shuffles)
      const int t = t0 + tid;
      const bool live = t < nstrips;
      const int r = live ? t % er_eff : 0, s = live ? t / er_eff : 0;
      float acc[16], cown[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = 0.f;
      if constexpr (WANT_DTHETA) {
        const float4* src = reinterpret_cast<const float4*>(sm.sX + r * E_LD + s * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float4 v = src[i]; cown[4*i] = v.x; cown[4*i+1] = v.y; cown[4*i+2] = v.z; cown[4*i+3] = v.w; }
#pragma unroll
        for (int i = 0; i < 16; ++i) {                     // owned tile: rows < BR, region columns HC .. HC + BC
          const int c = s * 16 + i;
          if (!live || r >= BR || c < HC || c >= HC + Cfg::BC) cown[i] = 0.f;
        }
      }
      for (int g0 = 0; g0 < G; g0 += 4) {                  // the loads of four heads are issued together
        float4 v[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int g2 = min(g0 + u, G - 1);
          const bool glob = (xme != nullptr) && g2 != grank;
          const float4* src = glob
              ? reinterpret_cast<const float4*>(xbase + kMixXchFloats + (size_t)g2 * xstride + r * E_LD + s * 16)
              : reinterpret_cast<const float4*>(cluster.map_shared_rank(sm.sE, g2) + r * E_LD + s * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) v[u][i] = glob ? __ldcg(src + i) : src[i];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float wv = (g0 + u < G) ? sm.sW[(g0 + u) * G + grank] : 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            acc[4*i] = fmaf(wv, v[u][i].x, acc[4*i]); acc[4*i+1] = fmaf(wv, v[u][i].y, acc[4*i+1]);
            acc[4*i+2] = fmaf(wv, v[u][i].z, acc[4*i+2]); acc[4*i+3] = fmaf(wv, v[u][i].w, acc[4*i+3]);
          }
          if constexpr (WANT_DTHETA) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              a = fmaf(cown[4*i], v[u][i].x, a); a = fmaf(cown[4*i+1], v[u][i].y, a);
              a = fmaf(cown[4*i+2], v[u][i].z, a); a = fmaf(cown[4*i+3], v[u][i].w, a);
            }
            a = warp_sum(a);
            if (lane == 0 && g0 + u < G) sm.sDW[warp * 64 + g0 + u] += a;
          }
        }
      }
      if (live) {
        float4* o = reinterpret_cast<float4*>(sm.sX + r * E_LD + s * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = make_float4(acc[4*i], acc[4*i+1], acc[4*i+2], acc[4*i+3]);
      }
    }
    if (xme != nullptr) __syncthreads();   // sX now holds this head's dC (the slots alternate between tiles: no barrier needed after the reads)
    else cluster.sync();                   // remote reads of sE done; sX now holds this head's dC
    dcfin = sm.sX;
  } else {
    __syncthreads();
  }

  // ---- 4. dTheta partial over the owned tile ----
  if constexpr (WANT_DTHETA && !Cfg::kNoConv) {
    const int r = tid & 63, s = tid >> 6;
    float dcv[16];
    {
      const float4* src = reinterpret_cast<const float4*>(dcfin + r * E_LD + HC + s * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) { float4 v = src[i]; dcv[4*i] = v.x; dcv[4*i+1] = v.y; dcv[4*i+2] = v.z; dcv[4*i+3] = v.w; }
    }
    float* dth = sm.sDTh + warp * (kMaxCQ * kThetaLd);
    if constexpr (CQ > 0) {
      constexpr int WIN_C = 2 * HC - (CK - 1) / 2;   // S column of tap b=0 for owned column 0
      constexpr int MIS = WIN_C & 3;
      constexpr int NLOAD = (MIS + 16 + CK - 1 + 3) / 4;
#pragma unroll 1
      for (int a = 0; a < CQ; ++a) {
        const float4* src = reinterpret_cast<const float4*>(sm.sS + (r + H1 - (CQ - 1) + a) * S_LD + s * 16 + WIN_C - MIS);
        float v[NLOAD * 4];
#pragma unroll
        for (int i = 0; i < NLOAD; ++i) { float4 t4 = src[i]; v[4*i] = t4.x; v[4*i+1] = t4.y; v[4*i+2] = t4.z; v[4*i+3] = t4.w; }
        float acc[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) {
          acc[b] = 0.f;
          if (b < CK) {
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[b] = fmaf(dcv[i], v[MIS + i + b], acc[b]);
          }
        }
        int idx;
        const float tot = reduce_scatter16(acc, lane, idx);
        if (!(lane & 1) && idx < CK) dth[a * kThetaLd + idx] += tot;
        if constexpr (CK > 16) {  // one extra tap column beyond the 16-wide butterfly
          float e = 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) e = fmaf(dcv[i], v[MIS + i + 16], e);
          e = warp_sum(e);
          if (lane == 0) dth[a * kThetaLd + 16] += e;
        }
      }
    } else {
      for (int a = 0; a < cq; ++a) {
        const float* row = sm.sS + (r + H1 - pq + a) * S_LD + s * 16 + 2 * HC - pk;
        for (int b = 0; b < ck; ++b) {
          float e = 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) e = fmaf(dcv[i], row[i + b], e);
          e = warp_sum(e);
          if (lane == 0) dth[a * kThetaLd + b] += e;
        }
      }
    }
  }

  // ---- 5. dS = adjoint conv(dC) on the owned tile, causal zero, bf16 ----
  {
    const int r = tid & 63, s = tid >> 6;
    float acc[16];
    if constexpr (!Cfg::kNoConv) {
      conv_strip<CQ, CK, HC - (CK - 1) / 2, true>(acc, dcfin, E_LD, r, s, 0, sm.sTheta, cq, ck, HC - pk);
    } else {
      const float4* src = reinterpret_cast<const float4*>(dcfin + r * E_LD + s * 16);
#pragma unroll
      for (int i = 0; i < 4; ++i) { float4 v = src[i]; acc[4*i] = v.x; acc[4*i+1] = v.y; acc[4*i+2] = v.z; acc[4*i+3] = v.w; }
    }
    const int qi = i0 + r;
    uint32_t* o = reinterpret_cast<uint32_t*>(sm.sDS + r * B_LD + s * 16);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int kj = j0 + s * 16 + 2 * i;
      float v0 = acc[2 * i], v1 = acc[2 * i + 1];
      if (causal) {
        if (kj > qi) v0 = 0.f;
        if (kj + 1 > qi) v1 = 0.f;
      }
      o[i] = pack_bf16(v0, v1);
    }
  }
  __syncthreads();
}

template <int D, int CQ, int CK, bool MIX>
FMTA_DEVINL void bwd_load_theta_w(const BwdSmem<D, CQ, CK, MIX>& sm, const TrainParams& p, int h, int cq, int ck, int tid) {
  using Cfg = BwdExactCfg<D, CQ, CK, MIX>;
  if constexpr (!Cfg::kNoConv) {
    for (int i = tid; i < cq * ck; i += Cfg::NT)
      sm.sTheta[(i / ck) * kThetaLd + (i % ck)] = p.theta[((size_t)h * cq) * ck + i];
  }
  if constexpr (MIX) {
    if (tid < p.G * p.G) sm.sW[tid] = p.Wmix[(size_t)(h / p.G) * p.G * p.G + tid];
  }
  for (int i = tid; i < 8 * kMaxCQ * kThetaLd; i += Cfg::NT) sm.sDTh[i] = 0.f;
  for (int i = tid; i < 8 * 64; i += Cfg::NT) sm.sDW[i] = 0.f;
}

template <int D, int CQ, int CK, bool MIX>
FMTA_DEVINL void bwd_load_rowstats(const BwdSmem<D, CQ, CK, MIX>& sm, const TrainParams& p, size_t bh, int i0, int tid) {
  using Cfg = BwdExactCfg<D, CQ, CK, MIX>;
  if (tid < Cfg::ER) {
    const int gi = i0 + tid;
    const bool ok = gi < p.N;
    sm.sLSE[tid] = ok ? p.LSE[bh * p.N + gi] : 0.f;
    sm.sDv[tid] = ok ? p.Dvec[bh * p.N + gi] : 0.f;
  }
}

// ------------------------------------------------------------------------------------------
template <int D, int CQ, int CK, bool MIX>
__global__ void __launch_bounds__(256, 1) bwd_dq_kernel(const TrainParams p) {
  using Cfg = BwdExactCfg<D, CQ, CK, MIX>;
  constexpr int BR = Cfg::BR, BC = Cfg::BC, H1 = Cfg::H1, HC = Cfg::HC, QK_LD = Cfg::QK_LD, B_LD = Cfg::B_LD;
  extern __shared__ __align__(16) unsigned char smem[];
  BwdSmem<D, CQ, CK, MIX> sm(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H;
  const int nQB = (N + BR - 1) / BR, nKB = (N + BC - 1) / BC;
  const int qb = nQB - 1 - (int)blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int i0 = qb * BR;
  const int cq = (CQ > 0) ? CQ : p.cq, ck = (CQ > 0) ? CK : p.ck;
  const bool causal = p.causal != 0;
  const size_t bh = (size_t)b * H + h;
  const bf16* Qg = p.Q + bh * (size_t)N * D;
  const bf16* Kg = p.K + bh * (size_t)N * D;
  const bf16* Vg = p.V + bh * (size_t)N * D;
  const bf16* dOg = p.dO + bh * (size_t)N * D;
  const int G = MIX ? p.G : 1, grank = MIX ? (h % G) : 0;
  // head mix through global memory when the caller gave the scratch: this CTA's slot pair and its group's
  // (two sets of slots, used by alternate tiles)
  const size_t xstride = (size_t)gridDim.x * 2 * kMixXchFloats;
  const size_t xset = (size_t)gridDim.x * gridDim.y * gridDim.z * 2 * kMixXchFloats;
  const float* xbase0 = (MIX && p.xchg) ? p.xchg + (((size_t)b * H + (h / G) * G) * gridDim.x + blockIdx.x) * 2 * kMixXchFloats : nullptr;
  float* xme0 = (MIX && p.xchg) ? p.xchg + (((size_t)b * H + h) * gridDim.x + blockIdx.x) * 2 * kMixXchFloats : nullptr;

  bwd_load_theta_w<D, CQ, CK, MIX>(sm, p, h, cq, ck, tid);
  bwd_load_rowstats<D, CQ, CK, MIX>(sm, p, bh, i0, tid);
  load_rows_async<D, Cfg::NT>(sm.sQ, QK_LD, Qg, i0 - H1, Cfg::SR, N, tid);
  load_rows_async<D, Cfg::NT>(sm.sdO, QK_LD, dOg, i0, Cfg::ER, N, tid);
  cp_async_commit();

  const int kb_begin = 0, kb_end = causal ? min(nKB - 1, (i0 + BR - 1) / BC) : nKB - 1;
  constexpr int ONT = D / 16;
  float accQ[ONT][4] = {};
  const int mt = warp & 3, nh = warp >> 2;

  for (int kb = kb_begin; kb <= kb_end; ++kb) {
    const int j0 = kb * BC;
    load_rows_async<D, Cfg::NT>(sm.sK, QK_LD, Kg, j0 - 2 * HC, Cfg::SR, N, tid);
    load_rows_async<D, Cfg::NT>(sm.sV, QK_LD, Vg, j0 - HC, Cfg::ER, N, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    bwd_tile<D, CQ, CK, MIX, true>(sm, p, i0, j0, cq, ck, G, grank, tid, xbase0 ? xbase0 + (size_t)(kb & 1) * xset : nullptr, xstride,
                                   xme0 ? xme0 + (size_t)(kb & 1) * xset : nullptr);
    // dQ += dS K   (K rows of the owned key block start at row 2*HC of sK)
    warp_gemm<ONT, false, true>(accQ, sm.sDS + mt * 16 * B_LD, B_LD, sm.sK + (2 * HC) * QK_LD + nh * (D / 2), QK_LD, BC, lane);
    __syncthreads();
  }
  cp_async_wait<0>();

  // dQ = scale * acc
  {
    const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
    for (int j = 0; j < ONT; ++j) {
      const int col = nh * (D / 2) + j * 8 + (lane & 3) * 2;
      if (i0 + r0 < N) {
        float2* o = reinterpret_cast<float2*>(p.dQ + (bh * N + i0 + r0) * D + col);
        float2 v = make_float2(accQ[j][0] * p.scale, accQ[j][1] * p.scale);
        *o = v;
      }
      if (i0 + r1 < N) {
        float2* o = reinterpret_cast<float2*>(p.dQ + (bh * N + i0 + r1) * D + col);
        float2 v = make_float2(accQ[j][2] * p.scale, accQ[j][3] * p.scale);
        *o = v;
      }
    }
  }
  // per-CTA partials of dTheta and dW (fixed summation order over warps)
  __syncthreads();
  const int slot = b * nQB + qb;
  if constexpr (!Cfg::kNoConv) {
    if (p.dTheta_part != nullptr) {
      for (int i = tid; i < cq * ck; i += Cfg::NT) {
        const int a = i / ck, bb = i % ck;
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) t += sm.sDTh[w * (kMaxCQ * kThetaLd) + a * kThetaLd + bb];
        p.dTheta_part[((size_t)slot * H + h) * (cq * ck) + i] = t;
      }
    }
  }
  if constexpr (MIX) {
    if (p.dW_part != nullptr && tid < G) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) t += sm.sDW[w * 64 + tid];
      // column `grank` of this group's G x G matrix: dW[tid, grank] = sum dC'_tid * C_grank
      p.dW_part[((size_t)slot * (H / G) + h / G) * (G * G) + tid * G + grank] = t;
    }
  }
}

// ------------------------------------------------------------------------------------------
template <int D, int CQ, int CK, bool MIX>
__global__ void __launch_bounds__(256, 1) bwd_dkdv_kernel(const TrainParams p) {
  using Cfg = BwdExactCfg<D, CQ, CK, MIX>;
  constexpr int BR = Cfg::BR, BC = Cfg::BC, H1 = Cfg::H1, HC = Cfg::HC, QK_LD = Cfg::QK_LD, B_LD = Cfg::B_LD;
  extern __shared__ __align__(16) unsigned char smem[];
  BwdSmem<D, CQ, CK, MIX> sm(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H;
  const int nQB = (N + BR - 1) / BR;
  const int kb = blockIdx.x;  // early key blocks see the most query blocks -> already longest first
  const int h = blockIdx.y, b = blockIdx.z;
  const int j0 = kb * BC;
  const int cq = (CQ > 0) ? CQ : p.cq, ck = (CQ > 0) ? CK : p.ck;
  const bool causal = p.causal != 0;
  const size_t bh = (size_t)b * H + h;
  const bf16* Qg = p.Q + bh * (size_t)N * D;
  const bf16* Kg = p.K + bh * (size_t)N * D;
  const bf16* Vg = p.V + bh * (size_t)N * D;
  const bf16* dOg = p.dO + bh * (size_t)N * D;
  const int G = MIX ? p.G : 1, grank = MIX ? (h % G) : 0;
  // head mix through global memory when the caller gave the scratch: this CTA's slot pair and its group's
  // (two sets of slots, used by alternate tiles)
  const size_t xstride = (size_t)gridDim.x * 2 * kMixXchFloats;
  const size_t xset = (size_t)gridDim.x * gridDim.y * gridDim.z * 2 * kMixXchFloats;
  const float* xbase0 = (MIX && p.xchg) ? p.xchg + (((size_t)b * H + (h / G) * G) * gridDim.x + blockIdx.x) * 2 * kMixXchFloats : nullptr;
  float* xme0 = (MIX && p.xchg) ? p.xchg + (((size_t)b * H + h) * gridDim.x + blockIdx.x) * 2 * kMixXchFloats : nullptr;

  bwd_load_theta_w<D, CQ, CK, MIX>(sm, p, h, cq, ck, tid);
  load_rows_async<D, Cfg::NT>(sm.sK, QK_LD, Kg, j0 - 2 * HC, Cfg::SR, N, tid);
  load_rows_async<D, Cfg::NT>(sm.sV, QK_LD, Vg, j0 - HC, Cfg::ER, N, tid);
  cp_async_commit();

  const int qb_begin = causal ? (j0 / BR) : 0, qb_end = nQB - 1;
  constexpr int ONT = D / 16;
  float accK[ONT][4] = {}, accV[ONT][4] = {};
  const int mt = warp & 3, nh = warp >> 2;

  for (int qb = qb_begin; qb <= qb_end; ++qb) {
    const int i0 = qb * BR;
    bwd_load_rowstats<D, CQ, CK, MIX>(sm, p, bh, i0, tid);
    load_rows_async<D, Cfg::NT>(sm.sQ, QK_LD, Qg, i0 - H1, Cfg::SR, N, tid);
    load_rows_async<D, Cfg::NT>(sm.sdO, QK_LD, dOg, i0, Cfg::ER, N, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    bwd_tile<D, CQ, CK, MIX, false>(sm, p, i0, j0, cq, ck, G, grank, tid, xbase0 ? xbase0 + (size_t)(qb & 1) * xset : nullptr, xstride,
                                    xme0 ? xme0 + (size_t)(qb & 1) * xset : nullptr);
    // dV += P^T dO ; dK += dS^T Q   (A operands stored [query][key] -> transposed loads)
    warp_gemm<ONT, true, true>(accV, sm.sPb + mt * 16, B_LD, sm.sdO + nh * (D / 2), QK_LD, BR, lane);
    warp_gemm<ONT, true, true>(accK, sm.sDS + mt * 16, B_LD, sm.sQ + H1 * QK_LD + nh * (D / 2), QK_LD, BR, lane);
    __syncthreads();
  }
  cp_async_wait<0>();

  const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
  for (int j = 0; j < ONT; ++j) {
    const int col = nh * (D / 2) + j * 8 + (lane & 3) * 2;
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int r = hh ? r1 : r0;
      if (j0 + r < N) {
        float2* ok_ = reinterpret_cast<float2*>(p.dK + (bh * N + j0 + r) * D + col);
        float2* ov_ = reinterpret_cast<float2*>(p.dV + (bh * N + j0 + r) * D + col);
        float2 vk = make_float2(accK[j][2 * hh] * p.scale, accK[j][2 * hh + 1] * p.scale);
        float2 vv = make_float2(accV[j][2 * hh], accV[j][2 * hh + 1]);
        *ok_ = vk; *ov_ = vv;
      }
    }
  }
}

}  // namespace fmta
