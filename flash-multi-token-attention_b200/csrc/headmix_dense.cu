// Head mixing without a key-query conv -- the reference's head_conv_attn kernels (fwd_kernel.py:7-279,
// bwd_dq_dw.py:8-370, bwd_dk_dv.py:8-404):   C'_g = sum_g' W[g,g'] * scale * Q_g' K_g'^T,  softmax,  P V.
//
// All G heads of a mixing group live in ONE CTA, as in the reference (its Triton program holds all
// heads of a batch element on a 16 x 16 tile): every head's score tile is produced where the mix
// needs it, so nothing is exchanged between CTAs and G = 32 is no different from G = 4.  (The
// cluster kernels in fwd_exact.cuh / bwd_exact.cuh, which keep one head per CTA and read the other
// heads' tiles through distributed shared memory, move G^2 tiles per step over the SM-to-SM
// network and stop at 16 heads; they remain the path for a mix that follows a key-query conv.)
//
// Tiles are small -- 16 keys per step, 16 to 64 query rows -- because G of them are resident at a
// time.  A CTA has 16 warps; for the per-head products (mma.sync, operands in shared memory) warp w
// owns the (head, 16-row tile) items w, w + 16, ..., and keeps their output accumulators in
// registers for the whole loop.  The mix itself is G FMAs per score entry on the FP32 pipe, taken
// straight from the fp32 score tiles in shared memory by threads that own (head, row, 8 keys)
// and go on to the softmax (forward) or to dC' = P (dP - D) (backward) in registers.
//
//   hm_fwd_kernel      : CTA = (row tile, group, batch); loops key steps; O, M, L (and LSE)
//   hm_bwd_dq_kernel   : CTA = (row tile, group, batch); loops key steps; dQ and one dW partial per CTA
//                        (summed in a fixed order by reduce_partials_kernel)
//   hm_bwd_dkdv_kernel : CTA = (key tile, group, batch); loops 16-row steps; dK and dV (one launch each where the
//                        accumulators of both do not fit the registers)
#include <cuda_runtime.h>

#include "fmta_common.cuh"
#include "fmta_params.h"
#include "launch_util.cuh"

namespace fmta {
namespace hm {

constexpr int NW = 16, NT = NW * 32;   // warps and threads per CTA
constexpr int BC = 16;                 // keys per step (forward, dQ) / query rows per step (dK, dV)

template <int D, int G>
struct Cfg {
  static constexpr int MT = (G >= NW) ? 1 : ((NW / G) > 4 ? 4 : (NW / G));   // 16-row tiles per head
  static constexpr int BR = 16 * MT;                    // rows (forward, dQ) / keys (dK, dV) per head and tile
  static constexpr int ITEMS = G * MT;                  // (head, 16-row tile) items of a per-head product
  static constexpr int IPW = (ITEMS + NW - 1) / NW;     // items per warp (1, or 2 with 32 heads)
  static constexpr int LD = D + 8;                      // bf16 row stride of the operand tiles
  static constexpr int S_LD = BC;                       // fp32 score rows: 16 floats
  static constexpr int P_LD = BC + 8;                   // bf16 probability rows (48 bytes: ldmatrix without conflicts)
  static constexpr int TSET = G * BR * LD * 2;          // bytes of one operand tile set with BR rows per head
  static constexpr int KSET = G * BC * LD * 2;          // ... with 16 rows per head
  static constexpr int SSET = G * BR * S_LD * 4;        // bytes of the fp32 score tiles
  static constexpr int PSET = G * BR * P_LD * 2;
};

// Copy rows [row0, row0 + rows) of every head of the group into [g][rows][ld]; rows outside [0, N) are zero.
template <int D>
FMTA_DEVINL void load_set(bf16* dst, int ld, int rows, const bf16* __restrict__ base, size_t head_stride, int G,
                          int row0, int N, int tid) {
  constexpr int CPR = D / 8;
  const int per_head = rows * CPR;
  for (int idx = tid; idx < G * per_head; idx += NT) {
    const int g = idx / per_head, rem = idx - g * per_head;
    const int r = rem / CPR, c = rem - r * CPR;
    const int gr = row0 + r;
    const bool ok = gr >= 0 && gr < N;
    cp_async16(dst + ((size_t)g * rows + r) * ld + c * 8, base + g * head_stride + (size_t)(ok ? gr : 0) * D + c * 8, ok);
  }
}

// The fp32 score tiles are rows of 16 floats = four 16-byte chunks; chunk c of row r is stored at chunk
// c ^ ((r >> 1) & 3), so that the eight lanes of a quarter-warp -- four rows, two 8-key strips -- read their
// chunks from different banks (unswizzled, rows two apart share them: every load took two wavefronts, every
// fragment store four; the kernels are bound by shared-memory wavefronts).
FMTA_DEVINL int sw_chunk(int row, int chunk) { return chunk ^ ((row >> 1) & 3); }

// item -> (head, 16-row tile)
template <int G, int MT>
FMTA_DEVINL void item_of(int item, int& g, int& mt) {
  if (G >= NW) { g = item; mt = 0; }
  else { g = item % G; mt = item / G; }
}

// out[g][r][c] (fp32, row stride S_LD) = alpha * A_g[r,:] . B_g[c,:] for every item; A tiles have `a_rows`
// rows per head, B tiles BC rows per head.
template <int D, int G>
FMTA_DEVINL void head_products(float* out, const bf16* sA, int a_rows, const bf16* sB, float alpha, int warp, int lane) {
  using C = Cfg<D, G>;
#pragma unroll
  for (int i = 0; i < C::IPW; ++i) {
    const int item = warp + i * NW;
    if (item < C::ITEMS) {
      int g, mt;
      item_of<G, C::MT>(item, g, mt);
      float acc[2][4] = {};
      warp_gemm<2, false, false>(acc, sA + ((size_t)g * a_rows + mt * 16) * C::LD, C::LD, sB + (size_t)g * BC * C::LD, C::LD, D, lane);
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int r = mt * 16 + (lane >> 2) + hh * 8, c = j * 8 + (lane & 3) * 2;
          *reinterpret_cast<float2*>(out + ((size_t)g * a_rows + r) * C::S_LD + sw_chunk(r, c >> 2) * 4 + (c & 3)) =
              make_float2(acc[j][2 * hh] * alpha, acc[j][2 * hh + 1] * alpha);
        }
    }
  }
}

// The mix of one (row, 4 keys) quad for TWO output heads: acc[h][c] = sum_g2 w2[g2].{x,y} * S[g2][row][4q + c].
// `w2` points at the pair of weights of input head 0; consecutive input heads are `wstride` floats apart.
// One 16-byte load of scores and one 8-byte broadcast load of weights feed 8 FMAs.
template <int G>
FMTA_DEVINL void mix_quad(float (&acc)[2][4], const float* sS, int rows, int row, int q, const float* w2, int wstride) {
#pragma unroll
  for (int c = 0; c < 4; ++c) acc[0][c] = acc[1][c] = 0.f;
  const float* sp = sS + (size_t)row * BC + sw_chunk(row, q) * 4;
#pragma unroll 4
  for (int g2 = 0; g2 < G; ++g2) {
    const float4 a = *reinterpret_cast<const float4*>(sp + (size_t)g2 * rows * BC);
    const float2 wv = *reinterpret_cast<const float2*>(w2 + g2 * wstride);
    acc[0][0] = fmaf(wv.x, a.x, acc[0][0]); acc[0][1] = fmaf(wv.x, a.y, acc[0][1]);
    acc[0][2] = fmaf(wv.x, a.z, acc[0][2]); acc[0][3] = fmaf(wv.x, a.w, acc[0][3]);
    acc[1][0] = fmaf(wv.y, a.x, acc[1][0]); acc[1][1] = fmaf(wv.y, a.y, acc[1][1]);
    acc[1][2] = fmaf(wv.y, a.z, acc[1][2]); acc[1][3] = fmaf(wv.y, a.w, acc[1][3]);
  }
}

// ------------------------------------------------------------------------------------------
template <int D, int G>
struct FwdSmem {
  using C = Cfg<D, G>;
  static constexpr int kOne = C::TSET + C::KSET + C::SSET + C::PSET + 3 * G * C::BR * 4 + G * G * 4;
  static constexpr bool TWO = kOne + C::KSET <= 227 * 1024;     // K and V in buffers of their own: both copies run a phase ahead
  static constexpr int oQ = 0;
  static constexpr int oKV = oQ + C::TSET;
  static constexpr int oV2 = TWO ? oKV + C::KSET : oKV;
  static constexpr int oS = oV2 + C::KSET;
  static constexpr int oP = oS + C::SSET;
  static constexpr int oStat = oP + C::PSET;                 // M, L, alpha: [G][BR] each
  static constexpr int oWt = oStat + 3 * G * C::BR * 4;        // W transposed: [input head][output head]
  static constexpr int kBytes = oWt + G * G * 4;
  static_assert(kBytes <= 227 * 1024, "forward: shared memory budget");
};

template <int D, int G>
__global__ void __launch_bounds__(NT, 1) hm_fwd_kernel(const TrainParams p) {
  using C = Cfg<D, G>;
  using SM = FwdSmem<D, G>;
  constexpr int BR = C::BR, LD = C::LD, P_LD = C::P_LD;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + SM::oQ);
  bf16* sKV = reinterpret_cast<bf16*>(smem + SM::oKV);       // K, and V too without a second buffer
  bf16* sV2 = reinterpret_cast<bf16*>(smem + SM::oV2);       // V (= sKV without a second buffer)
  float* sS = reinterpret_cast<float*>(smem + SM::oS);
  bf16* sP = reinterpret_cast<bf16*>(smem + SM::oP);
  float* sM = reinterpret_cast<float*>(smem + SM::oStat);
  float* sL = sM + G * BR;
  float* sAlpha = sL + G * BR;
  float* sWt = reinterpret_cast<float*>(smem + SM::oWt);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H;
  const int nQB = (N + BR - 1) / BR, nKB = (N + BC - 1) / BC;
  const int qb = nQB - 1 - (int)blockIdx.x;              // long (late) row tiles first
  const int grp = blockIdx.y, b = blockIdx.z;
  const int i0 = qb * BR;
  const bool causal = p.causal != 0;
  const size_t hs = (size_t)N * D;                       // elements between heads
  const size_t bh0 = (size_t)b * H + (size_t)grp * G;    // first (batch, head) of the group
  const bf16* Qg = p.Q + bh0 * hs;
  const bf16* Kg = p.K + bh0 * hs;
  const bf16* Vg = p.V + bh0 * hs;

  for (int i = tid; i < G * G; i += NT) sWt[(i % G) * G + i / G] = p.Wmix[(size_t)grp * G * G + i];
  for (int i = tid; i < G * BR; i += NT) { sM[i] = -INFINITY; sL[i] = 0.f; }
  constexpr int ONT = D / 8;
  float accO[C::IPW][ONT][4];
#pragma unroll
  for (int i = 0; i < C::IPW; ++i)
#pragma unroll
    for (int j = 0; j < ONT; ++j) accO[i][j][0] = accO[i][j][1] = accO[i][j][2] = accO[i][j][3] = 0.f;

  const int kb_end = causal ? min(nKB - 1, (i0 + BR - 1) / BC) : nKB - 1;
  load_set<D>(sQ, LD, BR, Qg, hs, G, i0, N, tid);
  load_set<D>(sKV, LD, BC, Kg, hs, G, 0, N, tid);
  cp_async_commit();
  if (SM::TWO) {
    load_set<D>(sV2, LD, BC, Vg, hs, G, 0, N, tid);
    cp_async_commit();
  }

  // Copy groups are committed in the order K(0) [V(0)] K(1) V(1) ...; with two buffers one later group may
  // still be in flight at each wait (empty groups keep the count uniform at the end of the loop).
  for (int kb = 0; kb <= kb_end; ++kb) {
    const int j0 = kb * BC;
    if (SM::TWO) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();                                     // K(kb) (and Q) have landed
    head_products<D, G>(sS, sQ, BR, sKV, p.scale, warp, lane);
    __syncthreads();                                     // score tiles complete, K no longer read
    if (SM::TWO) {
      if (kb < kb_end) load_set<D>(sKV, LD, BC, Kg, hs, G, j0 + BC, N, tid);   // K(kb+1) under the mix and PV
    } else {
      load_set<D>(sKV, LD, BC, Vg, hs, G, j0, N, tid);   // V(kb) arrives under the mix and the softmax
    }
    cp_async_commit();

    // ---- mix + online softmax: a thread owns (two output heads, row, 4 keys); the quads of a row sit in adjacent lanes ----
    for (int task = tid; task < (G / 2) * BR * 4; task += NT) {
      const int q = task & 3, row = (task >> 2) % BR, gp = task / (4 * BR);
      float c[2][4];
      mix_quad<G>(c, sS, BR, row, q, sWt + 2 * gp, G);
      const int qi = i0 + row;
      float m_old[2], m_new[2], sum[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int g = 2 * gp + h;
        float mx = -INFINITY;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int kj = j0 + q * 4 + k;
          if (kj >= N || (causal && kj > qi)) c[h][k] = -INFINITY;
          mx = fmaxf(mx, c[h][k]);
        }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        m_old[h] = sM[g * BR + row];
        m_new[h] = fmaxf(m_old[h], mx);
        const float m_use = (m_new[h] == -INFINITY) ? 0.f : m_new[h];
        float pr[4], sm = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) { pr[k] = exp2f((c[h][k] - m_use) * kLog2e); sm += pr[k]; }
        sm += __shfl_xor_sync(0xffffffffu, sm, 1);
        sm += __shfl_xor_sync(0xffffffffu, sm, 2);
        sum[h] = sm;
        *reinterpret_cast<uint2*>(sP + ((size_t)g * BR + row) * P_LD + q * 4) = make_uint2(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]));
      }
      __syncwarp();                                      // every quad of the row has read the old maximum
      if (q == 0) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int g = 2 * gp + h;
          const float m_use = (m_new[h] == -INFINITY) ? 0.f : m_new[h];
          const float alpha = (m_old[h] == -INFINITY) ? 0.f : exp2f((m_old[h] - m_use) * kLog2e);
          sM[g * BR + row] = m_new[h];
          sL[g * BR + row] = sL[g * BR + row] * alpha + sum[h];
          sAlpha[g * BR + row] = alpha;
        }
      }
    }
    if (SM::TWO) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();                                     // V(kb) has landed, P and alpha are complete

    // ---- O = alpha * O + P V ----
#pragma unroll
    for (int i = 0; i < C::IPW; ++i) {
      const int item = warp + i * NW;
      if (item < C::ITEMS) {
        int g, mt;
        item_of<G, C::MT>(item, g, mt);
        const float a0 = sAlpha[g * BR + mt * 16 + (lane >> 2)], a1 = sAlpha[g * BR + mt * 16 + (lane >> 2) + 8];
#pragma unroll
        for (int j = 0; j < ONT; ++j) { accO[i][j][0] *= a0; accO[i][j][1] *= a0; accO[i][j][2] *= a1; accO[i][j][3] *= a1; }
        warp_gemm<ONT, false, true>(accO[i], sP + ((size_t)g * BR + mt * 16) * P_LD, P_LD, sV2 + (size_t)g * BC * LD, LD, BC, lane);
      }
    }
    __syncthreads();                                     // V and P no longer read
    if (SM::TWO) {
      if (kb < kb_end) load_set<D>(sV2, LD, BC, Vg, hs, G, j0 + BC, N, tid);   // V(kb+1) under the next scores and mix
      cp_async_commit();
    } else if (kb < kb_end) {
      load_set<D>(sKV, LD, BC, Kg, hs, G, j0 + BC, N, tid);
      cp_async_commit();
    }
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- epilogue: normalise, write O, M, L (and LSE) ----
#pragma unroll
  for (int i = 0; i < C::IPW; ++i) {
    const int item = warp + i * NW;
    if (item < C::ITEMS) {
      int g, mt;
      item_of<G, C::MT>(item, g, mt);
      const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
      const float l0 = sL[g * BR + r0], l1 = sL[g * BR + r1];
      const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
      const size_t row_base = (bh0 + g) * (size_t)N;
#pragma unroll
      for (int j = 0; j < ONT; ++j) {
        const int col = j * 8 + (lane & 3) * 2;
        const float o00 = accO[i][j][0] * inv0, o01 = accO[i][j][1] * inv0, o10 = accO[i][j][2] * inv1, o11 = accO[i][j][3] * inv1;
        if (p.o_bf16) {
          bf16* O = reinterpret_cast<bf16*>(p.O);
          if (i0 + r0 < N) *reinterpret_cast<uint32_t*>(O + (row_base + i0 + r0) * D + col) = pack_bf16(o00, o01);
          if (i0 + r1 < N) *reinterpret_cast<uint32_t*>(O + (row_base + i0 + r1) * D + col) = pack_bf16(o10, o11);
        } else {
          float* O = reinterpret_cast<float*>(p.O);
          if (i0 + r0 < N) *reinterpret_cast<float2*>(O + (row_base + i0 + r0) * D + col) = make_float2(o00, o01);
          if (i0 + r1 < N) *reinterpret_cast<float2*>(O + (row_base + i0 + r1) * D + col) = make_float2(o10, o11);
        }
      }
    }
  }
  for (int i = tid; i < G * BR; i += NT) {
    const int g = i / BR, r = i - g * BR;
    if (i0 + r < N) {
      const size_t o = (bh0 + g) * (size_t)N + i0 + r;
      const float m = sM[i], l = sL[i];
      if (p.M) p.M[o] = m;
      if (p.L) p.L[o] = l;
      if (p.LSEout) p.LSEout[o] = m + logf(l);
    }
  }
}


// ------------------------------------------------------------------------------------------
// Backward.  Both kernels work on score tiles [head][outer][16] in shared memory: for dQ / dW the outer
// index is the query row (BR rows of a sub-tile) and the 16-wide strip runs over the keys of a step; for
// dK / dV (TR = true) the outer index is the key (BR keys of the CTA's tile) and the strip runs over the
// 16 query rows of a step -- the transposed tile, so that P^T and dS^T are the row-major A operands of
// dV += P^T dO and dK += dS^T Q.  Per step:
//   S   = scale * (outer operand) . (strip operand)^T          per head, mma.sync       -> sS  (fp32)
//   dP  = the same product of the dO / V pair                                            -> sDC (fp32)
//   C'  = mix of S over the heads;  P = exp(C' - LSE);  dC' = P (dP - D)                 -> sDC in place (P: sPb)
//   dW += dC'_g . S_g'  over the tile (dQ kernel only; per-thread partial sums, reduced at the end)
//   dS_g' = sum_g W[g,g'] dC'_g  -> bf16                                                  -> sDS (in the sS region)
//   dQ += dS K   |   dV += P^T dO,  dK += dS^T Q
// Operand tile sets that do not fit beside each other share a buffer and are copied again from L2.
template <int D, int G, bool TR>
struct BwdSmem {
  using C = Cfg<D, G>;
  // "big" sets have BR rows per head (Q, dO for dQ; K, V for dK/dV), "small" sets 16 (K, V; Q, dO)
  static constexpr int kFixed = 2 * C::SSET + 2 * G * C::BR * 4 + 2 * G * G * 4 + (TR ? 0 : 4096);
  static constexpr int kBase = C::TSET + C::KSET + kFixed;                    // one big + one small buffer
  static constexpr int kPb = TR ? C::PSET : 0;                                // dK/dV: P^T needs a place of its own beside a resident V
  static constexpr bool BIG2 = kBase + C::TSET + kPb <= 227 * 1024;           // second big buffer (dO | V resident)
  static constexpr bool SMALL2 = kBase + (BIG2 ? C::TSET + kPb : 0) + C::KSET <= 227 * 1024;   // second small buffer
  static constexpr int oBigA = 0;
  static constexpr int oBigB = BIG2 ? C::TSET : 0;
  static constexpr int oSmallA = oBigB + C::TSET;
  static constexpr int oSmallB = SMALL2 ? oSmallA + C::KSET : oSmallA;
  static constexpr int oS = oSmallB + C::KSET;
  static constexpr int oDC = oS + C::SSET;
  static constexpr int oPb = (TR && BIG2) ? oDC + C::SSET : oBigB;            // without a resident V, P^T takes V's place
  static constexpr int oStat = oDC + C::SSET + ((TR && BIG2) ? C::PSET : 0);  // LSE, D
  static constexpr int oW = oStat + 2 * G * C::BR * 4;
  static constexpr int oWt = oW + G * G * 4;                                  // W transposed: [input head][output head]
  static constexpr int oRed = oWt + G * G * 4;                                // dW reduction (dQ kernel)
  static constexpr int kBytes = oRed + (TR ? 0 : 4096);
  static_assert(kBytes <= 227 * 1024, "backward: shared memory budget");
  static_assert(C::PSET <= C::TSET && C::PSET <= C::SSET, "aliased bf16 tiles");
};

// P (optional, bf16) and dC' = P (dP - D) in place of dP, for all heads; a thread owns (two output heads, outer, 4 strip elements).
template <int G, int BR, bool TR, bool WANT_P, bool WANT_DC = true>
FMTA_DEVINL void bwd_mix_phase(const float* sS, float* sDC, bf16* sPb, const float* sWt, const float* sLSE, const float* sDv,
                               int o0, int s0, int N, bool causal, int tid) {
  constexpr int LR = TR ? BC : BR;                       // rows of the per-row statistics per head
  for (int task = tid; task < (G / 2) * BR * 4; task += NT) {
    const int q = task & 3, outer = (task >> 2) % BR, gp = task / (4 * BR);
    float c[2][4];
    mix_quad<G>(c, sS, BR, outer, q, sWt + 2 * gp, G);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int g = 2 * gp + h;
      float* dc = sDC + ((size_t)g * BR + outer) * BC + sw_chunk(outer, q) * 4;
      float4 d4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (WANT_DC) d4 = *reinterpret_cast<const float4*>(dc);
      const float dp[4] = {d4.x, d4.y, d4.z, d4.w};
      float pr[4], out[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int st = q * 4 + k;
        const int qi = TR ? s0 + st : o0 + outer, kj = TR ? o0 + outer : s0 + st;
        const int ri = g * LR + (TR ? st : outer);
        const bool ok = qi < N && kj < N && !(causal && kj > qi);
        pr[k] = ok ? exp2f((c[h][k] - sLSE[ri]) * kLog2e) : 0.f;
        out[k] = pr[k] * (dp[k] - sDv[ri]);
      }
      if (WANT_DC) *reinterpret_cast<float4*>(dc) = make_float4(out[0], out[1], out[2], out[3]);
      if (WANT_P)
        *reinterpret_cast<uint2*>(sPb + ((size_t)g * BR + outer) * (BC + 8) + q * 4) = make_uint2(pack_bf16(pr[0], pr[1]), pack_bf16(pr[2], pr[3]));
    }
  }
}

// dS_g' = sum_g W[g,g'] dC'_g as bf16 strips [g'][outer][P_LD]; a thread owns (two input heads g', outer, 4 strip elements)
template <int G, int BR>
FMTA_DEVINL void bwd_unmix_phase(const float* sDC, bf16* sDS, const float* sW, int tid) {
  for (int task = tid; task < (G / 2) * BR * 4; task += NT) {
    const int q = task & 3, outer = (task >> 2) % BR, gp = task / (4 * BR);
    float c[2][4];
    mix_quad<G>(c, sDC, BR, outer, q, sW + 2 * gp, G);   // columns 2gp, 2gp + 1 of W: the weights of head g sit at sW[g * G + ...]
#pragma unroll
    for (int h = 0; h < 2; ++h)
      *reinterpret_cast<uint2*>(sDS + ((size_t)(2 * gp + h) * BR + outer) * (BC + 8) + q * 4) =
          make_uint2(pack_bf16(c[h][0], c[h][1]), pack_bf16(c[h][2], c[h][3]));
  }
}

template <int D, int G>
__global__ void __launch_bounds__(NT, 1) hm_bwd_dq_kernel(const TrainParams p) {
  using C = Cfg<D, G>;
  using SM = BwdSmem<D, G, false>;
  constexpr int BR = C::BR, LD = C::LD, P_LD = C::P_LD;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sQ = reinterpret_cast<bf16*>(smem + SM::oBigA);
  bf16* sdO = reinterpret_cast<bf16*>(smem + SM::oBigB);     // = sQ without a second big buffer
  bf16* sK = reinterpret_cast<bf16*>(smem + SM::oSmallA);
  bf16* sV = reinterpret_cast<bf16*>(smem + SM::oSmallB);    // = sK without a second small buffer
  float* sS = reinterpret_cast<float*>(smem + SM::oS);
  float* sDC = reinterpret_cast<float*>(smem + SM::oDC);
  bf16* sDS = reinterpret_cast<bf16*>(smem + SM::oS);        // bf16 dS strips take the place of S
  float* sLSE = reinterpret_cast<float*>(smem + SM::oStat);
  float* sDv = sLSE + G * BR;
  float* sW = reinterpret_cast<float*>(smem + SM::oW);
  float* sWt = reinterpret_cast<float*>(smem + SM::oWt);
  float* sRed = reinterpret_cast<float*>(smem + SM::oRed);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H;
  const int nQB = (N + BR - 1) / BR, nKB = (N + BC - 1) / BC;
  const int qb = nQB - 1 - (int)blockIdx.x;              // long (late) row tiles first
  const int grp = blockIdx.y, b = blockIdx.z;
  const int i0 = qb * BR;
  const bool causal = p.causal != 0;
  const size_t hs = (size_t)N * D;
  const size_t bh0 = (size_t)b * H + (size_t)grp * G;
  const bf16* Qg = p.Q + bh0 * hs;
  const bf16* Kg = p.K + bh0 * hs;
  const bf16* Vg = p.V + bh0 * hs;
  const bf16* dOg = p.dO + bh0 * hs;

  for (int i = tid; i < G * G; i += NT) {
    const float wv = p.Wmix[(size_t)grp * G * G + i];
    sW[i] = wv;
    sWt[(i % G) * G + i / G] = wv;
  }

  // dW[g][g'] = sum over the tile of dC'_g * S_g': a thread owns a GB x GB block of (g, g') pairs and a share
  // of the tile's 4-float chunks (the shares of a block sit in adjacent lanes), so that 2 * GB loads feed
  // 4 * GB * GB FMAs; the shares are added at the end of the CTA, in a fixed order.
  constexpr int GB = G >= 4 ? 4 : G;
  constexpr int NBLK = (G / GB) * (G / GB), PARTS = NT / NBLK;
  constexpr int CH = BR * BC / 4;                          // 4-float chunks of one head's tile
  const int dw_part = tid % PARTS, dw_g0 = ((tid / PARTS) / (G / GB)) * GB, dw_h0 = ((tid / PARTS) % (G / GB)) * GB;
  float dwacc[GB][GB];
#pragma unroll
  for (int i = 0; i < GB; ++i)
#pragma unroll
    for (int j = 0; j < GB; ++j) dwacc[i][j] = 0.f;

  constexpr int ONT = D / 8;
  {
    float accQ[C::IPW][ONT][4];
#pragma unroll
    for (int i = 0; i < C::IPW; ++i)
#pragma unroll
      for (int j = 0; j < ONT; ++j) accQ[i][j][0] = accQ[i][j][1] = accQ[i][j][2] = accQ[i][j][3] = 0.f;
    for (int i = tid; i < G * BR; i += NT) {
      const int g = i / BR, r = i - g * BR;
      const bool ok = i0 + r < N;
      sLSE[i] = ok ? p.LSE[(bh0 + g) * (size_t)N + i0 + r] : 0.f;
      sDv[i] = ok ? p.Dvec[(bh0 + g) * (size_t)N + i0 + r] : 0.f;
    }
    if (SM::BIG2) {                                        // Q and dO stay for the whole key loop
      load_set<D>(sQ, LD, BR, Qg, hs, G, i0, N, tid);
      load_set<D>(sdO, LD, BR, dOg, hs, G, i0, N, tid);
      cp_async_commit();
    }
    const int kb_end = causal ? min(nKB - 1, (i0 + BR - 1) / BC) : nKB - 1;
    for (int kb = 0; kb <= kb_end; ++kb) {
      const int j0 = kb * BC;
      if (!SM::BIG2) load_set<D>(sQ, LD, BR, Qg, hs, G, i0, N, tid);
      load_set<D>(sK, LD, BC, Kg, hs, G, j0, N, tid);
      if (SM::SMALL2) load_set<D>(sV, LD, BC, Vg, hs, G, j0, N, tid);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
      head_products<D, G>(sS, sQ, BR, sK, p.scale, warp, lane);          // S
      if (!SM::BIG2 || !SM::SMALL2) {
        __syncthreads();                                                 // Q / K no longer read
        if (!SM::BIG2) load_set<D>(sdO, LD, BR, dOg, hs, G, i0, N, tid);
        if (!SM::SMALL2) load_set<D>(sV, LD, BC, Vg, hs, G, j0, N, tid);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
      }
      head_products<D, G>(sDC, sdO, BR, sV, 1.f, warp, lane);            // dP
      __syncthreads();
      if (!SM::SMALL2) {                                                 // K comes back under the element-wise phases
        load_set<D>(sK, LD, BC, Kg, hs, G, j0, N, tid);
        cp_async_commit();
      }
      bwd_mix_phase<G, BR, false, false>(sS, sDC, nullptr, sWt, sLSE, sDv, i0, j0, N, causal, tid);
      __syncthreads();
      // ---- dW partial sums ----
      for (int ch = dw_part; ch < CH; ch += PARTS) {
        float4 x[GB], y[GB];
#pragma unroll
        for (int i = 0; i < GB; ++i) {
          x[i] = reinterpret_cast<const float4*>(sDC + (size_t)(dw_g0 + i) * BR * BC)[ch];
          y[i] = reinterpret_cast<const float4*>(sS + (size_t)(dw_h0 + i) * BR * BC)[ch];
        }
#pragma unroll
        for (int i = 0; i < GB; ++i)
#pragma unroll
          for (int j = 0; j < GB; ++j) {
            float t = dwacc[i][j];
            t = fmaf(x[i].x, y[j].x, t); t = fmaf(x[i].y, y[j].y, t); t = fmaf(x[i].z, y[j].z, t); t = fmaf(x[i].w, y[j].w, t);
            dwacc[i][j] = t;
          }
      }
      __syncthreads();                                                   // S no longer read: dS strips may take its place
      bwd_unmix_phase<G, BR>(sDC, sDS, sW, tid);
      cp_async_wait<0>();
      __syncthreads();                                                   // dS complete, K back
      // ---- dQ += dS K ----
#pragma unroll
      for (int i = 0; i < C::IPW; ++i) {
        const int item = warp + i * NW;
        if (item < C::ITEMS) {
          int g, mt;
          item_of<G, C::MT>(item, g, mt);
          warp_gemm<ONT, false, true>(accQ[i], sDS + ((size_t)g * BR + mt * 16) * P_LD, P_LD, sK + (size_t)g * BC * LD, LD, BC, lane);
        }
      }
      __syncthreads();
    }
    // dQ = scale * acc
#pragma unroll
    for (int i = 0; i < C::IPW; ++i) {
      const int item = warp + i * NW;
      if (item < C::ITEMS) {
        int g, mt;
        item_of<G, C::MT>(item, g, mt);
        const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
        float* base = p.dQ + (bh0 + g) * hs;
#pragma unroll
        for (int j = 0; j < ONT; ++j) {
          const int col = j * 8 + (lane & 3) * 2;
          if (i0 + r0 < N) *reinterpret_cast<float2*>(base + (size_t)(i0 + r0) * D + col) = make_float2(accQ[i][j][0] * p.scale, accQ[i][j][1] * p.scale);
          if (i0 + r1 < N) *reinterpret_cast<float2*>(base + (size_t)(i0 + r1) * D + col) = make_float2(accQ[i][j][2] * p.scale, accQ[i][j][3] * p.scale);
        }
      }
    }
  }
  // ---- dW partial of this CTA: the shares of a block are added in a fixed order ----
  __syncthreads();
  if (p.dW_part != nullptr) {
    const int slot = b * nQB + qb;
    float* out = p.dW_part + ((size_t)slot * (H / G) + grp) * (G * G);
    constexpr int LP = PARTS < 32 ? PARTS : 32;              // shares of a block inside one warp
#pragma unroll
    for (int i = 0; i < GB; ++i)
#pragma unroll
      for (int j = 0; j < GB; ++j)
#pragma unroll
        for (int off = LP / 2; off > 0; off >>= 1) dwacc[i][j] += __shfl_xor_sync(0xffffffffu, dwacc[i][j], off);
    if (PARTS <= 32) {
      if (dw_part == 0) {
#pragma unroll
        for (int i = 0; i < GB; ++i)
#pragma unroll
          for (int j = 0; j < GB; ++j) out[(dw_g0 + i) * G + dw_h0 + j] = dwacc[i][j];
      }
    } else {
      constexpr int WPB = PARTS / 32;                        // warps per block
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < GB; ++i)
#pragma unroll
          for (int j = 0; j < GB; ++j) sRed[warp * 16 + i * GB + j] = dwacc[i][j];
      }
      __syncthreads();
      if (tid < NBLK * GB * GB) {
        const int blk = tid / (GB * GB), e = tid % (GB * GB);
        float t = 0.f;
        for (int w = 0; w < WPB; ++w) t += sRed[(blk * WPB + w) * 16 + e];
        const int g0 = (blk / (G / GB)) * GB, h0 = (blk % (G / GB)) * GB;
        out[(g0 + e / GB) * G + h0 + e % GB] = t;
      }
    }
  }
}

template <int D, int G>
struct DkvPass {
  // dK and dV accumulators of a warp's items: IPW * D / 8 tiles of 4 registers each.  Where both together pass
  // 64 registers (head dim 128, or 32 heads at head dim 64) dV and dK come from two launches (MODE 1: dV only,
  // no dP, no dS; MODE 2: dK only), else from one (MODE 0).
  static constexpr bool SPLIT = Cfg<D, G>::IPW * (D / 8) * 4 * 2 > 64;
};

template <int D, int G, int MODE>
__global__ void __launch_bounds__(NT, 1) hm_bwd_dkdv_kernel(const TrainParams p) {
  constexpr bool DO_V = MODE != 2, DO_K = MODE != 1;
  using C = Cfg<D, G>;
  using SM = BwdSmem<D, G, true>;
  constexpr int BR = C::BR, LD = C::LD, P_LD = C::P_LD;
  extern __shared__ __align__(16) unsigned char smem[];
  bf16* sK = reinterpret_cast<bf16*>(smem + SM::oBigA);
  bf16* sV = reinterpret_cast<bf16*>(smem + SM::oBigB);      // = sK without a second big buffer
  bf16* sQ = reinterpret_cast<bf16*>(smem + SM::oSmallA);
  bf16* sdO = reinterpret_cast<bf16*>(smem + SM::oSmallB);   // = sQ without a second small buffer
  float* sS = reinterpret_cast<float*>(smem + SM::oS);
  float* sDC = reinterpret_cast<float*>(smem + SM::oDC);
  bf16* sDS = reinterpret_cast<bf16*>(smem + SM::oS);
  bf16* sPb = reinterpret_cast<bf16*>(smem + SM::oPb);
  float* sLSE = reinterpret_cast<float*>(smem + SM::oStat);
  float* sDv = sLSE + G * BR;                                // (only G * 16 entries of each are used)
  float* sW = reinterpret_cast<float*>(smem + SM::oW);
  float* sWt = reinterpret_cast<float*>(smem + SM::oWt);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int N = p.N, H = p.H;
  const int nRB = (N + BC - 1) / BC;                         // 16-row steps
  const int kt = blockIdx.x;                                 // early key tiles see the most rows: longest first
  const int grp = blockIdx.y, b = blockIdx.z;
  const int j0 = kt * BR;
  const bool causal = p.causal != 0;
  const size_t hs = (size_t)N * D;
  const size_t bh0 = (size_t)b * H + (size_t)grp * G;
  const bf16* Qg = p.Q + bh0 * hs;
  const bf16* Kg = p.K + bh0 * hs;
  const bf16* Vg = p.V + bh0 * hs;
  const bf16* dOg = p.dO + bh0 * hs;

  for (int i = tid; i < G * G; i += NT) {
    const float wv = p.Wmix[(size_t)grp * G * G + i];
    sW[i] = wv;
    sWt[(i % G) * G + i / G] = wv;
  }
  constexpr int ONT = D / 8;
  float accK[DO_K ? C::IPW : 1][ONT][4], accV[DO_V ? C::IPW : 1][ONT][4];
#pragma unroll
  for (int i = 0; i < C::IPW; ++i)
#pragma unroll
    for (int j = 0; j < ONT; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (DO_K) accK[DO_K ? i : 0][j][e] = 0.f;
        if (DO_V) accV[DO_V ? i : 0][j][e] = 0.f;
      }

  if (SM::BIG2) {                                            // K and V stay for the whole row loop
    load_set<D>(sK, LD, BR, Kg, hs, G, j0, N, tid);
    if (DO_K) load_set<D>(sV, LD, BR, Vg, hs, G, j0, N, tid);
    cp_async_commit();
  }
  const int rb_begin = causal ? j0 / BC : 0;
  for (int rb = rb_begin; rb < nRB; ++rb) {
    const int i0 = rb * BC;
    __syncthreads();                                         // the previous step is done with every buffer
    for (int i = tid; i < G * BC; i += NT) {
      const int g = i / BC, r = i - g * BC;
      const bool ok = i0 + r < N;
      sLSE[i] = ok ? p.LSE[(bh0 + g) * (size_t)N + i0 + r] : 0.f;
      sDv[i] = ok ? p.Dvec[(bh0 + g) * (size_t)N + i0 + r] : 0.f;
    }
    if (!SM::BIG2) load_set<D>(sK, LD, BR, Kg, hs, G, j0, N, tid);
    load_set<D>(sQ, LD, BC, Qg, hs, G, i0, N, tid);
    if (SM::SMALL2) load_set<D>(sdO, LD, BC, dOg, hs, G, i0, N, tid);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    head_products<D, G>(sS, sK, BR, sQ, p.scale, warp, lane);            // S^T
    if (!SM::BIG2 || !SM::SMALL2) {
      __syncthreads();
      if (!SM::BIG2 && DO_K) load_set<D>(sV, LD, BR, Vg, hs, G, j0, N, tid);
      if (!SM::SMALL2) load_set<D>(sdO, LD, BC, dOg, hs, G, i0, N, tid);
      cp_async_commit();
      cp_async_wait<0>();
      __syncthreads();
    }
    if (DO_K) head_products<D, G>(sDC, sV, BR, sdO, 1.f, warp, lane);    // dP^T
    __syncthreads();                                                     // V no longer read: P^T may take its place
    bwd_mix_phase<G, BR, true, DO_V, DO_K>(sS, sDC, sPb, sWt, sLSE, sDv, j0, i0, N, causal, tid);
    __syncthreads();
    // ---- dV += P^T dO, and dS^T strips into the place of S^T ----
    if (DO_V) {
#pragma unroll
      for (int i = 0; i < C::IPW; ++i) {
        const int item = warp + i * NW;
        if (item < C::ITEMS) {
          int g, mt;
          item_of<G, C::MT>(item, g, mt);
          warp_gemm<ONT, false, true>(accV[DO_V ? i : 0], sPb + ((size_t)g * BR + mt * 16) * P_LD, P_LD, sdO + (size_t)g * BC * LD, LD, BC, lane);
        }
      }
    }
    if (DO_K) {
      bwd_unmix_phase<G, BR>(sDC, sDS, sW, tid);
      __syncthreads();
      if (!SM::SMALL2) {                                                 // Q again, in the place of dO
        load_set<D>(sQ, LD, BC, Qg, hs, G, i0, N, tid);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
      }
      // ---- dK += dS^T Q ----
#pragma unroll
      for (int i = 0; i < C::IPW; ++i) {
        const int item = warp + i * NW;
        if (item < C::ITEMS) {
          int g, mt;
          item_of<G, C::MT>(item, g, mt);
          warp_gemm<ONT, false, true>(accK[DO_K ? i : 0], sDS + ((size_t)g * BR + mt * 16) * P_LD, P_LD, sQ + (size_t)g * BC * LD, LD, BC, lane);
        }
      }
    }
  }
  // ---- dK = scale * acc, dV ----
#pragma unroll
  for (int i = 0; i < C::IPW; ++i) {
    const int item = warp + i * NW;
    if (item < C::ITEMS) {
      int g, mt;
      item_of<G, C::MT>(item, g, mt);
      const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
      float* bk = p.dK + (bh0 + g) * hs;
      float* bv = p.dV + (bh0 + g) * hs;
#pragma unroll
      for (int j = 0; j < ONT; ++j) {
        const int col = j * 8 + (lane & 3) * 2;
        if (j0 + r0 < N) {
          if (DO_K) *reinterpret_cast<float2*>(bk + (size_t)(j0 + r0) * D + col) = make_float2(accK[DO_K ? i : 0][j][0] * p.scale, accK[DO_K ? i : 0][j][1] * p.scale);
          if (DO_V) *reinterpret_cast<float2*>(bv + (size_t)(j0 + r0) * D + col) = make_float2(accV[DO_V ? i : 0][j][0], accV[DO_V ? i : 0][j][1]);
        }
        if (j0 + r1 < N) {
          if (DO_K) *reinterpret_cast<float2*>(bk + (size_t)(j0 + r1) * D + col) = make_float2(accK[DO_K ? i : 0][j][2] * p.scale, accK[DO_K ? i : 0][j][3] * p.scale);
          if (DO_V) *reinterpret_cast<float2*>(bv + (size_t)(j0 + r1) * D + col) = make_float2(accV[DO_V ? i : 0][j][2], accV[DO_V ? i : 0][j][3]);
        }
      }
    }
  }
}

}  // namespace hm

// ------------------------------------------------------------------------------------------
// host side
// dW partial slots of hm_bwd_dq_kernel: one per (batch, row tile)
int hm_dq_slots(int B, int N, int G) {
  const int mt = (G >= hm::NW) ? 1 : ((hm::NW / G) > 4 ? 4 : (hm::NW / G));
  return B * ((N + 16 * mt - 1) / (16 * mt));
}

bool hm_dense_supported(const TrainParams& p) {
  if (p.theta != nullptr || p.Wmix == nullptr) return false;
  if (p.G != 2 && p.G != 4 && p.G != 8 && p.G != 16 && p.G != 32) return false;
  if (p.d != 32 && p.d != 64 && p.d != 128) return false;
  if (p.G == 32 && p.d == 128) return false;             // two tile sets of 32 heads x 16 rows x 128 do not fit
  return true;
}

#define FMTA_HM_DISPATCH(p, ...)                                                                    \
  do {                                                                                              \
    const int d_ = (p).d, g_ = (p).G;                                                               \
    if (d_ == 32) { constexpr int D_ = 32; FMTA_HM_DISPATCH_G(g_, __VA_ARGS__) }                    \
    else if (d_ == 64) { constexpr int D_ = 64; FMTA_HM_DISPATCH_G(g_, __VA_ARGS__) }               \
    else if (d_ == 128) { constexpr int D_ = 128; FMTA_HM_DISPATCH_G16(g_, __VA_ARGS__) }           \
  } while (0)
#define FMTA_HM_DISPATCH_G16(g_, ...)                                   \
    if (g_ == 2) { constexpr int G_ = 2; __VA_ARGS__ }                  \
    else if (g_ == 4) { constexpr int G_ = 4; __VA_ARGS__ }             \
    else if (g_ == 8) { constexpr int G_ = 8; __VA_ARGS__ }             \
    else if (g_ == 16) { constexpr int G_ = 16; __VA_ARGS__ }
#define FMTA_HM_DISPATCH_G(g_, ...)                                     \
    FMTA_HM_DISPATCH_G16(g_, __VA_ARGS__)                               \
    else if (g_ == 32) { constexpr int G_ = 32; __VA_ARGS__ }

cudaError_t launch_hm_fwd(const TrainParams& p, cudaStream_t stream) {
  FMTA_HM_DISPATCH(p, {
    using C = hm::Cfg<D_, G_>;
    dim3 grid((p.N + C::BR - 1) / C::BR, p.H / p.G, p.B);
    return launch_kernel<TrainParams>(hm::hm_fwd_kernel<D_, G_>, grid, dim3(hm::NT), hm::FwdSmem<D_, G_>::kBytes, stream, 1, p);
  });
  return cudaErrorInvalidValue;
}

cudaError_t launch_hm_bwd_dq(const TrainParams& p, cudaStream_t stream) {
  FMTA_HM_DISPATCH(p, {
    dim3 grid((p.N + hm::Cfg<D_, G_>::BR - 1) / hm::Cfg<D_, G_>::BR, p.H / p.G, p.B);   // one dW partial slot per CTA
    return launch_kernel<TrainParams>(hm::hm_bwd_dq_kernel<D_, G_>, grid, dim3(hm::NT), hm::BwdSmem<D_, G_, false>::kBytes, stream, 1, p);
  });
  return cudaErrorInvalidValue;
}

cudaError_t launch_hm_bwd_dkdv(const TrainParams& p, cudaStream_t stream) {
  FMTA_HM_DISPATCH(p, {
    using C = hm::Cfg<D_, G_>;
    dim3 grid((p.N + C::BR - 1) / C::BR, p.H / p.G, p.B);
    constexpr int smem = hm::BwdSmem<D_, G_, true>::kBytes;
    if constexpr (hm::DkvPass<D_, G_>::SPLIT) {
      cudaError_t e = launch_kernel<TrainParams>(hm::hm_bwd_dkdv_kernel<D_, G_, 1>, grid, dim3(hm::NT), smem, stream, 1, p);
      if (e != cudaSuccess) return e;
      return launch_kernel<TrainParams>(hm::hm_bwd_dkdv_kernel<D_, G_, 2>, grid, dim3(hm::NT), smem, stream, 1, p);
    } else {
      return launch_kernel<TrainParams>(hm::hm_bwd_dkdv_kernel<D_, G_, 0>, grid, dim3(hm::NT), smem, stream, 1, p);
    }
  });
  return cudaErrorInvalidValue;
}

}  // namespace fmta
