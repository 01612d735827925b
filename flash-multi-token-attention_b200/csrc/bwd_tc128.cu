// Stacked-GEMM conv-attention backward on tcgen05 / TMEM / TMA for head dim 128 (entries off the
// causal band; the math is that of bwd_tc.cu).
//
// At d = 128 a stacked key tile is twice as large as at d = 64 and the accumulators twice as wide, so the
// plans of bwd_tc.cu do not fit the 227 KB of shared memory / 512 columns of tensor memory.  Both kernels
// here keep the query rows on the TMEM lanes for the scores (S = sum_a Q^(a) Kt_a^T, M = 128 rows, N = 64
// keys):
//
//   bwd_dq_tc128_kernel   : CTA = one tile of 128 dC rows (owning 120 dQ rows), loops 64-key blocks.  dO
//                           lives in tensor memory as the A operand of dP = dO V^T, which leaves shared
//                           memory for a ring of ten 16 KB key tiles; dQ (128 columns) accumulates in
//                           tensor memory with ONE 128 x 128 x 16 MMA per tap and 16 keys (B = Kt tile
//                           read MN-major across its two 128-byte-swizzled column slabs).
//   bwd_dkdv_tc128_kernel : CTA = 64 keys, loops 128-row query blocks.  The c_q stacked key tiles and V
//                           stay resident (112 KB).  The accumulators are kept TRANSPOSED, with the head
//                           dim on the lanes: dV^T[d, key] += dO^T P and dKt_a^T[d, key] += Q^(a)T dC are
//                           M = 128 MMAs whose A operand is the staged dO / Q tile read MN-major (for Q
//                           with the tap's row shift as a start-address offset of 128 bytes per row into
//                           the 128-byte-swizzled tile) and whose B operand is the
//                           bf16 P / dC tile exactly as the element-wise warps write it (one row per
//                           thread).  dV^T + 6 dKt^T take 448 columns; S and dP share the last 64
//                           (dP(0) | S(0) dP(1) | S(1) dP(2) ...), as in the d = 64 kernel.  Scores and dP
//                           are computed once per entry: no second pass over the head dim.
// Every mbarrier wait is bounded; no TMA multicast, no cluster, cta_group::1 only.
#include <cuda.h>
#include <cuda_runtime.h>

#include "bwd_tc.cuh"
#include "fmta_tc.cuh"
#include "launch_util.cuh"

namespace fmta {

// ==========================================================================================
// dQ, d = 128
// ==========================================================================================
struct Dq128Cfg {
  static constexpr int D = 128;
  static constexpr int BM = 128;               // dC rows per tile (= TMEM lanes)
  static constexpr int OWN = 120;              // dQ rows a tile owns (dQ row i needs dC rows i .. i + pad_q, pad_q <= 8)
  static constexpr int BC = 64;                // keys per block
  static constexpr int HALO = 16;
  static constexpr int QR = HALO + BM;         // 144 rows of Q
  static constexpr int DR = BM + 16;           // rows of the dC buffer (16 zero rows below)
  static constexpr int SLAB_BYTES = BC * 128;  // 64 keys x 64 elements, 128-byte swizzle
  static constexpr int TILE_BYTES = 2 * SLAB_BYTES;   // one Kt / V ring tile: two column slabs
  static constexpr int NSLOT = 10;
  static constexpr int Q_SLAB = QR * 128;      // 144 rows x 64 elements, 128-byte swizzle
  static constexpr int oQ = 0;                                  // two slabs
  static constexpr int odC = oQ + 2 * Q_SLAB;                   // [BC/8][DR][16 B]
  static constexpr int oRing = ((odC + (BC / 8) * DR * 16 + 1023) / 1024) * 1024;
  static constexpr int oBar = oRing + NSLOT * TILE_BYTES;
  static constexpr int kSmemBytes = oBar + 512 + 1024;
  static_assert(kSmemBytes <= 227 * 1024, "dQ kernel (d = 128): shared memory budget");
  static constexpr int kTmemCols = 512;        // S (two buffers) at 0 and 64, dP at 128, dQ at 192..319, dO (bf16 pairs) at 320..383
  static constexpr int colP = 128, colQ = 192, colO = 320;
  static constexpr int kEwWarps = 8;           // two element-wise warps per lane quarter, 32 key columns each
  static constexpr int kThreads = (kEwWarps + 1 + 2) * 32;   // element-wise warps, TMA warp, two MMA issuer warps
};

__global__ void __launch_bounds__(Dq128Cfg::kThreads, 1)
bwd_dq_tc128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKt,
                    const __grid_constant__ CUtensorMap tmV, const bf16* __restrict__ dO, const BwdTcParams p) {
  using Cfg = Dq128Cfg;
  constexpr int D = Cfg::D, BM = Cfg::BM, BC = Cfg::BC, HALO = Cfg::HALO, QR = Cfg::QR;
  const int OWN = p.own;                                 // 128 - pad_q dQ rows per tile of 128 dC rows
  constexpr int DR = Cfg::DR, NSLOT = Cfg::NSLOT;
  constexpr int NEW = Cfg::kEwWarps * 32;      // element-wise threads
  constexpr int W_TMA = Cfg::kEwWarps, W_S = Cfg::kEwWarps + 1, W_DQ = Cfg::kEwWarps + 2;   // warp roles
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem + Cfg::oQ;
  unsigned char* sdC = smem + Cfg::odC;
  unsigned char* sRing = smem + Cfg::oRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* full = bars;                 // [NSLOT]
  uint64_t* empty = bars + NSLOT;        // [NSLOT]  count 2: both issuers release every tile
  uint64_t* q_full = bars + 2 * NSLOT;   // Q staged
  uint64_t* do_full = q_full + 1;        // dO written to tensor memory (128 arrivals)
  uint64_t* sdp_full = do_full + 1;      // S and dP of the block complete
  uint64_t* s_free = sdp_full + 1;       // [2] S buffer b and dP of a block taken into registers (128 arrivals)
  uint64_t* dc_full = s_free + 2;        // dC tile written to shared memory (128 arrivals)
  uint64_t* dq_done = dc_full + 1;       // dQ MMAs of the block complete (dC buffer reusable)
  uint64_t* never_bar = dq_done + 1;     // nothing arrives here (expiry self-test)
  uint64_t* mma_drain = never_bar + 1;   // abort path: both issuers' MMAs have completed
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(mma_drain + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_issued = s_abort + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int band = pq + pk;
  const int nQB = (p.row_end - p.row_base + OWN - 1) / OWN;
  // length-major walk of the linear block order (longest row blocks first), as in the d = 64 kernel
  const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int nBH = gridDim.y * gridDim.z;
  const int qb = nQB - 1 - lin / nBH;
  const int h = (lin % nBH) % (int)gridDim.y, b = (lin % nBH) / (int)gridDim.y;
  const int bh = b * p.H + h;
  // tiles are laid out from the END of the window's rows, so that a partly filled tile is the first one (fewest
  // keys), not the last one (all keys); its rows before row_base are computed (negative rows as zero rows), not stored
  const int R0 = p.row_end - (nQB - qb) * OWN;
  const int nKB = (N + BC - 1) / BC;
  int nkb = 0;
  if (p.causal) {
    const int last = min(N - 1, R0 + BM - 1) - band;
    nkb = last >= 0 ? min(nKB, last / BC + 1) : 0;
  } else nkb = nKB;

  if (tid == 0) {
    for (int i = 0; i < NSLOT; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 2); }
    tc::mbar_init(q_full, 1); tc::mbar_init(do_full, NEW);
    tc::mbar_init(sdp_full, 1); tc::mbar_init(&s_free[0], NEW); tc::mbar_init(&s_free[1], NEW);
    tc::mbar_init(dc_full, NEW); tc::mbar_init(dq_done, 1);
    tc::mbar_init(never_bar, 1); tc::mbar_init(mma_drain, 2);
    *s_abort = 0; *s_issued = 0;
    tc::mbar_fence_init();
  }
  if (warp == W_S) {
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  // zero the dC buffer once: the 16 pad rows below the tile are read by the shifted views
  for (int i = tid; i < (BC / 8) * DR * 4; i += Cfg::kThreads) reinterpret_cast<uint32_t*>(sdC)[i] = 0u;
  tc::fence_proxy_async_smem();
  tc::tc_fence_before();
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory that a kernel of this library writes or reads back
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const int per_kb = cq + 1;   // ring tiles per key block

  if (warp == W_TMA) {
    // ===================== TMA producer =====================
    if (lane == 0 && nkb > 0) {
      tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmKt); tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, QR * D * 2);
      tc::tma_load_3d(sQ, &tmQ, q_full, 0, R0 - HALO, bh);
      tc::tma_load_3d(sQ + Cfg::Q_SLAB, &tmQ, q_full, 64, R0 - HALO, bh);
      int id = 0;
      bool ok = true;
      auto put = [&](const CUtensorMap* map, int y, int z) {
        const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
        if (!tc::mbar_wait(&empty[slot], ph ^ 1, s_abort)) { ok = false; return; }
        tc::mbar_expect_tx(&full[slot], Cfg::TILE_BYTES);
        tc::tma_load_3d(sRing + slot * Cfg::TILE_BYTES, map, &full[slot], 0, y, z);
        tc::tma_load_3d(sRing + slot * Cfg::TILE_BYTES + Cfg::SLAB_BYTES, map, &full[slot], 64, y, z);
        ++id;
        *s_issued = id;
      };
      for (int kb = 0; kb < nkb && ok; ++kb) {
        for (int a = 0; a < cq && ok; ++a) put(&tmKt, kb * BC, bh * cq + a);
        if (ok) put(&tmV, kb * BC, bh);
      }
    }
  } else if (warp > W_TMA) {
    // ===================== MMA issuers: one warp issues S and dP, the other dQ =====================
    const bool is_dq = warp == W_DQ;
    if (nkb > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescS = tc::make_idesc(BM, BC, 0, 0);    // S, dP: 128 x 64, K-major operands
      constexpr uint32_t idescQ = tc::make_idesc(BM, D, 0, 1);     // dQ: 128 x 128, B (Kt) MN-major
      // Q^(a): the swizzled tile with its start address moved by the tap's row shift, 128 bytes per row (the
      // tensor core swizzles the absolute shared-memory address, as TMA did when it wrote the tile)
      const uint64_t dQa = tc::make_sdesc(smem_u32(sQ) + (HALO - pq) * 128, 16, 1024, tc::kLayoutSW128);
      const uint64_t dCa = tc::make_sdesc(smem_u32(sdC), DR * 16, 128, tc::kLayoutNone);
      const uint64_t dKb = tc::make_sdesc(smem_u32(sRing), 16, 1024, tc::kLayoutSW128);
      // the same tile read MN-major, 128 columns wide: the second 64-column slab starts SLAB_BYTES further
      const uint64_t dKm = tc::make_sdesc(smem_u32(sRing), Cfg::SLAB_BYTES, 1024, tc::kLayoutSW128);
      const uint32_t q_hi = (uint32_t)(dQa >> 32), q_lo = (uint32_t)dQa;
      const uint32_t c_hi = (uint32_t)(dCa >> 32), c_lo = (uint32_t)dCa;
      const uint32_t k_hi = (uint32_t)(dKb >> 32), k_lo0 = (uint32_t)dKb;
      const uint32_t km_hi = (uint32_t)(dKm >> 32), km_lo0 = (uint32_t)dKm;
      const uint32_t tS = tmem, tP = tmem + Cfg::colP, tQ = tmem + Cfg::colQ, tO = tmem + Cfg::colO;
      bool ok = tc::mbar_wait_warp(q_full, 0, s_abort);
      if (!is_dq) {
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const uint32_t tSb = tS + 64 * (kb & 1);
          if (kb > 1) {      // the element-wise warps have taken S(kb-2) out of this buffer
            ok = tc::mbar_wait_warp(&s_free[kb & 1], ((kb >> 1) - 1) & 1, s_abort);
            tc::tc_fence_after();
          }
          for (int a = 0; a < cq && ok; ++a) {
            const int id = kb * per_kb + a, slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
            tc::tc_fence_after();
            const uint32_t b_lo = k_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
            const uint32_t a_lo = q_lo + (uint32_t)(a * (128 >> 4));
            tc::mma_ss2pe(tSb, a_lo, q_hi, b_lo, k_hi, idescS, a != 0);
#pragma unroll
            for (int k = 1; k < D / 16; ++k)
              tc::mma_ss2e<1>(tSb, a_lo + (uint32_t)((k >> 2) * (Cfg::Q_SLAB >> 4) + (k & 3) * 2), q_hi,
                              b_lo + (uint32_t)((k >> 2) * (Cfg::SLAB_BYTES >> 4) + (k & 3) * 2), k_hi, idescS);
            tc::mma_commit_e(&empty[slot]);      // (the dQ issuer holds the Kt tile until dQ(kb) is done)
          }
          if (!ok) break;
          const int id = kb * per_kb + cq, slot = id % NSLOT, ph = (id / NSLOT) & 1;
          if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
          if (kb == 0) {     // dO is in tensor memory
            ok = tc::mbar_wait_warp(do_full, 0, s_abort);
          } else {           // dP is single-buffered: block kb-1 must have left it
            ok = tc::mbar_wait_warp(&s_free[(kb - 1) & 1], ((kb - 1) >> 1) & 1, s_abort);
          }
          if (!ok) break;
          tc::tc_fence_after();
          {
            const uint32_t b_lo = k_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
            tc::mma_ts2e<0>(tP, tO, b_lo, k_hi, idescS);                 // dP = dO V^T, A from tensor memory
#pragma unroll
            for (int k = 1; k < D / 16; ++k)
              tc::mma_ts2e<1>(tP, tO + 8 * k, b_lo + (uint32_t)((k >> 2) * (Cfg::SLAB_BYTES >> 4) + (k & 3) * 2), k_hi, idescS);
          }
          tc::mma_commit_e(&empty[slot]);
          tc::mma_commit_e(sdp_full);
        }
      } else {
        for (int kb = 0; kb < nkb && ok; ++kb) {
          ok = tc::mbar_wait_warp(dc_full, kb & 1, s_abort);
          tc::tc_fence_after();
          for (int a = 0; a < cq && ok; ++a) {
            const int id = kb * per_kb + a, slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
            tc::tc_fence_after();
            const uint32_t b_lo = km_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
            const uint32_t a_lo = c_lo + (uint32_t)(pq - a);       // dC rows i' + pad_q - a
            tc::mma_ss2pe(tQ, a_lo, c_hi, b_lo, km_hi, idescQ, (kb != 0) || (a != 0));
#pragma unroll
            for (int k = 1; k < BC / 16; ++k)
              tc::mma_ss2e<1>(tQ, a_lo + (uint32_t)(2 * k * DR), c_hi, b_lo + (uint32_t)(k * (2048 / 16)), km_hi, idescQ);
            tc::mma_commit_e(&empty[slot]);
          }
          if (!ok) break;
          {   // the V tile of the block is not read here: release it right away
            const int id = kb * per_kb + cq, slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
            if (tc::elect_one()) tc::mbar_arrive(&empty[slot]);
          }
          tc::mma_commit_e(dq_done);
        }
      }
    }
  } else {
    // ===================== element-wise warps: one dC row per thread pair, 32 key columns per thread =====================
    constexpr int CW = BC / 2;                          // key columns per thread
    const int qtr = warp & 3, cg = warp >> 2;           // TMEM lane quarter, column half
    const int m = qtr * 32 + lane;                      // row within the tile = TMEM lane
    const int gi = R0 + m;                              // query index of this dC row
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const uint32_t tS = tmem + lane_base, tP = tS + Cfg::colP, tQ = tS + Cfg::colQ, tO = tS + Cfg::colO;
    const bool row_ok = gi >= 0 && gi < N;
    const float lse2 = row_ok ? p.LSE[(size_t)bh * N + gi] * kLog2e : 0.f;
    const float dvec = row_ok ? p.Dvec[(size_t)bh * N + gi] : 0.f;
    unsigned char* cbuf = sdC + m * 16 + cg * (CW / 8) * (DR * 16);
    bool ok = true;
    if (nkb > 0) {
      // this thread's half of the dO row goes to tensor memory as bf16 pairs (the A operand of dP = dO V^T)
      const uint4* src = reinterpret_cast<const uint4*>(dO + ((size_t)bh * N + (row_ok ? gi : 0)) * D) + cg * 8;
      uint32_t w[32];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 v = row_ok ? __ldg(src + i) : make_uint4(0u, 0u, 0u, 0u);
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
      }
      tc::tmem_st32u(tO + 32 * cg, w);
      tc::tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(do_full);
    }
    for (int kb = 0; kb < nkb && ok; ++kb) {
      ok = __all_sync(0xffffffffu, (p.selftest_expire && kb == 0)
                                       ? tc::mbar_wait(never_bar, 0, s_abort, tc::kSelfTestSpinLimit)
                                       : tc::mbar_wait(sdp_full, kb & 1, s_abort));
      if (!ok) break;
      tc::tc_fence_after();
      float s[CW], dp[CW];
      tc::tmem_ld32_nowait(tS + 64 * (kb & 1) + CW * cg, s);
      tc::tmem_ld32_nowait(tP + CW * cg, dp);
      tc::tmem_wait_ld();
      tc::tc_fence_before();
      tc::mbar_arrive(&s_free[kb & 1]);
      const int j0 = kb * BC + CW * cg;
      const int jlim = row_ok ? (p.causal ? min(N - 1, gi - band) : N - 1) : -1;   // last key owned here
      uint32_t pk32[CW / 2];
      if (__all_sync(0xffffffffu, j0 + CW - 1 <= jlim)) {      // whole block owned by every row of the warp: no masking
#pragma unroll
        for (int i = 0; i < CW; i += 2) {
          const float c0 = exp2f(s[i] - lse2) * (dp[i] - dvec);
          const float c1 = exp2f(s[i + 1] - lse2) * (dp[i + 1] - dvec);
          pk32[i / 2] = pack_bf16(c0, c1);
        }
      } else {
#pragma unroll
        for (int i = 0; i < CW; i += 2) {
          float c0 = exp2f(s[i] - lse2) * (dp[i] - dvec);
          float c1 = exp2f(s[i + 1] - lse2) * (dp[i + 1] - dvec);
          if (j0 + i > jlim) c0 = 0.f;
          if (j0 + i + 1 > jlim) c1 = 0.f;
          pk32[i / 2] = pack_bf16(c0, c1);
        }
      }
      if (kb > 0) {   // dQ(kb-1) has finished reading the dC buffer
        ok = __all_sync(0xffffffffu, tc::mbar_wait(dq_done, (kb - 1) & 1, s_abort));
        if (!ok) break;
      }
#pragma unroll
      for (int kc = 0; kc < CW / 8; ++kc)
        *reinterpret_cast<uint4*>(cbuf + kc * (DR * 16)) = make_uint4(pk32[4 * kc], pk32[4 * kc + 1], pk32[4 * kc + 2], pk32[4 * kc + 3]);
      tc::fence_proxy_async_smem();
      tc::mbar_arrive(dc_full);
    }
    // ---- epilogue: the owned dQ rows of this tile, 64 of the 128 columns per thread ----
    if (nkb > 0 && ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(dq_done, (nkb - 1) & 1, s_abort));
    tc::tc_fence_after();
    const bool have = (nkb > 0) && ok;
    const bool store = row_ok && (m < OWN) && (gi >= p.row_base) && (gi < p.row_end);
    float* orow = p.dQ + ((size_t)bh * N + (row_ok ? gi : 0)) * D + 64 * cg;
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      float o[32];
      if (have) {
        tc::tmem_ld32(tQ + 64 * cg + c * 32, o);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0.f;
      }
      if (store) {
#pragma unroll
        for (int i = 0; i < 32; i += 4)
          *reinterpret_cast<float4*>(orow + c * 32 + i) = make_float4(o[i] * kLn2, o[i + 1] * kLn2, o[i + 2] * kLn2, o[i + 3] * kLn2);
      }
    }
  }
  __syncwarp();

  tc::tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicExch(p.status, 1);
    // nothing of this CTA may still be in flight when its shared and tensor memory are given up
    if (warp > W_TMA) tc::mma_commit_e(mma_drain);
    if (tid == W_TMA * 32) {
      volatile int never = 0;
      if (nkb > 0) {
        tc::mbar_wait(q_full, 0, &never);
        const int issued = *s_issued;
        for (int id = max(0, issued - NSLOT); id < issued; ++id) tc::mbar_wait(&full[id % NSLOT], (id / NSLOT) & 1, &never);
      }
      tc::mbar_wait(mma_drain, 0, &never);
    }
    __syncthreads();
  }
  if (warp == W_S) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

// ==========================================================================================
// dK-tilde / dV, d = 128
// ==========================================================================================
struct Dkv128Cfg {
  static constexpr int D = 128;
  static constexpr int BK = 64;                // keys per CTA (= columns of the transposed accumulators)
  static constexpr int BR = 128;               // query rows per block (= TMEM lanes of S and dP)
  static constexpr int HALO = 16;
  static constexpr int QR = BR + HALO;         // 144 rows of Q per block
  static constexpr int MAXCQ = 6;              // resident Kt tiles
  static constexpr int SLAB_BYTES = BK * 128;  // 64 keys x 64 elements, 128-byte swizzle
  static constexpr int KT_BYTES = 2 * SLAB_BYTES;
  static constexpr int DO_SLAB = BR * 128;     // 128 rows x 64 elements, 128-byte swizzle
  static constexpr int oKt = 0;
  static constexpr int oV = oKt + MAXCQ * KT_BYTES;
  static constexpr int Q_SLAB = QR * 128;      // 144 rows x 64 elements, 128-byte swizzle
  static constexpr int oQ = oV + KT_BYTES;                      // two slabs
  static constexpr int odO = oQ + QR * D * 2;                   // two slabs
  static constexpr int oP = odO + 2 * DO_SLAB;                  // P  : [BK/8][BR][16 B]  (MN-major B operand)
  static constexpr int oDC = oP + (BK / 8) * BR * 16;           // dC : same layout
  static constexpr int oBar = oDC + (BK / 8) * BR * 16;
  static constexpr int kSmemBytes = oBar + 512 + 1024;
  static_assert(odO % 1024 == 0 && oV % 1024 == 0 && oQ % 1024 == 0 && Q_SLAB % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");
  static_assert(kSmemBytes <= 227 * 1024, "dK/dV kernel (d = 128): shared memory budget");
  static constexpr int kTmemCols = 512;        // dV^T at 0, dKt_a^T at 64 (1 + a), scratch X (S / dP) at 448
  static constexpr int colX = 448;
  static constexpr int kEwWarps = 8;
  static constexpr int kThreads = (kEwWarps + 4) * 32;   // + producer, issuer S, issuers A0 and A1
};

__global__ void __launch_bounds__(Dkv128Cfg::kThreads, 1)
bwd_dkdv_tc128_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                      const __grid_constant__ CUtensorMap tmKt, const __grid_constant__ CUtensorMap tmV,
                      const BwdTcParams p) {
  using Cfg = Dkv128Cfg;
  constexpr int D = Cfg::D, BK = Cfg::BK, BR = Cfg::BR, HALO = Cfg::HALO, QR = Cfg::QR;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sKt = smem + Cfg::oKt;
  unsigned char* sV = smem + Cfg::oV;
  unsigned char* sQ = smem + Cfg::oQ;
  unsigned char* sdO = smem + Cfg::odO;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* kv_full = bars;
  uint64_t* q_full = kv_full + 1;        // Q of the block staged
  uint64_t* q_free = q_full + 1;         // the three issuers are done with it (3 commits)
  uint64_t* do_full = q_free + 1;        // dO of the block staged
  uint64_t* do_free = do_full + 1;       // dP and dV^T of the block have read it (2 commits)
  uint64_t* st_full = do_free + 1;       // S in X
  uint64_t* xs_free = st_full + 1;       // S taken into registers (256 arrivals): X free for the next dP
  uint64_t* dpt_full = xs_free + 1;      // dP in X
  uint64_t* xd_free = dpt_full + 1;      // dP taken into registers (256 arrivals): X free for S
  uint64_t* pdc_full = xd_free + 1;      // P and dC (bf16) written to shared memory (256 arrivals)
  uint64_t* pdc_free = pdc_full + 1;     // the dV^T / dKt^T MMAs that read them have completed (2 commits)
  uint64_t* all_done = pdc_free + 1;
  uint64_t* never_bar = all_done + 1;
  uint64_t* mma_drain = never_bar + 1;
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(mma_drain + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_q_issued = s_abort + 1;    // blocks whose Q / dO copies the producer has issued
  volatile int* s_do_issued = s_abort + 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int band = pq + pk;
  int h, b, j0;
  dkdv_block_order(BK, h, b, j0);          // (batch, head)-major, key-tile-major tail
  j0 += p.key_base;
  const int bh = b * p.H + h;
  const int nQB = (N + BR - 1) / BR;
  const int qb_begin = p.causal ? min(nQB, (j0 + band) / BR) : 0;
  const int nblk = nQB - qb_begin;

  if (tid == 0) {
    tc::mbar_init(kv_full, 1);
    tc::mbar_init(q_full, 1); tc::mbar_init(q_free, 3);
    tc::mbar_init(do_full, 1); tc::mbar_init(do_free, 2);
    tc::mbar_init(st_full, 1); tc::mbar_init(xs_free, Cfg::kEwWarps * 32);
    tc::mbar_init(dpt_full, 1); tc::mbar_init(xd_free, Cfg::kEwWarps * 32);
    tc::mbar_init(pdc_full, Cfg::kEwWarps * 32); tc::mbar_init(pdc_free, 2);
    tc::mbar_init(all_done, 2);
    tc::mbar_init(never_bar, 1); tc::mbar_init(mma_drain, 3);
    *s_abort = 0; *s_q_issued = 0; *s_do_issued = 0;
    tc::mbar_fence_init();
  }
  if (warp == Cfg::kEwWarps + 1) {
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory that a kernel of this library writes or reads back
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tX = tmem + Cfg::colX;

  if (warp == Cfg::kEwWarps) {
    // ===================== producer warp (TMA) =====================
    if (nblk > 0) {
      if (lane == 0) {
        tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmdO); tc::tma_prefetch_desc(&tmKt); tc::tma_prefetch_desc(&tmV);
        tc::mbar_expect_tx(kv_full, (cq + 1) * Cfg::KT_BYTES);
        for (int a = 0; a < cq; ++a) {
          tc::tma_load_3d(sKt + a * Cfg::KT_BYTES, &tmKt, kv_full, 0, j0, bh * cq + a);
          tc::tma_load_3d(sKt + a * Cfg::KT_BYTES + Cfg::SLAB_BYTES, &tmKt, kv_full, 64, j0, bh * cq + a);
        }
        tc::tma_load_3d(sV, &tmV, kv_full, 0, j0, bh);
        tc::tma_load_3d(sV + Cfg::SLAB_BYTES, &tmV, kv_full, 64, j0, bh);
      }
      bool ok = true;
      for (int it = 0; it < nblk && ok; ++it) {
        const int i0 = (qb_begin + it) * BR;
        // ---- dO of block `it` (its buffer is free once dP and dV^T of block it-1 are done) ----
        if (it > 0) {
          ok = __all_sync(0xffffffffu, tc::mbar_wait(do_free, (it - 1) & 1, s_abort));
          if (!ok) break;
        }
        if (lane == 0) {
          tc::mbar_expect_tx(do_full, 2 * Cfg::DO_SLAB);
          tc::tma_load_3d(sdO, &tmdO, do_full, 0, i0, bh);
          tc::tma_load_3d(sdO + Cfg::DO_SLAB, &tmdO, do_full, 64, i0, bh);
          *s_do_issued = it + 1;
        }
        // ---- Q of block `it` (free once S and every dKt^T tap of block it-1 are done) ----
        if (it > 0) {
          ok = __all_sync(0xffffffffu, tc::mbar_wait(q_free, (it - 1) & 1, s_abort));
          if (!ok) break;
        }
        if (lane == 0) {
          tc::mbar_expect_tx(q_full, QR * D * 2);
          tc::tma_load_3d(sQ, &tmQ, q_full, 0, i0 - HALO, bh);
          tc::tma_load_3d(sQ + Cfg::Q_SLAB, &tmQ, q_full, 64, i0 - HALO, bh);
          *s_q_issued = it + 1;
        }
      }
    }
  } else if (warp == Cfg::kEwWarps + 1) {
    // ===================== MMA issuer S: dP and S of block `it` into the scratch columns X ==========
    if (nblk > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescT = tc::make_idesc(BR, BK, 0, 0);    // 128 x 64, K-major operands
      const uint64_t dKtB = tc::make_sdesc(smem_u32(sKt), 16, 1024, tc::kLayoutSW128);
      const uint32_t kt_hi = (uint32_t)(dKtB >> 32), kt_lo = (uint32_t)dKtB;
      const uint32_t v_lo = kt_lo + (uint32_t)((Cfg::oV - Cfg::oKt) >> 4);
      const uint64_t dOk = tc::make_sdesc(smem_u32(sdO), 16, 1024, tc::kLayoutSW128);
      const uint32_t o_lo = (uint32_t)dOk;                         // same high word as the Kt tiles
      // Q^(a), K-major: the same swizzled tile with the start address moved down by the tap's row shift.  The
      // tensor core applies the 128-byte swizzle to the absolute shared-memory address, exactly as TMA did when
      // it wrote the tile, so a start that is a multiple of 128 bytes (not of the 1024-byte pattern) reads the
      // shifted rows correctly.
      const uint64_t dQk = tc::make_sdesc(smem_u32(sQ) + (HALO - pq) * 128, 16, 1024, tc::kLayoutSW128);
      const uint32_t qk_lo = (uint32_t)dQk;                        // same high word as the Kt tiles
      bool ok = tc::mbar_wait_warp(kv_full, 0, s_abort);
      // X holds dP(it) first (taken into registers by the element-wise warps), then S(it):
      //   dP(0) | S(0) dP(1) | S(1) dP(2) | ...
      auto issue_dP = [&](int it) {
        if (!tc::mbar_wait_warp(do_full, it & 1, s_abort)) { ok = false; return; }
        tc::tc_fence_after();
        tc::mma_ss2e<0>(tX, o_lo, kt_hi, v_lo, kt_hi, idescT);               // dP = dO V^T
#pragma unroll
        for (int k = 1; k < D / 16; ++k)
          tc::mma_ss2e<1>(tX, o_lo + (uint32_t)((k >> 2) * (Cfg::DO_SLAB >> 4) + (k & 3) * 2), kt_hi,
                          v_lo + (uint32_t)((k >> 2) * (Cfg::SLAB_BYTES >> 4) + (k & 3) * 2), kt_hi, idescT);
        tc::mma_commit_e(dpt_full);
        tc::mma_commit_e(do_free);
      };
      if (ok) issue_dP(0);
      for (int it = 0; it < nblk && ok; ++it) {
        if (!tc::mbar_wait_warp(q_full, it & 1, s_abort)) { ok = false; break; }
        if (!tc::mbar_wait_warp(xd_free, it & 1, s_abort)) { ok = false; break; }   // dP(it) has left X
        tc::tc_fence_after();
        // S = sum_a Q^(a) Kt_a^T
        for (int a = 0; a < cq; ++a) {
          const uint32_t b_lo = kt_lo + (uint32_t)(a * (Cfg::KT_BYTES >> 4));
          const uint32_t a_lo = qk_lo + (uint32_t)(a * (128 >> 4));       // row shift = +128 B per row
          tc::mma_ss2pe(tX, a_lo, kt_hi, b_lo, kt_hi, idescT, a != 0);
#pragma unroll
          for (int k = 1; k < D / 16; ++k)
            tc::mma_ss2e<1>(tX, a_lo + (uint32_t)((k >> 2) * (Cfg::Q_SLAB >> 4) + (k & 3) * 2), kt_hi,
                            b_lo + (uint32_t)((k >> 2) * (Cfg::SLAB_BYTES >> 4) + (k & 3) * 2), kt_hi, idescT);
        }
        tc::mma_commit_e(st_full);
        tc::mma_commit_e(q_free);
        if (!tc::mbar_wait_warp(xs_free, it & 1, s_abort)) { ok = false; break; }   // S(it) has left X
        tc::tc_fence_after();
        if (it + 1 < nblk) issue_dP(it + 1);
      }
    }
  } else if (warp >= Cfg::kEwWarps + 2) {
    // ===================== MMA issuers A0 / A1: dV^T += dO^T P ; dKt_a^T += Q^(a)T dC =====================
    const int ai = warp - (Cfg::kEwWarps + 2);
    if (nblk > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescA = tc::make_idesc(D, BK, 1, 1);     // 128 (head dim) x 64 (keys), both operands MN-major
      // A0 takes dV^T and the first half of the taps, A1 the rest
      const int ntap = p.ntap, tap0 = p.tap0, accb = p.with_dv ? 1 : 0;
      const int t_half = ntap / 2;
      const int t_begin = ai == 0 ? 0 : t_half, t_end = ai == 0 ? t_half : ntap;
      // dO read MN-major (M = head dim across the two slabs, K = rows): 16 rows = 2048 bytes per step
      const uint64_t dOm = tc::make_sdesc(smem_u32(sdO), Cfg::DO_SLAB, 1024, tc::kLayoutSW128);
      // Q read MN-major (M = head dim across the two slabs, K = rows, shifted by the tap through the start address)
      const uint64_t dQm = tc::make_sdesc(smem_u32(sQ) + (HALO - pq) * 128, Cfg::Q_SLAB, 1024, tc::kLayoutSW128);
      // P / dC: N = keys in 8-key chunks BR * 16 bytes apart, K = rows 16 bytes apart
      const uint64_t dPb = tc::make_sdesc(smem_u32(smem + Cfg::oP), 128, BR * 16, tc::kLayoutNone);
      const uint64_t dCb = tc::make_sdesc(smem_u32(smem + Cfg::oDC), 128, BR * 16, tc::kLayoutNone);
      const uint32_t om_hi = (uint32_t)(dOm >> 32), om_lo = (uint32_t)dOm;
      const uint32_t qm_hi = (uint32_t)(dQm >> 32), qm_lo = (uint32_t)dQm;
      const uint32_t pb_hi = (uint32_t)(dPb >> 32), pb_lo = (uint32_t)dPb, cb_lo = (uint32_t)dCb;
      bool ok = true;
      for (int it = 0; it < nblk && ok; ++it) {
        const uint32_t acc_on = it != 0;
        if (!tc::mbar_wait_warp(q_full, it & 1, s_abort)) { ok = false; break; }
        if (ai == 0 && !tc::mbar_wait_warp(do_full, it & 1, s_abort)) { ok = false; break; }
        if (!tc::mbar_wait_warp(pdc_full, it & 1, s_abort)) { ok = false; break; }
        tc::tc_fence_after();
        if (ai == 0) {
          if (p.with_dv) {
            tc::mma_ss2pe(tmem, om_lo, om_hi, pb_lo, pb_hi, idescA, acc_on);
#pragma unroll
            for (int k = 1; k < BR / 16; ++k)
              tc::mma_ss2e<1>(tmem, om_lo + (uint32_t)(k * (2048 / 16)), om_hi, pb_lo + (uint32_t)(k * 16), pb_hi, idescA);
          }
          tc::mma_commit_e(do_free);
        }
        for (int i = t_begin; i < t_end; ++i) {
          const uint32_t dacc = tmem + 64 * (accb + i);
          const uint32_t a_lo = qm_lo + (uint32_t)((tap0 + i) * (128 >> 4));     // K (row) shift = +128 B per row
          tc::mma_ss2pe(dacc, a_lo, qm_hi, cb_lo, pb_hi, idescA, acc_on);
#pragma unroll
          for (int k = 1; k < BR / 16; ++k)
            tc::mma_ss2e<1>(dacc, a_lo + (uint32_t)(k * (2048 / 16)), qm_hi, cb_lo + (uint32_t)(k * 16), pb_hi, idescA);
        }
        tc::mma_commit_e(q_free);
        tc::mma_commit_e(pdc_free);
      }
      if (ok) tc::mma_commit_e(all_done);
    }
  } else {
    // ===================== element-wise warps: query row = lane, CW keys per thread =====================
    constexpr int NCG = Cfg::kEwWarps / 4, CW = BK / NCG;     // column groups (warps per lane quarter), columns each
    const int qtr = warp & 3, cg = warp >> 2;
    const int row = qtr * 32 + lane;
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const uint32_t tXl = tX + lane_base + CW * cg;
    bool ok = true;
    float dpc[CW];                                      // dP of the block about to be processed
    // every thread fetches the statistics of its own row (LSE in log2 units, D), one block ahead
    float lse2 = 0.f, dvec = 0.f;
    if (nblk > 0) {
      const int gi = qb_begin * BR + row;
      if (gi < N) { lse2 = p.LSE[(size_t)bh * N + gi] * kLog2e; dvec = p.Dvec[(size_t)bh * N + gi]; }
    }
    if (nblk > 0) {
      ok = __all_sync(0xffffffffu, p.selftest_expire ? tc::mbar_wait(never_bar, 0, s_abort, tc::kSelfTestSpinLimit)
                                                     : tc::mbar_wait(dpt_full, 0, s_abort));
      if (ok) {
        tc::tc_fence_after();
        tc::tmem_ldn(tXl, dpc);
        tc::tc_fence_before();
        tc::mbar_arrive(xd_free);
      }
    }
    for (int it = 0; it < nblk && ok; ++it) {
      const int i0 = (qb_begin + it) * BR;
      const int gi = i0 + row;
      float lse2_next = 0.f, dvec_next = 0.f;
      if (it + 1 < nblk && gi + BR < N) {
        lse2_next = p.LSE[(size_t)bh * N + gi + BR] * kLog2e;
        dvec_next = p.Dvec[(size_t)bh * N + gi + BR];
      }
      ok = __all_sync(0xffffffffu, tc::mbar_wait(st_full, it & 1, s_abort));
      if (!ok) break;
      tc::tc_fence_after();
      float s[CW];
      tc::tmem_ldn(tXl, s);
      tc::tc_fence_before();
      tc::mbar_arrive(xs_free);
      // P[i, key] = exp2(S - LSE_i), kept only where this kernel owns the entry; dC = P (dP - D_i)
      uint32_t pp[CW / 2], cc[CW / 2];
      const int kbase = j0 + CW * cg;
      if ((j0 + BK <= N) && (i0 + BR <= N) && (!p.causal || j0 + BK - 1 + band <= i0)) {   // block owned entirely
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
          const float p0 = exp2f(s[c] - lse2), p1 = exp2f(s[c + 1] - lse2);
          pp[c / 2] = pack_bf16(p0, p1);
          cc[c / 2] = pack_bf16(p0 * (dpc[c] - dvec), p1 * (dpc[c + 1] - dvec));
        }
      } else {
        const int jlim = (gi < N) ? (p.causal ? min(N - 1, gi - band) : N - 1) : -1;   // last key this row owns here
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
          const float p0 = (kbase + c <= jlim) ? exp2f(s[c] - lse2) : 0.f;
          const float p1 = (kbase + c + 1 <= jlim) ? exp2f(s[c + 1] - lse2) : 0.f;
          pp[c / 2] = pack_bf16(p0, p1);
          cc[c / 2] = pack_bf16(p0 * (dpc[c] - dvec), p1 * (dpc[c + 1] - dvec));
        }
      }
      if (it > 0) {   // the MMAs of block it-1 have finished reading the P / dC buffers
        ok = __all_sync(0xffffffffu, tc::mbar_wait(pdc_free, (it - 1) & 1, s_abort));
        if (!ok) break;
      }
      {
        unsigned char* pt = smem + Cfg::oP + row * 16;
        unsigned char* dc = smem + Cfg::oDC + row * 16;
#pragma unroll
        for (int q4 = 0; q4 < CW / 8; ++q4) {          // 8 keys (16 bytes) per chunk
          *reinterpret_cast<uint4*>(pt + ((CW / 8) * cg + q4) * (BR * 16)) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(dc + ((CW / 8) * cg + q4) * (BR * 16)) = make_uint4(cc[4 * q4], cc[4 * q4 + 1], cc[4 * q4 + 2], cc[4 * q4 + 3]);
        }
      }
      tc::fence_proxy_async_smem();
      tc::mbar_arrive(pdc_full);
      // dP of the next block: its dO is staged once dV^T of this block has read the buffer, which in turn
      // waits for the P tile just written -- so it can only be taken out of X here, not earlier
      if (it + 1 < nblk) {
        ok = __all_sync(0xffffffffu, tc::mbar_wait(dpt_full, (it + 1) & 1, s_abort));
        if (!ok) break;
        tc::tc_fence_after();
        tc::tmem_ldn(tXl, dpc);
        tc::tc_fence_before();
        tc::mbar_arrive(xd_free);
      }
      lse2 = lse2_next; dvec = dvec_next;
    }
    // ---- epilogue: the accumulators hold dV^T and dKt_a^T (lane = head dim, column = key); chunks of 32
    // keys are dealt round-robin to the two column groups ----
    if (nblk > 0 && ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(all_done, 0, s_abort));
    tc::tc_fence_after();
    const bool have = (nblk > 0) && ok;
    const int nacc = (p.with_dv ? 1 : 0) + p.ntap;
    const int dcol = qtr * 32 + lane;                   // head-dim index of this lane
    for (int ch = cg; ch < 2 * nacc; ch += NCG) {
      const int acc = ch >> 1, half = ch & 1;
      float o[32];
      if (have) {
        tc::tmem_ld32(tmem + lane_base + ch * 32, o);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0.f;
      }
      const int key0 = j0 + half * 32;
      if (p.with_dv && acc == 0) {
        float* dst = p.dV + ((size_t)bh * N + key0) * D + dcol;      // a warp writes 32 consecutive floats per key
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (key0 + i < N) dst[(size_t)i * D] = o[i];
      } else {
        // dKt_a leaves as bf16 [key][d]: neighbouring lanes pair up so that every lane stores one 4-byte word
        const int tap = p.tap0 + acc - (p.with_dv ? 1 : 0);
        bf16* dst = p.dKt + (((size_t)bh * cq + tap) * N + key0) * D + (dcol & ~1);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float mine_even = o[i], mine_odd = o[i + 1];
          const float other_even = __shfl_xor_sync(0xffffffffu, mine_even, 1);
          const float other_odd = __shfl_xor_sync(0xffffffffu, mine_odd, 1);
          // even lane: key i, columns (dcol, dcol + 1); odd lane: key i + 1, columns (dcol - 1, dcol)
          const bool odd = lane & 1;
          const uint32_t w = odd ? pack_bf16(other_odd, mine_odd) : pack_bf16(mine_even, other_even);
          const int key = key0 + i + (odd ? 1 : 0);
          if (key < N) *reinterpret_cast<uint32_t*>(dst + (size_t)(i + (odd ? 1 : 0)) * D) = w;
        }
      }
    }
  }
  __syncwarp();

  tc::tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicExch(p.status, 1);
    // MMAs and copies of this CTA are waited for (bounded) before its memories go
    if (warp > Cfg::kEwWarps) tc::mma_commit_e(mma_drain);
    if (tid == Cfg::kEwWarps * 32) {
      volatile int never = 0;
      if (nblk > 0) {
        tc::mbar_wait(kv_full, 0, &never);
        const int qi = *s_q_issued, di = *s_do_issued;
        if (qi > 0) tc::mbar_wait(q_full, (qi - 1) & 1, &never);
        if (di > 0) tc::mbar_wait(do_full, (di - 1) & 1, &never);
      }
      tc::mbar_wait(mma_drain, 0, &never);
    }
    __syncthreads();
  }
  if (warp == Cfg::kEwWarps + 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

// ==========================================================================================
// host side
// ==========================================================================================
cudaError_t launch_bwd_dq_tc128(const TrainParams& p, const __nv_bfloat16* Kt, int* status, cudaStream_t stream) {
  using Cfg = Dq128Cfg;
  constexpr int D = Cfg::D;
  const size_t BH = (size_t)p.B * p.H;
  alignas(64) CUtensorMap tmQ, tmKt, tmV;
  if (!make_tensor_map_bf16(&tmQ, p.Q, D, p.N, BH, 64, Cfg::QR, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmKt, Kt, D, p.N, BH * p.cq, 64, Cfg::BC, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmV, p.V, D, p.N, BH, 64, Cfg::BC, true)) return cudaErrorInvalidValue;
  BwdTcParams bp = {};
  bp.LSE = p.LSE; bp.Dvec = p.Dvec; bp.dQ = p.dQ; bp.status = status;
  bp.H = p.H; bp.N = p.N; bp.cq = p.cq; bp.ck = p.ck; bp.causal = p.causal;
  bp.selftest_expire = take_selftest_expire(kKernBwdDqTc);
  bp.row_base = win_lo(p); bp.row_end = win_hi(p); bp.row_anchor = bp.row_end;
  bp.own = Cfg::BM - (p.cq - 1);
  auto kern = bwd_dq_tc128_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((bp.row_end - bp.row_base + bp.own - 1) / bp.own, p.H, p.B);
  { ScopedKernelTimer timer_(kKernBwdDqTc, stream);
    e = launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tmQ, tmKt, tmV, p.dO, bp); }
  return e;
}

cudaError_t launch_bwd_dkdv_tc128(const TrainParams& p, const __nv_bfloat16* Kt, __nv_bfloat16* dKt, int* status, int with_dv,
                                  int key_lo, int key_hi, cudaStream_t stream) {
  using Cfg = Dkv128Cfg;
  constexpr int D = Cfg::D;
  const size_t BH = (size_t)p.B * p.H;
  alignas(64) CUtensorMap tmQ, tmdO, tmKt, tmV;
  if (!make_tensor_map_bf16(&tmQ, p.Q, D, p.N, BH, 64, Cfg::QR, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmdO, p.dO, D, p.N, BH, 64, Cfg::BR, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmKt, Kt, D, p.N, BH * p.cq, 64, Cfg::BK, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmV, p.V, D, p.N, BH, 64, Cfg::BK, true)) return cudaErrorInvalidValue;
  BwdTcParams bp = {};
  bp.LSE = p.LSE; bp.Dvec = p.Dvec; bp.dV = p.dV; bp.dKt = dKt; bp.status = status;
  bp.H = p.H; bp.N = p.N; bp.cq = p.cq; bp.ck = p.ck; bp.causal = p.causal;
  bp.tap0 = 0; bp.ntap = p.cq; bp.with_dv = with_dv;
  bp.key_base = key_lo;
  bp.selftest_expire = take_selftest_expire(kKernBwdDkdvTc);
  auto kern = bwd_dkdv_tc128_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((key_hi - key_lo + Cfg::BK - 1) / Cfg::BK, p.H, p.B);
  return launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tmQ, tmdO, tmKt, tmV, bp);
}

}  // namespace fmta
