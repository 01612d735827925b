// Stacked-GEMM conv-attention backward on tcgen05 / TMEM / TMA (entries off the causal band).
//
// With Kt_a[j] = scale * log2(e) * sum_b theta[a,b] k_{j+b-pad_k} (the forward's pre-pass) and
// Q^(a)[i] = q_{i-(pad_q-a)}, every entry with query - key >= pad_q + pad_k satisfies
//     C = sum_a Q^(a) Kt_a^T,   P = exp2(C - LSE*log2e),   dP = dO V^T,   dC = P * (dP - D)
//     dQ[i'] = ln2 * sum_a sum_j dC[i' + pad_q - a, j] Kt_a[j]
//     dKt_a  = dC^T Q^(a)  (gradient w.r.t. Kt_a / (scale*log2e) ... i.e. before the pre-pass scaling)     dV = P^T dO
// and dK / dTheta follow from dKt_a by the adjoint of the pre-pass (dk_post_mma_kernel).
// The band entries are handled by bwd_band_kernel (bwd_band.cu), which adds its part to the same
// outputs afterwards.
//
//   bwd_dq_tc_kernel   : CTA = NT query-row tiles, loops key blocks.  A tile computes dC for
//                        128 rows but owns only the first 120 of them as dQ rows: dQ row i'
//                        needs dC rows i'..i'+pad_q, so consecutive tiles overlap by 8 rows
//                        (recomputed, like the halo of the exact kernels) and no dQ row is
//                        ever shared between CTAs.  The row shift of dC is free: dC is staged
//                        in shared memory as a 128-byte-swizzled [rows][64 keys] tile, and the tensor
//                        core applies the swizzle to the absolute address, so a view shifted by s
//                        rows is the same tile with the descriptor start address moved by 128 s bytes.
//                        With STREAM the kernel also leaves P and dC in global memory (bwd_stream.cu).
//   bwd_dkdv_tc_kernel : CTA = 128 keys (= TMEM lanes), loops 64-row query blocks; transposed
//                        scores S^T = Kt_a Q^(a)T so that P^T and dC^T are produced with keys on the
//                        lanes (rows of the dV / dKt accumulators).  Q is staged once per block as a
//                        swizzled tile; its row-shifted views are start-address offsets as above.
// Head dim 64 here; head dim 128 in bwd_tc128.cu.
// Every mbarrier wait is bounded; no TMA multicast, no cluster, cta_group::1 only.
#include <cuda.h>
#include <cuda_runtime.h>

#include "fmta_params.h"
#include "bwd_tc.cuh"
#include "fmta_tc.cuh"
#include "launch_util.cuh"

namespace fmta {

// ==========================================================================================
// dQ
// ==========================================================================================
template <int D, bool STREAM = false>   // STREAM: the kernel also leaves P and dC in global memory (see bwd_stream.cu)
struct DqCfg {
  static_assert(D == 64, "the dQ tensor-core kernel is instantiated for d = 64");
  static constexpr int BM = 128;               // dC rows per tile (= TMEM lanes)
  static constexpr int OWN = 120;              // dQ rows a tile owns at most when its rows must start on a multiple of 8 (STREAM); else 128 - pad_q (dQ row i needs dC rows i .. i + pad_q)
  static constexpr int OWN_MAX = 128;
  static constexpr int BC = 64;                // keys per block
  static constexpr int NT = 2;                 // row tiles per CTA
  static constexpr int HALO = 16;
  // rows of Q staged: 264 are read; the buffer is 272 so that both TMA boxes of QR / 2 rows x 16 bytes land
  // on 128-byte boundaries of shared memory (a tiled TMA copy needs that of its destination)
  static constexpr int QR = ((HALO + OWN_MAX * (NT - 1) + BM + 15) / 16) * 16;
  static_assert((QR / 2 * 16) % 128 == 0, "TMA destination alignment");
  static constexpr int DR = BM + 16;           // rows of a dC buffer (16 zero rows below)
  static constexpr int TILE_BYTES = BC * 128;  // Kt / V ring tile: 64 keys x 64 elements
  static constexpr int NSLOT = STREAM ? 11 : 15;   // the Kt tiles of one key block held for its dQ MMAs (cq <= 7) while
                                               // the next block's cq + 1 tiles stream in: 2 cq + 1 slots (four of them
                                               // make room for the P tiles when P and dC are streamed out)
  static constexpr int oQ = 0;                                  // [D/8][QR][16 B]
  static constexpr int odO = oQ + QR * D * 2;                   // NT x [128 rows][128 B], 128B swizzle
  static constexpr int DC_BYTES = DR * 128;                     // one dC buffer: [DR rows][128 B], 128B swizzle
  static constexpr int odC = odO + NT * BM * 128;               // NT buffers
  static_assert(odC % 1024 == 0 && DC_BYTES % 1024 == 0, "swizzled dC buffers start on 1024-byte boundaries");
  static constexpr int P_BYTES = BM * 128;                      // STREAM: one P tile, [128 rows][128 B], 128B swizzle
  static constexpr int oP = odC + NT * DC_BYTES;
  static constexpr int oRing = ((oP + (STREAM ? NT * P_BYTES : 0) + 1023) / 1024) * 1024;
  static constexpr int oBar = oRing + NSLOT * TILE_BYTES;
  static constexpr int kSmemBytes = oBar + 512 + 1024;
  static constexpr int kTmemCols = 512;        // per tile t: S (two buffers) at 256t and 256t+64, dP at 256t+128, dQ at 256t+192
  static constexpr int kThreads = (NT * 4 + 1 + 2 * NT) * 32;   // element-wise warps, TMA warp, two MMA issuer warps per tile
};

template <int D, bool STREAM>
__global__ void __launch_bounds__(DqCfg<D, STREAM>::kThreads, 1)
bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                 const __grid_constant__ CUtensorMap tmKt, const __grid_constant__ CUtensorMap tmV,
                 const BwdTcParams p) {
  using Cfg = DqCfg<D, STREAM>;
  constexpr int BM = Cfg::BM, BC = Cfg::BC, NT = Cfg::NT, HALO = Cfg::HALO, QR = Cfg::QR;
  const int OWN = STREAM ? Cfg::OWN : p.own;
  constexpr int DR = Cfg::DR, NSLOT = Cfg::NSLOT;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem + Cfg::oQ;
  unsigned char* sdO = smem + Cfg::odO;
  unsigned char* sdC = smem + Cfg::odC;
  unsigned char* sRing = smem + Cfg::oRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* full = bars;                 // [NSLOT]
  uint64_t* empty = bars + NSLOT;        // [NSLOT]  count 2 NT
  uint64_t* q_full = bars + 2 * NSLOT;   // Q and dO staged
  uint64_t* sdp_full = q_full + 1;       // [NT] S and dP of the block complete
  uint64_t* s_free = sdp_full + 2;       // [NT][2] S buffer b and dP of a block taken into registers (128 arrivals)
  uint64_t* dc_full = s_free + 4;        // [NT] dC tile written to shared memory (128 arrivals)
  uint64_t* dq_done = dc_full + 2;       // [NT] dQ MMAs of the block complete (dC buffer reusable)
  uint64_t* never_bar = dq_done + 2;     // nothing arrives here (expiry self-test)
  uint64_t* mma_drain = never_bar + 1;   // abort path: every issuer's MMAs have completed (2 NT arrivals)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(mma_drain + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_issued = s_abort + 1;  // ring tiles the producer has issued

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int band = pq + pk;
  const int rows_per_cta = OWN * NT;
  const int nQB = (p.row_anchor - p.row_base + rows_per_cta - 1) / rows_per_cta;
  // CTAs are dispatched in linear block order; walk it length-major (all (batch, head) pairs of the
  // longest row block first) so that the greedy hardware scheduler ends with the short CTAs
  const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int nBH = gridDim.y * gridDim.z;
  const int qb = nQB - 1 - lin / nBH;
  const int h = (lin % nBH) % (int)gridDim.y, b = (lin % nBH) / (int)gridDim.y;
  const int bh = b * p.H + h;
  // The row blocks are laid out from the END of the rows: when their number is not a multiple of the block, the
  // partly filled block is the first one, which sees the fewest keys, not the last one, which sees them all
  // (N = 4096: the 18th block of 240 rows held 16 rows and walked every key block).  Its rows before row_base are
  // computed (negative rows as zero rows) and not stored.  The variant that leaves P and dC for the streaming dK/dV
  // kernel needs blocks that start at multiples of 8 rows: its anchor is row_end rounded up to one.
  const int R0 = p.row_anchor - (nQB - qb) * rows_per_cta;
  const int nKB = (N + BC - 1) / BC;
  int nkb_t[2] = {0, 0};
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int r0 = R0 + t * OWN;
    if (r0 >= p.row_end || r0 + OWN <= p.row_base) nkb_t[t] = 0;
    else if (p.causal) {
      const int last = min(N - 1, r0 + BM - 1) - band;
      nkb_t[t] = last >= 0 ? min(nKB, last / BC + 1) : 0;
    } else nkb_t[t] = nKB;
  }
  const int nkb = max(nkb_t[0], nkb_t[1]);

  if (tid == 0) {
    for (int i = 0; i < NSLOT; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 2 * NT); }   // every issuer releases every tile
    tc::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&sdp_full[i], 1); tc::mbar_init(&dc_full[i], BM);
      tc::mbar_init(&dq_done[i], 1);
    }
    for (int i = 0; i < 4; ++i) tc::mbar_init(&s_free[i], BM);
    tc::mbar_init(never_bar, 1); tc::mbar_init(mma_drain, 2 * NT);
    *s_abort = 0; *s_issued = 0;
    tc::mbar_fence_init();
  }
  if (warp == NT * 4 + 1) {
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  // zero the dC buffers once: the 16 pad rows below each tile are read by the shifted views
  for (int i = tid; i < NT * Cfg::DC_BYTES / 4; i += Cfg::kThreads) reinterpret_cast<uint32_t*>(sdC)[i] = 0u;
  tc::fence_proxy_async_smem();
  tc::tc_fence_before();
  pdl_trigger();   // the next kernel's CTAs may be scheduled once every CTA here has got this far
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp == NT * 4) {
    // ===================== TMA producer =====================
    if (lane == 0 && nkb > 0) {
      tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmdO); tc::tma_prefetch_desc(&tmKt); tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, QR * D * 2 + NT * BM * 128);
      for (int kc = 0; kc < D / 8; ++kc) {
        tc::tma_load_3d(sQ + kc * (QR * 16), &tmQ, q_full, kc * 8, R0 - HALO, bh);
        tc::tma_load_3d(sQ + kc * (QR * 16) + (QR / 2) * 16, &tmQ, q_full, kc * 8, R0 - HALO + QR / 2, bh);
      }
      for (int t = 0; t < NT; ++t) tc::tma_load_3d(sdO + t * (BM * 128), &tmdO, q_full, 0, R0 + t * OWN, bh);
      int id = 0;
      bool ok = true;
      auto put = [&](const CUtensorMap* map, int y, int z) {
        const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
        if (!tc::mbar_wait(&empty[slot], ph ^ 1, s_abort)) { ok = false; return; }
        tc::mbar_expect_tx(&full[slot], Cfg::TILE_BYTES);
        tc::tma_load_3d(sRing + slot * Cfg::TILE_BYTES, map, &full[slot], 0, y, z);
        ++id;
        *s_issued = id;
      };
      for (int kb = 0; kb < nkb && ok; ++kb) {
        for (int a = 0; a < cq && ok; ++a) put(&tmKt, kb * BC, bh * cq + a);
        if (ok) put(&tmV, kb * BC, bh);
      }
    }
  } else if (warp > NT * 4) {
    // ===================== MMA issuers: two per row tile =====================
    // One thread issues an MMA every 50-100 clocks whatever its size, so S/dP and dQ of a tile
    // are issued by different warps (warps NT*4+1+t: S and dP; warps NT*4+1+NT+t: dQ).
    const int wi = warp - (NT * 4 + 1);
    const int t = wi % NT;
    const bool is_dq = wi >= NT;
    if (nkb > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescS = tc::make_idesc(BM, BC, 0, 0);    // S, dP: 128 x 64, both K-major
      constexpr uint32_t idescQ = tc::make_idesc(BM, D, 0, 1);     // dQ: 128 x D, B (Kt) MN-major
      const uint64_t dQa = tc::make_sdesc(smem_u32(sQ) + (HALO + t * OWN - pq) * 16, QR * 16, 128, tc::kLayoutNone);
      const uint64_t dOa = tc::make_sdesc(smem_u32(sdO) + t * (BM * 128), 16, 1024, tc::kLayoutSW128);
      // dC is a 128-byte-swizzled [rows][64 keys] tile; its row-shifted views start 128 bytes per row further
      const uint64_t dCa = tc::make_sdesc(smem_u32(sdC) + t * Cfg::DC_BYTES, 16, 1024, tc::kLayoutSW128);
      const uint64_t dKb = tc::make_sdesc(smem_u32(sRing), 16, 1024, tc::kLayoutSW128);
      const uint32_t q_hi = (uint32_t)(dQa >> 32), q_lo = (uint32_t)dQa;
      const uint32_t o_hi = (uint32_t)(dOa >> 32), o_lo = (uint32_t)dOa;
      const uint32_t c_hi = (uint32_t)(dCa >> 32), c_lo = (uint32_t)dCa;
      const uint32_t k_hi = (uint32_t)(dKb >> 32), k_lo0 = (uint32_t)dKb;
      const uint32_t tS = tmem + t * 256, tP = tS + 128, tQ = tS + 192;   // S is double-buffered: tS + 64 * (kb & 1)
      const int my_nkb = nkb_t[t];
      const int per = cq + 1;                                // ring tiles per key block
      bool ok = tc::mbar_wait_warp(q_full, 0, s_abort);
      if (!is_dq) {
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const bool active = kb < my_nkb;
          const uint32_t tSb = tS + 64 * (kb & 1);
          if (active && kb > 1) {      // the element-wise warps have taken S(kb-2) out of this buffer
            ok = tc::mbar_wait_warp(&s_free[2 * t + (kb & 1)], ((kb >> 1) - 1) & 1, s_abort);
            tc::tc_fence_after();
          }
          for (int a = 0; a < cq && ok; ++a) {
            const int id = kb * per + a, slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
            if (active) {
              tc::tc_fence_after();
              const uint32_t b_lo = k_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
              const uint32_t a_lo = q_lo + (uint32_t)a;
              tc::mma_ss2pe(tSb, a_lo, q_hi, b_lo, k_hi, idescS, a != 0);
#pragma unroll
              for (int k = 1; k < D / 16; ++k)
                tc::mma_ss2e<1>(tSb, a_lo + (uint32_t)(2 * k * QR), q_hi, b_lo + (uint32_t)(2 * k), k_hi, idescS);
            }
            tc::mma_commit_e(&empty[slot]);      // (the dQ issuers hold the Kt tile until dQ(kb) is done)
          }
          if (!ok) break;
          const int id = kb * per + cq, slot = id % NSLOT, ph = (id / NSLOT) & 1;
          if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
          if (active && kb > 0) {      // dP is single-buffered: block kb-1 must have left it
            ok = tc::mbar_wait_warp(&s_free[2 * t + ((kb - 1) & 1)], ((kb - 1) >> 1) & 1, s_abort);
            if (!ok) break;
          }
          if (active) {
            tc::tc_fence_after();
            const uint32_t b_lo = k_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
            tc::mma_ss2e<0>(tP, o_lo, o_hi, b_lo, k_hi, idescS);
#pragma unroll
            for (int k = 1; k < D / 16; ++k)
              tc::mma_ss2e<1>(tP, o_lo + (uint32_t)(2 * k), o_hi, b_lo + (uint32_t)(2 * k), k_hi, idescS);
          }
          tc::mma_commit_e(&empty[slot]);
          if (active) tc::mma_commit_e(&sdp_full[t]);
        }
      } else {
        for (int kb = 0; kb < nkb && ok; ++kb) {
          const bool active = kb < my_nkb;
          if (active) {
            ok = tc::mbar_wait_warp(&dc_full[t], kb & 1, s_abort);
            tc::tc_fence_after();
            if constexpr (STREAM) {
              // P and dC of the tile's owned rows leave as they lie in shared memory (the swizzled image): the
              // global tensors are tile-major [B*H][row block of 64][key block of 64][64 rows x 128 bytes], a
              // tile's rows start at a multiple of 8, so a row keeps its swizzle phase and the streaming kernel
              // gets the same image with a plain copy.  One piece per 64-row block of the global layout.
              if (ok && tc::elect_one()) {
                const int r0 = R0 + t * OWN, r1 = min(N, r0 + OWN);
                const int nkb64 = p.ldp >> 6;
                const uint64_t pol_ef = tc::l2_policy_evict_first();
                for (int g = max(r0, 0); g < r1;) {
                  const int gend = min(r1, (g | 63) + 1);
                  const size_t tile = (((size_t)bh * ((N + 63) >> 6) + (g >> 6)) * nkb64 + kb) * 4096 + (size_t)(g & 63) * 64;
                  tc::bulk_store_hint(p.Pout + tile, smem + Cfg::oP + t * Cfg::P_BYTES + (g - r0) * 128, (uint32_t)(gend - g) * 128, pol_ef);
                  tc::bulk_store_hint(p.dCout + tile, sdC + t * Cfg::DC_BYTES + (g - r0) * 128, (uint32_t)(gend - g) * 128, pol_ef);
                  g = gend;
                }
                tc::tma_store_commit();
              }
            }
          }
          for (int a = 0; a < cq && ok; ++a) {
            const int id = kb * per + a, slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
            if (active) {
              tc::tc_fence_after();
              const uint32_t b_lo = k_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
              const uint32_t a_lo = c_lo + (uint32_t)((pq - a) * (128 >> 4));       // dC rows i' + pad_q - a
              tc::mma_ss2pe(tQ, a_lo, c_hi, b_lo, k_hi, idescQ, (kb != 0) || (a != 0));
#pragma unroll
              for (int k = 1; k < BC / 16; ++k)
                tc::mma_ss2e<1>(tQ, a_lo + (uint32_t)(2 * k), c_hi, b_lo + (uint32_t)(k * (2048 / 16)), k_hi, idescQ);
            }
            tc::mma_commit_e(&empty[slot]);
          }
          if (!ok) break;
          {   // the V tile of the block is not read here: release it right away
            const int id = kb * per + cq, slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; break; }
            if (tc::elect_one()) tc::mbar_arrive(&empty[slot]);
          }
          if constexpr (STREAM) {   // the bulk copies have read their tiles before the buffers are handed back
            if (active && tc::elect_one()) tc::tma_store_wait_read();
            __syncwarp();
          }
          if (active) tc::mma_commit_e(&dq_done[t]);
        }
        if constexpr (STREAM) {
          if (tc::elect_one()) tc::tma_store_wait_all();
          __syncwarp();
        }
      }
    }
  } else {
    // ===================== element-wise warpgroups: one dC row per thread =====================
    const int t = warp >> 2;
    const int m = tid & (BM - 1);
    const int gi = R0 + t * OWN + m;                    // query index of this dC row
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + t * 256 + lane_base, tP = tS + 128, tQ = tS + 192;
    const int my_nkb = nkb_t[t];
    const bool row_ok = gi >= 0 && gi < N;
    const float lse2 = row_ok ? p.LSE[(size_t)bh * N + gi] * kLog2e : 0.f;
    const float dvec = row_ok ? p.Dvec[(size_t)bh * N + gi] : 0.f;
    unsigned char* ctile = sdC + t * Cfg::DC_BYTES;     // this tile's dC buffer; chunk c of row r at r*128 + ((c ^ (r & 7)) << 4)
    unsigned char* cbuf = ctile + m * 128;
    // STREAM: P goes to a second swizzled tile beside dC; the dQ issuer of the tile sends both out with bulk copies
    unsigned char* pbuf = smem + Cfg::oP + t * Cfg::P_BYTES + m * 128;
    bool ok = true;
    for (int kb = 0; kb < my_nkb && ok; ++kb) {
      ok = __all_sync(0xffffffffu, (p.selftest_expire && kb == 0)
                                       ? tc::mbar_wait(never_bar, 0, s_abort, tc::kSelfTestSpinLimit)
                                       : tc::mbar_wait(&sdp_full[t], kb & 1, s_abort));
      if (!ok) break;
      tc::tc_fence_after();
      float s[BC], dp[BC];
      {
        float t0[32], t1[32], t2[32], t3[32];
        const uint32_t tSb = tS + 64 * (kb & 1);
        tc::tmem_ld32_nowait(tSb, t0); tc::tmem_ld32_nowait(tSb + 32, t1);
        tc::tmem_ld32_nowait(tP, t2); tc::tmem_ld32_nowait(tP + 32, t3);
        tc::tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) { s[i] = t0[i]; s[32 + i] = t1[i]; dp[i] = t2[i]; dp[32 + i] = t3[i]; }
      }
      tc::tc_fence_before();
      tc::mbar_arrive(&s_free[2 * t + (kb & 1)]);
      const int j0 = kb * BC;
      const int jlim = row_ok ? (p.causal ? min(N - 1, gi - band) : N - 1) : -1;   // last key owned here
      uint32_t pk32[BC / 2], pp32[STREAM ? BC / 2 : 1];
      if constexpr (!STREAM) {
        // one loop with the ownership mask always applied: two predicated selects per pair cost less than the
        // registers a separate unmasked copy of the loop takes (this kernel is capped at 128 registers)
#pragma unroll
        for (int i = 0; i < BC; i += 2) {
          float c0 = exp2f(s[i] - lse2) * (dp[i] - dvec);
          float c1 = exp2f(s[i + 1] - lse2) * (dp[i + 1] - dvec);
          if (j0 + i > jlim) c0 = 0.f;
          if (j0 + i + 1 > jlim) c1 = 0.f;
          pk32[i / 2] = pack_bf16(c0, c1);
        }
      } else {   // same arithmetic, keeping P as well
#pragma unroll
        for (int i = 0; i < BC; i += 2) {
          float p0 = exp2f(s[i] - lse2), p1 = exp2f(s[i + 1] - lse2);
          if (j0 + i > jlim) p0 = 0.f;
          if (j0 + i + 1 > jlim) p1 = 0.f;
          pp32[i / 2] = pack_bf16(p0, p1);
          pk32[i / 2] = pack_bf16(p0 * (dp[i] - dvec), p1 * (dp[i + 1] - dvec));
        }
      }
      if (kb > 0) {   // dQ(kb-1) has finished reading the dC buffer (STREAM: and the bulk copies of block kb-1 both tiles)
        ok = __all_sync(0xffffffffu, tc::mbar_wait(&dq_done[t], (kb - 1) & 1, s_abort));
        if (!ok) break;
      }
#pragma unroll
      for (int kc = 0; kc < BC / 8; ++kc) {
        *reinterpret_cast<uint4*>(cbuf + ((kc ^ (m & 7)) << 4)) = make_uint4(pk32[4 * kc], pk32[4 * kc + 1], pk32[4 * kc + 2], pk32[4 * kc + 3]);
        if constexpr (STREAM)
          *reinterpret_cast<uint4*>(pbuf + ((kc ^ (m & 7)) << 4)) = make_uint4(pp32[4 * kc], pp32[4 * kc + 1], pp32[4 * kc + 2], pp32[4 * kc + 3]);
      }
      tc::fence_proxy_async_smem();
      tc::mbar_arrive(&dc_full[t]);
    }
    // ---- streaming outputs: zero the key blocks this tile did not visit but a 64-row x 128-key tile of the
    // dK/dV kernel that holds one of its rows may read: up to the end of the 128-key tile of key
    // (last row + 63 - band); without a causal mask, up to ldp ----
    if (STREAM && row_ok && m < OWN) {
      const int nkb64 = p.ldp >> 6;
      const size_t tile_row = ((size_t)bh * ((N + 63) >> 6) + (gi >> 6)) * nkb64 * 4096 + (size_t)(gi & 63) * 64;
      bf16* prow = p.Pout + tile_row;     // key block kz of this row: + kz * 4096
      bf16* crow = p.dCout + tile_row;
      const int r_last = R0 + t * OWN + BM - 1;
      const int fill_end = p.causal ? min(p.ldp, (max(r_last + 63 - band, 0) / 128 + 1) * 128) : p.ldp;
      for (int kz = my_nkb; kz * BC < fill_end; ++kz)
#pragma unroll
        for (int c = 0; c < BC / 8; ++c) {
          *reinterpret_cast<uint4*>(prow + (size_t)kz * 4096 + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
          *reinterpret_cast<uint4*>(crow + (size_t)kz * 4096 + 8 * c) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    // ---- epilogue: the owned dQ rows of this tile ----
    if (my_nkb > 0 && ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(&dq_done[t], (my_nkb - 1) & 1, s_abort));
    tc::tc_fence_after();
    const bool have = (my_nkb > 0) && ok;
    const bool store = row_ok && (m < OWN) && (gi >= p.row_base) && (gi < p.row_end);
    float* orow = p.dQ + ((size_t)bh * N + (row_ok ? gi : 0)) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      float o[32];
      if (have) {
        tc::tmem_ld32(tQ + c * 32, o);
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
    // nothing of this CTA may still be in flight when its shared and tensor memory are given up: every
    // issuer commits behind its last MMA; one thread waits (bounded) for those commits, for the Q / dO
    // copies and for the latest copy issued into each ring slot
    if (warp > NT * 4) tc::mma_commit_e(mma_drain);
    if (tid == NT * 4 * 32 && nkb > 0) {
      volatile int never = 0;
      tc::mbar_wait(q_full, 0, &never);
      const int issued = *s_issued;
      for (int id = max(0, issued - NSLOT); id < issued; ++id) tc::mbar_wait(&full[id % NSLOT], (id / NSLOT) & 1, &never);
    }
    if (tid == NT * 4 * 32) { volatile int never = 0; tc::mbar_wait(mma_drain, 0, &never); }
    __syncthreads();
  }
  if (warp == NT * 4 + 1) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

// ==========================================================================================
// dK-tilde / dV
// ==========================================================================================
template <int D, int CQMAX, bool PAIR>   // PAIR: two adjacent taps share one 128-wide MMA
struct DkvCfg {
  static_assert(D == 64, "the dK/dV tensor-core kernel is instantiated for d = 64");
  static constexpr int BK = 128;               // keys per CTA (= TMEM lanes)
  static constexpr int BR = 64;                // query rows per block
  static constexpr int HALO = 8;               // rows of Q staged above the block (pad_q <= 5)
  static constexpr int QR = BR + HALO;         // 72 rows of Q per stage
  static constexpr int MAXCQ = CQMAX;          // resident Kt tiles; at most 7 accumulators of 64 columns + 64 scratch = 512
  static constexpr int NSTG = (CQMAX <= 6) ? 4 : 3;   // query-block stages in flight (a seventh resident tile leaves room for three)
  static constexpr int KT_BYTES = BK * 128;    // one resident Kt / V tile
  static constexpr int oKt = 0;                                   // MAXCQ x [128 keys][128 B], 128B swizzle
  static constexpr int oV = oKt + MAXCQ * KT_BYTES;
  static constexpr int oStage = oV + KT_BYTES;
  static constexpr int sgdO = 0;                                  // [64 rows][128 B], 128B swizzle
  static constexpr int sgQ = BR * 128;                            // [QR rows][128 B], 128B swizzle (one TMA copy)
  static constexpr int sgLD = sgQ + QR * 128;                     // LSE*log2e [64], D [64]
  static constexpr int STAGE_BYTES = ((sgLD + 2 * BR * 4 + 1023) / 1024) * 1024;
  static constexpr int oPT = oStage + NSTG * STAGE_BYTES;         // P^T : [BR/8][128 keys][16 B] (K-major A operand)
  static constexpr int oDCT = oPT + (BR / 8) * BK * 16;           // dC^T: same layout
  static constexpr int oBar = oDCT + (BR / 8) * BK * 16;
  static constexpr int kSmemBytes = oBar + 512 + 1024;
  static_assert(kSmemBytes <= 227 * 1024, "dK/dV kernel: shared memory budget");
  static constexpr int kTmemCols = 512;        // dV at 0, dKt_a at 64*(1+a), scratch X at 448
  static constexpr int colX = 448;
  static constexpr int kEwWarps = 16;
  static constexpr int kThreads = (kEwWarps + 4) * 32;   // + producer, issuer S, issuers A0 and A1
};

template <int D, int CQMAX, bool PAIR>
__global__ void __launch_bounds__(DkvCfg<D, CQMAX, PAIR>::kThreads, 1)
bwd_dkdv_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmKt, const __grid_constant__ CUtensorMap tmV,
                   const __grid_constant__ CUtensorMap tmdKt, const __grid_constant__ CUtensorMap tmdV,
                   const BwdTcParams p) {
  using Cfg = DkvCfg<D, CQMAX, PAIR>;
  constexpr int BK = Cfg::BK, BR = Cfg::BR, HALO = Cfg::HALO, QR = Cfg::QR, NSTG = Cfg::NSTG;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sKt = smem + Cfg::oKt;
  unsigned char* sV = smem + Cfg::oV;
  unsigned char* sStage = smem + Cfg::oStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* full = bars;                 // [NSTG]
  uint64_t* empty = bars + NSTG;         // [NSTG]
  uint64_t* kv_full = bars + 2 * NSTG;
  uint64_t* st_full = kv_full + 1;       // S^T in X
  uint64_t* xs_free = st_full + 1;       // S^T taken into registers (256 arrivals): X free for the next dP^T
  uint64_t* dpt_full = xs_free + 1;      // dP^T in X
  uint64_t* xd_free = dpt_full + 1;      // dP^T taken into registers (256 arrivals): X free for S^T
  uint64_t* pdc_full = xd_free + 1;      // P^T and dC^T (bf16) written to shared memory (256 arrivals)
  uint64_t* pdc_free = pdc_full + 1;     // the dV / dKt MMAs that read them have completed
  uint64_t* all_done = pdc_free + 1;
  uint64_t* never_bar = all_done + 1;    // nothing arrives here (expiry self-test)
  uint64_t* mma_drain = never_bar + 1;   // abort path: every issuer's MMAs have completed (3 arrivals)
  uint64_t* v_full = mma_drain + 1;      // the V tile alone: dP^T(0) starts on it while the Kt tiles are still in flight
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(v_full + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_issued = s_abort + 1;  // stages the producer has issued
  volatile int* s_kt_issued = s_abort + 2;   // the copies of the Kt tiles have been issued

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int band = pq + pk;
  // (batch, head)-major block order: the key tiles of one (batch, head) run side by side and share its
  // Q / dO stream in L2 (the length-major order of the dQ kernel was 7 % slower here)
  // block order: see dkdv_block_order
  int h, b, j0;
  dkdv_block_order(BK, h, b, j0);
  j0 += p.key_base;
  const int bh = b * p.H + h;
  const int nQB = (N + BR - 1) / BR;
  const int qb_begin = p.causal ? min(nQB, (j0 + band) / BR) : 0;
  const int nblk = nQB - qb_begin;

  if (tid == 0) {
    for (int i = 0; i < NSTG; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 3); }   // three issuers release a stage
    tc::mbar_init(kv_full, 1); tc::mbar_init(v_full, 1);
    tc::mbar_init(st_full, 1); tc::mbar_init(xs_free, Cfg::kEwWarps * 32);
    tc::mbar_init(dpt_full, 1); tc::mbar_init(xd_free, Cfg::kEwWarps * 32);
    tc::mbar_init(pdc_full, Cfg::kEwWarps * 32); tc::mbar_init(pdc_free, 2);
    tc::mbar_init(all_done, 2);
    tc::mbar_init(never_bar, 1); tc::mbar_init(mma_drain, 3);
    *s_abort = 0; *s_issued = 0; *s_kt_issued = 0;
    tc::mbar_fence_init();
  }
  if (warp == Cfg::kEwWarps + 1) {
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tX = tmem + Cfg::colX;

  if (warp == Cfg::kEwWarps) {
    // ===================== producer warp (TMA + row statistics) =====================
    if (nblk > 0) {
      if (lane == 0) {
        tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmdO); tc::tma_prefetch_desc(&tmKt); tc::tma_prefetch_desc(&tmV);
        // V first, then (below) the first query block, then the Kt tiles: that is the order in which the
        // first MMAs need them (dP^T(0) = V dO^T, then S^T(0))
        tc::mbar_expect_tx(v_full, Cfg::KT_BYTES);
        tc::tma_load_3d(sV, &tmV, v_full, 0, j0, bh);
      }
      bool ok = true;
      for (int it = 0; it < nblk && ok; ++it) {
        const int st = it % NSTG, ph = (it / NSTG) & 1;
        const int i0 = (qb_begin + it) * BR;
        unsigned char* sg = sStage + st * Cfg::STAGE_BYTES;
        ok = __all_sync(0xffffffffu, tc::mbar_wait(&empty[st], ph ^ 1, s_abort));
        if (!ok) break;
        // LSE * log2(e) and D of the 64 rows: two rows per lane, plain loads and stores
        float* ld = reinterpret_cast<float*>(sg + Cfg::sgLD);
#pragma unroll
        for (int r = lane; r < BR; r += 32) {
          const int gi = i0 + r;
          ld[r] = gi < N ? p.LSE[(size_t)bh * N + gi] * kLog2e : 0.f;
          ld[BR + r] = gi < N ? p.Dvec[(size_t)bh * N + gi] : 0.f;
        }
        __syncwarp();
        if (lane == 0) {
          tc::mbar_expect_tx(&full[st], BR * 128 + QR * 128);
          tc::tma_load_3d(sg + Cfg::sgdO, &tmdO, &full[st], 0, i0, bh);
          tc::tma_load_3d(sg + Cfg::sgQ, &tmQ, &full[st], 0, i0 - HALO, bh);
          *s_issued = it + 1;
          if (it == 0) {
            tc::mbar_expect_tx(kv_full, cq * Cfg::KT_BYTES);
            for (int a = 0; a < cq; ++a) tc::tma_load_3d(sKt + a * Cfg::KT_BYTES, &tmKt, kv_full, 0, j0, bh * cq + a);
            *s_kt_issued = 1;
          }
        }
      }
    }
  } else if (warp == Cfg::kEwWarps + 1) {
    // ===================== MMA issuer S: S^T and dP^T of block `it` into the scratch columns X ==========
    // One thread issues an MMA every 50-100 clocks whatever its size, so the three MMA streams of a
    // block (S^T/dP^T, dV + first half of the dKt taps, second half of the taps) have a warp each.
    if (nblk > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescT = tc::make_idesc(BK, BR, 0, 0);    // 128 x 64, K-major operands
      const uint64_t dKtA = tc::make_sdesc(smem_u32(sKt), 16, 1024, tc::kLayoutSW128);
      const uint32_t kt_hi = (uint32_t)(dKtA >> 32), kt_lo = (uint32_t)dKtA;
      const uint32_t v_lo = kt_lo + (uint32_t)((Cfg::oV - Cfg::oKt) >> 4);
      bool ok = tc::mbar_wait_warp(v_full, 0, s_abort);
      // X holds dP^T(it) first (taken by the element-wise warps one block ahead), then S^T(it):
      //   dP^T(0) | S^T(0) dP^T(1) | S^T(1) dP^T(2) | ...
      auto issue_dPT = [&](int it) {
        const int st = it % NSTG, ph = (it / NSTG) & 1;
        const uint64_t dOk = tc::make_sdesc(smem_u32(sStage + st * Cfg::STAGE_BYTES) + Cfg::sgdO, 16, 1024, tc::kLayoutSW128);
        const uint32_t o_hi = (uint32_t)(dOk >> 32), o_lo = (uint32_t)dOk;
        if (!tc::mbar_wait_warp(&full[st], ph, s_abort)) { ok = false; return; }
        tc::tc_fence_after();
        tc::mma_ss2e<0>(tX, v_lo, kt_hi, o_lo, o_hi, idescT);               // dP^T = V dO^T
#pragma unroll
        for (int k = 1; k < D / 16; ++k)
          tc::mma_ss2e<1>(tX, v_lo + (uint32_t)(2 * k), kt_hi, o_lo + (uint32_t)(2 * k), o_hi, idescT);
        tc::mma_commit_e(dpt_full);
      };
      if (ok) issue_dPT(0);
      for (int it = 0; it < nblk && ok; ++it) {
        const int st = it % NSTG;
        const uint32_t sg = smem_u32(sStage + st * Cfg::STAGE_BYTES);
        // Q^(a), K-major, N = rows: the swizzled tile with its start address moved by the tap's row shift,
        // 128 bytes per row (the tensor core swizzles the absolute shared-memory address, as TMA did)
        const uint64_t dQk = tc::make_sdesc(sg + Cfg::sgQ + (HALO - pq) * 128, 16, 1024, tc::kLayoutSW128);
        const uint32_t qk_hi = (uint32_t)(dQk >> 32), qk_lo = (uint32_t)dQk;
        if (it == 0 && !tc::mbar_wait_warp(kv_full, 0, s_abort)) { ok = false; break; }   // the Kt tiles
        if (!tc::mbar_wait_warp(xd_free, it & 1, s_abort)) { ok = false; break; }   // dP^T(it) has left X
        tc::tc_fence_after();
        // S^T = sum_a Kt_a Q^(a)T
        for (int a = 0; a < cq; ++a) {
          const uint32_t a_lo = kt_lo + (uint32_t)(a * (Cfg::KT_BYTES >> 4));
          const uint32_t b_lo = qk_lo + (uint32_t)(a * (128 >> 4));
          tc::mma_ss2pe(tX, a_lo, kt_hi, b_lo, qk_hi, idescT, a != 0);
#pragma unroll
          for (int k = 1; k < D / 16; ++k)
            tc::mma_ss2e<1>(tX, a_lo + (uint32_t)(2 * k), kt_hi, b_lo + (uint32_t)(2 * k), qk_hi, idescT);
        }
        tc::mma_commit_e(st_full);
        tc::mma_commit_e(&empty[st]);        // this issuer's reads of the stage (dO for dP^T, Q for S^T) are done then
        if (!tc::mbar_wait_warp(xs_free, it & 1, s_abort)) { ok = false; break; }   // S^T(it) has left X
        tc::tc_fence_after();
        if (it + 1 < nblk) issue_dPT(it + 1);
      }
    }
  } else if (warp >= Cfg::kEwWarps + 2) {
    // ===================== MMA issuers A0 / A1: dV += P^T dO ; dKt_a += dC^T Q^(a) =====================
    const int ai = warp - (Cfg::kEwWarps + 2);
    if (nblk > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescA = tc::make_idesc(BK, D, 0, 1);     // 128 x D, B MN-major
      constexpr uint32_t idescA2 = tc::make_idesc(BK, 2 * D, 0, 1); // 128 x 2D: two adjacent taps at once
      // this launch accumulates taps [tap0, tap0 + ntap) (accumulator i at column 64 * (with_dv + i)) and
      // dV (column 0) when with_dv; A0 takes dV and the first half of the tap groups, A1 the rest.  With
      // PAIR a group is two adjacent taps in one 128-wide MMA (an odd last tap goes alone).
      const int ntap = p.ntap, tap0 = p.tap0, accb = p.with_dv ? 1 : 0;
      const int pairs = PAIR ? ntap / 2 : 0, singles = ntap - 2 * pairs;     // groups: `pairs` pairs, then `singles` single taps
      const int ngrp = pairs + singles, g_half = ngrp / 2;
      const int g_begin = ai == 0 ? 0 : g_half, g_end = ai == 0 ? g_half : ngrp;
      const uint64_t dPTa = tc::make_sdesc(smem_u32(smem + Cfg::oPT), BK * 16, 128, tc::kLayoutNone);
      const uint64_t dDCa = tc::make_sdesc(smem_u32(smem + Cfg::oDCT), BK * 16, 128, tc::kLayoutNone);
      const uint32_t pt_hi = (uint32_t)(dPTa >> 32), pt_lo = (uint32_t)dPTa, dc_lo = (uint32_t)dDCa;
      bool ok = true;
      for (int it = 0; it < nblk && ok; ++it) {
        const int st = it % NSTG, ph = (it / NSTG) & 1;
        const uint32_t sg = smem_u32(sStage + st * Cfg::STAGE_BYTES);
        // the same tile read MN-major (N = head dim, K = rows shifted by the tap).  A second 64-column atom
        // placed 128 bytes = ONE ROW after the first is the next tap's operand, so ONE 128 x 128 MMA
        // accumulates two adjacent filter taps (dKt_a | dKt_{a+1}) += dC^T [Q^(a) | Q^(a+1)] from one copy of Q
        const uint64_t dQm = tc::make_sdesc(sg + Cfg::sgQ + (HALO - pq) * 128, 128, 1024, tc::kLayoutSW128);
        const uint64_t dOk = tc::make_sdesc(sg + Cfg::sgdO, 16, 1024, tc::kLayoutSW128);
        const uint32_t qm_hi = (uint32_t)(dQm >> 32), qm_lo = (uint32_t)dQm;
        const uint32_t o_hi = (uint32_t)(dOk >> 32), o_lo = (uint32_t)dOk;
        const uint32_t acc_on = it != 0;
        if (!tc::mbar_wait_warp(&full[st], ph, s_abort)) { ok = false; break; }
        if (!tc::mbar_wait_warp(pdc_full, it & 1, s_abort)) { ok = false; break; }
        tc::tc_fence_after();
        if (ai == 0 && p.with_dv) {
          tc::mma_ss2pe(tmem, pt_lo, pt_hi, o_lo, o_hi, idescA, acc_on);
#pragma unroll
          for (int k = 1; k < BR / 16; ++k)
            tc::mma_ss2e<1>(tmem, pt_lo + (uint32_t)(2 * k * BK), pt_hi, o_lo + (uint32_t)(k * (2048 / 16)), o_hi, idescA);
        }
        for (int gi = g_begin; gi < g_end; ++gi) {
          const bool pair = gi < pairs;
          const int i = pair ? 2 * gi : 2 * pairs + (gi - pairs);        // first accumulator / tap of the group
          const uint32_t dacc = tmem + 64 * (accb + i);
          const uint32_t b_lo = qm_lo + (uint32_t)((tap0 + i) * (128 >> 4));
          const uint32_t idg = pair ? idescA2 : idescA;
          tc::mma_ss2pe(dacc, dc_lo, pt_hi, b_lo, qm_hi, idg, acc_on);
#pragma unroll
          for (int k = 1; k < BR / 16; ++k)
            tc::mma_ss2e<1>(dacc, dc_lo + (uint32_t)(2 * k * BK), pt_hi, b_lo + (uint32_t)(k * (2048 / 16)), qm_hi, idg);
        }
        tc::mma_commit_e(&empty[st]);
        tc::mma_commit_e(pdc_free);
      }
      if (ok) tc::mma_commit_e(all_done);
    }
  } else {
    // ===================== element-wise warps: key = lane, CW query rows per thread =====================
    constexpr int NCG = Cfg::kEwWarps / 4, CW = BR / NCG;     // column groups (warps per lane quarter), columns each
    const int qtr = warp & 3, cg = warp >> 2;
    const int key = j0 + qtr * 32 + lane;
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    const uint32_t tXl = tX + lane_base + CW * cg;
    bool ok = true;
    float dpc[CW];                                      // dP^T of the block about to be processed
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
      const int st = it % NSTG, ph = (it / NSTG) & 1;
      const int i0 = (qb_begin + it) * BR;
      const float* ld = reinterpret_cast<const float*>(sStage + st * Cfg::STAGE_BYTES + Cfg::sgLD) + CW * cg;
      ok = __all_sync(0xffffffffu, tc::mbar_wait(&full[st], ph, s_abort));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, tc::mbar_wait(st_full, it & 1, s_abort));
      if (!ok) break;
      tc::tc_fence_after();
      float s[CW];
      tc::tmem_ldn(tXl, s);
      tc::tc_fence_before();
      tc::mbar_arrive(xs_free);
      // take the next block's dP^T out of X right away, so that its S^T can start while this
      // block's arithmetic runs
      float dpn[CW];
      if (it + 1 < nblk) {
        ok = __all_sync(0xffffffffu, tc::mbar_wait(dpt_full, (it + 1) & 1, s_abort));
        if (!ok) break;
        tc::tc_fence_after();
        tc::tmem_ldn(tXl, dpn);
        tc::tc_fence_before();
        tc::mbar_arrive(xd_free);
      }
      // P^T[key, i] = exp2(S^T - LSE_i), kept only where this kernel owns the entry; dC^T = P^T (dP^T - D_i)
      uint32_t pp[CW / 2], cc[CW / 2];
      if ((j0 + BK <= N) && (i0 + BR <= N) && (!p.causal || j0 + BK - 1 + band <= i0)) {   // block owned entirely
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
          const float p0 = exp2f(s[c] - ld[c]), p1 = exp2f(s[c + 1] - ld[c + 1]);
          pp[c / 2] = pack_bf16(p0, p1);
          cc[c / 2] = pack_bf16(p0 * (dpc[c] - ld[BR + c]), p1 * (dpc[c + 1] - ld[BR + c + 1]));
        }
      } else {
#pragma unroll
        for (int c = 0; c < CW; c += 2) {
          const int gi = i0 + CW * cg + c;
          const bool own0 = (key < N) && (gi < N) && (!p.causal || key <= gi - band);
          const bool own1 = (key < N) && (gi + 1 < N) && (!p.causal || key <= gi + 1 - band);
          const float p0 = own0 ? exp2f(s[c] - ld[c]) : 0.f;
          const float p1 = own1 ? exp2f(s[c + 1] - ld[c + 1]) : 0.f;
          pp[c / 2] = pack_bf16(p0, p1);
          cc[c / 2] = pack_bf16(p0 * (dpc[c] - ld[BR + c]), p1 * (dpc[c + 1] - ld[BR + c + 1]));
        }
      }
#pragma unroll
      for (int c = 0; c < CW; ++c) dpc[c] = dpn[c];
      if (it > 0) {   // the MMAs of block it-1 have finished reading the P^T / dC^T buffers
        ok = __all_sync(0xffffffffu, tc::mbar_wait(pdc_free, (it - 1) & 1, s_abort));
        if (!ok) break;
      }
      {
        unsigned char* pt = smem + Cfg::oPT + (qtr * 32 + lane) * 16;
        unsigned char* dc = smem + Cfg::oDCT + (qtr * 32 + lane) * 16;
#pragma unroll
        for (int q4 = 0; q4 < CW / 8; ++q4) {          // 8 rows (16 bytes) per K-chunk
          *reinterpret_cast<uint4*>(pt + ((CW / 8) * cg + q4) * (BK * 16)) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
          *reinterpret_cast<uint4*>(dc + ((CW / 8) * cg + q4) * (BK * 16)) = make_uint4(cc[4 * q4], cc[4 * q4 + 1], cc[4 * q4 + 2], cc[4 * q4 + 3]);
        }
      }
      tc::fence_proxy_async_smem();
      tc::mbar_arrive(pdc_full);
    }
    // ---- epilogue: dV and dKt_a rows of this key; 14 chunks of 32 columns dealt round-robin to the column groups ----
    if (nblk > 0 && ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(all_done, 0, s_abort));
    tc::tc_fence_after();
    const bool have = (nblk > 0) && ok;
    const int nacc = (p.with_dv ? 1 : 0) + p.ntap;
    // Everything leaves through shared memory and TMA tile stores, as whole lines: dKt_a as bf16 (its adjoint
    // kernel feeds it to mma.sync as it is) through the Kt tiles, dV as fp32 through the first query-block
    // stage -- neither is read by an MMA any more.  Tiles are [128 keys][128 B] with the 128-byte swizzle, so
    // that the lanes of a warp (one key row each) store without bank conflicts.  The 2 * nacc chunks of 32
    // columns go round by round to the NCG column groups; a round completes two accumulators, whose tiles
    // are sent off at once, so that only the last round's copies are waited for at the end.
    unsigned char* sdV = sStage;                       // columns 0-31 | columns 32-63, KT_BYTES each
    const int row = qtr * 32 + lane;
    const int nrounds = (2 * nacc + NCG - 1) / NCG;
    for (int r = 0; r < nrounds; ++r) {
      const int ch = r * NCG + cg;
      if (ch < 2 * nacc) {
        const int acc = ch >> 1, half = ch & 1;
        float o[32];
        if (have) {
          tc::tmem_ld32(tmem + lane_base + ch * 32, o);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (p.with_dv && acc == 0) {
          unsigned char* tile = sdV + half * Cfg::KT_BYTES + row * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(tile + ((i ^ (row & 7)) << 4)) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        } else {
          unsigned char* tile = sKt + (acc - (p.with_dv ? 1 : 0)) * Cfg::KT_BYTES + row * 128;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(tile + (((half * 4 + i) ^ (row & 7)) << 4)) =
                make_uint4(pack_bf16(o[8 * i], o[8 * i + 1]), pack_bf16(o[8 * i + 2], o[8 * i + 3]),
                           pack_bf16(o[8 * i + 4], o[8 * i + 5]), pack_bf16(o[8 * i + 6], o[8 * i + 7]));
        }
      }
      tc::fence_proxy_async_smem();
      tc::named_bar_sync(1, Cfg::kEwWarps * 32);
      if (tid == 0) {                                  // one thread owns the bulk group of every round
        for (int acc = 2 * r; acc < min(2 * r + 2, nacc); ++acc) {
          if (p.with_dv && acc == 0) {
            tc::tma_store_3d(&tmdV, sdV, 0, j0, bh);
            tc::tma_store_3d(&tmdV, sdV + Cfg::KT_BYTES, 32, j0, bh);
          } else {
            const int t = acc - (p.with_dv ? 1 : 0);
            tc::tma_store_3d(&tmdKt, sKt + t * Cfg::KT_BYTES, 0, j0, bh * cq + p.tap0 + t);
          }
        }
        tc::tma_store_commit();
      }
    }
    if (tid == 0) tc::tma_store_wait_read();
  }
  __syncwarp();

  tc::tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicExch(p.status, 1);
    // as in the dQ kernel: MMAs and copies of this CTA are waited for (bounded) before its memories go
    if (warp > Cfg::kEwWarps) tc::mma_commit_e(mma_drain);
    if (tid == Cfg::kEwWarps * 32) {
      volatile int never = 0;
      if (nblk > 0) {
        tc::mbar_wait(v_full, 0, &never);
        if (*s_kt_issued) tc::mbar_wait(kv_full, 0, &never);
        const int issued = *s_issued;
        for (int it = max(0, issued - NSTG); it < issued; ++it) tc::mbar_wait(&full[it % NSTG], (it / NSTG) & 1, &never);
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

// ------------------------------------------------------------------------------------------
// Adjoint of the Kt pre-pass:   dK[j] = sum_{a,b} scale*theta[a,b] * dKt_a[j - b + pad_k]
//                      dTheta[a,b]   += scale * sum_j <dKt_a[j], k_{j+b-pad_k}>
// Both are small GEMMs on mma.sync, fed straight from the bf16 dKt_a rows in shared memory:
//   dK tile (16 keys x 64) = sum_a T_a (16 x 32) X_a (32 rows x 64), T_a[x, r] = scale*theta[a, x + pad_k + 8 - r]
//       the banded Toeplitz form of filter row a, held as a bf16 (hi, lo) pair so that theta keeps
//       16 mantissa bits, X_a the dKt_a rows from 8 above the tile's first key on;
//   dTheta^T (filter columns x taps) = A B with the contraction over (key, column) pairs:
//       A[b, (j, d)] = k_{j + b - pad_k}[d],  B[(j, d), a] = dKt_a[j, d]  -- for a fixed key the 16
//       contraction steps are 16 consecutive columns, so every fragment row is 16 contiguous bytes
//       of shared memory and the products land in the accumulator already summed per (a, b).
// The rows are staged by TMA (two mbarrier batches, bounded waits), the Toeplitz tiles by one bulk copy.
// One CTA per (64 keys, batch*head); dTheta leaves as one partial per CTA.
#ifndef FMTA_DKPOST_THETA_LO
#define FMTA_DKPOST_THETA_LO 1
#endif
constexpr bool kThetaLo = FMTA_DKPOST_THETA_LO != 0;
struct DkPostCfg {
  static constexpr int D = 64, NT = 256;
  static constexpr int KEYS = 64, HALO = 8, ROWS = KEYS + 2 * HALO;   // c_k <= 17
  // A staged tile is [ROWS][128 B] as TMA writes it with the 128-byte swizzle: the 16-byte chunk c of
  // a row sits at chunk c ^ (address bits 7..9).  Consecutive tiles start 128 bytes further along that
  // pattern, so that the same row of the c_q tap tiles (one dTheta fragment) covers all banks.
  static constexpr int TILE_BYTES = ROWS * 128;
  static constexpr int TILE_STRIDE = TILE_BYTES + 128;
  static constexpr int T_LD = 40, T_ELEMS = 16 * T_LD;        // one 16 x 32 Toeplitz tile (bf16), rows 80 bytes apart
  static constexpr int RED_LD = 7 * 24;              // floats per warp in the dTheta reduction buffer
  __host__ __device__ static constexpr int t_bytes(int cq) { return 2 * cq * T_ELEMS * 2; }
  static constexpr int smem_bytes(int cq) {           // alignment slack + key rows + c_q tap tiles + max(Toeplitz tiles, reduction buffer) + barriers
    return 1024 + (cq + 1) * TILE_STRIDE + (t_bytes(cq) > 8 * RED_LD * 4 ? t_bytes(cq) : 8 * RED_LD * 4) + 64;
  }
};

// The Toeplitz tiles of every head, [H][c_q][hi, lo][16][T_LD] bf16: T[x, r] = scale * theta[a, x + pad_k + 8 - r].
__global__ void dk_post_toeplitz_kernel(const float* __restrict__ theta, bf16* __restrict__ Tg, int cq, int ck, float scale) {
  constexpr int T_LD = DkPostCfg::T_LD, T_ELEMS = DkPostCfg::T_ELEMS, HALO = DkPostCfg::HALO;
  const int h = blockIdx.x, pk = (ck - 1) / 2;
  pdl_trigger();
  for (int i = threadIdx.x; i < cq * 16 * T_LD; i += blockDim.x) {
    const int a = i / (16 * T_LD), x = (i / T_LD) % 16, r = i % T_LD;
    const int bb = x + pk + HALO - r;
    const float w = (r < 32 && bb >= 0 && bb < ck) ? theta[((size_t)h * cq + a) * ck + bb] * scale : 0.f;
    const bf16 hi = __float2bfloat16_rn(w);
    bf16* dst = Tg + ((size_t)h * cq + a) * 2 * T_ELEMS + x * T_LD + r;
    dst[0] = hi;
    dst[T_ELEMS] = __float2bfloat16_rn(w - __bfloat162float(hi));
  }
  // the tiles depend on the filter only, so they are built while the kernel before this one still runs; waiting
  // here keeps "this kernel has completed" implying that one has, which the adjoint kernel behind it relies on
  pdl_wait();
}

__global__ void __launch_bounds__(DkPostCfg::NT, 2)
dk_post_mma_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmX,
                   const bf16* __restrict__ Tg, float* __restrict__ dK, float* __restrict__ dTheta_part, int* status,
                   int H, int N, int cq, int ck, float scale, int n_jblocks, int dfull, int j_base) {
  using Cfg = DkPostCfg;
  constexpr int D = Cfg::D, NT = Cfg::NT, KEYS = Cfg::KEYS, HALO = Cfg::HALO;
  constexpr int T_LD = Cfg::T_LD, T_ELEMS = Cfg::T_ELEMS, RED_LD = Cfg::RED_LD;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // tile 0: key rows, tile 1 + a: dKt_a rows; row r of a tile is key J0 - HALO + r
  unsigned char* sTb = smem + (cq + 1) * Cfg::TILE_STRIDE;
  bf16* sT = reinterpret_cast<bf16*>(sTb);                  // [cq][hi, lo][16][T_LD]
  float* sRed = reinterpret_cast<float*>(sTb);               // takes the place of the Toeplitz tiles once the dK GEMMs are done
  const int t_or_red = Cfg::t_bytes(cq) > 8 * RED_LD * 4 ? Cfg::t_bytes(cq) : 8 * RED_LD * 4;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sTb + t_or_red);
  volatile int* s_abort = reinterpret_cast<volatile int*>(bars + 2);
  // last (batch, head) first: the dK/dV kernel wrote its dKt rows most recently, so they are still in L2
  const int bh = gridDim.y - 1 - blockIdx.y, h = bh % H, b = bh / H;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pk = (ck - 1) / 2;
  const int J0 = j_base + blockIdx.x * KEYS;                 // j_base: the first key of the call's window
  const int col0 = blockIdx.z * D;                           // a CTA handles 64 of the head's `dfull` columns
  const int half = (cq + 1) / 2;                             // the taps arrive in two batches
  // 16-byte chunk c of row r of tile t
  auto at = [&](int t, int r, int c) -> const void* {
    return smem + t * Cfg::TILE_STRIDE + r * 128 + (((c ^ (r + t)) & 7) << 4);
  };

  if (tid == 0) {
    tc::tma_prefetch_desc(&tmK); tc::tma_prefetch_desc(&tmX);
    tc::mbar_init(&bars[0], 1); tc::mbar_init(&bars[1], 1);
    *s_abort = 0;
    tc::mbar_fence_init();
  }
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory
  if (tid == 0) {
    tc::mbar_expect_tx(&bars[0], (1 + half) * Cfg::TILE_BYTES + Cfg::t_bytes(cq));
    tc::tma_load_3d(smem, &tmK, &bars[0], col0, J0 - HALO, bh);
    tc::bulk_load(sTb, Tg + (size_t)h * cq * 2 * T_ELEMS, Cfg::t_bytes(cq), &bars[0]);
    for (int a = 0; a < half; ++a) tc::tma_load_3d(smem + (a + 1) * Cfg::TILE_STRIDE, &tmX, &bars[0], col0, J0 - HALO, bh * cq + a);
    if (cq > half) {
      tc::mbar_expect_tx(&bars[1], (cq - half) * Cfg::TILE_BYTES);
      for (int a = half; a < cq; ++a) tc::tma_load_3d(smem + (a + 1) * Cfg::TILE_STRIDE, &tmX, &bars[1], col0, J0 - HALO, bh * cq + a);
    }
  }
  bool ok = true;

  // ---- dK: warp = (32 keys, 16 columns).  Its two 16-key tiles share the middle one of their three
  // 16-row steps through X_a, and the Toeplitz fragments are the same for every tile ----
  const int cgp = warp & 3, kh = warp >> 2;
  float acc[2][2][4] = {};
  {
    const int l8 = lane & 7, q = lane >> 3;
    const int t_off = (l8 + (q & 1) * 8) * T_LD + (q >> 1) * 8;
    const int x_row = 32 * kh + l8 + (q & 1) * 8, x_chunk = 2 * cgp + (q >> 1);
#pragma unroll
    for (int a = 0; a < 7; ++a) {
      if (a < cq) {
        if (a == 0 || a == half) {
          ok = ok && tc::mbar_wait(&bars[a == 0 ? 0 : 1], 0, s_abort);
        }
        uint32_t ah[2][4], al[2][4];
        ldsm_x4(ah[0], sT + 2 * a * T_ELEMS + t_off);
        ldsm_x4(ah[1], sT + 2 * a * T_ELEMS + t_off + 16);
        if (kThetaLo) {
          ldsm_x4(al[0], sT + (2 * a + 1) * T_ELEMS + t_off);
          ldsm_x4(al[1], sT + (2 * a + 1) * T_ELEMS + t_off + 16);
        }
#pragma unroll
        for (int st = 0; st < 3; ++st) {
          uint32_t bfr[4];
          ldsm_x4_t(bfr, at(a + 1, x_row + 16 * st, x_chunk));
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            const int m = st - ks;                           // the tile whose step ks these rows are
            if (m >= 0 && m < 2) {
              mma_bf16(acc[m][0], ah[ks], bfr[0], bfr[1]);
              mma_bf16(acc[m][1], ah[ks], bfr[2], bfr[3]);
              if (kThetaLo) {
                mma_bf16(acc[m][0], al[ks], bfr[0], bfr[1]);
                mma_bf16(acc[m][1], al[ks], bfr[2], bfr[3]);
              }
            }
          }
        }
      }
    }
  }
  {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int key = J0 + 32 * kh + 16 * m + g + 8 * hh;
          if (key < N)
            *reinterpret_cast<float2*>(dK + ((size_t)bh * N + key) * dfull + col0 + 16 * cgp + 8 * j + 2 * t4) = make_float2(acc[m][j][2 * hh], acc[m][j][2 * hh + 1]);
        }
  }

  // ---- dTheta^T (filter columns x taps): warp = 8 keys, two 32-column contraction steps each ----
  float th[2][4][4] = {};                                    // [16 filter columns][four independent accumulation chains]
  {
    const int l8 = lane & 7, q = lane >> 3;
    const int m0 = l8 + (q & 1) * 8;                         // A fragment row = filter column (past c_k: column 0, unused results)
    const int sA0 = (m0 < ck ? m0 : 0) - pk, sA1 = (m0 + 16 < ck ? m0 + 16 : 0) - pk;
    const int bt = 1 + (l8 < cq ? l8 : 0);                   // B fragment row = tap (past c_q: tap 0); four 8-column slabs
    const bool wide = ck > 16;
#pragma unroll 4
    for (int kk = 0; kk < 8; ++kk) {
      const int row = HALO + 8 * warp + kk;                  // shared-memory row of this key
#pragma unroll
      for (int c0 = 0; c0 < D / 8; c0 += 4) {
        uint32_t bfr[4], a0[4], a1[4];
        ldsm_x4(bfr, at(bt, row, c0 + q));
        ldsm_x4(a0, at(0, row + sA0, c0 + (q >> 1)));
        ldsm_x4(a1, at(0, row + sA0, c0 + 2 + (q >> 1)));
        const int ch = (c0 >> 1) & 2;                        // chains 0, 1 for columns 0..31, 2, 3 for columns 32..63
        mma_bf16(th[0][ch], a0, bfr[0], bfr[1]);
        mma_bf16(th[0][ch + 1], a1, bfr[2], bfr[3]);
        if (wide) {
          ldsm_x4(a0, at(0, row + sA1, c0 + (q >> 1)));
          ldsm_x4(a1, at(0, row + sA1, c0 + 2 + (q >> 1)));
          mma_bf16(th[1][ch], a0, bfr[0], bfr[1]);
          mma_bf16(th[1][ch + 1], a1, bfr[2], bfr[3]);
        }
      }
    }
  }
  __syncthreads();                                           // every warp is done with the Toeplitz tiles
  {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int bb = 16 * m + 8 * hh + g, a = 2 * t4 + u;
          if (a < cq && bb < 24) sRed[warp * RED_LD + a * 24 + bb] = (th[m][0][2 * hh + u] + th[m][1][2 * hh + u]) + (th[m][2][2 * hh + u] + th[m][3][2 * hh + u]);
        }
  }
  __syncthreads();
  const int slot = (b * (int)gridDim.z + (int)blockIdx.z) * n_jblocks + blockIdx.x;   // one partial per CTA
  for (int i = tid; i < cq * ck; i += NT) {
    const int a = i / ck, bb = i % ck;
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += sRed[w * RED_LD + a * 24 + bb];
    dTheta_part[((size_t)slot * H + h) * (cq * ck) + i] = t * scale;
  }
  if (!ok) atomicExch(status, 1);
}

// ==========================================================================================
// host side
// ==========================================================================================
cudaError_t launch_ktilde(const TrainParams& p, __nv_bfloat16* Kt, cudaStream_t stream);

bool bwd_tc_supported(const TrainParams& p) {
  // head dim 64: up to seven query taps (two launches of the dK/dV kernel for the seventh); head dim 128:
  // up to six (the resident stacked key tiles of the dK/dV kernel fill its shared memory)
  const bool shape_ok = (p.d == 64 && p.cq <= 7) || (p.d == 128 && p.cq <= 6);
  return p.theta != nullptr && p.Wmix == nullptr && shape_ok && p.cq >= 1 && tensor_maps_available();
}

size_t bwd_tc_workspace_bytes(int B, int H, int N, int d, int cq) {
  const size_t rows = (size_t)B * H * N;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  // Kt (bf16) + dKt (bf16) + status + the Toeplitz tiles of the dKt adjoint
  return up(rows * cq * d * 2) + up(rows * cq * d * 2) + 2048 + up((size_t)H * DkPostCfg::t_bytes(cq));
}

size_t bwd_tc_stream_workspace_bytes(int B, int H, int N, int d, int cq) {
  return bwd_tc_workspace_bytes(B, H, N, d, cq) + bwd_stream_extra_bytes(B, H, N);
}

// where the streamed P / dC tensors sit in a workspace of bwd_tc_stream_workspace_bytes
static void stream_buffers(const TrainParams& p, void* workspace, __nv_bfloat16** P, __nv_bfloat16** dC, int* ldp) {
  unsigned char* w = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~uintptr_t(1023));
  w += bwd_tc_workspace_bytes(p.B, p.H, p.N, p.d, p.cq);
  *ldp = (p.N + 127) / 128 * 128;
  const size_t one = ((size_t)p.B * p.H * (size_t)((p.N + 63) / 64 * 64) * (size_t)*ldp * 2 + 1023) / 1024 * 1024;
  *P = reinterpret_cast<__nv_bfloat16*>(w);
  *dC = reinterpret_cast<__nv_bfloat16*>(w + one);
}

// Rows N .. 64*ceil(N/64)-1 of the last row block of the tile-major P / dC tensors are read by the streaming
// dK/dV kernel (a whole 64-row tile at a time) but written by nobody: zero them (a few KB per (batch, head)).
__global__ void zero_tail_rows_kernel(bf16* __restrict__ P, bf16* __restrict__ dC, int N, int nkb64) {
  const int nrb = (N + 63) >> 6, r0 = N & 63;
  const size_t tile = ((size_t)blockIdx.y * nrb + (nrb - 1)) * nkb64 + blockIdx.x;
  uint4* p4 = reinterpret_cast<uint4*>(P + tile * 4096 + (size_t)r0 * 64);
  uint4* c4 = reinterpret_cast<uint4*>(dC + tile * 4096 + (size_t)r0 * 64);
  for (int i = threadIdx.x; i < (64 - r0) * 8; i += blockDim.x) { p4[i] = make_uint4(0u, 0u, 0u, 0u); c4[i] = make_uint4(0u, 0u, 0u, 0u); }
}

cudaError_t launch_bwd_dq_tc(const TrainParams& p, void* workspace, bool keep_pdc, cudaStream_t stream) {
  constexpr int D = 64;
  using Cfg = DqCfg<D, false>;
  const size_t rows = (size_t)p.B * p.H * p.N, BH = (size_t)p.B * p.H;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  unsigned char* w = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(w); w += up(rows * p.cq * p.d * 2);
  if (p.Kt_ext) Kt = p.Kt_ext;                        // the stacked key operand kept from the forward
  w += up(rows * p.cq * p.d * 2);
  int* status = nullptr;
  cudaError_t e = status_word_of(reinterpret_cast<int*>(w), stream, &status);
  if (e != cudaSuccess) return e;
  if (!(p.Kt_ext && p.kt_valid)) {
    e = launch_ktilde(p, Kt, stream);
    if (e != cudaSuccess) return e;
  }
  if (p.d == 128) return launch_bwd_dq_tc128(p, Kt, status, stream);
  alignas(64) CUtensorMap tmQ, tmdO, tmKt, tmV;
  if (!make_tensor_map_bf16(&tmQ, p.Q, D, p.N, BH, 8, Cfg::QR / 2, false)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmdO, p.dO, D, p.N, BH, 64, Cfg::BM, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmKt, Kt, D, p.N, BH * p.cq, 64, Cfg::BC, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmV, p.V, D, p.N, BH, 64, Cfg::BC, true)) return cudaErrorInvalidValue;
  BwdTcParams bp = {};
  bp.LSE = p.LSE; bp.Dvec = p.Dvec; bp.dQ = p.dQ; bp.status = status;
  bp.H = p.H; bp.N = p.N; bp.cq = p.cq; bp.ck = p.ck; bp.causal = p.causal;
  bp.selftest_expire = take_selftest_expire(kKernBwdDqTc);
  bp.row_base = win_lo(p); bp.row_end = win_hi(p);
  bp.row_anchor = keep_pdc ? (bp.row_end + 7) / 8 * 8 : bp.row_end;
  bp.own = keep_pdc ? Cfg::OWN : Cfg::BM - (p.cq - 1);
  const int rows_per_cta = bp.own * Cfg::NT;
  dim3 grid((bp.row_anchor - bp.row_base + rows_per_cta - 1) / rows_per_cta, p.H, p.B);
  if (keep_pdc) {
    stream_buffers(p, workspace, &bp.Pout, &bp.dCout, &bp.ldp);
    if (p.N % 64 != 0) zero_tail_rows_kernel<<<dim3(bp.ldp / 64, (unsigned)BH), 128, 0, stream>>>(bp.Pout, bp.dCout, p.N, bp.ldp / 64);
    using CfgS = DqCfg<D, true>;
    auto kern = bwd_dq_tc_kernel<D, true>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, CfgS::kSmemBytes);
    if (e != cudaSuccess) return e;
    ScopedKernelTimer timer_(kKernBwdDqTc, stream);
    kern<<<grid, CfgS::kThreads, CfgS::kSmemBytes, stream>>>(tmQ, tmdO, tmKt, tmV, bp);
    return cudaGetLastError();
  }
  auto kern = bwd_dq_tc_kernel<D, false>;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  { ScopedKernelTimer timer_(kKernBwdDqTc, stream);
    e = launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tmQ, tmdO, tmKt, tmV, bp); }
  return e;
}


// One launch of the dK/dV kernel for the taps [tap0, tap0 + ntap) (and dV).
template <int CQMAX, bool PAIR>
static cudaError_t launch_dkdv_pass(const TrainParams& p, const __nv_bfloat16* Kt, __nv_bfloat16* dKt, int* status, int tap0,
                                    int ntap, int with_dv, int key_lo, int key_hi, cudaStream_t stream) {
  constexpr int D = 64;
  using Cfg = DkvCfg<D, CQMAX, PAIR>;
  const size_t BH = (size_t)p.B * p.H;
  alignas(64) CUtensorMap tmQ, tmdO, tmKt, tmV, tmdKt, tmdV;
  if (!make_tensor_map_bf16(&tmdKt, dKt, D, p.N, BH * p.cq, 64, Cfg::BK, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_f32(&tmdV, p.dV, D, p.N, BH, 32, Cfg::BK, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmQ, p.Q, D, p.N, BH, 64, Cfg::QR, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmdO, p.dO, D, p.N, BH, 64, Cfg::BR, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmKt, Kt, D, p.N, BH * p.cq, 64, Cfg::BK, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmV, p.V, D, p.N, BH, 64, Cfg::BK, true)) return cudaErrorInvalidValue;
  BwdTcParams bp = {};
  bp.LSE = p.LSE; bp.Dvec = p.Dvec; bp.dV = p.dV; bp.dKt = dKt; bp.status = status;
  bp.H = p.H; bp.N = p.N; bp.cq = p.cq; bp.ck = p.ck; bp.causal = p.causal;
  bp.tap0 = tap0; bp.ntap = ntap; bp.with_dv = with_dv;
  bp.key_base = key_lo;
  bp.selftest_expire = take_selftest_expire(kKernBwdDkdvTc);
  auto kern = bwd_dkdv_tc_kernel<D, CQMAX, PAIR>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((key_hi - key_lo + Cfg::BK - 1) / Cfg::BK, p.H, p.B);
  return launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tmQ, tmdO, tmKt, tmV, tmdKt, tmdV, bp);
}

cudaError_t launch_bwd_dkdv_tc(const TrainParams& p, void* workspace, float* dTheta_part_tc, bool keep_pdc, cudaStream_t stream) {
  const int D = p.d;
  const size_t rows = (size_t)p.B * p.H * p.N, BH = (size_t)p.B * p.H;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  unsigned char* w = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~uintptr_t(1023));
  __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(w); w += up(rows * p.cq * D * 2);
  if (p.Kt_ext) Kt = p.Kt_ext;
  __nv_bfloat16* dKt = reinterpret_cast<__nv_bfloat16*>(w); w += up(rows * p.cq * D * 2);
  int* status = registered_status_word();               // else the workspace word the dQ launch cleared
  if (status == nullptr) status = reinterpret_cast<int*>(w);
  cudaError_t e;
  { ScopedKernelTimer timer_(kKernBwdDkdvTc, stream);
    // A call with a window computes dV and dK of its keys [lo, hi).  dK needs dKt of pad_k keys on either side
    // (the adjoint of the pre-pass), so one key tile before and one after the window are computed too, without dV.
    const int BK = (D == 128) ? 64 : 128;
    const int lo = win_lo(p), hi = win_hi(p);
    const int seg_lo[3] = {lo, max(0, lo - BK), hi}, seg_hi[3] = {hi, lo, min(p.N, hi + BK)}, seg_dv[3] = {1, 0, 0};
    e = cudaSuccess;
    if (keep_pdc) {
      __nv_bfloat16 *Pb, *dCb; int ldp;
      stream_buffers(p, workspace, &Pb, &dCb, &ldp);
      e = launch_bwd_dkdv_stream(p, Pb, dCb, ldp, dKt, status, stream);
    } else {
      for (int sg = 0; sg < 3 && e == cudaSuccess; ++sg) {
        const int klo = seg_lo[sg], khi = seg_hi[sg], dv = seg_dv[sg];
        if (khi <= klo) continue;
        if (D == 128) {
          e = launch_bwd_dkdv_tc128(p, Kt, dKt, status, dv, klo, khi, stream);
        } else if (p.cq <= 6) {
          e = launch_dkdv_pass<6, true>(p, Kt, dKt, status, 0, p.cq, dv, klo, khi, stream);
        } else {
          // seven taps: dV + 7 accumulators + the scratch columns exceed the tensor memory, so the taps are
          // split over two launches (each recomputes S^T and dP^T)
          e = launch_dkdv_pass<7, false>(p, Kt, dKt, status, 0, 4, dv, klo, khi, stream);
          if (e == cudaSuccess) e = launch_dkdv_pass<7, false>(p, Kt, dKt, status, 4, p.cq - 4, 0, klo, khi, stream);
        }
      }
    } }
  if (e != cudaSuccess) return e;
  const int j_base = win_lo(p);
  const int njb = (win_hi(p) - j_base + DkPostCfg::KEYS - 1) / DkPostCfg::KEYS;
  dim3 g2(njb, (unsigned)BH, D / DkPostCfg::D);      // one CTA per 64 keys and 64 columns of the head dim
  const int smem = DkPostCfg::smem_bytes(p.cq);
  auto kern = dk_post_mma_kernel;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  __nv_bfloat16* Tg = reinterpret_cast<__nv_bfloat16*>(w + 1024);   // status word first
  alignas(64) CUtensorMap tmK, tmX;
  if (!make_tensor_map_bf16(&tmK, p.K, D, p.N, BH, 64, DkPostCfg::ROWS, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmX, dKt, D, p.N, BH * p.cq, 64, DkPostCfg::ROWS, true)) return cudaErrorInvalidValue;
  // (the maps span the full head dim; each CTA fetches its 64-column slab)
  ScopedKernelTimer timer2_(kKernDkPost, stream);
  e = launch_pdl(dk_post_toeplitz_kernel, dim3(p.H), dim3(256), 0, stream, p.theta, Tg, p.cq, p.ck, p.scale);
  if (e != cudaSuccess) return e;
  return launch_pdl(kern, g2, dim3(DkPostCfg::NT), (size_t)smem, stream, tmK, tmX, Tg, p.dK, dTheta_part_tc, status, p.H, p.N, p.cq,
                    p.ck, p.scale, njb, D, j_base);
}

// slots of dTheta partials written by the dKt adjoint kernel: one per CTA
int bwd_tc_theta_slots(int B, int N, int d) {
  return B * (d > DkPostCfg::D ? d / DkPostCfg::D : 1) * ((N + DkPostCfg::KEYS - 1) / DkPostCfg::KEYS);
}


}  // namespace fmta
