// Stacked-GEMM conv-attention forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// Off the causal band (query - key >= pad_q + pad_k) the conv'd logits are a plain GEMM with a
// stacked contraction:
//     C[i,j] = sum_a  q_{i-(pad_q-a)} . Kt_a[j],     Kt_a[j] = scale * sum_b theta[a,b] k_{j+b-pad_k}
// so those tiles are FlashAttention with c_q accumulating MMAs per score tile and no work on the
// FP32 pipe.  This file holds
//   ktilde_kernel : the memory-bound pre-pass that writes the c_q bf16 operands Kt_a;
//   fwd_tc_kernel : the warp-specialised main kernel (1 TMA warp, 1 MMA warp, 2 softmax warpgroups);
//   launch_fwd_tc : tensor maps + launches.
// Ownership is per score entry: the stacked kernel takes every entry with query - key >= pad_q +
// pad_k (masking the rest of a diagonal tile), the band kernel (fwd_band.cu) takes the band entries.  The
// kernel leaves an UN-normalised partial (O, m, l) per query row; the band kernel continues the
// online softmax from that state over the band and writes the final O, M, L.
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
  // one thread = one 16-byte chunk of one output row of ONE tap (blockIdx.z): light threads, many of them
  constexpr int CPR = D / 8;          // 16-byte chunks per row
  constexpr int RPB = 256 / CPR;      // rows per block
  __shared__ float sTh[20];
  const int bh = blockIdx.y, h = bh % H, a = blockIdx.z;
  if (threadIdx.x < ck) sTh[threadIdx.x] = theta[((size_t)h * cq + a) * ck + threadIdx.x] * scale;   // scale carries log2(e)
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory that a kernel of this library writes or reads back
  const int j = blockIdx.x * RPB + threadIdx.x / CPR, c = threadIdx.x % CPR;
  if (j >= N) return;
  const int pk = (ck - 1) / 2;
  const bf16* Kb = K + (size_t)bh * N * D + c * 8;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll 4
  for (int b = 0; b < ck; ++b) {
    const int jj = j + b - pk;
    if (jj < 0 || jj >= N) continue;
    const uint4 kv = *reinterpret_cast<const uint4*>(Kb + (size_t)jj * D);
    const float w = sTh[b];
    const uint32_t w32[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc[2 * e] = fmaf(w, __uint_as_float(w32[e] << 16), acc[2 * e]);
      acc[2 * e + 1] = fmaf(w, __uint_as_float(w32[e] & 0xffff0000u), acc[2 * e + 1]);
    }
  }
  uint4 o;
  o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
  o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
  *reinterpret_cast<uint4*>(Kt + (((size_t)bh * cq + a) * N + j) * D + c * 8) = o;
}

// Same pre-pass with the filter width known at compile time: one thread owns one 16-byte column
// chunk of RR consecutive rows and produces all c_q taps from a register window of RR + CK - 1
// key rows, so every key row is loaded once per RR outputs instead of once per output and tap.
template <int D, int CK, int RR>
__global__ void __launch_bounds__(256) ktilde_window_kernel(const bf16* __restrict__ K, const float* __restrict__ theta,
                                                            bf16* __restrict__ Kt, int H, int N, int cq, float scale) {
  constexpr int CPR = D / 8, RUNS = 256 / CPR, PK = (CK - 1) / 2, WIN = RR + CK - 1;
  __shared__ float sTh[16 * CK];
  const int bh = blockIdx.y, h = bh % H;
  for (int i = threadIdx.x; i < cq * CK; i += 256) sTh[i] = theta[(size_t)h * cq * CK + i] * scale;
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory that a kernel of this library writes or reads back
  const int j0 = (blockIdx.x * RUNS + threadIdx.x / CPR) * RR, c = threadIdx.x % CPR;
  if (j0 >= N) return;
  const bf16* Kb = K + (size_t)bh * N * D + c * 8;
  uint4 win[WIN];
#pragma unroll
  for (int r = 0; r < WIN; ++r) {
    const int jj = j0 + r - PK;
    win[r] = (jj >= 0 && jj < N) ? *reinterpret_cast<const uint4*>(Kb + (size_t)jj * D) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int a = 0; a < cq; ++a) {
    float w[CK];
#pragma unroll
    for (int b = 0; b < CK; ++b) w[b] = sTh[a * CK + b];
    bf16* out = Kt + (((size_t)bh * cq + a) * N + j0) * D + c * 8;
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
      for (int b = 0; b < CK; ++b) {
        const uint4 kv = win[r + b];
        const uint32_t w32[4] = {kv.x, kv.y, kv.z, kv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[2 * e] = fmaf(w[b], __uint_as_float(w32[e] << 16), acc[2 * e]);
          acc[2 * e + 1] = fmaf(w[b], __uint_as_float(w32[e] & 0xffff0000u), acc[2 * e + 1]);
        }
      }
      if (j0 + r < N) {
        uint4 o;
        o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
        o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(out + (size_t)r * D) = o;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------
struct TcParams {
  float* Opart;   // [B,H,N,D] un-normalised
  float* Mpart;   // [B,H,N]  row max, natural-log units
  float* Lpart;
  int* status;    // device word: set non-zero when a bounded wait expired
  int H, N, cq, ck, causal;
  int qb_hi;      // the grid covers the row blocks [qb_hi - gridDim.x, qb_hi) (all of them unless the call has a window)
  int selftest_expire;   // failure-detection self-test: the softmax warps' first wait is on a barrier nothing arrives at
};

// One CTA owns two row tiles of 128 query rows (one softmax warpgroup and one TMEM lane per row).
// Every Kt / V tile staged in shared memory feeds the MMAs of both row tiles.  Tensor memory per row
// tile: S (BC columns, fp32), P (BC / 2 columns, bf16 pairs) and O (D columns, fp32); S is released to
// the next block's MMAs as soon as the softmax threads have loaded it into registers.
//   d = 64 : key blocks are 128 wide, so that every score MMA is 128 x 128 x 16 (a 64-wide MMA is bound
//            by shared-memory operand fetch: 4 KB of A per 2 KB of B);
//   d = 128: two row tiles only fit the tensor memory with 64-key blocks (2 x (64 + 32 + 128) = 448
//            columns).  A single 128-row tile with 128-key blocks has the cheaper MMAs, but streams
//            fourteen 16 KB tiles per block for 128 rows -- 62 bytes per cycle, more than eleven ring
//            slots cover at the latency of a TMA copy (tensor pipe 42 % busy); sharing every tile between
//            256 rows halves that.
template <int D, int NT_ = 2>
struct TcCfg {
  static constexpr int BM = 128;               // rows per tile (= TMEM lanes)
  static constexpr int BC = (D == 64) ? 128 : 64;   // keys per block
  static constexpr int NT = NT_;               // row tiles per CTA (TMEM: NT * (BC + BC / 2 + D) <= 512); 2, or 1 for
                                               // grids that would leave SMs without a CTA (one long sequence, few heads)
  static constexpr int HALO = 16;              // rows staged above the block (pad_q <= 15)
  static constexpr int QR = NT * BM + HALO;    // rows of Q in shared memory
  static constexpr int QBOX = QR / 2;          // Q is fetched as two boxes per 16-byte column slab
  static constexpr int SLABS = D / 64;         // 64-element (128-byte) column slabs per row
  static constexpr int TILE_BYTES = BC * 128;  // one ring tile: BC keys x 64 elements, 128B-swizzled
  static constexpr int NSLOT = (D == 64) ? 11 : 19;
  static constexpr int oQ = 0;
  static constexpr int oRing = ((oQ + QR * D * 2 + 1023) / 1024) * 1024;
  static constexpr int oBar = oRing + NSLOT * TILE_BYTES;
  static constexpr int kSmemBytes = oBar + 512 + 1024;   // + alignment slack
  static constexpr int kTmemCols = 512;
  static constexpr int colS = 0;               // S[t] at colS + t*BC
  static constexpr int colP = NT * BC;         // P[t] at colP + t*BC/2
  static constexpr int colO = NT * BC + NT * BC / 2;   // O[t] at colO + t*D
  static constexpr int kThreads = (NT * 4 + 1 + NT) * 32;   // softmax warpgroups, TMA warp, one MMA warp per row tile
  static_assert(NT * (BC + BC / 2 + D) <= kTmemCols, "TMEM budget");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
  static_assert(QR <= 512 && QBOX <= 256, "TMA box limit");
};

constexpr float kRescaleTau = 8.f;   // log2 units: P may reach 2^8 before O is rescaled

template <int D, int NT_>
__global__ void __launch_bounds__(TcCfg<D, NT_>::kThreads, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKt,
              const __grid_constant__ CUtensorMap tmV, const TcParams p) {
  using Cfg = TcCfg<D, NT_>;
  constexpr int BM = Cfg::BM, BC = Cfg::BC, HALO = Cfg::HALO, QR = Cfg::QR, NSLOT = Cfg::NSLOT, NT = Cfg::NT;
  constexpr int SLABS = Cfg::SLABS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem + Cfg::oQ;
  unsigned char* sRing = smem + Cfg::oRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* full = bars;                 // [NSLOT]  TMA -> MMA
  uint64_t* empty = bars + NSLOT;        // [NSLOT]  MMA -> TMA
  uint64_t* q_full = bars + 2 * NSLOT;
  uint64_t* s_full = q_full + 1;         // [NT]  S[t] ready (one commit per key block)
  uint64_t* s_free = s_full + 2;         // [NT]  S[t] loaded into registers (128 arrivals)
  uint64_t* p_full = s_free + 2;         // [NT]  P[t] written to tensor memory (128 arrivals)
  uint64_t* o_full = p_full + 2;         // [NT]  PV(t, kb) completed
  uint64_t* never_bar = o_full + 2;      // nothing arrives here (expiry self-test)
  uint64_t* mma_drain = never_bar + 1;   // abort path: every issuer's MMAs have completed (NT arrivals)
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(mma_drain + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_issued = s_abort + 1;
  volatile int* s_consumed = s_abort + 2;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int band = pq + pk;              // entries with query - key < band belong to the band kernel
  const int nQB = (N + NT * BM - 1) / (NT * BM);
  // CTAs are dispatched in linear block order; walk it length-major (all (batch, head) pairs of the
  // longest row block first) so that the greedy hardware scheduler ends with the short CTAs
  const int lin = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
  const int nBH = gridDim.y * gridDim.z;
  const int qb = p.qb_hi - 1 - lin / nBH;
  const int h = (lin % nBH) % (int)gridDim.y, b = (lin % nBH) / (int)gridDim.y;
  const int bh = b * p.H + h;
  const int i0 = qb * NT * BM;
  const int nKB = (N + BC - 1) / BC;
  int nkb_t[2] = {0, 0};
#pragma unroll
  for (int t = 0; t < NT; ++t) {
    const int r0 = i0 + t * BM;
    if (r0 >= N) nkb_t[t] = 0;
    else if (p.causal) {
      // key blocks that hold at least one key j <= (last row) - band
      const int last = min(N - 1, r0 + BM - 1) - band;
      nkb_t[t] = last >= 0 ? min(nKB, last / BC + 1) : 0;
    } else nkb_t[t] = nKB;
  }
  const int nkb = max(nkb_t[0], nkb_t[1]);

  if (tid == 0) {
    for (int i = 0; i < NSLOT; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], NT); }   // every MMA warp releases a slot
    tc::mbar_init(q_full, 1);
    tc::mbar_init(never_bar, 1); tc::mbar_init(mma_drain, NT);
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&s_full[i], 1); tc::mbar_init(&s_free[i], BM); tc::mbar_init(&p_full[i], BM); tc::mbar_init(&o_full[i], 1); }
    *s_abort = 0; *s_issued = 0; *s_consumed = 0;
    tc::mbar_fence_init();
  }
  if (warp == NT * 4 + 1) {   // the first MMA warp owns the tensor-memory allocation
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  pdl_trigger();
  __syncthreads();
  pdl_wait();      // nothing before this line touches global memory that a kernel of this library writes or reads back
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp == NT * 4) {
    // ===================== TMA producer =====================
    if (lane == 0 && nkb > 0) {
      tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmKt); tc::tma_prefetch_desc(&tmV);
      tc::mbar_expect_tx(q_full, QR * D * 2);
      for (int kc = 0; kc < D / 8; ++kc) {   // 16-byte-wide column slabs -> [kc][row][8 elements]
        tc::tma_load_3d(sQ + kc * (QR * 16), &tmQ, q_full, kc * 8, i0 - HALO, bh);
        tc::tma_load_3d(sQ + kc * (QR * 16) + Cfg::QBOX * 16, &tmQ, q_full, kc * 8, i0 - HALO + Cfg::QBOX, bh);
      }
      int id = 0;
      bool ok = true;
      auto put = [&](const CUtensorMap* map, int x, int y, int z) {
        const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
        if (!tc::mbar_wait(&empty[slot], ph ^ 1, s_abort)) { ok = false; return; }
        tc::mbar_expect_tx(&full[slot], Cfg::TILE_BYTES);
        tc::tma_load_3d(sRing + slot * Cfg::TILE_BYTES, map, &full[slot], x, y, z);
        ++id;
        *s_issued = id;
      };
      // same order as the MMA warp consumes: S(0); then S(kb+1), V(kb)
      for (int a = 0; a < cq && ok; ++a)
        for (int sl = 0; sl < SLABS && ok; ++sl) put(&tmKt, sl * 64, 0, bh * cq + a);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        if (kb + 1 < nkb)
          for (int a = 0; a < cq && ok; ++a)
            for (int sl = 0; sl < SLABS && ok; ++sl) put(&tmKt, sl * 64, (kb + 1) * BC, bh * cq + a);
        for (int sl = 0; sl < SLABS && ok; ++sl) put(&tmV, sl * 64, kb * BC, bh);
      }
    }
  } else if (warp > NT * 4) {
    // ===================== MMA issuers: one warp (one elected thread) per row tile =====================
    // Both walk the same tile stream; a ring slot is released when every issuer has committed
    // its MMAs on it.  Two issuers keep the tensor pipe fed while one of them sits in a barrier
    // wait or a commit.
    const int t = warp - (NT * 4 + 1);
    if (nkb > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescS = tc::make_idesc(BM, BC, 0, 0);
      constexpr uint32_t idescPV = tc::make_idesc(BM, 64, 0, 1);
      // descriptors split into a constant high word and a low word that carries the start address
      const uint64_t dQ0 = tc::make_sdesc(smem_u32(sQ) + (t * BM + HALO - pq) * 16, QR * 16, 128, tc::kLayoutNone);
      const uint64_t dK0 = tc::make_sdesc(smem_u32(sRing), 16, 1024, tc::kLayoutSW128);
      const uint32_t aS_hi = (uint32_t)(dQ0 >> 32), aS_lo = (uint32_t)dQ0;
      const uint32_t b_hi = (uint32_t)(dK0 >> 32), b_lo0 = (uint32_t)dK0;
      const uint32_t dS = tmem + Cfg::colS + t * BC;
      const uint32_t aP = tmem + Cfg::colP + t * (BC / 2);      // bf16 pairs: 8 columns per 16 keys
      const int my_nkb = nkb_t[t];
      int id = 0;
      bool ok = tc::mbar_wait_warp(q_full, 0, s_abort);
      auto issue_S = [&](int kb) {
        const bool active = kb < my_nkb;
        // S[t] is single-buffered: wait until the softmax threads have taken block kb-1 out of it
        if (active && kb > 0) {
          ok = tc::mbar_wait_warp(&s_free[t], (kb - 1) & 1, s_abort);
          tc::tc_fence_after();
        }
        for (int a = 0; a < cq && ok; ++a) {
#pragma unroll
          for (int sl = 0; sl < SLABS; ++sl) {
            const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
            if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; return; }
            if (active) {
              tc::tc_fence_after();
              const uint32_t b_lo = b_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
              const uint32_t a_lo = aS_lo + (uint32_t)(a + sl * 8 * QR);   // row shift = +16 B per row
              if (a == 0 && sl == 0) tc::mma_ss2e<0>(dS, a_lo, aS_hi, b_lo, b_hi, idescS);
              else tc::mma_ss2e<1>(dS, a_lo, aS_hi, b_lo, b_hi, idescS);
#pragma unroll
              for (int k = 1; k < 4; ++k)
                tc::mma_ss2e<1>(dS, a_lo + (uint32_t)(2 * k * QR), aS_hi, b_lo + (uint32_t)(k * 2), b_hi, idescS);
            }
            tc::mma_commit_e(&empty[slot]);
            ++id;
          }
        }
        if (ok && active) tc::mma_commit_e(&s_full[t]);
      };
      auto issue_PV = [&](int kb) {
        const bool active = kb < my_nkb;
#pragma unroll
        for (int sl = 0; sl < SLABS; ++sl) {
          const int slot = id % NSLOT, ph = (id / NSLOT) & 1;
          if (!tc::mbar_wait_warp(&full[slot], ph, s_abort)) { ok = false; return; }
          if (active) {
            if (sl == 0 && !tc::mbar_wait_warp(&p_full[t], kb & 1, s_abort)) { ok = false; return; }
            tc::tc_fence_after();
            const uint32_t b_lo = b_lo0 + (uint32_t)(slot * (Cfg::TILE_BYTES >> 4));
            const uint32_t dO = tmem + Cfg::colO + t * D + sl * 64;
            if (kb == 0) tc::mma_ts2e<0>(dO, aP, b_lo, b_hi, idescPV);
            else tc::mma_ts2e<1>(dO, aP, b_lo, b_hi, idescPV);
#pragma unroll
            for (int k = 1; k < BC / 16; ++k)
              tc::mma_ts2e<1>(dO, aP + 8 * k, b_lo + (uint32_t)(k * (2048 / 16)), b_hi, idescPV);
            if (sl == SLABS - 1) tc::mma_commit_e(&o_full[t]);
          }
          tc::mma_commit_e(&empty[slot]);
          ++id;
        }
      };
      if (ok) issue_S(0);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        if (kb + 1 < nkb) issue_S(kb + 1);
        if (ok) issue_PV(kb);
      }
      if (t == 0) *s_consumed = id;
    }
  } else {
    // ===================== softmax warpgroups: one query row per thread =====================
    const int t = warp >> 2;                            // row tile of this warpgroup
    const int m = tid & (BM - 1);                       // row within the tile = TMEM lane
    const int gi = i0 + t * BM + m;                     // query index
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + Cfg::colS + t * BC + lane_base;
    const uint32_t tP = tmem + Cfg::colP + t * (BC / 2) + lane_base;
    const uint32_t tO = tmem + Cfg::colO + t * D + lane_base;
    const int my_nkb = nkb_t[t];
    float m_run = -INFINITY, l_run = 0.f;               // log2 units (Kt carries scale * log2(e))
    float m_true = -INFINITY;                           // true row max (m_run lags it by up to tau)
    bool ok = true;
    for (int kb = 0; kb < my_nkb && ok; ++kb) {
      ok = __all_sync(0xffffffffu, (p.selftest_expire && kb == 0)
                                       ? tc::mbar_wait(never_bar, 0, s_abort, tc::kSelfTestSpinLimit)
                                       : tc::mbar_wait(&s_full[t], kb & 1, s_abort));
      if (!ok) break;   // warp-uniform: the TMEM accesses below are warp-collective
      tc::tc_fence_after();
      float s[BC];
#pragma unroll
      for (int c = 0; c < BC / 32; ++c) tc::tmem_ld32_nowait(tS + 32 * c, reinterpret_cast<float(&)[32]>(s[32 * c]));
      tc::tmem_wait_ld();
      // S[t] is in registers: let the MMA warp overwrite it with the next key block
      tc::tc_fence_before();
      tc::mbar_arrive(&s_free[t]);
      const int j0 = kb * BC;
      // mask: keys past N, and (causal) entries on or above the band, which the band kernel owns
      const int jlim = p.causal ? min(N - 1, gi - band) : N - 1;   // last key this row may see here
      if (j0 + BC - 1 > jlim) {
#pragma unroll
        for (int i = 0; i < BC; ++i) if (j0 + i > jlim) s[i] = -INFINITY;
      }
      float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]), mx2 = fmaxf(s[4], s[5]), mx3 = fmaxf(s[6], s[7]);
#pragma unroll
      for (int i = 8; i < BC; i += 8) {
        mx0 = fmaxf(mx0, fmaxf(s[i], s[i + 1])); mx1 = fmaxf(mx1, fmaxf(s[i + 2], s[i + 3]));
        mx2 = fmaxf(mx2, fmaxf(s[i + 4], s[i + 5])); mx3 = fmaxf(mx3, fmaxf(s[i + 6], s[i + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      m_true = fmaxf(m_true, mx);
      // lazy rescale: keep the reference max until a block exceeds it by more than tau
      float alpha = 1.f;
      bool need = false;
      if (m_run == -INFINITY) {
        m_run = mx;                                     // O and l are still zero: nothing to rescale
      } else if (mx > m_run + kRescaleTau) {
        alpha = exp2f(m_run - mx);
        m_run = mx;
        need = true;
      }
      const float mref = (m_run == -INFINITY) ? 0.f : m_run;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pk32[BC / 2];
#pragma unroll
      for (int i = 0; i < BC; i += 4) {
        const float p0 = exp2f(s[i] - mref), p1 = exp2f(s[i + 1] - mref);
        const float p2 = exp2f(s[i + 2] - mref), p3 = exp2f(s[i + 3] - mref);
        sum0 += p0 + p1; sum1 += p2 + p3;
        pk32[i / 2] = pack_bf16(p0, p1); pk32[i / 2 + 1] = pack_bf16(p2, p3);
      }
      l_run = l_run * alpha + (sum0 + sum1);
      if (kb > 0) {
        // PV(kb-1) complete: P[t] may be overwritten and O touched.  Waited for on every block
        // (not only when O is rescaled) so that the parity wait never aliases an older phase.
        ok = __all_sync(0xffffffffu, tc::mbar_wait(&o_full[t], (kb - 1) & 1, s_abort));
        if (!ok) break;
        tc::tc_fence_after();
      }
      if (__any_sync(0xffffffffu, need)) {   // O *= alpha (need is false on the first block)
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tc::tmem_ld32(tO + c * 32, o);
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] *= alpha;
          tc::tmem_st32(tO + c * 32, o);
        }
      }
#pragma unroll
      for (int c = 0; c < BC / 64; ++c) tc::tmem_st32u(tP + 32 * c, reinterpret_cast<const uint32_t(&)[32]>(pk32[32 * c]));
      tc::tmem_wait_st();
      tc::tc_fence_before();
      tc::mbar_arrive(&p_full[t]);
    }
    // ---- epilogue: un-normalised partial row ----
    if (my_nkb > 0 && ok) ok = __all_sync(0xffffffffu, tc::mbar_wait(&o_full[t], (my_nkb - 1) & 1, s_abort));
    tc::tc_fence_after();
    const bool have = (my_nkb > 0) && ok;               // warp-uniform
    // re-reference the partial to the true row max (what the reference reports as M)
    const float fix = (m_true == -INFINITY) ? 0.f : exp2f(m_run - m_true);
    float* orow = p.Opart + ((size_t)bh * N + (gi < N ? gi : 0)) * D;
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      float o[32];
      if (have) {
        tc::tmem_ld32(tO + c * 32, o);                  // warp-collective: every lane takes part
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0.f;
      }
      if (gi < N) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(orow + c * 32 + i) = make_float4(o[i] * fix, o[i + 1] * fix, o[i + 2] * fix, o[i + 3] * fix);
      }
    }
    if (gi < N) {
      const bool any = have && (m_run != -INFINITY);
      p.Mpart[(size_t)bh * N + gi] = any ? m_true * 0.6931471805599453f : -INFINITY;
      p.Lpart[(size_t)bh * N + gi] = any ? l_run * fix : 0.f;
    }
  }
  __syncwarp();

  // ===================== teardown =====================
  tc::tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicExch(p.status, 1);
    // nothing of this CTA may still be in flight when its shared and tensor memory are given up: every
    // issuer commits behind its last MMA, one thread waits (bounded) for those commits and for the
    // copies that were issued but never consumed
    if (warp > NT * 4) tc::mma_commit_e(mma_drain);
    if (tid == NT * 4 * 32) {
      volatile int never = 0;
      for (int id = *s_consumed; id < *s_issued; ++id) tc::mbar_wait(&full[id % NSLOT], (id / NSLOT) & 1, &never);
      tc::mbar_wait(mma_drain, 0, &never);
    }
    __syncthreads();
  }
  if (warp == NT * 4 + 1) {
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
}  // namespace

bool tensor_maps_available() { return get_encode_fn() != nullptr; }

bool make_tensor_map_bf16(CUtensorMap* map, const void* base, int D, int rows, size_t outer, int box_x, int box_rows, bool sw128) {
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

// fp32 tensor viewed as [outer][rows][D] (D contiguous); box = {box_x, box_rows, 1}; box_x * 4 <= 128 with the swizzle
bool make_tensor_map_f32(CUtensorMap* map, const void* base, int D, int rows, size_t outer, int box_x, int box_rows, bool sw128) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)outer};
  cuuint64_t strides[2] = {(cuuint64_t)D * 4, (cuuint64_t)rows * D * 4};
  cuuint32_t box[3] = {(cuuint32_t)box_x, (cuuint32_t)box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims, strides, box, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Pre-pass: Kt = scale * log2(e) * (theta applied along the key axis of K), c_q bf16 copies.
cudaError_t launch_ktilde(const TrainParams& p, __nv_bfloat16* Kt, cudaStream_t stream) {
  ScopedKernelTimer timer_(kKernKtilde, stream);
  const size_t BH = (size_t)p.B * p.H;
  const float sc = p.scale * kLog2e;
  if ((p.ck == 11 || p.ck == 7 || p.ck == 5 || p.ck == 3) && p.cq <= 16) {      // filter widths with a register-window instantiation
    constexpr int RR = 4;
#define FMTA_KT_WIN(DD, CKK)                                                                                      \
    { constexpr int RUNS = 256 / (DD / 8);                                                                        \
      dim3 grid((p.N + RUNS * RR - 1) / (RUNS * RR), (unsigned)BH);                                               \
      (void)launch_pdl(ktilde_window_kernel<DD, CKK, RR>, grid, dim3(256), 0, stream, p.K, p.theta, Kt, p.H, p.N, p.cq, sc); }
    if (p.d == 64) {
      if (p.ck == 11) FMTA_KT_WIN(64, 11) else if (p.ck == 7) FMTA_KT_WIN(64, 7) else if (p.ck == 5) FMTA_KT_WIN(64, 5) else FMTA_KT_WIN(64, 3)
    } else {
      if (p.ck == 11) FMTA_KT_WIN(128, 11) else if (p.ck == 7) FMTA_KT_WIN(128, 7) else if (p.ck == 5) FMTA_KT_WIN(128, 5) else FMTA_KT_WIN(128, 3)
    }
#undef FMTA_KT_WIN
    return cudaGetLastError();
  }
  if (p.d == 64) {
    constexpr int RPB = 256 / (64 / 8);
    dim3 grid((p.N + RPB - 1) / RPB, (unsigned)BH, p.cq);
    ktilde_kernel<64><<<grid, 256, 0, stream>>>(p.K, p.theta, Kt, p.H, p.N, p.cq, p.ck, sc);
  } else {
    constexpr int RPB = 256 / (128 / 8);
    dim3 grid((p.N + RPB - 1) / RPB, (unsigned)BH, p.cq);
    ktilde_kernel<128><<<grid, 256, 0, stream>>>(p.K, p.theta, Kt, p.H, p.N, p.cq, p.ck, sc);
  }
  return cudaGetLastError();
}

namespace {

template <int D, int NT_>
cudaError_t launch_tc_t(const TrainParams& p, bf16* Kt, float* Opart, float* Mpart, float* Lpart, int* status,
                        cudaStream_t stream) {
  using Cfg = TcCfg<D, NT_>;
  const size_t BH = (size_t)p.B * p.H;
  alignas(64) CUtensorMap tmQ, tmKt, tmV;
  if (!make_tensor_map_bf16(&tmQ, p.Q, D, p.N, BH, 8, Cfg::QBOX, false)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmKt, Kt, D, p.N, BH * p.cq, 64, Cfg::BC, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmV, p.V, D, p.N, BH, 64, Cfg::BC, true)) return cudaErrorInvalidValue;
  TcParams tp;
  tp.Opart = Opart; tp.Mpart = Mpart; tp.Lpart = Lpart; tp.status = status;
  tp.H = p.H; tp.N = p.N; tp.cq = p.cq; tp.ck = p.ck; tp.causal = p.causal;
  tp.selftest_expire = take_selftest_expire(kKernFwdTc);
  auto kern = fwd_tc_kernel<D, NT_>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  constexpr int RB = Cfg::NT * Cfg::BM;                           // rows per CTA; a window starts on a multiple of it
  tp.qb_hi = (win_hi(p) + RB - 1) / RB;
  dim3 grid(tp.qb_hi - win_lo(p) / RB, p.H, p.B);
  { ScopedKernelTimer timer_(kKernFwdTc, stream);
    e = launch_pdl(kern, grid, dim3(Cfg::kThreads), Cfg::kSmemBytes, stream, tmQ, tmKt, tmV, tp); }
  return e;
}

int sm_count() {
  static int n[16] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return 148;
  if (n[dev] == 0 && cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n[dev] = 148;
  return n[dev];
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

// Runs the pre-pass and the stacked kernel; on return p_out describes where the band kernel
// must pick up (Opart / Mpart / Lpart).
cudaError_t launch_fwd_tc(const TrainParams& p, void* workspace, const float** Opart, const float** Mpart,
                          const float** Lpart, cudaStream_t stream) {
  const size_t rows = (size_t)p.B * p.H * p.N;
  auto up = [](size_t x) { return (x + 1023) / 1024 * 1024; };
  unsigned char* w = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(workspace) + 1023) & ~uintptr_t(1023));
  bf16* Kt = reinterpret_cast<bf16*>(w); w += up(rows * p.cq * p.d * 2);
  if (p.Kt_ext) Kt = p.Kt_ext;                      // the caller keeps the stacked key operand (for the backward)
  float* Op = reinterpret_cast<float*>(w); w += up(rows * p.d * 4);
  float* Mp = reinterpret_cast<float*>(w); w += up(rows * 4);
  float* Lp = reinterpret_cast<float*>(w); w += up(rows * 4);
  int* status = nullptr;
  cudaError_t e = status_word_of(reinterpret_cast<int*>(w), stream, &status);
  if (e != cudaSuccess) return e;
  if (!(p.Kt_ext && p.kt_valid)) {
    e = launch_ktilde(p, Kt, stream);
    if (e != cudaSuccess) return e;
  }
  // Two row tiles per CTA share every key tile they stage; when that leaves SMs without a CTA (fewer CTAs than SMs:
  // a window of one long sequence with few heads) one tile per CTA doubles the CTAs instead.
  const long ctas2 = (long)((win_hi(p) - win_lo(p) + 255) / 256) * p.B * p.H;
  const bool one_tile = ctas2 < sm_count();
  if (p.d == 64) e = one_tile ? launch_tc_t<64, 1>(p, Kt, Op, Mp, Lp, status, stream) : launch_tc_t<64, 2>(p, Kt, Op, Mp, Lp, status, stream);
  else e = one_tile ? launch_tc_t<128, 1>(p, Kt, Op, Mp, Lp, status, stream) : launch_tc_t<128, 2>(p, Kt, Op, Mp, Lp, status, stream);
  *Opart = Op; *Mpart = Mp; *Lpart = Lp;
  return e;
}


}  // namespace fmta
