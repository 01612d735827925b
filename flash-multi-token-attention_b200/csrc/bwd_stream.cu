// dK-tilde / dV by streaming (head dim 64): when the dQ kernel has left the off-band P and dC = P (dP - D)
// in global memory (bf16, tile-major [B*H][row block][key block][64 rows][64 keys]), dV = P^T dO and dKt_a = dC^T Q^(a) are plain
// accumulating GEMMs over the query rows -- no score recomputation, no exponentials, no element-wise
// phase.  A CTA owns 128 keys (= TMEM lanes) and walks 64-row query blocks; a stage holds the P and dC
// tiles of the block (64 rows x 128 keys each, two 128-byte-swizzled slabs), dO and Q:
//   dV  [128 keys x 64]  += A(P tile read MN-major: M = keys across the two slabs, K = rows) * dO
//   dKt [128 keys x 128] += A(dC tile, same form) * [Q^(a) | Q^(a+1)]   (two taps per MMA, the second column
//                            atom one row = 128 bytes later in the same swizzled Q tile)
// The tiles are used exactly as the dQ kernel wrote them: a row-major [query][key] tile IS the transposed
// operand when it is read MN-major, so nothing is transposed anywhere.  Tensor memory: dV + up to 7 dKt
// accumulators = 512 columns (no scratch columns are needed, so seven taps fit one pass).
// Per score entry the kernel moves 4 bytes of P / dC from HBM and executes 2 d (c_q + 1) tensor FLOPs, against
// 2 d (2 c_q + 2) for the recomputing kernel: it is bound by the HBM stream, not by the tensor pipe.
// Every mbarrier wait is bounded; no TMA multicast, no cluster, cta_group::1 only.
#include <cuda.h>
#include <cuda_runtime.h>

#include "bwd_tc.cuh"
#include "fmta_tc.cuh"
#include "launch_util.cuh"

namespace fmta {

struct DkvStreamCfg {
  static constexpr int D = 64;
  static constexpr int BK = 128;               // keys per CTA (= TMEM lanes)
  static constexpr int BR = 64;                // query rows per block
  static constexpr int HALO = 8;               // rows of Q staged above the block (pad_q <= 6)
  static constexpr int QR = BR + HALO;         // 72 rows of Q per stage
  static constexpr int MAXCQ = 7;
  static constexpr int NSTG = 4;
  static constexpr int SLAB = BR * 128;        // 64 rows x 64 keys (or 64 head dims), 128-byte swizzle
  static constexpr int sgP = 0;                // two slabs
  static constexpr int sgDC = 2 * SLAB;        // two slabs
  static constexpr int sgdO = 4 * SLAB;
  static constexpr int sgQ = 5 * SLAB;         // [QR rows][128 B]
  static constexpr int STAGE_BYTES = 5 * SLAB + QR * 128;
  static_assert(STAGE_BYTES % 1024 == 0, "stages start on 1024-byte boundaries");
  static constexpr int KT_BYTES = BK * 128;    // one dKt tile on its way out (epilogue; takes the place of the stages)
  static constexpr int oStage = 0;
  static constexpr int oBar = NSTG * STAGE_BYTES;
  static constexpr int kSmemBytes = oBar + 512 + 1024;
  static_assert(MAXCQ * KT_BYTES <= NSTG * STAGE_BYTES, "epilogue tiles fit the stage memory");
  static_assert(kSmemBytes <= 227 * 1024, "streaming dK/dV kernel: shared memory budget");
  static constexpr int kTmemCols = 512;        // dV at 0, dKt_a at 64 (1 + a)
  static constexpr int kEpWarps = 8;           // write-out warps (two per TMEM lane quarter)
  static constexpr int kThreads = (kEpWarps + 3) * 32;   // + producer, issuers A0 and A1
};

__global__ void __launch_bounds__(DkvStreamCfg::kThreads, 1)
bwd_dkdv_stream_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                       const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmdC,
                       const __grid_constant__ CUtensorMap tmdKt, const BwdTcParams p) {
  using Cfg = DkvStreamCfg;
  constexpr int D = Cfg::D, BK = Cfg::BK, BR = Cfg::BR, HALO = Cfg::HALO, QR = Cfg::QR, NSTG = Cfg::NSTG;
  constexpr int W_TMA = Cfg::kEpWarps, W_A0 = Cfg::kEpWarps + 1;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sStage = smem + Cfg::oStage;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::oBar);
  uint64_t* full = bars;                 // [NSTG]
  uint64_t* empty = bars + NSTG;         // [NSTG]  both issuers release a stage
  uint64_t* all_done = bars + 2 * NSTG;  // the last MMAs of both issuers have completed
  uint64_t* never_bar = all_done + 1;    // nothing arrives here (expiry self-test)
  uint64_t* mma_drain = never_bar + 1;   // abort path
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(mma_drain + 1);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  volatile int* s_issued = s_abort + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int N = p.N, cq = p.cq, pq = cq - 1, pk = (p.ck - 1) / 2;
  const int band = pq + pk;
  int h, b, j0;
  dkdv_block_order(BK, h, b, j0);          // (batch, head)-major, key-tile-major tail
  const int bh = b * p.H + h;
  const int nQB = (N + BR - 1) / BR;
  const int qb_begin = p.causal ? min(nQB, (j0 + band) / BR) : 0;
  const int nblk = nQB - qb_begin;

  if (tid == 0) {
    for (int i = 0; i < NSTG; ++i) { tc::mbar_init(&full[i], 1); tc::mbar_init(&empty[i], 2); }
    tc::mbar_init(all_done, 2);
    tc::mbar_init(never_bar, 1); tc::mbar_init(mma_drain, 2);
    *s_abort = 0; *s_issued = 0;
    tc::mbar_fence_init();
  }
  if (warp == W_A0) {
    tc::tmem_alloc(s_tmem, Cfg::kTmemCols);
    tc::tmem_relinquish();
  }
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const uint32_t tmem = *s_tmem;

  if (warp == W_TMA) {
    // ===================== producer =====================
    if (lane == 0 && nblk > 0) {
      tc::tma_prefetch_desc(&tmQ); tc::tma_prefetch_desc(&tmdO); tc::tma_prefetch_desc(&tmP); tc::tma_prefetch_desc(&tmdC);
      bool ok = true;
      for (int it = 0; it < nblk && ok; ++it) {
        const int st = it % NSTG, ph = (it / NSTG) & 1;
        const int i0 = (qb_begin + it) * BR;
        unsigned char* sg = sStage + st * Cfg::STAGE_BYTES;
        if (!tc::mbar_wait(&empty[st], ph ^ 1, s_abort)) { ok = false; break; }
        tc::mbar_expect_tx(&full[st], Cfg::STAGE_BYTES);
        // P / dC are tile-major ([B*H][row block][key block][64 rows][64 keys]): a slab is one 8 KB tile
        const int tile = ((bh * nQB + qb_begin + it) * p.ldp + j0) >> 6;      // p.ldp / 64 key blocks per row block
        tc::tma_load_3d(sg + Cfg::sgP, &tmP, &full[st], 0, 0, tile);
        tc::tma_load_3d(sg + Cfg::sgP + Cfg::SLAB, &tmP, &full[st], 0, 0, tile + 1);
        tc::tma_load_3d(sg + Cfg::sgDC, &tmdC, &full[st], 0, 0, tile);
        tc::tma_load_3d(sg + Cfg::sgDC + Cfg::SLAB, &tmdC, &full[st], 0, 0, tile + 1);
        tc::tma_load_3d(sg + Cfg::sgdO, &tmdO, &full[st], 0, i0, bh);
        tc::tma_load_3d(sg + Cfg::sgQ, &tmQ, &full[st], 0, i0 - HALO, bh);
        *s_issued = it + 1;
      }
    }
  } else if (warp > W_TMA) {
    // ===================== MMA issuers A0 / A1 =====================
    const int ai = warp - W_A0;
    if (nblk > 0) {   // all lanes run the loop; one elected lane issues (see tc::elect_one)
      constexpr uint32_t idescV = tc::make_idesc(BK, D, 1, 1);        // 128 x 64, both operands MN-major
      constexpr uint32_t idescK2 = tc::make_idesc(BK, 2 * D, 1, 1);   // 128 x 128: two adjacent taps at once
      // A0 takes dV and the first half of the tap groups, A1 the rest; a group is two adjacent taps (an odd
      // last tap goes alone)
      const int pairs = cq / 2, singles = cq - 2 * pairs;
      const int ngrp = pairs + singles, g_half = ngrp / 2;
      const int g_begin = ai == 0 ? 0 : g_half, g_end = ai == 0 ? g_half : ngrp;
      bool ok = true;
      for (int it = 0; it < nblk && ok; ++it) {
        const int st = it % NSTG, ph = (it / NSTG) & 1;
        const uint32_t sg = smem_u32(sStage + st * Cfg::STAGE_BYTES);
        // P / dC read MN-major: M = keys across the two slabs (leading-dimension offset = slab size), K = rows
        const uint64_t dPa = tc::make_sdesc(sg + Cfg::sgP, Cfg::SLAB, 1024, tc::kLayoutSW128);
        const uint64_t dCa = tc::make_sdesc(sg + Cfg::sgDC, Cfg::SLAB, 1024, tc::kLayoutSW128);
        // dO read MN-major (N = head dim, K = rows); Q likewise with the tap's row shift as a start-address
        // offset and the next tap as a second column atom one row (128 bytes) later
        const uint64_t dOb = tc::make_sdesc(sg + Cfg::sgdO, 16, 1024, tc::kLayoutSW128);
        const uint64_t dQb = tc::make_sdesc(sg + Cfg::sgQ + (HALO - pq) * 128, 128, 1024, tc::kLayoutSW128);
        const uint32_t pa_hi = (uint32_t)(dPa >> 32), pa_lo = (uint32_t)dPa, ca_lo = (uint32_t)dCa;
        const uint32_t ob_hi = (uint32_t)(dOb >> 32), ob_lo = (uint32_t)dOb;
        const uint32_t qb_hi = (uint32_t)(dQb >> 32), qb_lo = (uint32_t)dQb;
        const uint32_t acc_on = it != 0;
        if (!tc::mbar_wait_warp(&full[st], ph, s_abort)) { ok = false; break; }
        tc::tc_fence_after();
        if (ai == 0) {
          tc::mma_ss2pe(tmem, pa_lo, pa_hi, ob_lo, ob_hi, idescV, acc_on);
#pragma unroll
          for (int k = 1; k < BR / 16; ++k)
            tc::mma_ss2e<1>(tmem, pa_lo + (uint32_t)(k * (2048 / 16)), pa_hi, ob_lo + (uint32_t)(k * (2048 / 16)), ob_hi, idescV);
        }
        for (int gi = g_begin; gi < g_end; ++gi) {
          const bool pair = gi < pairs;
          const int i = pair ? 2 * gi : 2 * pairs + (gi - pairs);        // first accumulator / tap of the group
          const uint32_t dacc = tmem + 64 * (1 + i);
          const uint32_t b_lo = qb_lo + (uint32_t)(i * (128 >> 4));
          const uint32_t idg = pair ? idescK2 : idescV;
          tc::mma_ss2pe(dacc, ca_lo, pa_hi, b_lo, qb_hi, idg, acc_on);
#pragma unroll
          for (int k = 1; k < BR / 16; ++k)
            tc::mma_ss2e<1>(dacc, ca_lo + (uint32_t)(k * (2048 / 16)), pa_hi, b_lo + (uint32_t)(k * (2048 / 16)), qb_hi, idg);
        }
        tc::mma_commit_e(&empty[st]);
      }
      if (ok) tc::mma_commit_e(all_done);
    }
  } else {
    // ===================== write-out warps: dV and dKt_a rows of this key =====================
    constexpr int NCG = Cfg::kEpWarps / 4;
    const int qtr = warp & 3, cg = warp >> 2;
    const int key = j0 + qtr * 32 + lane;
    const uint32_t lane_base = (uint32_t)(qtr * 32) << 16;
    bool ok = true;
    if (nblk > 0) ok = __all_sync(0xffffffffu, p.selftest_expire ? tc::mbar_wait(never_bar, 0, s_abort, tc::kSelfTestSpinLimit)
                                                                  : tc::mbar_wait(all_done, 0, s_abort));
    tc::tc_fence_after();
    const bool have = (nblk > 0) && ok;
    const bool store = key < N;
    const size_t krow = (size_t)(store ? key : 0);
    const int nacc = 1 + cq;
    for (int ch = cg; ch < 2 * nacc; ch += NCG) {
      const int acc = ch >> 1, half = ch & 1;
      float o[32];
      if (have) {
        tc::tmem_ld32(tmem + lane_base + ch * 32, o);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] = 0.f;
      }
      if (acc == 0) {
        if (store) {
          float* dst = p.dV + ((size_t)bh * N + krow) * D + half * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
        }
      } else {
        // dKt_a leaves as bf16 through shared memory (the stages are free once every MMA has completed):
        // [128 keys][128 B] with the 128-byte swizzle, then one TMA tile store per tap
        const int row = qtr * 32 + lane;
        unsigned char* tile = sStage + (acc - 1) * Cfg::KT_BYTES + row * 128;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(tile + (((half * 4 + i) ^ (row & 7)) << 4)) =
              make_uint4(pack_bf16(o[8 * i], o[8 * i + 1]), pack_bf16(o[8 * i + 2], o[8 * i + 3]),
                         pack_bf16(o[8 * i + 4], o[8 * i + 5]), pack_bf16(o[8 * i + 6], o[8 * i + 7]));
      }
    }
    tc::fence_proxy_async_smem();
    tc::named_bar_sync(1, Cfg::kEpWarps * 32);
    if (warp == 0 && tc::elect_one()) {
      for (int t = 0; t < cq; ++t) tc::tma_store_3d(&tmdKt, sStage + t * Cfg::KT_BYTES, 0, j0, bh * cq + t);
      tc::tma_store_commit();
      tc::tma_store_wait_read();
    }
  }
  __syncwarp();

  tc::tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    if (tid == 0) atomicExch(p.status, 1);
    // MMAs and copies of this CTA are waited for (bounded) before its memories go
    if (warp > W_TMA) tc::mma_commit_e(mma_drain);
    if (tid == W_TMA * 32) {
      volatile int never = 0;
      const int issued = *s_issued;
      for (int it = max(0, issued - NSTG); it < issued; ++it) tc::mbar_wait(&full[it % NSTG], (it / NSTG) & 1, &never);
      tc::mbar_wait(mma_drain, 0, &never);
    }
    __syncthreads();
  }
  if (warp == W_A0) {
    tc::tc_fence_after();
    tc::tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

size_t bwd_stream_extra_bytes(int B, int H, int N) {
  const size_t ldp = ((size_t)N + 127) / 128 * 128, nr = ((size_t)N + 63) / 64 * 64;
  return 2 * (((size_t)B * H * nr * ldp * 2 + 1023) / 1024 * 1024);
}

cudaError_t launch_bwd_dkdv_stream(const TrainParams& p, const __nv_bfloat16* Pbuf, const __nv_bfloat16* dCbuf, int ldp,
                                   __nv_bfloat16* dKt, int* status, cudaStream_t stream) {
  using Cfg = DkvStreamCfg;
  constexpr int D = Cfg::D;
  const size_t BH = (size_t)p.B * p.H;
  alignas(64) CUtensorMap tmQ, tmdO, tmP, tmdC, tmdKt;
  if (!make_tensor_map_bf16(&tmdKt, dKt, D, p.N, BH * p.cq, 64, Cfg::BK, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmQ, p.Q, D, p.N, BH, 64, Cfg::QR, true)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmdO, p.dO, D, p.N, BH, 64, Cfg::BR, true)) return cudaErrorInvalidValue;
  const size_t n_tiles = BH * (size_t)((p.N + 63) / 64) * (size_t)(ldp / 64);      // 64 x 64 tiles of 8 KB
  if (n_tiles >= (size_t)1 << 31) return cudaErrorInvalidValue;
  // the tiles are stored as the swizzled shared-memory image the dQ kernel held, so they are copied as they are
  if (!make_tensor_map_bf16(&tmP, Pbuf, 64, 64, n_tiles, 64, 64, false)) return cudaErrorInvalidValue;
  if (!make_tensor_map_bf16(&tmdC, dCbuf, 64, 64, n_tiles, 64, 64, false)) return cudaErrorInvalidValue;
  BwdTcParams bp = {};
  bp.dV = p.dV; bp.dKt = dKt; bp.status = status;
  bp.H = p.H; bp.N = p.N; bp.cq = p.cq; bp.ck = p.ck; bp.causal = p.causal; bp.ldp = ldp;
  bp.selftest_expire = take_selftest_expire(kKernBwdDkdvTc);
  auto kern = bwd_dkdv_stream_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
  if (e != cudaSuccess) return e;
  dim3 grid((p.N + Cfg::BK - 1) / Cfg::BK, p.H, p.B);
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tmQ, tmdO, tmP, tmdC, tmdKt, bp);
  return cudaGetLastError();
}

}  // namespace fmta
