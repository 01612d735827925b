// Decode (fwd_inference) kernel: last-query-row conv attention over a KV cache, split-K.
//
// Memory-bound: K and V are each read once from HBM with 16-byte loads straight into
// registers (no shared-memory staging, no block-level barrier in the key loop).  Every warp
// owns a contiguous key range of its split and keeps its own online-softmax state:
//   per 16-key step   S_a[j] = scale * q_a . k_j   for the <=16 most recent query rows   (mma.sync)
//                     -> fp32 ring buffer in shared memory (per warp, 64 keys deep)
//   one step later    C[j]  = sum_{a,b} theta[a,b] S_a[j+b-pad_k]   (needs +-pad_k neighbours)
//                     p = exp(C - m), O += p V                                        (FP32 pipe)
// The MMA contraction index is permuted so that each lane's B fragment is one contiguous
// 16-byte piece of a K row (A = Q is laid out to match once, in registers).
// Warps are merged in shared memory, splits by combine_splits_kernel on the same stream
// (result normalised into split 0, as the reference leaves it).  With `offset_causal` the score of
// a key later than a query row's own position is zeroed before the conv, as in the training
// forward, so that the result equals the last row of the training forward over the same sequence.
#pragma once
#include "fmta_common.cuh"
#include "fmta_params.h"

namespace fmta {

constexpr int kDecWarps = 4;
constexpr int kDecRing = 64;   // keys kept per warp for the conv window
constexpr int kDecMaxPages = 2048;   // block-table entries of one sequence kept in shared memory (paged cache)

FMTA_DEVINL uint4 ldg_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
FMTA_DEVINL float bf_lo(uint32_t x) { return __uint_as_float(x << 16); }
FMTA_DEVINL float bf_hi(uint32_t x) { return __uint_as_float(x & 0xffff0000u); }

// keys handled by one split, a multiple of 16 * kDecWarps
__host__ __device__ inline int decode_keys_per_split(int Nk, int k_splits) {
  const int per = (Nk + k_splits - 1) / k_splits;
  return ((per + 16 * kDecWarps - 1) / (16 * kDecWarps)) * (16 * kDecWarps);
}

template <int D, bool R16, bool PAGED>
__global__ void __launch_bounds__(kDecWarps * 32, 4) decode_kernel(const DecodeParams p) {
  constexpr int KS = D / 16;       // k-steps of the MMA
  constexpr int CH = D / 32;       // 32-element chunks per row (one 16-byte load per lane each)
  constexpr int LPR = D / 8;       // lanes covering one V row with 16-byte loads
  constexpr int KPL = 32 / LPR;    // V rows fetched by one warp-wide load
  constexpr int VL = 16 / KPL;     // V loads per 16-key step
  __shared__ float sRing[kDecWarps][16][kDecRing];
  __shared__ float sTheta[16 * 20];
  __shared__ float sMergeO[kDecWarps][D];
  __shared__ float sMergeML[kDecWarps][2];
  __shared__ int sTable[PAGED ? kDecMaxPages : 1];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  // a per-sequence length comes from device memory the caller may have left stale: clamp it to the range the
  // block table (and the shared-memory copy of its row) was sized for
  const int Nk = (PAGED && p.seq_lens) ? min(max(p.seq_lens[b], 1), p.Nk) : p.Nk;
  const int cq = p.cq, ck = p.ck, pk = (ck - 1) / 2;
  const int rows = min(p.q_len, cq);          // query rows that the last output row sees
  const size_t bh = (size_t)b * p.H + h;
  const bf16* Kg = PAGED ? p.K : p.K + bh * (size_t)Nk * D;
  const bf16* Vg = PAGED ? p.V : p.V + bh * (size_t)Nk * D;
  // A 16-key step never straddles a page (pages hold a multiple of 16 keys), so the page lookup is
  // done once per step: step_base(kb) is the element offset of key (kb rounded down to its page),
  // and a key's row follows at (key - that) * D.
  const int page_mask = PAGED ? p.page_size - 1 : 0;
  auto step_base = [&](int kb) -> size_t {
    if (PAGED) {
      const int pg = max(kb, 0) >> p.page_shift;
      return ((size_t)sTable[pg] * p.H + h) * p.page_size * D;
    }
    return 0;
  };
  auto row_in = [&](int key) -> size_t { return PAGED ? (size_t)(key & page_mask) * D : (size_t)key * D; };
  if (PAGED) {
    const int npg = (Nk + p.page_size - 1) >> p.page_shift;
    for (int i = tid; i < npg; i += kDecWarps * 32) sTable[i] = p.block_table[(size_t)b * p.max_pages + i];
  }
  const bf16* Qg = p.Q + (bh * p.q_len + (p.q_len - rows)) * (size_t)D;

  // theta rows that see a real query row: tap a = cq - rows + r  <->  ring row r
  for (int i = tid; i < rows * ck; i += kDecWarps * 32)
    sTheta[(i / ck) * 20 + (i % ck)] = p.theta[((size_t)h * cq + (cq - rows) + i / ck) * ck + (i % ck)];
  for (int i = tid; i < kDecWarps * 16 * kDecRing; i += kDecWarps * 32) (&sRing[0][0][0])[i] = 0.f;

  // A fragments of Q in the permuted-k layout (rows >= `rows` are zero)
  uint32_t qa[KS][R16 ? 4 : 2];
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    uint2 lo = make_uint2(0u, 0u), lo2 = lo, hi = lo, hi2 = lo;
    if (g < rows) {
      const uint4 v = *reinterpret_cast<const uint4*>(Qg + (size_t)g * D + c * 32 + t * 8);
      lo = make_uint2(v.x, v.y); lo2 = make_uint2(v.z, v.w);
    }
    if (R16 && g + 8 < rows) {
      const uint4 v = *reinterpret_cast<const uint4*>(Qg + (size_t)(g + 8) * D + c * 32 + t * 8);
      hi = make_uint2(v.x, v.y); hi2 = make_uint2(v.z, v.w);
    }
    if (R16) {
      qa[2 * c][0] = lo.x; qa[2 * c][1] = hi.x; qa[2 * c][2] = lo.y; qa[2 * c][3] = hi.y;
      qa[2 * c + 1][0] = lo2.x; qa[2 * c + 1][1] = hi2.x; qa[2 * c + 1][2] = lo2.y; qa[2 * c + 1][3] = hi2.y;
    } else {
      qa[2 * c][0] = lo.x; qa[2 * c][1] = lo.y;
      qa[2 * c + 1][0] = lo2.x; qa[2 * c + 1][1] = lo2.y;
    }
  }
  __syncthreads();

  const int keys_per_split = decode_keys_per_split(Nk, p.k_splits);   // (per sequence when lengths differ)
  const int keys_per_warp = keys_per_split / kDecWarps;
  const int k_lo = split * keys_per_split + warp * keys_per_warp;
  const int k_hi = min(k_lo + keys_per_warp, ((Nk + 15) / 16) * 16);

  float m_run = -INFINITY, l_run = 0.f;
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = 0.f;
  float* ring = &sRing[warp][0][0];
  const int vrow = lane / LPR, vcol = (lane % LPR) * 8;
  const int ckey = lane & 15, chalf = lane >> 4;
  const int ra = chalf ? (rows + 1) / 2 : 0, rb = chalf ? rows : (rows + 1) / 2;

  if (k_lo < k_hi) {
    for (int kb = k_lo - 16; kb <= k_hi; kb += 16) {
      // ---- issue loads: K block [kb, kb+16), V block [kb-16, kb) ----
      uint4 kf[2][CH];
      const bf16* Kst = Kg + step_base(kb);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int key = kb + 8 * j + g;
        const bool ok = key >= 0 && key < Nk;
#pragma unroll
        for (int c = 0; c < CH; ++c)
          kf[j][c] = ok ? ldg_nc_v4(Kst + row_in(key) + c * 32 + t * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
      const bool do_pv = (kb - 16 >= k_lo);
      uint4 vf[VL];
      if (do_pv) {
        const bf16* Vst = Vg + step_base(kb - 16);
#pragma unroll
        for (int i = 0; i < VL; ++i) {
          const int key = kb - 16 + i * KPL + vrow;
          vf[i] = (key < Nk) ? ldg_nc_v4(Vst + row_in(key) + vcol) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // ---- S for the K block -> ring ----
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          if (R16) {
            const uint32_t a0[4] = {qa[2 * c][0], qa[2 * c][1], qa[2 * c][2], qa[2 * c][3]};
            const uint32_t a1[4] = {qa[2 * c + 1][0], qa[2 * c + 1][1], qa[2 * c + 1][2], qa[2 * c + 1][3]};
            mma_bf16(acc, a0, kf[j][c].x, kf[j][c].y);
            mma_bf16(acc, a1, kf[j][c].z, kf[j][c].w);
          } else {
            const uint32_t a0[4] = {qa[2 * c][0], 0u, qa[2 * c][1], 0u};
            const uint32_t a1[4] = {qa[2 * c + 1][0], 0u, qa[2 * c + 1][1], 0u};
            mma_bf16(acc, a0, kf[j][c].x, kf[j][c].y);
            mma_bf16(acc, a1, kf[j][c].z, kf[j][c].w);
          }
        }
        const int kcol = (kb + 8 * j + 2 * t) & (kDecRing - 1);
        float v0 = acc[0] * p.scale, v1 = acc[1] * p.scale, v2 = acc[2] * p.scale, v3 = acc[3] * p.scale;
        if (p.offset_causal && kb + 16 > Nk - rows) {   // only the last keys of the cache can lie in a row's future
          const int key0 = kb + 8 * j + 2 * t, lim = Nk - rows + g;
          if (key0 > lim) v0 = 0.f;
          if (key0 + 1 > lim) v1 = 0.f;
          if (key0 > lim + 8) v2 = 0.f;
          if (key0 + 1 > lim + 8) v3 = 0.f;
        }
        *reinterpret_cast<float2*>(ring + g * kDecRing + kcol) = make_float2(v0, v1);
        if (R16) *reinterpret_cast<float2*>(ring + (g + 8) * kDecRing + kcol) = make_float2(v2, v3);
      }
      __syncwarp();
      // ---- conv + softmax + PV for the previous block [kb-16, kb) ----
      if (do_pv) {
        const int key = kb - 16 + ckey;
        float cpart = 0.f;
        for (int a = ra; a < rb; ++a) {
          const float* srow = ring + a * kDecRing;
          const float* trow = sTheta + a * 20;
          for (int bb = 0; bb < ck; ++bb)
            cpart = fmaf(trow[bb], srow[(key + bb - pk) & (kDecRing - 1)], cpart);
        }
        float cval = cpart + __shfl_xor_sync(0xffffffffu, cpart, 16);
        if (key >= Nk) cval = -INFINITY;
        float mx = cval;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        const float m_new = fmaxf(m_run, mx);      // finite: key kb-16 < Nk is always valid here
        const float pj = exp2f((cval - m_new) * kLog2e);
        float ps = pj;
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
        const float alpha = exp2f((m_run - m_new) * kLog2e);   // m_run = -inf -> 0
        l_run = l_run * alpha + ps;
        m_run = m_new;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] *= alpha;
#pragma unroll
        for (int i = 0; i < VL; ++i) {
          const float pv = __shfl_sync(0xffffffffu, pj, i * KPL + vrow);
          o[0] = fmaf(pv, bf_lo(vf[i].x), o[0]); o[1] = fmaf(pv, bf_hi(vf[i].x), o[1]);
          o[2] = fmaf(pv, bf_lo(vf[i].y), o[2]); o[3] = fmaf(pv, bf_hi(vf[i].y), o[3]);
          o[4] = fmaf(pv, bf_lo(vf[i].z), o[4]); o[5] = fmaf(pv, bf_hi(vf[i].z), o[5]);
          o[6] = fmaf(pv, bf_lo(vf[i].w), o[6]); o[7] = fmaf(pv, bf_hi(vf[i].w), o[7]);
        }
      }
      __syncwarp();
    }
  }
  // ---- merge the V-row parities inside the warp, then the warps of the CTA ----
#pragma unroll
  for (int off = LPR; off < 32; off <<= 1)
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] += __shfl_xor_sync(0xffffffffu, o[i], off);
  if (lane < LPR) {
#pragma unroll
    for (int i = 0; i < 8; ++i) sMergeO[warp][vcol + i] = o[i];
  }
  if (lane == 0) { sMergeML[warp][0] = m_run; sMergeML[warp][1] = l_run; }
  __syncthreads();
  float m = -INFINITY;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, sMergeML[w][0]);
  float wgt[kDecWarps], l = 0.f;
#pragma unroll
  for (int w = 0; w < kDecWarps; ++w) {
    wgt[w] = (sMergeML[w][0] == -INFINITY) ? 0.f : exp2f((sMergeML[w][0] - m) * kLog2e);
    l += sMergeML[w][1] * wgt[w];
  }
  const size_t so = (bh * p.k_splits + split);
  for (int dcol = tid; dcol < D; dcol += kDecWarps * 32) {
    float acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) acc += sMergeO[w][dcol] * wgt[w];
    p.O_splits[so * D + dcol] = acc;   // un-normalised partial
  }
  if (tid == 0) { p.M_splits[so] = m; p.L_splits[so] = l; }
}

// Merge the split partials of one (batch, head) and leave the normalised result in split 0
// (fwd_inference.cu:332-367 keeps the same convention).
__global__ void combine_splits_kernel(float* __restrict__ O_splits, float* __restrict__ M_splits,
                                      float* __restrict__ L_splits, int k_splits, int D) {
  const size_t bh = blockIdx.x;
  float* Ms = M_splits + bh * k_splits;
  float* Ls = L_splits + bh * k_splits;
  float m = -INFINITY;
  for (int s = 0; s < k_splits; ++s) m = fmaxf(m, Ms[s]);
  float l = 0.f;
  for (int s = 0; s < k_splits; ++s) l += (Ms[s] == -INFINITY) ? 0.f : Ls[s] * exp2f((Ms[s] - m) * kLog2e);
  const float inv = 1.f / l;
  for (int dcol = threadIdx.x; dcol < D; dcol += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < k_splits; ++s) {
      const float w = (Ms[s] == -INFINITY) ? 0.f : exp2f((Ms[s] - m) * kLog2e);
      acc += O_splits[(bh * k_splits + s) * D + dcol] * w;
    }
    O_splits[(bh * k_splits) * D + dcol] = acc * inv;
  }
  __syncthreads();
  if (threadIdx.x == 0) { Ms[0] = m; Ls[0] = l; }
}

// Append n_new key/value rows per sequence to a paged cache: row r of sequence b goes to position
// seq_lens[b] + r (seq_lens is not modified; the caller advances it).  One 16-byte chunk per thread.
template <int D>
__global__ void kv_append_paged_kernel(bf16* __restrict__ Kpool, bf16* __restrict__ Vpool,
                                       const int* __restrict__ block_table, const int* __restrict__ seq_lens,
                                       const bf16* __restrict__ Knew, const bf16* __restrict__ Vnew, int H, int n_new,
                                       int page_size, int page_shift, int max_pages) {
  constexpr int CPR = D / 8;
  const int b = blockIdx.z, h = blockIdx.y;
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n_new * CPR) return;
  const int r = idx / CPR, c = idx % CPR;
  const int pos = seq_lens[b] + r;
  if (pos < 0 || (pos >> page_shift) >= max_pages) return;   // past the block table: the row is dropped, nothing is written
  const int pg = block_table[(size_t)b * max_pages + (pos >> page_shift)], in = pos & (page_size - 1);
  const size_t dst = (((size_t)pg * H + h) * page_size + in) * D + c * 8;
  const size_t src = (((size_t)b * H + h) * n_new + r) * D + c * 8;
  *reinterpret_cast<uint4*>(Kpool + dst) = *reinterpret_cast<const uint4*>(Knew + src);
  *reinterpret_cast<uint4*>(Vpool + dst) = *reinterpret_cast<const uint4*>(Vnew + src);
}

}  // namespace fmta
