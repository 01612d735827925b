// Key-query convolution of a score tile held in shared memory (fp32), on the FP32 pipe.
//
// Math (per head):  C[i,j] = sum_{a<c_q, b<c_k} theta[a,b] * S[i + a - pad_q, j + b - pad_k]
// with pad_q = c_q-1, pad_k = (c_k-1)/2, and its adjoint
//                  dS[i,j] = sum_{a,b} theta[a,b] * dC[i - a + pad_q, j - b + pad_k].
// Both are "correlate a window of the source tile with a small filter"; the adjoint uses
// the filter flipped in both directions and a window that extends to LATER rows.
//
// Each thread produces a 1 x 16 strip: for every filter row it loads the 16+c_k-1 source
// values once (aligned float4 loads) and issues 16*c_k FMAs against them, so the loop is
// FMA-bound rather than shared-memory bound.  Lanes of a warp walk consecutive tile rows;
// with a source row stride that is an odd multiple of 4 floats the float4 loads are free
// of bank conflicts.
#pragma once
#include "fmta_common.cuh"

namespace fmta {

constexpr int kMaxCQ = 16;  // filter rows supported by the generic path (halo of 16 rows)
constexpr int kMaxCK = 17;  // filter columns (odd) supported (halo of 8 columns per side)
constexpr int kThetaLd = 20;

// Compile-time filter shape.  src points at the tile element that output (0,0) reads with
// tap (0,0), i.e. the caller has already applied the (-pad_q, -pad_k) / adjoint offsets, and
// `col_mis` = (that column index) mod 4 so that loads can be aligned down.
//   FLIP == false: out[r][c] = sum theta[a][b]         * src[r+a][c+b]
//   FLIP == true : out[r][c] = sum theta[CQ-1-a][CK-1-b] * src[r+a][c+b]
template <int CQ, int CK, int COL_MIS, bool FLIP>
FMTA_DEVINL void conv_strip16(float (&acc)[16], const float* __restrict__ src_aligned, int src_ld,
                              const float* __restrict__ theta /* smem [CQ][kThetaLd] */) {
  constexpr int NLOAD = (COL_MIS + 16 + CK - 1 + 3) / 4;  // float4 loads per source row
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
#pragma unroll
  for (int a = 0; a < CQ; ++a) {
    float v[NLOAD * 4];
    const float4* p = reinterpret_cast<const float4*>(src_aligned + a * src_ld);
#pragma unroll
    for (int i = 0; i < NLOAD; ++i) {
      float4 t = p[i];
      v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
    const int ta = FLIP ? (CQ - 1 - a) : a;
#pragma unroll
    for (int b = 0; b < CK; ++b) {
      const float w = theta[ta * kThetaLd + (FLIP ? (CK - 1 - b) : b)];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fmaf(w, v[COL_MIS + i + b], acc[i]);
    }
  }
}

// Run-time filter shape (any c_q <= kMaxCQ, odd c_k <= kMaxCK); slower, used for shapes
// without a compiled specialisation.  `src` is the un-aligned window origin.
template <bool FLIP>
FMTA_DEVINL void conv_strip16_rt(float (&acc)[16], const float* __restrict__ src, int src_ld,
                                 const float* __restrict__ theta, int cq, int ck) {
#pragma unroll
  for (int i = 0; i < 16; ++i) acc[i] = 0.f;
  for (int a = 0; a < cq; ++a) {
    const float* row = src + a * src_ld;
    const int ta = FLIP ? (cq - 1 - a) : a;
    for (int b = 0; b < ck; ++b) {
      const float w = theta[ta * kThetaLd + (FLIP ? (ck - 1 - b) : b)];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fmaf(w, row[i + b], acc[i]);
    }
  }
}

// Dispatch helper: CQ == 0 selects the run-time path.  (r, c16) is the strip, win_r/win_c the
// tile coordinates of the window origin for output (0,0).
template <int CQ, int CK, int WIN_C, bool FLIP>
FMTA_DEVINL void conv_strip(float (&acc)[16], const float* __restrict__ tile, int ld, int r, int c16,
                            int win_r, const float* __restrict__ theta, int cq, int ck, int win_c_rt) {
  if constexpr (CQ > 0) {
    constexpr int MIS = WIN_C & 3;
    const float* p = tile + (r + win_r) * ld + (c16 * 16 + WIN_C - MIS);
    conv_strip16<CQ, CK, MIS, FLIP>(acc, p, ld, theta);
  } else {
    const float* p = tile + (r + win_r) * ld + (c16 * 16 + win_c_rt);
    conv_strip16_rt<FLIP>(acc, p, ld, theta, cq, ck);
  }
}

// acc[16] += sum_g2 w[g2 * wstride] * (16 floats at `off` of head g2's copy of `buf`), the other heads' copies read
// through distributed shared memory.  A remote load costs several hundred cycles and G is a run-time value, so
// the loads of four heads are issued together before any of them is used (with two heads the clamped extra
// loads carry weight zero).
template <typename Cluster>
FMTA_DEVINL void mix_remote16(float (&acc)[16], Cluster& cluster, float* buf, int off, const float* w, int wstride, int G) {
  for (int g0 = 0; g0 < G; g0 += 4) {
    float4 v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float4* src = reinterpret_cast<const float4*>(cluster.map_shared_rank(buf, min(g0 + u, G - 1)) + off);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[u][i] = src[i];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float wv = (g0 + u < G) ? w[(g0 + u) * wstride] : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[4 * i] = fmaf(wv, v[u][i].x, acc[4 * i]); acc[4 * i + 1] = fmaf(wv, v[u][i].y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(wv, v[u][i].z, acc[4 * i + 2]); acc[4 * i + 3] = fmaf(wv, v[u][i].w, acc[4 * i + 3]);
      }
    }
  }
}

// The same sum with the heads' tiles published in global memory (one slot of `xstride` floats per head of the
// group, `xbase` = slot of head 0): measured on B200, tiles read back from L2 arrive about three times faster
// than through distributed shared memory (4.3 bytes per cycle and SM there).
// The CTA's own tile (head `self`) is taken from its shared-memory copy `own`.
FMTA_DEVINL void mix_global16(float (&acc)[16], const float* xbase, size_t xstride, int off, const float* w, int wstride, int G,
                              int self, const float* own) {
  for (int g0 = 0; g0 < G; g0 += 4) {
    float4 v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int g2 = min(g0 + u, G - 1);
      if (g2 == self) {
        const float4* src = reinterpret_cast<const float4*>(own + off);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[u][i] = src[i];
      } else {
        const float4* src = reinterpret_cast<const float4*>(xbase + (size_t)g2 * xstride + off);
#pragma unroll
        for (int i = 0; i < 4; ++i) v[u][i] = __ldcg(src + i);
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float wv = (g0 + u < G) ? w[(g0 + u) * wstride] : 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        acc[4 * i] = fmaf(wv, v[u][i].x, acc[4 * i]); acc[4 * i + 1] = fmaf(wv, v[u][i].y, acc[4 * i + 1]);
        acc[4 * i + 2] = fmaf(wv, v[u][i].z, acc[4 * i + 2]); acc[4 * i + 3] = fmaf(wv, v[u][i].w, acc[4 * i + 3]);
      }
    }
  }
}

}  // namespace fmta
