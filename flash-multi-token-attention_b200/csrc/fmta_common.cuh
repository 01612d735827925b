// Shared device helpers for the conv-attention kernels (sm_100a).
//
// Register-fragment tensor-core helpers (ldmatrix + mma.sync m16n8k16 bf16, fp32
// accumulate) used by the exact tile kernels, the band kernels and the decode kernel, cp.async
// tile loaders with zero fill, and small warp utilities.  The TMA / tcgen05 / TMEM
// helpers used by the stacked-GEMM forward live in fmta_tc.cuh.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmta {

typedef __nv_bfloat16 bf16;

#define FMTA_DEVINL __device__ __forceinline__

FMTA_DEVINL uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- cp.async (16-byte, L2 only) with zero fill when `valid` is false -------------------
FMTA_DEVINL void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem_dst)),
               "l"(gsrc), "r"(sz)
               : "memory");
}
FMTA_DEVINL void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
FMTA_DEVINL void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// wait until at most n (0..6) of this thread's cp.async groups are pending
FMTA_DEVINL void cp_async_wait_dyn(int n) {
  switch (n) {
    case 0: cp_async_wait<0>(); break;
    case 1: cp_async_wait<1>(); break;
    case 2: cp_async_wait<2>(); break;
    case 3: cp_async_wait<3>(); break;
    case 4: cp_async_wait<4>(); break;
    case 5: cp_async_wait<5>(); break;
    default: cp_async_wait<6>(); break;
  }
}

// Copy rows [row0, row0+nrows) of a row-major [n_rows_total, D] bf16 matrix into shared
// memory with row stride `ld` elements.  Rows outside [0, n_rows_total) become zero.
template <int D, int NT>
FMTA_DEVINL void load_rows_async(bf16* dst, int ld, const bf16* __restrict__ src, int row0, int nrows,
                                 int n_rows_total, int tid) {
  constexpr int CPR = D / 8;  // 16-byte chunks per row
  for (int idx = tid; idx < nrows * CPR; idx += NT) {
    const int r = idx / CPR, c = idx % CPR;
    const int gr = row0 + r;
    const bool ok = (gr >= 0) && (gr < n_rows_total);
    const bf16* g = src + (size_t)(ok ? gr : 0) * D + c * 8;
    cp_async16(dst + r * ld + c * 8, g, ok);
  }
}

// ---- ldmatrix / mma.sync -----------------------------------------------------------------
FMTA_DEVINL void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
FMTA_DEVINL void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
FMTA_DEVINL void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One warp: acc[NT][4] += A(16 x Kdim) * B(Kdim x 8*NT), operands bf16 in shared memory.
//   A_T == false: A stored [m][k] (ld = lda), pointer at element (m0, k0)
//   A_T == true : A stored [k][m],           pointer at element (k0, m0)
//   B_T == false: B stored [n][k] (ld = ldb), pointer at element (n0, k0)
//   B_T == true : B stored [k][n],           pointer at element (k0, n0)
// NT must be even.  Fragment ownership of acc follows mma.m16n8k16: for n-tile j,
// acc[j][0..1] = (row lane/4, cols 8j + 2*(lane%4) + {0,1}), acc[j][2..3] = same cols, row + 8.
template <int NT, bool A_T, bool B_T>
FMTA_DEVINL void warp_gemm(float (*acc)[4], const bf16* A, int lda, const bf16* B, int ldb, int Kdim,
                           int lane) {
  static_assert(NT % 2 == 0, "NT must be even");
  const int l8 = lane & 7, q = lane >> 3;
  for (int k0 = 0; k0 < Kdim; k0 += 16) {
    uint32_t a[4];
    if (!A_T) {
      ldsm_x4(a, A + (l8 + (q & 1) * 8) * lda + k0 + (q >> 1) * 8);
    } else {
      ldsm_x4_t(a, A + (k0 + l8 + (q >> 1) * 8) * lda + (q & 1) * 8);
    }
#pragma unroll
    for (int j = 0; j < NT; j += 2) {
      uint32_t b[4];
      if (!B_T) {
        // matrices: (n 0-7,k 0-7) (n 0-7,k 8-15) (n 8-15,k 0-7) (n 8-15,k 8-15)
        ldsm_x4(b, B + (j * 8 + l8 + (q >> 1) * 8) * ldb + k0 + (q & 1) * 8);
      } else {
        // stored [k][n]: matrices (k 0-7,n 0-7) (k 8-15,n 0-7) (k 0-7,n 8-15) (k 8-15,n 8-15)
        ldsm_x4_t(b, B + (k0 + l8 + (q & 1) * 8) * ldb + j * 8 + (q >> 1) * 8);
      }
      mma_bf16(acc[j], a, b[0], b[1]);
      mma_bf16(acc[j + 1], a, b[2], b[3]);
    }
  }
}

FMTA_DEVINL float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
FMTA_DEVINL float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

FMTA_DEVINL uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}

constexpr float kLog2e = 1.4426950408889634f;

}  // namespace fmta
