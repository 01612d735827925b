// Parameter block and host-side declarations shared by the tensor-core backward kernels
// (bwd_tc.cu: head dim 64; bwd_tc128.cu: head dim 128).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "fmta_common.cuh"
#include "fmta_params.h"

namespace fmta {

constexpr float kLn2 = 0.6931471805599453f;


struct BwdTcParams {
  const float* LSE;   // [B,H,N] natural log
  const float* Dvec;  // [B,H,N]
  float* dQ;          // [B,H,N,D]   (dq kernel: overwritten)
  float* dV;          // [B,H,N,D]   (dkdv kernel: overwritten)
  bf16* dKt;          // [B,H,cq,N,D] bf16 (dkdv kernel: overwritten)
  int* status;
  int H, N, cq, ck, causal;
  // dK/dV kernel: the filter taps whose dKt this launch accumulates ([tap0, tap0 + ntap)) and whether it
  // accumulates dV as well; seven taps do not fit the tensor memory at once and take two launches
  int tap0, ntap, with_dv;
  // window of the call: the dQ kernel tiles the rows [row_base, row_end) and writes no other row; the dK/dV
  // kernel's key tile 0 starts at key_base (whole sequence: 0, N, 0)
  int row_base, row_end, key_base;
  int own;          // dQ kernels: dQ rows a tile of 128 dC rows owns (128 - pad_q; 120 where tiles must start on multiples of 8 rows)
  int row_anchor;   // dQ kernels: the row blocks are laid out backwards from this row (row_end, rounded up to a multiple of 8 by the variant that leaves P and dC)
  int selftest_expire;   // failure-detection self-test: the element-wise warps' first wait is on a barrier nothing arrives at
  // dQ kernel (optional outputs): the off-band P and dC = P (dP - D) of every entry, bf16, tile-major
  // [B*H][row block of 64][key block of 64][64 rows][64 keys] with ldp / 64 key blocks (ldp = N rounded up to
  // 128), so that the dK/dV kernel can stream them instead of recomputing them
  bf16* Pout;
  bf16* dCout;
  int ldp;
};


bool make_tensor_map_bf16(CUtensorMap* map, const void* base, int D, int rows, size_t outer, int box_x, int box_rows, bool sw128);
bool make_tensor_map_f32(CUtensorMap* map, const void* base, int D, int rows, size_t outer, int box_x, int box_rows, bool sw128);
bool tensor_maps_available();

// streaming dK/dV (bwd_stream.cu): P and dC left in global memory by the dQ kernel
size_t bwd_stream_extra_bytes(int B, int H, int N);
cudaError_t launch_bwd_dkdv_stream(const TrainParams& p, const __nv_bfloat16* Pbuf, const __nv_bfloat16* dCbuf, int ldp,
                                   __nv_bfloat16* dKt, int* status, cudaStream_t stream);

// head dim 128 (bwd_tc128.cu)
cudaError_t launch_bwd_dq_tc128(const TrainParams& p, const __nv_bfloat16* Kt, int* status, cudaStream_t stream);
cudaError_t launch_bwd_dkdv_tc128(const TrainParams& p, const __nv_bfloat16* Kt, __nv_bfloat16* dKt, int* status, int with_dv,
                                  int key_lo, int key_hi, cudaStream_t stream);

// Work assignment of the dK/dV kernels (grid: key tiles x heads x batch).  (batch, head)-major: the key tiles
// of one (batch, head) run side by side and share its Q / dO stream in L2 (a fully length-major order was 7 %
// slower), early key tiles, which see the most query blocks, first.  The last pairs (about 3.5 CTAs per SM)
// are walked key-tile-major instead, so that the grid ends on the shortest CTAs of several pairs and not on
// one whole pair (before, the SMs idled 7 % of the kernel at its end).
#ifdef __CUDACC__
__device__ __forceinline__ void dkdv_block_order(int BK, int& h, int& b, int& j0) {
  const int nKT = gridDim.x, nBH = gridDim.y * gridDim.z;
  const int lin = blockIdx.x + nKT * (blockIdx.y + gridDim.y * blockIdx.z);
  const int X = min(nBH, max(1, (512 + nKT / 2) / nKT));      // pairs in the key-tile-major tail
  const int head_ctas = (nBH - X) * nKT;
  int bhl, kt;
  if (lin < head_ctas) { bhl = lin / nKT; kt = lin - bhl * nKT; }
  else { const int r = lin - head_ctas; kt = r / X; bhl = nBH - X + (r - kt * X); }
  j0 = kt * BK;                                               // + the window's first key, added by the caller
  h = bhl % (int)gridDim.y; b = bhl / (int)gridDim.y;
}
#endif

}  // namespace fmta
