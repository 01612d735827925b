// Launch parameter blocks shared between the C-ABI layer (capi.cu) and the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmta {

struct TrainParams {
  const __nv_bfloat16* Q;
  const __nv_bfloat16* K;
  const __nv_bfloat16* V;
  const __nv_bfloat16* dO;   // backward only
  const float* theta;        // [H, cq, ck] fp32 (nullptr = no key-query conv)
  const float* Wmix;         // [H/G, G, G] fp32 head-mix matrices (nullptr = no mix)
  const float* LSE;          // backward: [B,H,N] log-sum-exp of the forward
  const float* Dvec;         // backward: [B,H,N] rowsum(dO*O)
  void* O;                   // forward: [B,H,N,d] fp32 or bf16
  float* M;                  // forward: [B,H,N] row max
  float* L;                  // forward: [B,H,N] row sum of exp(C - M)
  float* LSEout;             // forward (optional): M + log L
  const float* Opart;        // forward band kernel: un-normalised partial (O, m, l) left by the tensor-core kernel
  const float* Mpart;
  const float* Lpart;
  float* dQ;                 // backward outputs, fp32
  float* dK;
  float* dV;
  float* dTheta_part;        // [n_slots, H, cq*ck] per-CTA-slot partial sums (reduced later)
  float* dW_part;            // [n_slots, H/G, G*G]
  __nv_bfloat16* Kt_ext;     // tensor-core path: caller-owned stacked key operand [B,H,cq,N,d] instead of the workspace's (nullptr: none)
  int kt_valid;              //   ... which already holds the operand of these K / theta / scale: the pre-pass is skipped
  int row_lo, row_hi;        // tensor-core path: the window of sequence positions this call computes (output rows of the
                             //   forward; dQ rows, dK / dV keys and the dTheta terms of the backward); 0, 0 = the whole sequence
  float* xchg;               // conv + mix cluster kernels: optional global scratch, 2 sets x 2 * kMixXchFloats floats per CTA (nullptr: exchange through distributed shared memory)
  int B, H, N, d, cq, ck, G;
  float scale;
  int causal;
  int o_bf16;
  int n_slots;
};

#ifdef __CUDACC__
// Programmatic dependent launch.  A kernel launched with launch_pdl may start while the kernel before it in the
// stream is still running; it must call pdl_wait() before it reads anything an earlier kernel wrote or writes
// anything one reads (pdl_wait returns once the preceding kernel has completed and its writes are visible; every CTA
// calls it before it exits, so that "this kernel has completed" keeps implying "every earlier one has").
// pdl_trigger() lets the NEXT kernel's CTAs be scheduled as soon as every CTA of this one has called it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

// The window of a call: [win_lo(p), win_hi(p))
__host__ __device__ inline int win_lo(const TrainParams& p) { return p.row_hi > 0 ? p.row_lo : 0; }
__host__ __device__ inline int win_hi(const TrainParams& p) { return p.row_hi > 0 ? p.row_hi : p.N; }

// One exchanged tile of the conv + mix cluster kernels: the backward's 80 x 84 fp32 region (the forward's 64 x 68 tile fits)
constexpr int kMixXchFloats = 80 * 84;

struct DecodeParams {
  const __nv_bfloat16* Q;    // [B,H,q_len,d]
  const __nv_bfloat16* K;    // [B,H,Nk,d]
  const __nv_bfloat16* V;
  const float* theta;        // [H,cq,ck]
  float* O_splits;           // [B,H,k_splits,d]
  float* M_splits;           // [B,H,k_splits]
  float* L_splits;
  int B, H, q_len, Nk, d, cq, ck, k_splits;
  float scale;
  int offset_causal;         // zero the scores of keys later than each query row's position (row r sits at Nk - rows + r)
  // paged cache (block_table != nullptr): K and V point at pools [n_pages, H, page_size, d]; page p of
  // sequence b is pool page block_table[b * max_pages + p]; seq_lens (optional) gives Nk per sequence
  const int* block_table;
  const int* seq_lens;
  int page_size, page_shift, max_pages;
};

}  // namespace fmta
