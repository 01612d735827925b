// Launch parameter blocks shared between the C-ABI layer (capi.cu) and the kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fmta {

// Which key blocks of a query block a kernel walks.
enum KMode : int {
  kAllTiles = 0,      // every (causally reachable) key block
  kBandTiles = 1,     // only key blocks that touch the causal band i-j < pad_q+pad_k
};

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
  const float* Opart;        // forward (optional): un-normalised partial O to start from
  const float* Mpart;
  const float* Lpart;
  float* dQ;                 // backward outputs, fp32
  float* dK;
  float* dV;
  float* dTheta_part;        // [n_slots, H, cq*ck] per-CTA-slot partial sums (reduced later)
  float* dW_part;            // [n_slots, H/G, G*G]
  int B, H, N, d, cq, ck, G;
  float scale;
  int causal;
  int o_bf16;
  int kmode;
  int accumulate;            // backward: add into dQ/dK/dV instead of overwriting
  int n_slots;
  // band mode (kmode == kBandTiles): one 64x64 tile per CTA, placed so that it holds every band entry
  // of the rows (keys) the CTA owns: key tile starts band_off before the first owned row
  int band_off;              // 16 or 32
  int band_ownq;             // query rows owned per CTA (forward, dQ kernel)
  int band_ownk;             // keys owned per CTA (dK/dV kernel)
};

// Geometry of the band tiles for a filter shape (see TrainParams::band_*).
inline void band_geometry(int cq, int ck, int* off, int* ownq, int* ownk) {
  const int pq = cq - 1, pk = (ck - 1) / 2, band = pq + pk;
  *off = (band + pk <= 17) ? 16 : 32;
  int oq = 64 - *off;
  if (72 - *off - pq < oq) oq = 72 - *off - pq;
  *ownq = oq;
  int ok = 65 - band - pq;
  if (ok > 48) ok = 48;
  *ownk = ok;
}

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
};

}  // namespace fmta
