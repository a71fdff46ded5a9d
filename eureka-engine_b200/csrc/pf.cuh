// pf.cuh -- host interface of the prompt path (pf.cu): the dense tcgen05 GEMM and the row-batched ops of a chunk.
#pragma once
#include "model.cuh"

#define PF_MAXMAT 4
struct PfMat {
  const uint8_t *W;     // device layout, row stride dev_row_bytes(fmt, K)
  float *out;           // [ksplit][PF rows][ostride]
  int rows, ostride;
  long long split_stride;
};
struct PfArgs {
  PfMat m[PF_MAXMAT];
  int nmat;
  int t128[PF_MAXMAT + 1];   // prefix sums of 128-row tiles
  int K, ksplit, R;          // columns, K-slices, rows of the chunk in use (<= PF_RMAX)
  const __half *x;           // activations, k-group major
  unsigned int *err;
};


int pf_setup(void);
int pf_wait_errors_clear(void);
int pf_wait_errors(void);                         // 1 when a bounded wait of the dense GEMM ran out
int pf_pick_ksplit(int ntiles, int nsb, int sms);
int pf_gemm(cudaStream_t s, int fmt, PfArgs &a);  // fills the tile table; a.ksplit <= K / 256
int op_pf_embed(cudaStream_t s, int fmt, const uint8_t *W, int d, const int *ids, int R, float *x);
int op_pf_norm(cudaStream_t s, const float *xin, PartIn add, const float *w, float eps, int d, float *xout, __half *kg, int kg_K, int kg_col0, float *hn_out, int R);
int op_pf_silu(cudaStream_t s, PartIn g, PartIn u, int f, __half *kg, int R);
int op_pf_delta(cudaStream_t s, PartIn qkv, PartIn z, PartIn bp, PartIn ap, float *ring, int ring_ks, const float *cw, const float *dt, const float *sa,
                const float *nw, DeltaShape sh, float *S, const SpecCtl *ctl, float *y, float *beta, float *decay, float *o, __half *kg, int p0, int R);
