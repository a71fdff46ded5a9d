// gemm.cuh -- dequant-fused skinny GEMM: Y[t][r] = sum_c W[r][c] * x[t][c] for T <= 16 rows of
// activations against Q4_K / Q5_K / Q6_K / Q8_0 weights.  This is the weight-streaming term of the
// reference's T-row verify leaves (tools/payload-spec.patch:46-238: spec_q4v, spec_q8c, spec_q6v)
// re-designed for sm_100a:
//
//  * the quantised integers go to the tensor cores UNCONVERTED: a 4/5/6/8-bit code placed in the
//    low bits of an fp16 lane is the subnormal value code * 2^-24 (exact), so mma.m16n8k16 computes
//    sum(code * x) per 32- or 16-column scale group exactly in fp32; the group's scale and
//    min/offset are applied to that partial sum in fp32.  No weight is ever rounded;
//  * activations are fp16 hi/lo planes (common.cuh), T <= 4 rows fill the n = 8 tile exactly; 8 rows take two
//    n-tiles, 16 rows four (the rows of several streams verified in one pass);
//  * every warp streams its own 16-row weight tiles through a private cp.async ring in shared
//    memory (16-byte coalesced copies of the packed super-blocks, bank-conflict-free row stride),
//    prefetching across tile boundaries so HBM requests never drain between tiles (the kernel
//    itself is k_gemm2 in gemm2.cuh; this file holds the arithmetic of a staged chunk and the epilogue);
//  * up to four matrices that share the activations run in one launch (gate|up, q|k|v,
//    qkv|z|beta|alpha), and K can be split into slices whose partial sums the consumer adds in a
//    fixed order (deterministic, no atomics).
#pragma once
#include "common.cuh"

#define GEMM_MAXMAT 4
#define GEMM_MAXSPLIT 16

struct GemmMat {
  const uint8_t *W;   // device layout, row stride dev_row_bytes(fmt, K)
  float *out;         // [ksplit][T][ostride] partial sums (row index within this matrix)
  int rows;
  int ostride;        // floats between consecutive tokens of one partial
  long long split_stride;  // floats between consecutive K-slices
  const int *tok_slot;     // optional: token t is written to row-block tok_slot[t] instead of t
  // several streams in one pass (tok_per > 0): token t is row t % tok_per of stream z = t / tok_per, whose slot array
  // lies tok_stride ints after the previous stream's and whose row-blocks start at z * tok_add
  int tok_per, tok_stride, tok_add;
};

__device__ __forceinline__ int gemm_out_block(const GemmMat &M, int t) {
  if (!M.tok_slot) return t;
  if (M.tok_per <= 0) return M.tok_slot[t];
  const int z = t / M.tok_per;
  return M.tok_slot[(size_t)z * M.tok_stride + (t - z * M.tok_per)] + z * M.tok_add;
}

struct GemmArgs {
  GemmMat m[GEMM_MAXMAT];
  int nmat;
  int tile0[GEMM_MAXMAT + 1];  // prefix sums of 16-row tiles
  int K, nsb;                  // columns, super-blocks (256 columns) per row
  int ksplit;
  XPlanes xp;
  int planes;                  // 2: hi/lo columns are folded into T = NC/2 tokens; 1: NC independent tokens
  int T;                       // tokens actually written
};

// a routed-expert launch (moe.cuh)
struct MoeArgs {
  const uint8_t *W;     // GU or D stack
  long long es;         // bytes per expert block
  const int *ids;       // [T][nslot]
  int nslot;            // k + 1
  int ne;               // block ne is the shared expert; ids are clamped to 0..ne
  int ef, d, T;
  const int *n_rows;    // rows of the pass in flight (<= T); tiles of later rows are not computed
  float *g, *u;         // k_moe_gu: [T][nslot * ef]
  float *out;           // k_moe_dn: [ksplit][T][d]
  long long split_stride;
};

// the 8 six-bit scales and 8 six-bit mins of a Q4_K / Q5_K super-block as four byte-packed words
// (tools/qwen35_engine.c:66-72, all eight pairs at once)
__device__ __forceinline__ void k4_scales(uint32_t u0, uint32_t u1, uint32_t u2, uint32_t &scA, uint32_t &scB,
                                          uint32_t &mnA, uint32_t &mnB) {
  scA = u0 & 0x3f3f3f3fu;
  mnA = u1 & 0x3f3f3f3fu;
  scB = (u2 & 0x0f0f0f0fu) | (((u0 >> 6) & 0x03030303u) << 4);
  mnB = ((u2 >> 4) & 0x0f0f0f0fu) | (((u1 >> 6) & 0x03030303u) << 4);
}
// byte i of w as a float without the conversion pipe: 0x4B0000bb is 2^23 + bb exactly
__device__ __forceinline__ float byte_f(uint32_t w, int i) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | (uint32_t)i)) - 8388608.0f;
}

// the same times a power of two, in one FMA: (2^23 + bb) * s - 2^23 * s is exact
__device__ __forceinline__ float byte_f_scaled(uint32_t w, int i, float s) {
  return fmaf(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7650u | (uint32_t)i)), s, -8388608.0f * s);
}

#define TWO24 16777216.0f

// a * b + c on two fp16 lanes
__device__ __forceinline__ uint32_t g2_hfma2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// ---- epilogue of one (row tile, K-slice) unit ---------------------------------------------------
// Folds the planes and writes the unit's partial sums; the consumer adds the K-slices in index order.
template <int NT>
__device__ __forceinline__ void gemm_epilogue(const GemmArgs &a, const GemmMat &M, int ks, int tile, int row0, float (&acc)[NT][4], int lane) {
  const int gid = lane >> 2, j = lane & 3;
  float val[NT][4];
  size_t idx[NT][4];
  bool on[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) { val[nt][i] = 0.0f; idx[nt][i] = 0; on[nt][i] = false; }
  if (a.planes == 2) {
    if constexpr (NT == 1) {
      // one n-tile: columns 0..3 the hi halves of rows 0..3, columns 4..7 their lo halves (held by lane j ^ 2)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const float lo = __shfl_xor_sync(0xffffffffu, acc[0][i], 2);
        const int t = 2 * j + (i & 1), r = row0 + gid + ((i >> 1) << 3);
        on[0][i] = j < 2 && t < a.T && r < M.rows;
        if (on[0][i]) { idx[0][i] = (size_t)gemm_out_block(M, t) * M.ostride + r; val[0][i] = acc[0][i] + lo * XP_LO_INV; }
      }
    } else {
      // n-tiles 0 .. NT/2-1 the hi halves of rows 8 nt .. 8 nt + 7, n-tiles NT/2 .. NT-1 their lo halves
#pragma unroll
      for (int nt = 0; nt < NT / 2; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
          const int t = nt * 8 + 2 * j + (i & 1), r = row0 + gid + ((i >> 1) << 3);
          on[nt][i] = t < a.T && r < M.rows;
          if (on[nt][i]) { idx[nt][i] = (size_t)gemm_out_block(M, t) * M.ostride + r; val[nt][i] = acc[nt][i] + acc[nt + NT / 2][i] * XP_LO_INV; }
        }
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int t = nt * 8 + 2 * j + (i & 1), r = row0 + gid + ((i >> 1) << 3);
        on[nt][i] = t < a.T && r < M.rows;
        if (on[nt][i]) { idx[nt][i] = (size_t)gemm_out_block(M, t) * M.ostride + r; val[nt][i] = acc[nt][i]; }
      }
  }
  float *out = M.out + (size_t)ks * M.split_stride;
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) if (on[nt][i]) out[idx[nt][i]] = val[nt][i];
}
