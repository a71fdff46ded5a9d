// pfmm.cuh -- the prompt path's dense GEMM on the fifth-generation tensor cores: Y[r][n] = sum_k W[n][k] X[r][k] for a
// chunk of up to 256 prompt rows against Q4_K / Q5_K / Q6_K / Q8_0 weights.  It replaces, for this library, the
// reference's chunked tensor-core prefill GEMM (tools/pf27/pfmm.cuh:311-384: int8 mma.sync + cp.async on sm_86; its
// caller host/llb_pf.h:551 pf_take) with a design for sm_100a:
//
//   * the multiply is tcgen05.mma (kind::f16, M = 128 weight rows, N = 256 prompt rows, K = 16 per instruction) issued
//     by ONE thread, both operands in shared memory, the fp32 accumulator in TENSOR MEMORY (two accumulators of 256
//     columns: the epilogue of one tile runs while the next tile multiplies);
//   * the activation operand arrives by TMA: the chunk's activations are kept in global memory in the order the
//     operand wants (k-group major, see PF_KG below), so a 64-column stage of all 256 rows is ONE contiguous 32 KB
//     cp.async.bulk that completes on an mbarrier (plain bulk copy of this GPU's own memory, no multicast);
//   * the weight operand is dequantised on the fly: eight warps read the packed super-blocks (each thread one row's 32
//     weights of a stage), turn the integer codes into fp16 exactly (0x6400 | code is 1024 + code), apply the sub-block
//     scale and min in one fp16 FMA and store 16-byte core-matrix rows; stores of a warp are conflict-free;
//   * a four-stage ring of (16 KB weights, 32 KB activations) with full / empty mbarriers decouples the three roles;
//     four more warps read finished accumulators with tcgen05.ld and write Y as f32, coalesced along the weight rows;
//   * every wait is bounded: a wait that runs out sets *err, and all roles then run through without waiting, so the
//     kernel returns, frees its tensor memory and leaves the context usable (llb_b200_wait_errors() reports it).
//
// Numerics: weights and activations are rounded to fp16 (11 bits) before the multiply, sums are fp32.  That is the
// prompt path's trade (the reference's fast prefill rounds to int8); the T-row verify path keeps about 22 bits.
#pragma once
#include "gemm3.cuh"

#define PF_R 256              // rows of a prompt chunk = N of the MMA
#define PF_KS 64              // columns per ring stage
#define PF_STAGES 4
#define PF_A_BYTES (128 * PF_KS * 2)
#define PF_B_BYTES (PF_R * PF_KS * 2)
#define PF_STAGE_BYTES (PF_A_BYTES + PF_B_BYTES)
#define PF_SMEM (1024 + PF_STAGES * PF_STAGE_BYTES)
#define PF_THREADS 512        // warps 0-7 dequantise, 8 loads activations, 9 issues MMAs, 12-15 write results
#define PF_IDESC 0x08400010u  // kind::f16: D f32, A / B f16 K-major, N = 256, M = 128
#define PF_MAXMAT 4

// Activations of a chunk for the dense GEMM, "k-group major": element (row r, column k) of a [PF_R][K] matrix sits at
// half index ((k >> 3) * PF_R + r) * 8 + pf_perm(k & 7): eight consecutive columns of one row are one 16-byte
// core-matrix row, the 256 rows of a k-group are contiguous (4 KB), and a 64-column stage is one 32 KB run.  Inside the
// eight the stored order is 0 2 1 3 4 6 5 7, the order in which the weight unpack produces its codes (both operands
// use it, so the contraction is unchanged).
__host__ __device__ inline size_t pf_kg_halves(int K) { return (size_t)K * PF_R; }
__device__ __forceinline__ size_t pf_kg_index4(int r, int k) { return ((size_t)(k >> 3) * PF_R + r) * 8 + (k & 4); }   // k a multiple of 4
// four consecutive columns k .. k+3 of row r (stored 0 2 1 3)
__device__ __forceinline__ void pf_kg_store4(__half *x, int r, int k, float v0, float v1, float v2, float v3) {
  const __half2 a = __floats2half2_rn(v0, v2), b = __floats2half2_rn(v1, v3);
  *(uint2 *)(x + pf_kg_index4(r, k)) = make_uint2(*(const uint32_t *)&a, *(const uint32_t *)&b);
}

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
  int K, ksplit, R;          // columns, K-slices, rows of the chunk in use (<= PF_R)
  const __half *x;           // activations, k-group major
  unsigned int *err;
};

// half2 helpers on raw words
__device__ __forceinline__ uint32_t pf_hsub2(uint32_t a, uint32_t b) { uint32_t d; asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t pf_hmul2(uint32_t a, uint32_t b) { uint32_t d; asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t pf_h2(float v) { const __half2 h = __float2half2_rn(v); return *(const uint32_t *)&h; }

__device__ __forceinline__ void pf_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void pf_bulk_load(uint32_t dst_s, const void *src, uint32_t bytes, uint32_t bar_s) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_s), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_s), "l"(src), "r"(bytes), "r"(bar_s)
               : "memory");
}
