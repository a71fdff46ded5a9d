// ffn_fused.cuh -- the SwiGLU FFN of a layer as ONE launch: gate|up GEMM, silu(gate) * up, down GEMM.
//
// A GEMM launch costs about 6 us before it streams at full rate: its CTAs take a whole SM each, so they cannot
// start before the previous launch has left, then they wait for the producer of their activations and stage them.
// Here the CTAs stay: when a CTA has finished its gate|up tiles it fills its ring with ffn_down weights, meets the
// other CTAs at a grid-wide barrier (all gate|up outputs are then in L2), builds its K-slice of silu(gate) * up as
// activation planes directly in shared memory (no plane array in global memory, no separate kernel), and streams
// its ffn_down tiles.  Replaces llb_spec_gu + llb_t_siluq + llb_spec_re of the reference's spec_ffn
// (host/llb_host.c:1701-1711) with one launch instead of three.
//
// The barrier: every CTA of the launch is resident (at most one per SM, grid <= SM count), arrives with one
// atomic add and polls the counter.  The poll is bounded; a wait that runs out sets *err and goes on (the results
// of that launch are then invalid, llb_b200_wait_errors() reports it).  The last CTA to leave resets the counters.
#pragma once
#include "gemm2.cuh"

#define FFN_SYNC_LIMIT (1u << 22)

__device__ __forceinline__ void ffn_grid_sync(unsigned int *sync, unsigned int nblocks, unsigned int *err) {
  __threadfence();   // this thread's gate|up outputs, before the CTA says it is done
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(sync, 1u);
    unsigned int seen = 0, it = 0;
    do {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(sync) : "memory");
    } while (seen < nblocks && ++it < FFN_SYNC_LIMIT);
    if (seen < nblocks && err) atomicExch(err, 1u);
    // everybody who increments the second counter has left the loop above: the last one may reset both
    if (atomicAdd(sync + 1, 1u) == nblocks - 1) { sync[0] = 0; sync[1] = 0; __threadfence(); }
  }
  __syncthreads();
}

// silu(g) * u of 32 consecutive slice columns (lane = column) of token t into the planes and the side array in
// shared memory, laid out exactly as G2StagePlanes would have copied them from global memory
template <int FMT> __device__ __forceinline__ void ffn_store32(uint8_t *xh_s, uint8_t *xsf_s, int CS, int t, int blk32, float v, int lane) {
  constexpr int NC = 8, NH = 4;
  const int c = blk32 * 32 + lane, pc = (c & ~7) | ((c & 4) | ((c & 1) << 1) | ((c & 2) >> 1));
  const __half hi = __float2half_rn(v);
  float hif = __half2float(hi);
  const __half lo = __float2half_rn((v - hif) * XP_LO_SCALE);
  float lof = __half2float(lo);
  ((__half *)(xh_s + (size_t)t * CS))[pc] = hi;
  ((__half *)(xh_s + (size_t)(NH + t) * CS))[pc] = lo;
#pragma unroll
  for (int m = 1; m < 16; m <<= 1) {
    hif += __shfl_xor_sync(0xffffffffu, hif, m);
    lof += __shfl_xor_sync(0xffffffffu, lof, m);
  }
  const float hi32 = hif + __shfl_xor_sync(0xffffffffu, hif, 16), lo32 = lof + __shfl_xor_sync(0xffffffffu, lof, 16);
  if constexpr (FMT == LLB_FM_Q6_K) {
    if ((lane & 15) == 0) {   // f32 sums of 16 columns: [16-column group][NC]
      float *x16 = (float *)xsf_s + (size_t)(blk32 * 2 + (lane >> 4)) * NC;
      x16[t] = hif; x16[NH + t] = lof;
    }
  } else {
    if (lane == 0) {          // 32-column means as fp16 hi / rest, in the order the min-term MMA's B fragment reads them
      const int sb = blk32 >> 3, b = blk32 & 7;
      __half *f = (__half *)xsf_s + ((size_t)sb * NC + t) * 16 + 4 * (b >> 1) + (b & 1);
      float m = hi32 * 0.03125f;
      __half h1 = __float2half_rn(m);
      f[0] = h1; f[2] = __float2half_rn(m - __half2float(h1));
      f += (size_t)NH * 16;
      m = lo32 * 0.03125f;
      h1 = __float2half_rn(m);
      f[0] = h1; f[2] = __float2half_rn(m - __half2float(h1));
    }
  }
}

template <int FMT> struct FfnStageSilu {
  const float *g, *u;      // gate and up outputs [T][f], complete (their launch used one K-slice)
  int f, T;
  unsigned int *sync, *err;
  __device__ __forceinline__ void operator()(uint8_t *xh_s, uint8_t *xsf_s, int CS, int sb0, int nsl) const {
    ffn_grid_sync(sync, gridDim.x, err);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    // tasks: (token t of 4 plane pairs, 32-column block); rows t >= T are zero planes.  Eight tasks at a time: their
    // sixteen loads are in flight together (one trip to L2 per batch, not per task)
    const int ntask = 4 * nsl * 8;
    for (int t0 = warp; t0 < ntask; t0 += 8 * nwarp) {
      float gv[8], uv[8];
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const int task = t0 + q * nwarp, t = task & 3, blk32 = task >> 2;
        gv[q] = 0.0f; uv[q] = 0.0f;
        if (task < ntask && t < T) {
          const size_t i = (size_t)t * f + (size_t)sb0 * 256 + blk32 * 32 + lane;
          gv[q] = __ldcg(g + i); uv[q] = __ldcg(u + i);
        }
      }
#pragma unroll
      for (int q = 0; q < 8; q++) {
        const int task = t0 + q * nwarp;
        if (task < ntask) ffn_store32<FMT>(xh_s, xsf_s, CS, task & 3, task >> 2, (gv[q] / (1.0f + expf(-gv[q]))) * uv[q], lane);
      }
    }
    __syncthreads();
  }
};

template <int FMT2>
__global__ void __launch_bounds__(512, 1) k_ffn(const GemmArgs a1, const GemmArgs a2, const int cps1, const int cps2, unsigned int *sync,
                                                unsigned int *err) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  g2_phase<LLB_FM_Q4_K, 1>(a1, cps1, (int)blockIdx.x, smem, G2StagePlanes<LLB_FM_Q4_K, 1>{a1});
  __syncthreads();   // the CTA is done with the first launch's shared memory
  g2_phase<FMT2, 1>(a2, cps2, (int)blockIdx.x, smem, FfnStageSilu<FMT2>{a1.m[0].out, a1.m[1].out, a1.m[0].rows, a1.T, sync, err});
}
