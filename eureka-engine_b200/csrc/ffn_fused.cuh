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

__device__ __forceinline__ void ffn_grid_sync(unsigned int *sync, unsigned int nblocks, unsigned int *err, unsigned int limit = FFN_SYNC_LIMIT) {
  __threadfence();   // this thread's gate|up outputs, before the CTA says it is done
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(sync, 1u);
    unsigned int seen = 0, it = 0;
    do {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(sync) : "memory");
    } while (seen < nblocks && ++it < limit);
    if (seen < nblocks && err) atomicExch(err, 1u);
    // everybody who increments the second counter has left the loop above: the last one may reset both
    if (atomicAdd(sync + 1, 1u) == nblocks - 1) { sync[0] = 0; sync[1] = 0; __threadfence(); }
  }
  __syncthreads();
}

// silu(g) * u of FOUR consecutive slice columns c .. c+3 (c a multiple of 4; the eight lanes 8j .. 8j+7 of a warp hold
// one aligned group of 32 columns) of token t into the planes and the side array in shared memory, laid out exactly as
// G2StagePlanes would have copied them from global memory.  Stored order inside the four: 0 2 1 3.
template <int FMT> __device__ __forceinline__ void ffn_store4(uint8_t *xh_s, uint8_t *xsf_s, int CS, int t, int c, const float (&v)[4], int lane) {
  constexpr int NC = 8, NH = 4;
  __half hi[4], lo[4];
  float hs = 0.0f, ls = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    hi[i] = __float2half_rn(v[i]);
    const float hf = __half2float(hi[i]);
    lo[i] = __float2half_rn((v[i] - hf) * XP_LO_SCALE);
    hs += hf; ls += __half2float(lo[i]);
  }
  {
    const __half2 a = __halves2half2(hi[0], hi[2]), b = __halves2half2(hi[1], hi[3]);
    *(uint2 *)(xh_s + (size_t)t * CS + (size_t)c * 2) = make_uint2(*(const uint32_t *)&a, *(const uint32_t *)&b);
    const __half2 e = __halves2half2(lo[0], lo[2]), f = __halves2half2(lo[1], lo[3]);
    *(uint2 *)(xh_s + (size_t)(NH + t) * CS + (size_t)c * 2) = make_uint2(*(const uint32_t *)&e, *(const uint32_t *)&f);
  }
  hs += __shfl_xor_sync(0xffffffffu, hs, 1); ls += __shfl_xor_sync(0xffffffffu, ls, 1);
  hs += __shfl_xor_sync(0xffffffffu, hs, 2); ls += __shfl_xor_sync(0xffffffffu, ls, 2);   // 16 columns
  if constexpr (FMT == LLB_FM_Q6_K) {
    if ((lane & 3) == 0) {   // f32 sums of 16 columns: [16-column group][NC]
      float *x16 = (float *)xsf_s + (size_t)(c >> 4) * NC;
      x16[t] = hs; x16[NH + t] = ls;
    }
  } else {
    const float h32 = hs + __shfl_xor_sync(0xffffffffu, hs, 4), l32 = ls + __shfl_xor_sync(0xffffffffu, ls, 4);
    if ((lane & 7) == 0) {   // 32-column means as fp16 hi / rest, in the order the min-term MMA's B fragment reads them
      const int sb = c >> 8, b = (c >> 5) & 7;
      __half *f = (__half *)xsf_s + ((size_t)sb * NC + t) * 16 + 4 * (b >> 1) + (b & 1);
      float m = h32 * 0.03125f;
      __half h1 = __float2half_rn(m);
      f[0] = h1; f[2] = __float2half_rn((m - __half2float(h1)) * XP_LO_SCALE);
      f += (size_t)NH * 16;
      m = l32 * 0.03125f;
      h1 = __float2half_rn(m);
      f[0] = h1; f[2] = __float2half_rn((m - __half2float(h1)) * XP_LO_SCALE);
    }
  }
}

template <int FMT> struct FfnStageSilu {
  const float *g, *u;      // gate and up outputs [T][f], complete (their launch used one K-slice)
  int f, T;
  unsigned int *sync, *err;
  __device__ __forceinline__ void operator()(uint8_t *xh_s, uint8_t *xsf_s, int CS, int sb0, int nsl) const {
    ffn_grid_sync(sync, gridDim.x, err);
    const int lane = threadIdx.x & 31;
    // thread task = (token t of the 4 plane pairs, group of four columns); rows t >= T are zero planes.  The slice
    // has nsl * 64 groups per token; up to six tasks of a thread are loaded together (one trip to L2)
    const int ngrp = nsl * 64, ntask = 4 * ngrp;
    for (int t0 = threadIdx.x; t0 < ntask; t0 += 6 * blockDim.x) {
      float4 gv[6], uv[6];
#pragma unroll
      for (int q = 0; q < 6; q++) {
        const int task = t0 + q * blockDim.x, t = task / ngrp, c = 4 * (task - t * ngrp);
        gv[q] = make_float4(0.f, 0.f, 0.f, 0.f); uv[q] = gv[q];
        if (task < ntask && t < T) {
          const size_t i = (size_t)t * f + (size_t)sb0 * 256 + c;
          gv[q] = __ldcg((const float4 *)(g + i)); uv[q] = __ldcg((const float4 *)(u + i));
        }
      }
#pragma unroll
      for (int q = 0; q < 6; q++) {
        const int task = t0 + q * blockDim.x, t = task / ngrp, c = 4 * (task - t * ngrp);
        if (task < ntask) {   // whole warps: ngrp and blockDim are multiples of 32
          const float h[4] = {(gv[q].x / (1.0f + expf(-gv[q].x))) * uv[q].x, (gv[q].y / (1.0f + expf(-gv[q].y))) * uv[q].y,
                              (gv[q].z / (1.0f + expf(-gv[q].z))) * uv[q].z, (gv[q].w / (1.0f + expf(-gv[q].w))) * uv[q].w};
          ffn_store4<FMT>(xh_s, xsf_s, CS, t, c, h, lane);
        }
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
  g2_phase<LLB_FM_Q4_K, 1>(a1, cps1, (int)blockIdx.x, smem, G2StagePlanes<LLB_FM_Q4_K, 1>{a1}, G2MatsPlain<LLB_FM_Q4_K>{a1});
  __syncthreads();   // the CTA is done with the first launch's shared memory
  g2_phase<FMT2, 1>(a2, cps2, (int)blockIdx.x, smem, FfnStageSilu<FMT2>{a1.m[0].out, a1.m[1].out, a1.m[0].rows, a1.T, sync, err}, G2MatsPlain<FMT2>{a2});
}
