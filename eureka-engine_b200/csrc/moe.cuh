// moe.cuh -- the routed-expert FFN's two GEMMs (llb_moe_gu, llb_moe_dn of tools/payload-moeany.patch;
// host side host/llb_host.c:622-724) for the T <= 16 rows of a verify pass (the rows of several streams), on the
// K-quant GEMM phase of gemm2.cuh.
//
// Device layout of a layer's experts: two stacks of ne + 1 blocks, the shared expert being block ne,
//   GU  block e = [ef gate rows][ef up rows] of d columns      (es_gu bytes per block)
//   D   block e = d rows of ef columns                         (es_d bytes per block)
// A token's slots are its k chosen experts in rank order and then the shared expert: ids[t][0..k],
// wt[t][0..k] (the router kernel writes them; the shared slot carries sigmoid(shared gate)).
//
//   k_moe_gu   one virtual matrix per (token, slot): the 2 ef rows of the slot's expert against the
//              activation planes of ALL rows (an MMA has 8 columns whether one is wanted or four); the
//              epilogue keeps the slot's own token: g, u [T][(k+1) ef]
//   (k_silu_xp then builds planes of wt * silu(g) * u, (k+1) ef columns per token; with T <= 4 the down launch
//   builds its slice of them in shared memory itself, k_moe_dn_silu)
//   k_moe_dn   one virtual matrix per token: d rows of (k+1) ef columns whose super-blocks come from
//              the token's experts in rank order, so that the MMA accumulation IS the rank-order
//              weighted sum plus the gated shared expert; the epilogue keeps the token's own column.
// Two tokens that chose the same expert read its bytes twice; the second read comes from L2.
// Column t of a launch is computed by the same instructions whatever the other columns hold, so a row's
// result does not depend on which rows share its pass.
#pragma once
#include "gemm2.cuh"
#include "ffn_fused.cuh"


// A pass of 16 rows stages 32 plane columns but multiplies a weight tile with two n-tiles of them only: the hi and the
// lo tile of the eight rows its own row t is among (columns 8 (t / 8) .. and 16 + 8 (t / 8) ..).
template <int NT> constexpr int moe_ntc() { return NT > 2 ? 2 : NT; }
// column t of a finished tile: hi + lo / 2048, rows gid and gid + 8 (every lane takes part in the shuffles); with two
// n-tiles they are the hi and lo tiles of rows 8 (t / 8) ..
template <int NTC> __device__ __forceinline__ void moe_col(const float (&acc)[NTC][4], int t, int lane, float &v0, float &v1, bool &mine) {
  const int j = lane & 3, i = t & 1;
  float lo[4];
  if constexpr (NTC == 1) {
#pragma unroll
    for (int q = 0; q < 4; q++) lo[q] = __shfl_xor_sync(0xffffffffu, acc[0][q], 2);
    mine = j < 2 && (t >> 1) == j;
  } else {
#pragma unroll
    for (int q = 0; q < 4; q++) lo[q] = acc[1][q];
    mine = ((t & 7) >> 1) == j;
  }
  v0 = acc[0][i] + lo[i] * XP_LO_INV;
  v1 = acc[0][i + 2] + lo[i + 2] * XP_LO_INV;
}

template <int FMT> struct MoeGuMats {
  static constexpr bool EARLY = false;
  const MoeArgs &m;
  struct Cur { const uint8_t *W; };
  __device__ __forceinline__ int ntiles() const { return min(*m.n_rows, m.T) * m.nslot * (m.ef >> 3); }   // 2 ef / 16 tiles per slot
  __device__ __forceinline__ size_t row_bytes() const { return dev_row_bytes(FMT, m.d); }
  __device__ __forceinline__ void locate(int tile, int sb0, Cur &c, int &row0, int &rows) const {
    const int tps = m.ef >> 3, slot = tile / tps;
    const int e = min(max(m.ids[slot], 0), m.ne);
    row0 = (tile - slot * tps) * 16; rows = 2 * m.ef;
    c.W = m.W + (size_t)e * m.es + (size_t)sb0 * G2Traits<FMT>::SB;
  }
  __device__ __forceinline__ const uint8_t *src(const Cur &c, int sb0, int pc) const { return c.W + (size_t)pc * G2Traits<FMT>::SB; }
  __device__ __forceinline__ int col0(int tile) const { return ((tile / (m.ef >> 3)) / m.nslot) & ~7; }
  template <int NT> __device__ __forceinline__ void epilogue(int ks, int tile, float (&acc)[NT][4], int lane) const {
    const int tps = m.ef >> 3, slot = tile / tps, t = slot / m.nslot, jx = slot - t * m.nslot;
    float v0, v1;
    bool mine;
    moe_col<NT>(acc, t, lane, v0, v1, mine);
    if (!mine) return;
    const int r = (tile - slot * tps) * 16 + (lane >> 2);          // rows r and r + 8 of [gate | up]; a tile is all gate or all up
    float *dst = (r < m.ef ? m.g : m.u) + (size_t)t * m.nslot * m.ef + (size_t)jx * m.ef + (r < m.ef ? r : r - m.ef);
    dst[0] = v0; dst[8] = v1;
  }
};

template <int FMT> struct MoeDnMats {
  static constexpr bool EARLY = false;
  const MoeArgs &m;
  struct Cur { const int *ids; };
  __device__ __forceinline__ int ntiles() const { return min(*m.n_rows, m.T) * (m.d >> 4); }
  __device__ __forceinline__ size_t row_bytes() const { return dev_row_bytes(FMT, m.ef); }
  __device__ __forceinline__ void locate(int tile, int sb0, Cur &c, int &row0, int &rows) const {
    const int tpt = m.d >> 4, t = tile / tpt;
    row0 = (tile - t * tpt) * 16; rows = m.d;
    c.ids = m.ids + t * m.nslot;
  }
  __device__ __forceinline__ const uint8_t *src(const Cur &c, int sb0, int pc) const {
    const int eb = m.ef >> 8, sbi = sb0 + pc, g = sbi / eb;
    const int e = min(max(c.ids[g], 0), m.ne);
    return m.W + (size_t)e * m.es + (size_t)(sbi - g * eb) * G2Traits<FMT>::SB;
  }
  __device__ __forceinline__ int col0(int tile) const { return (tile / (m.d >> 4)) & ~7; }
  template <int NT> __device__ __forceinline__ void epilogue(int ks, int tile, float (&acc)[NT][4], int lane) const {
    const int tpt = m.d >> 4, t = tile / tpt;
    float v0, v1;
    bool mine;
    moe_col<NT>(acc, t, lane, v0, v1, mine);
    if (!mine) return;
    float *dst = m.out + (size_t)ks * m.split_stride + (size_t)t * m.d + (tile - t * tpt) * 16 + (lane >> 2);
    dst[0] = v0; dst[8] = v1;
  }
};

template <int FMT, int NT>
__global__ void __launch_bounds__(g2_warps<FMT>(8 * NT, moe_ntc<NT>() != NT) * 32, G2_CPSM) k_moe_gu(const GemmArgs a, const MoeArgs m, const int cps) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  g2_phase<FMT, NT, G2StagePlanes<FMT, NT>, MoeGuMats<FMT>, moe_ntc<NT>()>(a, cps, (int)blockIdx.x, smem, G2StagePlanes<FMT, NT>{a}, MoeGuMats<FMT>{m});
}
// The down launch's activation slice built in shared memory from the gate|up outputs (T <= 4 rows): wt * silu(g) * u
// of the CTA's K-slice, planes and side array exactly as k_silu_xp + G2StagePlanes would have left them, without the
// launch in between.  Every CTA of a K-slice computes the same few thousand values.
template <int FMT> struct MoeStageSilu {
  const MoeArgs &m;
  const float *wt;   // [T][nslot]
  __device__ __forceinline__ void operator()(uint8_t *xh_s, uint8_t *xsf_s, int CS, int sb0, int nsl) const {
    pdl_wait();
    const int lane = threadIdx.x & 31, T = min(*m.n_rows, m.T), f = m.nslot * m.ef;
    const int ngrp = nsl * 64, ntask = 4 * ngrp;   // (row of the 4 plane pairs, group of four columns); rows >= T are zero planes
    for (int t0 = threadIdx.x; t0 < ntask; t0 += 4 * blockDim.x) {
      float4 gv[4], uv[4];
      float w[4];
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int task = t0 + q * blockDim.x, t = task / ngrp, c = 4 * (task - t * ngrp);
        gv[q] = make_float4(0.f, 0.f, 0.f, 0.f); uv[q] = gv[q]; w[q] = 0.0f;
        if (task < ntask && t < T) {
          const int cg = sb0 * 256 + c;
          const size_t i = (size_t)t * f + cg;
          gv[q] = __ldcg((const float4 *)(m.g + i)); uv[q] = __ldcg((const float4 *)(m.u + i));
          w[q] = __ldcg(wt + (size_t)t * m.nslot + cg / m.ef);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; q++) {
        const int task = t0 + q * blockDim.x, t = task / ngrp, c = 4 * (task - t * ngrp);
        if (task < ntask) {   // whole warps: ngrp and blockDim are multiples of 32
          const float h[4] = {(gv[q].x / (1.0f + expf(-gv[q].x))) * uv[q].x * w[q], (gv[q].y / (1.0f + expf(-gv[q].y))) * uv[q].y * w[q],
                              (gv[q].z / (1.0f + expf(-gv[q].z))) * uv[q].z * w[q], (gv[q].w / (1.0f + expf(-gv[q].w))) * uv[q].w * w[q]};
          ffn_store4<FMT>(xh_s, xsf_s, CS, t, c, h, lane);
        }
      }
    }
    __syncthreads();
  }
};

template <int FMT>
__global__ void __launch_bounds__(G2Traits<FMT>::WARPS * 32, G2_CPSM) k_moe_dn_silu(const GemmArgs a, const MoeArgs m, const float *wt, const int cps) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  g2_phase<FMT, 1>(a, cps, (int)blockIdx.x, smem, MoeStageSilu<FMT>{m, wt}, MoeDnMats<FMT>{m});
}

template <int FMT, int NT>
__global__ void __launch_bounds__(g2_warps<FMT>(8 * NT, moe_ntc<NT>() != NT) * 32, G2_CPSM) k_moe_dn(const GemmArgs a, const MoeArgs m, const int cps) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  g2_phase<FMT, NT, G2StagePlanes<FMT, NT>, MoeDnMats<FMT>, moe_ntc<NT>()>(a, cps, (int)blockIdx.x, smem, G2StagePlanes<FMT, NT>{a}, MoeDnMats<FMT>{m});
}
