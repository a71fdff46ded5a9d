// gemm3.cuh -- the Q4_K skinny GEMM on the fifth-generation tensor cores (tcgen05), T <= 4.
//
// Same arithmetic as gemm2.cuh -- 4-bit codes as fp16 subnormal integers, fp16 hi/lo activation
// planes, sub-block scales applied to fp32 partial sums, the "min" term as one extra MMA per
// super-block -- but the multiply runs as tcgen05.mma (M = 128 rows, N = 16, K = 16) with the weight
// operand in TENSOR MEMORY: a thread owns one row and a pair of sub-blocks, unpacks its 32 bytes of
// nibbles into 32 registers (five instructions per four) and stores them with tcgen05.st; one thread
// issues the 17 MMAs of a 128-row x 256-column super-block; the accumulators come back with
// tcgen05.ld, one row per thread, so the scale step is 18 FMAs per thread and super-block.  The mma.sync
// kernel spends 380 warp instructions per 16 rows x 256 columns; this one about 250 for the same bytes.
//
//   TMEM columns (512 allocated):  A buffers at 0 and 136 (128 columns of codes + 8 of mins),
//   D buffers at 272 and 376.  Issuing a tcgen05.mma costs one thread about 100 cycles, so four warps
//   issue, each the four MMAs of one sub-block pair (the last also the min term).  The MMA's N is 16 but
//   only 8 columns are real (4 tokens x hi/lo): issuer i accumulates sub-block 2i at D + 24i and
//   2i + 1 at D + 24i + 8, whose first MMA overwrites the unused upper half of the one before (the MMAs
//   of one thread execute in issue order); the min term sits at D + 88.
//   Shared memory: activation planes of the CTA's K-slice as K-major core matrices
//   [k/8][column][8 halves] (the planes' stored k-order 0 2 1 3 4 6 5 7 is the order the unpack
//   produces), the sub-block means for the min term, a ring of raw 128-row x 144-byte stages filled
//   with cp.async, and the buffer the four threads of a row reduce through.
//   Every wait on an mbarrier is bounded; a wait that runs out sets *err and the kernel drains, frees
//   its tensor memory and returns.
#pragma once
#include "gemm.cuh"
#include "tc5.cuh"
static_assert(GEMM_MAXMAT == 4, "k_gemm3 finds a tile's matrix with three compares");

#define G3_THREADS 512        // worker threads; four more warps issue the MMAs
#define G3_BLOCK (G3_THREADS + 128)
#define G3_STAGES 6
#define G3_STAGE_BYTES (128 * 144)
#define G3_RED_BYTES (5 * 128 * 8 * 4)   // four partial sums per row and column, and the row's min terms
#define G3_HDR_BYTES 128
#define G3_SMEM_MAX 232448
#define G3_TMEM_COLS 512
#define G3_A_COLS 136
#define G3_D0 272
#define G3_D_COLS 104
#define G3_IDESC 0x08040010u   // kind::f16: D f32, A/B f16 K-major, N = 16, M = 128

// bytes of shared memory for a K-slice of nsl super-blocks (NC = 8 activation columns)
__host__ __device__ inline int g3_xp_bytes(int nsl) { return nsl * (32 * 8 * 16 + 2 * 8 * 16) + 256; }
inline int g3_smem_bytes(int nsl) { return G3_HDR_BYTES + g3_xp_bytes(nsl) + G3_RED_BYTES + G3_STAGES * G3_STAGE_BYTES; }
inline int g3_max_slice_sb() { return (G3_SMEM_MAX - G3_HDR_BYTES - 256 - G3_RED_BYTES - G3_STAGES * G3_STAGE_BYTES) / (32 * 8 * 16 + 2 * 8 * 16); }

__device__ __forceinline__ void workers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(G3_THREADS) : "memory"); }
__device__ __forceinline__ void quarter_sync(int q) { asm volatile("bar.sync %0, 128;" ::"r"(2 + q) : "memory"); }

__global__ void __launch_bounds__(G3_BLOCK, 1) k_gemm3(const GemmArgs a, const int cps, unsigned int *__restrict__ err) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int q = warp & 3, c = (warp >> 2) & 3, r = 32 * q + lane;   // TMEM lane quarter, sub-block pair, row of the tile
  const int ks = blockIdx.x % a.ksplit, ci = blockIdx.x / a.ksplit;
  const int sb0 = (int)(((long long)ks * a.nsb) / a.ksplit), nsl = (int)(((long long)(ks + 1) * a.nsb) / a.ksplit) - sb0;
  uint32_t *tmem_slot = (uint32_t *)(smem + 40);
  volatile uint32_t *dead = (volatile uint32_t *)(smem + 44);
  uint8_t *Bp = smem + G3_HDR_BYTES, *Bm = Bp + (size_t)nsl * 4096 + 128;
  float *red = (float *)(Bm + (size_t)nsl * 256 + 128);
  uint8_t *ring = (uint8_t *)red + G3_RED_BYTES;
  // barriers: D_full[2] at +0, +8 (one commit per issuing warp), A_full[2] at +24, +32 (16 worker warps)
  const uint32_t bar_s = smem_u32(smem), Bp_s = smem_u32(Bp), Bm_s = smem_u32(Bm);
  auto dfull = [&](int i) { return bar_s + 8u * (uint32_t)i; };
  auto afull = [&](int i) { return bar_s + 24u + 8u * (uint32_t)i; };
  int t128[GEMM_MAXMAT + 1];
  t128[0] = 0;
#pragma unroll
  for (int m = 0; m < GEMM_MAXMAT; m++) t128[m + 1] = t128[m] + (m < a.nmat ? (a.m[m].rows + 127) / 128 : 0);
  const int ntiles = t128[GEMM_MAXMAT];
  const int my_tiles = ci < ntiles ? (ntiles - ci + cps - 1) / cps : 0, n_items = my_tiles * nsl;
  const size_t rb = dev_row_bytes(LLB_FM_Q4_K, a.K);

  // The four warps of a lane quarter load the quarter's 32 rows x 144 bytes of a super-block together:
  // 288 sixteen-byte pieces, piece i = tq + 128 * it of thread tq = 32 c + lane, nine consecutive pieces per row.
  const int tq = 32 * c + lane;
  uint8_t *qring = ring + (size_t)q * 4608;
  const uint32_t qring_s = smem_u32(qring);
  int p_tile = ci, p_c = 0, p_stage = 0, p_left = n_items;
  const uint8_t *p_W = nullptr;
  uint32_t p_off[3];
  auto plan_tile = [&](int tile) {
    if (tile >= ntiles) return;
    const int m = (tile >= t128[1]) + (tile >= t128[2]) + (tile >= t128[3]);   // t128[k] = ntiles beyond the last matrix
    const int row0 = (tile - (m == 0 ? 0 : m == 1 ? t128[1] : m == 2 ? t128[2] : t128[3])) * 128 + 32 * q, rows = a.m[m].rows;
    p_W = a.m[m].W + (size_t)sb0 * 144;
#pragma unroll
    for (int it = 0; it < 3; it++) {
      const int i = tq + 128 * it, rr = i / 9, pp = i - rr * 9;
      p_off[it] = (uint32_t)min(row0 + rr, rows - 1) * (uint32_t)rb + pp * 16;
    }
  };
  auto issue = [&]() {
    if (p_left > 0) {
      const uint8_t *src = p_W + (size_t)p_c * 144;
      const uint32_t dst = qring_s + p_stage * G3_STAGE_BYTES + tq * 16;
      cp_async16(dst, src + p_off[0]);
      cp_async16(dst + 2048, src + p_off[1]);
      if (tq < 32) cp_async16(dst + 4096, src + p_off[2]);
      p_left--;
      if (++p_c == nsl) { p_c = 0; p_tile += cps; plan_tile(p_tile); }
      p_stage = p_stage + 1 == G3_STAGES ? 0 : p_stage + 1;
    }
    cp_async_commit();
  };
  const bool worker = warp < G3_THREADS / 32;
  pdl_trigger();
  if (worker) {
    plan_tile(p_tile);
#pragma unroll 1
    for (int s = 0; s < G3_STAGES - 1; s++) issue();   // weights depend on no kernel: in flight before the wait
  }
  if (tid == 0) {
    mbar_init(dfull(0), 4);
    mbar_init(dfull(1), 4);
    mbar_init(afull(0), 16);
    mbar_init(afull(1), 16);
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)G3_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();
  if (worker) {
    const int per_col = nsl * 32;   // k-groups of the slice
    for (int i = tid; i < 8 * per_col; i += G3_THREADS) {
      const int n = i / per_col, g = i - n * per_col;
      cp_async16(Bp_s + (g * 8 + n) * 16, (const uint8_t *)(a.xp.xh + (size_t)n * a.K + (size_t)sb0 * 256) + g * 16);
    }
    for (int i = tid; i < nsl * 16; i += G3_THREADS) {   // (sb, n, h): 16 halves of means -> chunk h of column n
      const int sb = i >> 4, n = (i >> 1) & 7, h = i & 1;
      cp_async16(Bm_s + ((sb * 2 + h) * 8 + n) * 16, (const uint8_t *)(a.xp.xsf + ((size_t)(sb0 + sb) * 8 + n) * 16) + h * 16);
    }
    if (tid < 8) *(uint4 *)(Bp + (size_t)nsl * 4096 + tid * 16) = make_uint4(0, 0, 0, 0);
    else if (tid < 16) *(uint4 *)(Bm + (size_t)nsl * 256 + (tid - 8) * 16) = make_uint4(0, 0, 0, 0);
    cp_async_commit();
    cp_async_wait<0>();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMAs read these bytes through the async proxy
  }
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (!worker) {
    // ---- four issuing warps: lane 0 of warp 16 + i feeds the tensor core sub-block pair i ---------
    if (lane == 0) {
      const int i4 = warp - G3_THREADS / 32;
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      int c_c = 0;
      for (int s = 0; s < n_items; s++) {
        const int buf = s & 1;
        if (!*dead && !mbar_wait(afull(buf), (uint32_t)(s >> 1) & 1u)) {
          *dead = 1;
          if (err) atomicExch(err, 1u);
        }
        t5_fence_after();
        const uint32_t abuf = tmem_base + (uint32_t)(buf * G3_A_COLS + 32 * i4), dbuf = tmem_base + (uint32_t)(G3_D0 + buf * G3_D_COLS + 24 * i4);
        const uint64_t bd = g3_desc(Bp_s + c_c * 4096 + i4 * 1024, 128, 128);   // + 8 per 128 bytes: the address field counts 16-byte units
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
          for (int u = 0; u < 2; u++) t5_mma_f16_ts(dbuf + 8 * h, abuf + 16 * h + 8 * u, bd + (uint64_t)((4 * h + 2 * u) * 8), G3_IDESC, u);
        if (i4 == 3) t5_mma_f16_ts(dbuf + 16, tmem_base + (uint32_t)(buf * G3_A_COLS + 128), g3_desc(Bm_s + c_c * 256, 128, 128), G3_IDESC, 0);
        t5_commit(dfull(buf));
        if (++c_c == nsl) c_c = 0;
      }
      // nothing of this CTA may still be running on the tensor core when its tensor memory is freed
      if (n_items > 0 && !*dead) mbar_wait(dfull((n_items - 1) & 1), (uint32_t)((n_items - 1) >> 1) & 1u);
    }
  } else {
    // ---- 512 workers: unpack super-block s into tensor memory, scale super-block s - 1 out of it ---
    const uint32_t lane_off = (uint32_t)(32 * q) << 16;
    float acc[8], accm[2] = {0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < 8; j++) acc[j] = 0.0f;
    float s0_p = 0.0f, s1_p = 0.0f, dm_p = 0.0f;
    int c_stage = 0;             // ring stage of the item being unpacked
    int e_tile = ci, e_c = 0;    // the item whose accumulators are read (one behind)
#pragma unroll 1
    for (int s = 0; s <= n_items; s++) {
      const int buf = s & 1;
      float s0 = 0.0f, s1 = 0.0f, dm = 0.0f;
      if (s < n_items) {
        cp_async_wait<G3_STAGES - 2>();   // this thread's pieces of item s have landed
        quarter_sync(q);                  // ... and those of the quarter's other three warps; they are done with item s - 1
        issue();                          // item s + G3_STAGES - 1 into the stage item s - 1 left
        const uint8_t *rowp = qring + (size_t)c_stage * G3_STAGE_BYTES + lane * 144;
        const uint4 hdr = *(const uint4 *)rowp, qa = *(const uint4 *)(rowp + 16 + 32 * c), qb = *(const uint4 *)(rowp + 32 + 32 * c);
        c_stage = c_stage + 1 == G3_STAGES ? 0 : c_stage + 1;
        uint32_t sc0, sc1, mn0, mn1;
        if (c < 2) {
          const uint32_t sv = hdr.y >> (16 * c), mv = hdr.z >> (16 * c);
          sc0 = sv & 63; sc1 = (sv >> 8) & 63; mn0 = mv & 63; mn1 = (mv >> 8) & 63;
        } else {
          const uint32_t hv = hdr.w >> (16 * (c - 2)), lo = hdr.y >> (16 * (c - 2)), mi = hdr.z >> (16 * (c - 2));
          sc0 = (hv & 15) | ((lo >> 2) & 0x30); sc1 = ((hv >> 8) & 15) | ((lo >> 10) & 0x30);
          mn0 = ((hv >> 4) & 15) | ((mi >> 2) & 0x30); mn1 = ((hv >> 12) & 15) | ((mi >> 10) & 0x30);
        }
        const float d = h2f_bits(hdr.x & 0xffffu), dmin = h2f_bits(hdr.x >> 16);
        s0 = d * (float)sc0 * TWO24; s1 = d * (float)sc1 * (TWO24 * 0.0625f); dm = dmin * 32.0f;
        const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const uint32_t w8 = w[i] >> 8;
          v[2 * i] = w[i] & 0x000f000fu; v[2 * i + 1] = w8 & 0x000f000fu;            // sub-block 2c: low nibbles
          v[16 + 2 * i] = w[i] & 0x00f000f0u; v[16 + 2 * i + 1] = w8 & 0x00f000f0u;  // sub-block 2c+1: high nibbles, x16
        }
        // A[buf] is free: this thread waited for the MMAs of item s - 2 when it read their accumulators
        const uint32_t abuf = tmem_base + lane_off + (uint32_t)(buf * G3_A_COLS);
        t5_st32(abuf + 32 * c, v);
        // the pair's mins as fp16 numbers (0x6400 | m is 1024 + m): m against the means' hi halves, m / 2048 against
        // their lo halves, which are stored times 2048
        const uint32_t mt = mn0 | (mn1 << 16) | 0x64006400u;
        t5_st2(abuf + 128 + 2 * c, g2_hfma2(mt, 0x3c003c00u, 0xe400e400u), g2_hfma2(mt, 0x10001000u, 0xb800b800u));
        t5_wait_st();
        t5_fence_before();
        __syncwarp();
        // also says: this warp has read the accumulators of item s - 2, whose buffer item s takes
        if (lane == 0) mbar_arrive(afull(buf));
      } else {
        cp_async_wait<0>();
      }
      if (s >= 1) {
        const int it = s - 1, eb = it & 1;
        if (!*dead && !mbar_wait(dfull(eb), (uint32_t)(it >> 1) & 1u)) {
          *dead = 1;
          if (err) atomicExch(err, 1u);
        }
        t5_fence_after();
        float v[16], vm[2];
        const uint32_t dcol = tmem_base + lane_off + (uint32_t)(G3_D0 + eb * G3_D_COLS);
        t5_ld16(dcol + 24 * c, v);
        t5_ld2(dcol + 88 + 2 * c, vm);
        t5_wait_ld();
        t5_fence_before();
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] += s0_p * v[j] + s1_p * v[8 + j];
        accm[0] += dm_p * vm[0];
        accm[1] += dm_p * vm[1];
        if (++e_c == nsl) {
          // tile done: the four threads of a row add up through shared memory
          // (the min term of a column is subtracted after the four partial sums are added, so that a
          // column's result does not depend on which column of the launch it is)
          float4 *rp = (float4 *)(red + ((size_t)c * 128 + r) * 8);
          rp[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
          rp[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
          *(float2 *)(red + (size_t)(4 * 128 + r) * 8 + 2 * c) = make_float2(accm[0], accm[1]);
          quarter_sync(q);
          if (c == 0) {
            float sum[8];
#pragma unroll
            for (int j = 0; j < 8; j++) sum[j] = 0.0f;
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
              const float4 x0 = *(const float4 *)(red + ((size_t)cc * 128 + r) * 8), x1 = *(const float4 *)(red + ((size_t)cc * 128 + r) * 8 + 4);
              sum[0] += x0.x; sum[1] += x0.y; sum[2] += x0.z; sum[3] += x0.w; sum[4] += x1.x; sum[5] += x1.y; sum[6] += x1.z; sum[7] += x1.w;
            }
            {
              const float4 m0 = *(const float4 *)(red + (size_t)(4 * 128 + r) * 8), m1 = *(const float4 *)(red + (size_t)(4 * 128 + r) * 8 + 4);
              sum[0] -= m0.x; sum[1] -= m0.y; sum[2] -= m0.z; sum[3] -= m0.w; sum[4] -= m1.x; sum[5] -= m1.y; sum[6] -= m1.z; sum[7] -= m1.w;
            }
            const int m = (e_tile >= t128[1]) + (e_tile >= t128[2]) + (e_tile >= t128[3]);
            const GemmMat &M = a.m[m];
            const int row = (e_tile - (m == 0 ? 0 : m == 1 ? t128[1] : m == 2 ? t128[2] : t128[3])) * 128 + r;
            if (row < M.rows) {
              float *out = M.out + (size_t)ks * M.split_stride;
#pragma unroll
              for (int t = 0; t < 8; t++) {
                if (t < a.T && (a.planes == 1 || t < 4)) {
                  const float val = a.planes == 2 ? sum[t & 3] + sum[4 + (t & 3)] * XP_LO_INV : sum[t];
                  out[(size_t)gemm_out_block(M, t) * M.ostride + row] = val;
                }
              }
            }
          }
          quarter_sync(q);   // the quarter's part of red is free again
#pragma unroll
          for (int j = 0; j < 8; j++) acc[j] = 0.0f;
          accm[0] = accm[1] = 0.0f;
          e_c = 0;
          e_tile += cps;
        }
      }
      s0_p = s0; s1_p = s1; dm_p = dm;
    }
  }
  t5_fence_before();
  __syncthreads();
  if (warp == 0) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)G3_TMEM_COLS) : "memory");
  }
}
