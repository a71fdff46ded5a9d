// pfmm.cuh -- the prompt path's dense GEMM on the fifth-generation tensor cores: Y[r][n] = sum_k W[n][k] X[r][k] for a
// chunk of up to PF_R = 256 prompt rows against Q4_K / Q5_K / Q6_K / Q8_0 weights.  It replaces, for this library, the
// reference's chunked tensor-core prefill GEMM (tools/pf27/pfmm.cuh:311-384: int8 mma.sync + cp.async on sm_86; its
// caller host/llb_pf.h:551 pf_take) with a design for sm_100a:
//
//   * the multiply is tcgen05.mma (kind::f16, M = 128 weight rows, N = 256 prompt rows, K = 16 per instruction), both
//     operands in shared memory, fp32 accumulators in TENSOR MEMORY;
//   * BOTH operands are two fp16 planes, hi = fp16(v) and lo = fp16((v - hi) * 2048) (about 22 bits of v, as the T-row
//     path's activation planes): a 16-column step is three MMAs, hi.hi into one accumulator of 256 columns and the
//     two cross terms hi.lo and lo.hi into another (together all 512 columns of tensor memory); the epilogue adds the
//     cross terms divided by 2048 (lo.lo is below fp32 resolution).  With one fp16 plane per operand every GEMM output carried a relative error of 4e-4, which a
//     random 8-layer model amplified past the path's 2e-2 bar;
//   * N = 256 because the kernel is bound by turning codes into fp16 planes (14.5 thread instructions per weight; with
//     N = 128 the tensor pipe was 40 % busy): a dequantised weight stage now serves twice the rows.  Measured on the
//     27B shape's gate|up launch: N = 128, three stages, three accumulators 174 us per 128 rows; two units of N = 128
//     per stage (four accumulators) 262 us per 256 rows; N = 256 238 us per 256 rows;
//   * the activation planes arrive by TMA: the chunk's activations are kept in global memory in the order the operand
//     wants (k-group major, common.cuh), so a 64-column stage of one plane is ONE contiguous 16 KB cp.async.bulk that
//     completes on an mbarrier (plain bulk copies of this GPU's own memory, no multicast);
//   * the weight planes are made on the fly: eight warps read the packed super-blocks (each thread one row's 32 weights
//     of a stage), dequantise in fp32 (the formulas of tools/qwen35_engine.c:233-307, one FMA per weight), split
//     each weight into its two planes and store 16-byte core-matrix rows; stores of a warp are conflict-free;
//   * a two-stage ring of (32 KB weights, 64 KB activations) with full / empty mbarriers decouples the roles, so
//     loads and dequantisation run ahead of the MMAs; four more warps read a finished tile out with tcgen05.ld.
//     (Separate rings -- three weight stages and four half-stages of 32 activation columns, which fit the same shared
//     memory -- were measured and dropped: the issuing threads then wait and commit twice as often, and a gate|up launch
//     took 319 us against 262 us);
//   * every wait is bounded: a wait that runs out sets *err, and all roles then run through without waiting, so the
//     kernel returns, frees its tensor memory and leaves the context usable (llb_b200_wait_errors() reports it).
#pragma once
#include "gemm.cuh"
#include "tc5.cuh"
#include "pf.cuh"

#define PF_KS 64              // columns per ring stage
#define PF_STAGES 2
#define PF_A_BYTES (128 * PF_KS * 2)     // one plane of 128 weight rows
#define PF_B_BYTES (PF_R * PF_KS * 2)    // one plane of one unit of the chunk's rows
#define PF_NUN (PF_RMAX / PF_R)   // units of a chunk
#define PF_STAGE_BYTES (2 * PF_A_BYTES + 2 * PF_NUN * PF_B_BYTES)   // [A hi | A lo | per unit: B hi | B lo]
#define PF_SMEM (1024 + PF_STAGES * PF_STAGE_BYTES)
#define PF_THREADS 512        // warps 0-7 dequantise, 8 loads activations, 9-11 issue MMAs, 12-15 write results
#define PF_IDESC (0x08000010u | ((uint32_t)(PF_R >> 3) << 17))  // kind::f16: D f32, A / B f16 K-major, N = PF_R, M = 128


__device__ __forceinline__ void pf_mma_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void pf_bulk_copy(uint32_t dst_s, const void *src, uint32_t bytes, uint32_t bar_s) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_s), "l"(src), "r"(bytes), "r"(bar_s)
               : "memory");
}

// ---- weights: packed super-blocks -> fp16 core-matrix rows ------------------------------------------
// A thread takes the 32 weights of one row that start at column c0 (a multiple of 32): raw words with pf_load, fp32
// values with pf_deq, then pf_split8 turns every eight of them into a 16-byte row of each plane (k-groups c0/8 .. + 3).
struct PfRaw { uint32_t w[8], x[8], h[4]; };

template <int FMT> __device__ __forceinline__ void pf_load(const uint8_t *row, int K, int c0, PfRaw &r) {
  if constexpr (FMT == LLB_FM_Q8_0) {
    const uint4 a = ldg128(row + c0), b = ldg128(row + c0 + 16);
    r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w; r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
    r.h[0] = *(const unsigned short *)(row + K + 2 * (c0 >> 5));
  } else if constexpr (FMT == LLB_FM_Q6_K) {
    const uint8_t *blk = row + (size_t)(c0 >> 8) * 224;
    const int j8 = (c0 >> 5) & 7, hf = j8 >> 2, qd = j8 & 3;
    const uint4 a = ldg128(blk + 64 * hf + 32 * (qd & 1)), b = ldg128(blk + 64 * hf + 32 * (qd & 1) + 16);
    const uint4 c = ldg128(blk + 128 + 32 * hf), d = ldg128(blk + 128 + 32 * hf + 16);
    r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w; r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
    r.x[0] = c.x; r.x[1] = c.y; r.x[2] = c.z; r.x[3] = c.w; r.x[4] = d.x; r.x[5] = d.y; r.x[6] = d.z; r.x[7] = d.w;
    r.h[0] = *(const unsigned short *)(blk + 192 + 8 * hf + 2 * qd);   // the two int8 scales of this quarter
    r.h[1] = *(const unsigned short *)(blk + 208);
  } else {
    constexpr int SB = FMT == LLB_FM_Q4_K ? 144 : 176, QOFF = FMT == LLB_FM_Q4_K ? 16 : 48;
    const uint8_t *blk = row + (size_t)(c0 >> 8) * SB;
    const int g = (c0 >> 6) & 3;
    const uint4 hd = ldg128(blk), a = ldg128(blk + QOFF + 32 * g), b = ldg128(blk + QOFF + 32 * g + 16);
    r.h[0] = hd.x; r.h[1] = hd.y; r.h[2] = hd.z; r.h[3] = hd.w;
    r.w[0] = a.x; r.w[1] = a.y; r.w[2] = a.z; r.w[3] = a.w; r.w[4] = b.x; r.w[5] = b.y; r.w[6] = b.z; r.w[7] = b.w;
    if constexpr (FMT == LLB_FM_Q5_K) {
      const uint4 c = ldg128(blk + 16), d = ldg128(blk + 32);
      r.x[0] = c.x; r.x[1] = c.y; r.x[2] = c.z; r.x[3] = c.w; r.x[4] = d.x; r.x[5] = d.y; r.x[6] = d.z; r.x[7] = d.w;
    }
  }
}

// An integer code c < 128 sitting in bits 16.. of a word becomes the float 128 + c by OR-ing 0x43000000 (no conversion
// instruction); one FMA then gives scale * c - offset: fmaf(128 + c, scale, -(128 scale + offset)).  The constant is rounded
// once per sub-block (about 1e-6 of a weight), instead of every weight being rounded twice as in the reference's
// d * sc * q - dmin * m; both planes together still carry the result to about 22 bits.
__device__ __forceinline__ float pf_code_f(uint32_t x, int j, uint32_t mask) {
  // byte j of x, masked, moved to bits 16..: shifts by 16, 8, 0, -8
  const uint32_t v = j == 0 ? x << 16 : j == 1 ? x << 8 : j == 2 ? x : x >> 8;
  return __uint_as_float((v & (mask << 16)) | 0x43000000u);
}

// the 32 weights as fp32
template <int FMT> __device__ __forceinline__ void pf_deq(const PfRaw &r, int c0, float (&w)[32]) {
  if constexpr (FMT == LLB_FM_Q8_0) {
    const float d = h2f_bits(r.h[0]), c = -384.0f * d;     // byte = q + 128, float = 256 + byte
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t x = r.w[i] ^ 0x80808080u;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const uint32_t v = j == 0 ? x << 15 : j == 1 ? x << 7 : j == 2 ? x >> 1 : x >> 9;
        w[4 * i + j] = fmaf(__uint_as_float((v & (0xffu << 15)) | 0x43800000u), d, c);
      }
    }
  } else if constexpr (FMT == LLB_FM_Q6_K) {
    const int qd = (c0 >> 5) & 3;
    const float d = h2f_bits(r.h[1]);
    const float s0 = __fmul_rn(d, (float)(int8_t)(r.h[0] & 0xff)), s1 = __fmul_rn(d, (float)(int8_t)(r.h[0] >> 8));
    const float k0 = -160.0f * s0, k1 = -160.0f * s1;      // (128 + code) - 160 = code - 32
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const uint32_t x = qd < 2 ? r.w[i] : r.w[i] >> 4, hb = (r.x[i] >> (2 * qd)) & 0x03030303u;
      const uint32_t c6 = (x & 0x0f0f0f0fu) | (hb << 4);   // four six-bit codes, one a byte
#pragma unroll
      for (int j = 0; j < 4; j++) w[4 * i + j] = fmaf(pf_code_f(c6, j, 0x3fu), i < 4 ? s0 : s1, i < 4 ? k0 : k1);
    }
  } else {
    const int j8 = (c0 >> 5) & 7, hi = j8 & 1;
    uint32_t scA, scB, mnA, mnB;
    k4_scales(r.h[1], r.h[2], r.h[3], scA, scB, mnA, mnB);
    const float sc = (float)(((j8 < 4 ? scA : scB) >> (8 * (j8 & 3))) & 0xffu), mn = (float)(((j8 < 4 ? mnA : mnB) >> (8 * (j8 & 3))) & 0xffu);
    const float ds = __fmul_rn(h2f_bits(r.h[0] & 0xffffu), sc), dm = __fmul_rn(h2f_bits(r.h[0] >> 16), mn);
    const float c = -fmaf(128.0f, ds, dm);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      uint32_t x = (hi ? r.w[i] >> 4 : r.w[i]) & 0x0f0f0f0fu;
      if constexpr (FMT == LLB_FM_Q5_K) x |= ((r.x[i] >> j8) & 0x01010101u) << 4;   // the fifth bit of column l is bit j8 of qh byte l
#pragma unroll
      for (int j = 0; j < 4; j++) w[4 * i + j] = fmaf(pf_code_f(x, j, 0x1fu), ds, c);
    }
  }
}
// eight weights -> one 16-byte row of the hi plane and one of the lo plane.  hi is the weight with its low 13 mantissa
// bits cleared (exactly an fp16 number for normal magnitudes), lo the exact remainder times 2048.
__device__ __forceinline__ void pf_split8(const float *w, uint4 &hi, uint4 &lo) {
  uint32_t h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const float a = w[2 * i], b = w[2 * i + 1];
    const float ah = __uint_as_float(__float_as_uint(a) & 0xffffe000u), bh = __uint_as_float(__float_as_uint(b) & 0xffffe000u);
    const __half2 hh = __floats2half2_rn(ah, bh), ll = __floats2half2_rn((a - ah) * XP_LO_SCALE, (b - bh) * XP_LO_SCALE);
    h[i] = *(const uint32_t *)&hh; l[i] = *(const uint32_t *)&ll;
  }
  hi = make_uint4(h[0], h[1], h[2], h[3]);
  lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// ---- the kernel ------------------------------------------------------------------------------------------------
// Work unit = (128-row tile, K-slice); CTA b takes units b, b + grid, ...  Every role walks the same unit sequence.
__device__ __forceinline__ void pf_locate(const PfArgs &a, int tile, int &m, int &row0) {
  m = 0;
  while (m + 1 < a.nmat && tile >= a.t128[m + 1]) m++;
  row0 = (tile - a.t128[m]) * 128;
}
// K-slices are whole super-blocks, as equal as they come: first column and 64-column stages of unit u
__device__ __forceinline__ void pf_slice(const PfArgs &a, int u, int ntiles, int &kbase, int &nst) {
  const int ks = u / ntiles, nsb = a.K >> 8;
  const int sb0 = (int)(((long long)ks * nsb) / a.ksplit), sb1 = (int)(((long long)(ks + 1) * nsb) / a.ksplit);
  kbase = sb0 << 8; nst = (sb1 - sb0) << 2;
}

template <int FMT>
__global__ void __launch_bounds__(PF_THREADS, 1) k_pfmm(const PfArgs a) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // header: full_a[4] +0, full_b[4] +32, empty[4] +64, acc_full +128, acc_empty +136, tensor-memory address +144, dead +148
  const uint32_t bar_s = smem_u32(smem);
  auto full_a = [&](int s) { return bar_s + 8u * (uint32_t)s; };
  auto full_b = [&](int s) { return bar_s + 32u + 8u * (uint32_t)s; };
  auto empty = [&](int s) { return bar_s + 64u + 8u * (uint32_t)s; };
  auto acc_full = [&](int b) { return bar_s + 128u + 8u * (uint32_t)b; };
  auto acc_empty = [&](int b) { return bar_s + 136u + 8u * (uint32_t)b; };
  uint32_t *tmem_slot = (uint32_t *)(smem + 144);
  volatile uint32_t *dead = (volatile uint32_t *)(smem + 148);
  uint8_t *ring = smem + 1024;
  const uint32_t ring_s = smem_u32(ring);
  const int ntiles = a.t128[a.nmat], nunits = ntiles * a.ksplit;
  const size_t rb = dev_row_bytes(FMT, a.K);
  const int nun = a.R > PF_R ? 2 : 1;   // units of PF_R rows in this chunk

  pdl_trigger();
  if (tid == 0) {
    for (int s = 0; s < PF_STAGES; s++) { mbar_init(full_a(s), 8); mbar_init(full_b(s), 1); mbar_init(empty(s), 3); }
    mbar_init(acc_full(0), 3); mbar_init(acc_empty(0), 4);
    *dead = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 10) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  pdl_wait();              // the activations come from the kernel in front
  t5_fence_before();
  __syncthreads();
  t5_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // a bounded wait that gives up for the whole CTA
  auto wait = [&](uint32_t bar, uint32_t parity) {
    if (*dead) return;
    if (!mbar_wait(bar, parity)) { *dead = 1; if (a.err) atomicExch(a.err, 1u); }
  };

  if (warp < 8) {
    // ---- weights: thread = (row r of the tile, half h of the stage's 64 columns) ----
    const int r = tid & 127, h = tid >> 7;
    PfRaw raw0, raw1;                                  // two stages of raw words in flight (never indexed: they stay in registers)
    int it = 0;                                        // stages produced so far by this CTA
    // the loads run two stages ahead of the conversion: cursor (lu, ls) is the stage to load next
    int lu = blockIdx.x, ls = 0, lkbase = 0, lnst = 0, lm = 0, lrow0 = 0;
    const uint8_t *lrow = nullptr;
    auto lplan = [&]() {
      if (lu < nunits) {
        pf_locate(a, lu % ntiles, lm, lrow0);
        pf_slice(a, lu, ntiles, lkbase, lnst);
        lrow = a.m[lm].W + (size_t)min(lrow0 + r, a.m[lm].rows - 1) * rb;
      }
    };
    auto lnext = [&](PfRaw &dst) {
      if (lu < nunits) {
        pf_load<FMT>(lrow, a.K, lkbase + ls * PF_KS + 32 * h, dst);
        if (++ls == lnst) { ls = 0; lu += gridDim.x; lplan(); }
      }
    };
    // converts the stage held in rw (columns c0 ..), refills rw with the stage two ahead, publishes the stage
    auto one = [&](PfRaw &rw, int c0) {
      const int slot = it % PF_STAGES;
      float w[32];
      pf_deq<FMT>(rw, c0, w);
      lnext(rw);
      if (it >= PF_STAGES) wait(empty(slot), (uint32_t)((it / PF_STAGES) + 1) & 1u);
      uint8_t *A = ring + (size_t)slot * PF_STAGE_BYTES;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        uint4 hi, lo;
        pf_split8(w + 8 * j, hi, lo);
        *(uint4 *)(A + ((size_t)(4 * h + j) * 128 + r) * 16) = hi;
        *(uint4 *)(A + PF_A_BYTES + ((size_t)(4 * h + j) * 128 + r) * 16) = lo;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads these bytes through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(full_a(slot));
      it++;
    };
    lplan();
    lnext(raw0);
    lnext(raw1);
    for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
      int kbase, nst;
      pf_slice(a, u, ntiles, kbase, nst);
      for (int s = 0; s < nst; s += 2) {               // nst is a multiple of four: a K-slice is whole super-blocks
        one(raw0, kbase + 32 * h + s * PF_KS);
        one(raw1, kbase + 32 * h + (s + 1) * PF_KS);
      }
    }
  } else if (warp == 8) {
    // ---- activations: one 16 KB bulk copy per unit, plane and stage ----
    if (lane == 0) {
      int it = 0;
      for (int u = blockIdx.x; u < nunits; u += gridDim.x) {
        int kbase, nst;
        pf_slice(a, u, ntiles, kbase, nst);
        for (int s = 0; s < nst; s++, it++) {
          const int slot = it % PF_STAGES;
          if (it >= PF_STAGES) wait(empty(slot), (uint32_t)((it / PF_STAGES) + 1) & 1u);
          if (*dead) continue;
          const __half *src = a.x + (size_t)((kbase + s * PF_KS) >> 3) * PF_R * 8;
          const uint32_t dst = ring_s + slot * PF_STAGE_BYTES + 2 * PF_A_BYTES;
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_b(slot)), "r"((uint32_t)(nun * 2 * PF_B_BYTES)) : "memory");
          for (int un = 0; un < nun; un++) {   // a unit's planes follow the previous unit's in global memory (common.cuh)
            const __half *su = src + (size_t)un * pf_kg_halves(a.K);
            pf_bulk_copy(dst + un * 2 * PF_B_BYTES, su, PF_B_BYTES, full_b(slot));
            pf_bulk_copy(dst + un * 2 * PF_B_BYTES + PF_B_BYTES, su + (size_t)a.K * PF_R, PF_B_BYTES, full_b(slot));
          }
        }
      }
    }
  } else if (warp >= 9 && warp < 12) {
    // ---- the tensor core.  Issuing one tcgen05.mma costs a thread 100 to 200 cycles, more than a 128 x 128 x 16 MMA
    // takes to execute, so the products of a step are spread over three threads; MMAs into one accumulator come from
    // one thread (a thread's MMAs execute in its issue order, MMAs of different threads would not be ordered):
    //   warp 9: hi.hi -> D1     warp 10: hi.lo and lo.hi -> D23     result = D1 + D23 / 2048
    //   (tensor-memory columns: D1 at 0, D23 at PF_R.  The code is written for PF_RMAX / PF_R units of PF_R rows, unit un
    //   with its pair of accumulators at 2 un PF_R and warp 10 + un issuing its cross terms; PF_R = 256 leaves one unit)
    if (lane == 0) {
      const int which = warp - 9;
      int it = 0, i = 0;
      for (int u = blockIdx.x; u < nunits; u += gridDim.x, i++) {
        int kbase, nst;
        pf_slice(a, u, ntiles, kbase, nst);
        if (i >= 1) wait(acc_empty(0), (uint32_t)(i - 1) & 1u);   // the previous tile has been read out of tensor memory
        t5_fence_after();
        for (int s = 0; s < nst; s++, it++) {
          const int slot = it % PF_STAGES;
          wait(full_a(slot), (uint32_t)(it / PF_STAGES) & 1u);
          wait(full_b(slot), (uint32_t)(it / PF_STAGES) & 1u);
          t5_fence_after();
          const uint32_t st = ring_s + slot * PF_STAGE_BYTES, b0 = st + 2 * PF_A_BYTES;
          const uint64_t a_hi = g3_desc(st, 2048, 128), a_lo = g3_desc(st + PF_A_BYTES, 2048, 128);
          if (!*dead) {
#pragma unroll
            for (int k = 0; k < PF_KS / 16; k++) {   // a step is two k-groups further on: the address field counts 16-byte units
              const uint64_t ka = (uint64_t)(k * 2 * 2048 / 16), kb = (uint64_t)(k * 2 * PF_R * 16 / 16);
              const uint32_t first = (s | k) != 0;
              if (which == 0) {
                for (int un = 0; un < nun; un++)
                  pf_mma_ss(tmem_base + (uint32_t)(un * 2 * PF_R), a_hi + ka, g3_desc(b0 + un * 2 * PF_B_BYTES, PF_R * 16, 128) + kb, PF_IDESC, first);
              } else if (which - 1 < nun) {
                const int un = which - 1;
                const uint32_t d = tmem_base + (uint32_t)(un * 2 * PF_R + PF_R);
                const uint64_t b_hi = g3_desc(b0 + un * 2 * PF_B_BYTES, PF_R * 16, 128) + kb, b_lo = g3_desc(b0 + un * 2 * PF_B_BYTES + PF_B_BYTES, PF_R * 16, 128) + kb;
                pf_mma_ss(d, a_hi + ka, b_lo, PF_IDESC, first);
                pf_mma_ss(d, a_lo + ka, b_hi, PF_IDESC, 1u);
              }
            }
          }
          t5_commit(empty(slot));        // arrives when this thread's MMAs have read the stage
        }
        t5_commit(acc_full(0));          // ... and when this thread's share of the tile is in tensor memory
      }
      // nothing of this CTA may still run on the tensor core when its tensor memory is freed
      if (i > 0) wait(acc_full(0), (uint32_t)(i - 1) & 1u);
    }
  } else if (warp >= 12) {
    // ---- results: lane quarter q of the accumulators, one weight row per thread ----
    const int q = warp - 12;
    int i = 0;
    for (int u = blockIdx.x; u < nunits; u += gridDim.x, i++) {
      int m, row0;
      pf_locate(a, u % ntiles, m, row0);
      const PfMat &M = a.m[m];
      const int row = row0 + 32 * q + lane;
      float *out = M.out + (size_t)(u / ntiles) * M.split_stride + row;
      wait(acc_full(0), (uint32_t)i & 1u);
      t5_fence_after();
      const uint32_t t0 = tmem_base + ((uint32_t)(32 * q) << 16);
      for (int c = 0; c < a.R; c += 16) {     // chunk rows c .. c + 15: unit c / 128, its columns c % 128 ..
        float v[16], v2[16];
        const uint32_t col = (uint32_t)((c / PF_R) * 2 * PF_R + (c % PF_R));
        t5_ld16(t0 + col, v);
        t5_ld16(t0 + col + PF_R, v2);
        t5_wait_ld();
        if (row < M.rows) {
#pragma unroll
          for (int j = 0; j < 16; j++)
            if (c + j < a.R) out[(size_t)(c + j) * M.ostride] = v[j] + v2[j] * XP_LO_INV;
        }
      }
      t5_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty(0));
    }
  }
  t5_fence_before();
  __syncthreads();
  if (warp == 10) {
    t5_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}
