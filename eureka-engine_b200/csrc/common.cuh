// common.cuh -- shared device helpers of the B200 speculative-decoding library.
//
// Weight formats are the reference's (host/llb_formats.h:4-15).  Device layouts:
//   Q8_0  as stored in a pack: row = [cols x int8][cols/32 x f16]          (tools/q8_pack.py:7-10)
//   Q4_K  as stored: 144-byte super-blocks                                  (tools/qwen35_engine.c:258-272)
//   Q5_K  as stored: 176-byte super-blocks                                  (tools/qwen35_engine.c:273-289)
//   Q6_K  re-sliced at load: each 210-byte super-block is padded to 224 bytes
//         [ql 128 | qh 64 | scales 16 | d 2 | zero 14] so that every super-block starts on a
//         16-byte boundary (the stored 210-byte stride does not); values are unchanged.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLB_FM_F32 0
#define LLB_FM_Q8_0 1
#define LLB_FM_Q4_K 3
#define LLB_FM_Q6_K 4
#define LLB_FM_Q5_K 9

// bytes of one row in the DEVICE layout
__host__ __device__ inline size_t dev_row_bytes(int fmt, int cols) {
  switch (fmt) {
    case LLB_FM_F32: return (size_t)cols * 4;
    case LLB_FM_Q8_0: return (size_t)cols / 32 * 34;
    case LLB_FM_Q4_K: return (size_t)cols / 256 * 144;
    case LLB_FM_Q5_K: return (size_t)cols / 256 * 176;
    case LLB_FM_Q6_K: return (size_t)cols / 256 * 224;
  }
  return 0;
}
// bytes of one row as stored in a pack (host/llb_formats.h:17)
__host__ __device__ inline size_t pack_row_bytes(int fmt, int cols) {
  return fmt == LLB_FM_Q6_K ? (size_t)cols / 256 * 210 : dev_row_bytes(fmt, cols);
}

// ---- activation planes -------------------------------------------------------------------------
// A GEMM reads its T <= 8 activation rows as fp16 "planes": column t (< NH) holds hi = fp16(x),
// column NH + t holds lo = fp16((x - hi) * 2048), NH = NC / 2, so hi + lo/2048 carries about 22
// bits of x.  NC is 8 (T <= 4) or 16 (T <= 8).  With planes == 1 all NC columns are independent
// rows (bf16/fp16 inputs that need no second plane).
//   xh   [NC][K]    fp16, K-index permuted inside every aligned group of 8: stored order
//                   0 2 1 3 4 6 5 7, which is the order the tensor-core B fragments consume
//   xs16 [K/16][NC] f32 sums of the fp16 values over 16 consecutive columns
//   xs32 [K/32][NC] f32 sums over 32 consecutive columns
//   xsf  [K/256][NC][16] fp16: the eight 32-column MEANS of a super-block as hi/lo pairs (hi = fp16(m),
//                   lo = fp16((m - hi) * 2048), like the planes), in the order the min-term MMA's B fragment
//                   reads them: for j = 0..3: hi(2j) hi(2j+1) lo(2j) lo(2j+1)
struct XPlanes {
  __half *xh;
  float *xs16;
  float *xs32;
  __half *xsf;
  int K;
  int NC;
};
__host__ __device__ inline size_t xp_bytes(int K, int NC) {
  return (size_t)NC * K * 2 + (size_t)(K / 16) * NC * 4 + (size_t)(K / 32) * NC * 4 + (size_t)(K / 256) * NC * 32;
}
__host__ __device__ inline XPlanes xp_carve(void *base, int K, int NC) {
  char *b = (char *)base;
  XPlanes xp;
  xp.xh = (__half *)b; b += (size_t)NC * K * 2;
  xp.xs16 = (float *)b; b += (size_t)(K / 16) * NC * 4;
  xp.xs32 = (float *)b; b += (size_t)(K / 32) * NC * 4;
  xp.xsf = (__half *)b;
  xp.K = K; xp.NC = NC;
  return xp;
}
#define XP_LO_SCALE 2048.0f
#define XP_LO_INV (1.0f / 2048.0f)

__host__ __device__ inline int xp_perm(int c) { return (c & ~7) | ((c & 4) | ((c & 1) << 1) | ((c & 2) >> 1)); }

// Warp-cooperative store of 32 consecutive columns (lane = column c0 + lane) of row t.
__device__ __forceinline__ void xp_store32(const XPlanes &xp, int t, int planes, int c0, float v, int lane) {
  int c = c0 + lane, NH = xp.NC >> 1;
  __half hi = __float2half_rn(v);
  float hif = __half2float(hi);
  float lof = 0.0f;
  xp.xh[(size_t)t * xp.K + xp_perm(c)] = hi;
  if (planes == 2) {
    __half lo = __float2half_rn((v - hif) * XP_LO_SCALE);
    lof = __half2float(lo);
    xp.xh[(size_t)(NH + t) * xp.K + xp_perm(c)] = lo;
  }
#pragma unroll
  for (int m = 1; m < 16; m <<= 1) {
    hif += __shfl_xor_sync(0xffffffffu, hif, m);
    lof += __shfl_xor_sync(0xffffffffu, lof, m);
  }
  float hi32 = hif + __shfl_xor_sync(0xffffffffu, hif, 16);
  float lo32 = lof + __shfl_xor_sync(0xffffffffu, lof, 16);
  if ((lane & 15) == 0) {
    xp.xs16[(size_t)(c >> 4) * xp.NC + t] = hif;
    if (planes == 2) xp.xs16[(size_t)(c >> 4) * xp.NC + NH + t] = lof;
  }
  if (lane == 0) {
    xp.xs32[(size_t)(c >> 5) * xp.NC + t] = hi32;
    if (planes == 2) xp.xs32[(size_t)(c >> 5) * xp.NC + NH + t] = lo32;
    const int b = (c >> 5) & 7;
    __half *f = xp.xsf + ((size_t)(c >> 8) * xp.NC + t) * 16 + 4 * (b >> 1) + (b & 1);
    float v = hi32 * 0.03125f;
    __half h1 = __float2half_rn(v);
    f[0] = h1; f[2] = __float2half_rn((v - __half2float(h1)) * XP_LO_SCALE);
    if (planes == 2) {
      f += (size_t)NH * 16;
      v = lo32 * 0.03125f;
      h1 = __float2half_rn(v);
      f[0] = h1; f[2] = __float2half_rn((v - __half2float(h1)) * XP_LO_SCALE);
    }
  }
}

// The same for a thread that holds FOUR consecutive columns c .. c+3 (c a multiple of 4) of row t; the eight
// lanes 8j .. 8j+7 of a warp must hold one aligned group of 32 columns.  `on` is false for a thread past
// the row's end (it still takes part in the shuffles).  Stored order inside the four: 0 2 1 3.
__device__ __forceinline__ void xp_store4(const XPlanes &xp, int t, int planes, int c, const float (&v)[4], int lane, bool on) {
  const int NH = xp.NC >> 1;
  __half hi[4];
  float hs = 0.0f, ls = 0.0f, hif[4];
#pragma unroll
  for (int i = 0; i < 4; i++) { hi[i] = __float2half_rn(on ? v[i] : 0.0f); hif[i] = __half2float(hi[i]); hs += hif[i]; }
  if (on) {
    const __half2 a = __halves2half2(hi[0], hi[2]), b = __halves2half2(hi[1], hi[3]);
    *(uint2 *)(xp.xh + (size_t)t * xp.K + c) = make_uint2(*(const uint32_t *)&a, *(const uint32_t *)&b);
  }
  if (planes == 2) {
    __half lo[4];
#pragma unroll
    for (int i = 0; i < 4; i++) { lo[i] = __float2half_rn(on ? (v[i] - hif[i]) * XP_LO_SCALE : 0.0f); ls += __half2float(lo[i]); }
    if (on) {
      const __half2 a = __halves2half2(lo[0], lo[2]), b = __halves2half2(lo[1], lo[3]);
      *(uint2 *)(xp.xh + (size_t)(NH + t) * xp.K + c) = make_uint2(*(const uint32_t *)&a, *(const uint32_t *)&b);
    }
  }
  hs += __shfl_xor_sync(0xffffffffu, hs, 1); ls += __shfl_xor_sync(0xffffffffu, ls, 1);
  hs += __shfl_xor_sync(0xffffffffu, hs, 2); ls += __shfl_xor_sync(0xffffffffu, ls, 2);
  const float h32 = hs + __shfl_xor_sync(0xffffffffu, hs, 4), l32 = ls + __shfl_xor_sync(0xffffffffu, ls, 4);
  if (!on) return;
  if ((lane & 3) == 0) {
    xp.xs16[(size_t)(c >> 4) * xp.NC + t] = hs;
    if (planes == 2) xp.xs16[(size_t)(c >> 4) * xp.NC + NH + t] = ls;
  }
  if ((lane & 7) == 0) {
    xp.xs32[(size_t)(c >> 5) * xp.NC + t] = h32;
    if (planes == 2) xp.xs32[(size_t)(c >> 5) * xp.NC + NH + t] = l32;
    const int b = (c >> 5) & 7;
    __half *f = xp.xsf + ((size_t)(c >> 8) * xp.NC + t) * 16 + 4 * (b >> 1) + (b & 1);
    float m = h32 * 0.03125f;
    __half h1 = __float2half_rn(m);
    f[0] = h1; f[2] = __float2half_rn((m - __half2float(h1)) * XP_LO_SCALE);
    if (planes == 2) {
      f += (size_t)NH * 16;
      m = l32 * 0.03125f;
      h1 = __float2half_rn(m);
      f[0] = h1; f[2] = __float2half_rn((m - __half2float(h1)) * XP_LO_SCALE);
    }
  }
}

// ---- activations of a prompt chunk ----------------------------------------------------------------
#define PF_R 256              // rows of a prompt chunk (= N of the dense GEMM's MMA, pfmm.cuh)
#define PF_RMAX 256           // ... of PF_RMAX / PF_R units multiplied against the same dequantised weight stage (one)
// Activations of a chunk for the dense GEMM, "k-group major", as two fp16 planes like the T-row planes: hi = fp16(x),
// lo = fp16((x - hi) * 2048), about 22 bits of x.  Element (row r, column k) of a [PF_R][K] matrix sits at half index
// ((k >> 3) * PF_R + r) * 8 + (k & 7) of its plane; the lo plane follows the hi plane (K * PF_R halves further on).  Eight
// consecutive columns of one row are one 16-byte core-matrix row, the PF_R rows of a k-group are contiguous (2 KB), and
// a 64-column stage of one plane is one contiguous run (32 KB).  A chunk of more than PF_R rows is two such matrices one after the other.
__host__ __device__ inline size_t pf_kg_halves(int K) { return (size_t)2 * K * PF_R; }
// four consecutive columns k .. k+3 (k a multiple of 4) of row r into both planes
__device__ __forceinline__ void pf_kg_store4(__half *x, int K, int r, int k, float v0, float v1, float v2, float v3) {
  if (r >= PF_R) { x += pf_kg_halves(K); r -= PF_R; }   // a second unit of a chunk follows the first
  const size_t i = ((size_t)(k >> 3) * PF_R + r) * 8 + (k & 4);
  const __half2 a = __floats2half2_rn(v0, v1), b = __floats2half2_rn(v2, v3);
  const float2 af = __half22float2(a), bf = __half22float2(b);
  const __half2 c = __floats2half2_rn((v0 - af.x) * XP_LO_SCALE, (v1 - af.y) * XP_LO_SCALE), d = __floats2half2_rn((v2 - bf.x) * XP_LO_SCALE, (v3 - bf.y) * XP_LO_SCALE);
  *(uint2 *)(x + i) = make_uint2(*(const uint32_t *)&a, *(const uint32_t *)&b);
  *(uint2 *)(x + (size_t)K * PF_R + i) = make_uint2(*(const uint32_t *)&c, *(const uint32_t *)&d);
}
// ---- programmatic dependent launch --------------------------------------------------------------
// Every kernel of a pass is launched with the programmatic-serialization attribute: the next kernel's
// CTAs may become resident while this one still runs, do whatever does not depend on it (a GEMM
// prefetches its first weight chunks), and park in pdl_wait() until this grid has completed and its
// writes are visible.  Each kernel calls pdl_trigger() first and pdl_wait() before its first
// dependent read or any global write, so completion order stays the launch order.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- small PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
// D += A(16x16, row) * B(16x8, col), fp16 inputs, fp32 accumulate
__device__ __forceinline__ void mma16816(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 ldg128(const void *p) { return __ldg((const uint4 *)p); }
__device__ __forceinline__ uint2 ldg64(const void *p) { return __ldg((const uint2 *)p); }
__device__ __forceinline__ float2 ldg_f2(const void *p) { return __ldg((const float2 *)p); }

__device__ __forceinline__ float h2f_bits(uint32_t h16) { return __half2float(__ushort_as_half((unsigned short)h16)); }

// ---- per-format scalar dequantisers (bit-exact with tools/qwen35_engine.c:233-307) -------------
// Each returns weight (row, c) of a matrix in DEVICE layout.  __fmul_rn/__fsub_rn keep the
// reference's one-rounding-per-operation arithmetic (no FMA contraction).
__device__ __forceinline__ void q4k_scale_min(const uint8_t *s, int j, int &sc, int &mn) {
  if (j < 4) { sc = s[j] & 63; mn = s[j + 4] & 63; }
  else { sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4); mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}
__device__ __forceinline__ float deq_elem(int fmt, const uint8_t *row, int cols, int c) {
  if (fmt == LLB_FM_F32) return ((const float *)row)[c];
  if (fmt == LLB_FM_Q8_0) {
    float d = h2f_bits(((const unsigned short *)(row + cols))[c >> 5]);
    return __fmul_rn((float)((const int8_t *)row)[c], d);
  }
  int b = c >> 8, i = c & 255;
  if (fmt == LLB_FM_Q4_K || fmt == LLB_FM_Q5_K) {
    const uint8_t *blk = row + (size_t)b * (fmt == LLB_FM_Q4_K ? 144 : 176);
    float d = h2f_bits(blk[0] | (blk[1] << 8)), dm = h2f_bits(blk[2] | (blk[3] << 8));
    int g = i >> 6, hi = (i >> 5) & 1, l = i & 31, sc, mn;
    q4k_scale_min(blk + 4, 2 * g + hi, sc, mn);
    const uint8_t *qs = blk + (fmt == LLB_FM_Q4_K ? 16 : 48);
    int q = hi ? (qs[32 * g + l] >> 4) : (qs[32 * g + l] & 15);
    if (fmt == LLB_FM_Q5_K) q += ((blk[16 + l] >> (2 * g + hi)) & 1) * 16;
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dm, (float)mn));
  }
  if (fmt == LLB_FM_Q6_K) {
    const uint8_t *blk = row + (size_t)b * 224;
    int hf = i >> 7, qd = (i >> 5) & 3, l = i & 31;
    uint8_t lq = blk[64 * hf + 32 * (qd & 1) + l];
    int nib = qd < 2 ? (lq & 15) : (lq >> 4);
    int code = (nib | (((blk[128 + 32 * hf + l] >> (2 * qd)) & 3) << 4)) - 32;
    float d = h2f_bits(blk[208] | (blk[209] << 8));
    float sc = (float)((const int8_t *)(blk + 192))[8 * hf + 2 * qd + (l >> 4)];
    return __fmul_rn(__fmul_rn(d, sc), (float)code);
  }
  return 0.0f;
}
