// gemm.cuh -- dequant-fused skinny GEMM: Y[t][r] = sum_c W[r][c] * x[t][c] for T <= 8 rows of
// activations against Q4_K / Q5_K / Q6_K / Q8_0 weights.  This is the weight-streaming term of the
// reference's T-row verify leaves (tools/payload-spec.patch:46-238: spec_q4v, spec_q8c, spec_q6v)
// re-designed for sm_100a:
//
//  * the quantised integers go to the tensor cores UNCONVERTED: a 4/5/6/8-bit code placed in the
//    low bits of an fp16 lane is the subnormal value code * 2^-24 (exact), so mma.m16n8k16 computes
//    sum(code * x) per 32- or 16-column scale group exactly in fp32; the group's scale and
//    min/offset are applied to that partial sum in fp32.  No weight is ever rounded;
//  * activations are fp16 hi/lo planes (common.cuh), T <= 4 rows fill the n = 8 tile exactly;
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
};

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

template <int FMT> struct FmtTraits;
template <> struct FmtTraits<LLB_FM_Q4_K> { enum { SB = 144, RS = 288, STAGES = 4 }; };
template <> struct FmtTraits<LLB_FM_Q5_K> { enum { SB = 176, RS = 352, STAGES = 4 }; };
template <> struct FmtTraits<LLB_FM_Q6_K> { enum { SB = 224, RS = 480, STAGES = 3 }; };
template <> struct FmtTraits<LLB_FM_Q8_0> { enum { SB = 272, RS = 544, STAGES = 3 }; };  // 256 int8 + 16 B of scales


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

// ---- one chunk (<= 2 super-blocks = 512 columns) of a 16-row tile ------------------------------
// st: this warp's stage, rows at stride RS; kc0: first column of the chunk; acc[nt][4]: the C
// fragment (rows gid, gid+8; columns 2j, 2j+1 of n-tile nt).
template <int FMT, int NT>
__device__ __forceinline__ void consume_chunk(const uint8_t *st, int csb, int kc0, const GemmArgs &a, float (&acc)[NT][4],
                                              int lane) {
  const int gid = lane >> 2, j = lane & 3;
  const int K = a.K, NC = a.xp.NC;
  const __half *xh = a.xp.xh;
  constexpr int RS = FmtTraits<FMT>::RS;
  const uint8_t *r0 = st + gid * RS, *r1 = r0 + 8 * RS;

  if constexpr (FMT == LLB_FM_Q4_K || FMT == LLB_FM_Q5_K) {
    constexpr int SB = FmtTraits<FMT>::SB;
    constexpr int QOFF = FMT == LLB_FM_Q4_K ? 16 : 48;
    for (int sb = 0; sb < csb; sb++) {
      const uint8_t *b0 = r0 + sb * SB, *b1 = r1 + sb * SB;
      uint4 h0 = *(const uint4 *)b0, h1 = *(const uint4 *)b1;
      uint32_t scA0, scB0, mnA0, mnB0, scA1, scB1, mnA1, mnB1;
      k4_scales(h0.y, h0.z, h0.w, scA0, scB0, mnA0, mnB0);
      k4_scales(h1.y, h1.z, h1.w, scA1, scB1, mnA1, mnB1);
      float sS[NT][4], sM[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) sS[nt][i] = sM[nt][i] = 0.0f;
      uint32_t qh0 = 0, qh1 = 0, qh0b = 0, qh1b = 0;
      if constexpr (FMT == LLB_FM_Q5_K) {
        uint2 t0 = *(const uint2 *)(b0 + 16 + 8 * j), t1 = *(const uint2 *)(b1 + 16 + 8 * j);
        qh0 = t0.x; qh0b = t0.y; qh1 = t1.x; qh1b = t1.y;
      }
#pragma unroll
      for (int g = 0; g < 4; g++) {
        uint2 a0 = *(const uint2 *)(b0 + QOFF + 32 * g + 8 * j), a1 = *(const uint2 *)(b1 + QOFF + 32 * g + 8 * j);
        const int kc = kc0 + sb * 256 + 64 * g;
        // fifth bits (Q5_K): bit 2g of qh byte l belongs to the low nibble's column, bit 2g+1 to the high one
        uint32_t f0l = 0, f0h = 0, f1l = 0, f1h = 0, f0lb = 0, f0hb = 0, f1lb = 0, f1hb = 0;
        if constexpr (FMT == LLB_FM_Q5_K) {
          f0l = (qh0 >> (2 * g)) & 0x01010101u; f0h = (qh0 >> (2 * g + 1)) & 0x01010101u;
          f1l = (qh1 >> (2 * g)) & 0x01010101u; f1h = (qh1 >> (2 * g + 1)) & 0x01010101u;
          f0lb = (qh0b >> (2 * g)) & 0x01010101u; f0hb = (qh0b >> (2 * g + 1)) & 0x01010101u;
          f1lb = (qh1b >> (2 * g)) & 0x01010101u; f1hb = (qh1b >> (2 * g + 1)) & 0x01010101u;
        }
        const float sc0l = byte_f(g < 2 ? scA0 : scB0, (2 * g) & 3), sc0h = byte_f(g < 2 ? scA0 : scB0, (2 * g + 1) & 3);
        const float sc1l = byte_f(g < 2 ? scA1 : scB1, (2 * g) & 3), sc1h = byte_f(g < 2 ? scA1 : scB1, (2 * g + 1) & 3);
        const float mn0l = byte_f(g < 2 ? mnA0 : mnB0, (2 * g) & 3), mn0h = byte_f(g < 2 ? mnA0 : mnB0, (2 * g + 1) & 3);
        const float mn1l = byte_f(g < 2 ? mnA1 : mnB1, (2 * g) & 3), mn1h = byte_f(g < 2 ? mnA1 : mnB1, (2 * g + 1) & 3);
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          const __half *xr = xh + (size_t)(nt * 8 + gid) * K + kc + 8 * j;
          uint4 bl = ldg128(xr), bh = ldg128(xr + 32);
          float pl[4] = {0.f, 0.f, 0.f, 0.f}, ph[4] = {0.f, 0.f, 0.f, 0.f};
          // low nibbles: columns kc + 8j + {0,2 | 1,3} then {4,6 | 5,7}; code * 2^-24
          mma16816(pl, (a0.x & 0x000f000fu) | ((f0l & 0x00010001u) << 4), (a1.x & 0x000f000fu) | ((f1l & 0x00010001u) << 4),
                   ((a0.x >> 8) & 0x000f000fu) | (((f0l >> 8) & 0x00010001u) << 4),
                   ((a1.x >> 8) & 0x000f000fu) | (((f1l >> 8) & 0x00010001u) << 4), bl.x, bl.y);
          mma16816(pl, (a0.y & 0x000f000fu) | ((f0lb & 0x00010001u) << 4), (a1.y & 0x000f000fu) | ((f1lb & 0x00010001u) << 4),
                   ((a0.y >> 8) & 0x000f000fu) | (((f0lb >> 8) & 0x00010001u) << 4),
                   ((a1.y >> 8) & 0x000f000fu) | (((f1lb >> 8) & 0x00010001u) << 4), bl.z, bl.w);
          // high nibbles: columns kc + 32 + ...; code * 16 * 2^-24
          mma16816(ph, (a0.x & 0x00f000f0u) | ((f0h & 0x00010001u) << 8), (a1.x & 0x00f000f0u) | ((f1h & 0x00010001u) << 8),
                   ((a0.x >> 8) & 0x00f000f0u) | (((f0h >> 8) & 0x00010001u) << 8),
                   ((a1.x >> 8) & 0x00f000f0u) | (((f1h >> 8) & 0x00010001u) << 8), bh.x, bh.y);
          mma16816(ph, (a0.y & 0x00f000f0u) | ((f0hb & 0x00010001u) << 8), (a1.y & 0x00f000f0u) | ((f1hb & 0x00010001u) << 8),
                   ((a0.y >> 8) & 0x00f000f0u) | (((f0hb >> 8) & 0x00010001u) << 8),
                   ((a1.y >> 8) & 0x00f000f0u) | (((f1hb >> 8) & 0x00010001u) << 8), bh.z, bh.w);
          const float *xs = a.xp.xs32 + (size_t)(kc >> 5) * NC + nt * 8 + 2 * j;
          float2 xl = ldg_f2(xs), xhh = ldg_f2(xs + NC);
          sS[nt][0] += sc0l * pl[0] + (sc0h * 0.0625f) * ph[0];
          sS[nt][1] += sc0l * pl[1] + (sc0h * 0.0625f) * ph[1];
          sS[nt][2] += sc1l * pl[2] + (sc1h * 0.0625f) * ph[2];
          sS[nt][3] += sc1l * pl[3] + (sc1h * 0.0625f) * ph[3];
          sM[nt][0] += mn0l * xl.x + mn0h * xhh.x;
          sM[nt][1] += mn0l * xl.y + mn0h * xhh.y;
          sM[nt][2] += mn1l * xl.x + mn1h * xhh.x;
          sM[nt][3] += mn1l * xl.y + mn1h * xhh.y;
        }
      }
      const float d0 = h2f_bits(h0.x & 0xffffu) * TWO24, dm0 = h2f_bits(h0.x >> 16);
      const float d1 = h2f_bits(h1.x & 0xffffu) * TWO24, dm1 = h2f_bits(h1.x >> 16);
#pragma unroll
      for (int nt = 0; nt < NT; nt++) {
        acc[nt][0] += d0 * sS[nt][0] - dm0 * sM[nt][0];
        acc[nt][1] += d0 * sS[nt][1] - dm0 * sM[nt][1];
        acc[nt][2] += d1 * sS[nt][2] - dm1 * sM[nt][2];
        acc[nt][3] += d1 * sS[nt][3] - dm1 * sM[nt][3];
      }
    }
  } else if constexpr (FMT == LLB_FM_Q8_0) {
    // per 256 columns: 256 int8 at r + sb*256, their 8 f16 scales at r + 512 + sb*16
    for (int sb = 0; sb < csb; sb++) {
#pragma unroll
      for (int b = 0; b < 8; b++) {
        uint2 a0 = *(const uint2 *)(r0 + sb * 256 + 32 * b + 8 * j), a1 = *(const uint2 *)(r1 + sb * 256 + 32 * b + 8 * j);
        a0.x ^= 0x80808080u; a0.y ^= 0x80808080u; a1.x ^= 0x80808080u; a1.y ^= 0x80808080u;  // code = q + 128
        const float d0 = h2f_bits(*(const unsigned short *)(r0 + 512 + sb * 16 + 2 * b));
        const float d1 = h2f_bits(*(const unsigned short *)(r1 + 512 + sb * 16 + 2 * b));
        const int kc = kc0 + sb * 256 + 32 * b;
#pragma unroll
        for (int nt = 0; nt < NT; nt++) {
          uint4 bx = ldg128(xh + (size_t)(nt * 8 + gid) * K + kc + 8 * j);
          float p[4] = {0.f, 0.f, 0.f, 0.f};
          mma16816(p, __byte_perm(a0.x, 0, 0x4240), __byte_perm(a1.x, 0, 0x4240), __byte_perm(a0.x, 0, 0x4341),
                   __byte_perm(a1.x, 0, 0x4341), bx.x, bx.y);
          mma16816(p, __byte_perm(a0.y, 0, 0x4240), __byte_perm(a1.y, 0, 0x4240), __byte_perm(a0.y, 0, 0x4341),
                   __byte_perm(a1.y, 0, 0x4341), bx.z, bx.w);
          float2 xs = ldg_f2(a.xp.xs32 + (size_t)(kc >> 5) * NC + nt * 8 + 2 * j);
          acc[nt][0] += d0 * (p[0] * TWO24 - 128.0f * xs.x);
          acc[nt][1] += d0 * (p[1] * TWO24 - 128.0f * xs.y);
          acc[nt][2] += d1 * (p[2] * TWO24 - 128.0f * xs.x);
          acc[nt][3] += d1 * (p[3] * TWO24 - 128.0f * xs.y);
        }
      }
    }
  } else {  // Q6_K, 224-byte device super-blocks
    for (int sb = 0; sb < csb; sb++) {
      const uint8_t *b0 = r0 + sb * 224, *b1 = r1 + sb * 224;
      const float d0 = h2f_bits(*(const unsigned short *)(b0 + 208)), d1 = h2f_bits(*(const unsigned short *)(b1 + 208));
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
          // 16 columns l = 16u + 4j + {0..3} of each quarter qd of this half
          const int o = 16 * u + 4 * j;
          const uint32_t la0 = *(const uint32_t *)(b0 + 64 * hf + o), lb0 = *(const uint32_t *)(b0 + 64 * hf + 32 + o);
          const uint32_t la1 = *(const uint32_t *)(b1 + 64 * hf + o), lb1 = *(const uint32_t *)(b1 + 64 * hf + 32 + o);
          const uint32_t hq0 = *(const uint32_t *)(b0 + 128 + 32 * hf + o), hq1 = *(const uint32_t *)(b1 + 128 + 32 * hf + o);
#pragma unroll
          for (int qd = 0; qd < 4; qd++) {
            const uint32_t l0 = (qd & 1) ? lb0 : la0, l1 = (qd & 1) ? lb1 : la1;
            // code (0..63) in fp16 lanes: quarters 0,1 -> code * 2^-24; quarters 2,3 -> 16 * code * 2^-24
            const uint32_t nm = qd < 2 ? 0x000f000fu : 0x00f000f0u, hm = qd < 2 ? 0x00300030u : 0x03000300u;
            const int hs = 4 - 2 * (qd & 1);  // qd 0,2: qh << 4 ; qd 1,3: qh << 2 (after the quarter's own >> 2qd, << 4|8)
            const uint32_t e0 = (l0 & nm) | ((hq0 << hs) & hm), e1 = (l1 & nm) | ((hq1 << hs) & hm);
            const uint32_t o0 = ((l0 >> 8) & nm) | (((hq0 >> 8) << hs) & hm), o1 = ((l1 >> 8) & nm) | (((hq1 >> 8) << hs) & hm);
            const float w = qd < 2 ? TWO24 : TWO24 * 0.0625f;
            const float s0 = d0 * (float)((const int8_t *)(b0 + 192))[8 * hf + 2 * qd + u];
            const float s1 = d1 * (float)((const int8_t *)(b1 + 192))[8 * hf + 2 * qd + u];
            const int kc = kc0 + sb * 256 + 128 * hf + 32 * qd + 16 * u;
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
              uint2 bx = ldg64(xh + (size_t)(nt * 8 + gid) * K + kc + 4 * j);
              float p[4] = {0.f, 0.f, 0.f, 0.f};
              mma16816(p, e0, e1, o0, o1, bx.x, bx.y);
              float2 xs = ldg_f2(a.xp.xs16 + (size_t)(kc >> 4) * NC + nt * 8 + 2 * j);
              acc[nt][0] += s0 * (p[0] * w - 32.0f * xs.x);
              acc[nt][1] += s0 * (p[1] * w - 32.0f * xs.y);
              acc[nt][2] += s1 * (p[2] * w - 32.0f * xs.x);
              acc[nt][3] += s1 * (p[3] * w - 32.0f * xs.y);
            }
          }
        }
      }
    }
  }
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
    float lo[4];
    if constexpr (NT == 1) {
#pragma unroll
      for (int i = 0; i < 4; i++) lo[i] = __shfl_xor_sync(0xffffffffu, acc[0][i], 2);
    } else {
#pragma unroll
      for (int i = 0; i < 4; i++) lo[i] = acc[NT - 1][i];
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int t = 2 * j + (i & 1), r = row0 + gid + ((i >> 1) << 3);
      on[0][i] = (NT == 2 || j < 2) && t < a.T && r < M.rows;
      if (on[0][i]) { idx[0][i] = (size_t)(M.tok_slot ? M.tok_slot[t] : t) * M.ostride + r; val[0][i] = acc[0][i] + lo[i] * XP_LO_INV; }
    }
  } else {
#pragma unroll
    for (int nt = 0; nt < NT; nt++)
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int t = nt * 8 + 2 * j + (i & 1), r = row0 + gid + ((i >> 1) << 3);
        on[nt][i] = t < a.T && r < M.rows;
        if (on[nt][i]) { idx[nt][i] = (size_t)(M.tok_slot ? M.tok_slot[t] : t) * M.ostride + r; val[nt][i] = acc[nt][i]; }
      }
  }
  float *out = M.out + (size_t)ks * M.split_stride;
#pragma unroll
  for (int nt = 0; nt < NT; nt++)
#pragma unroll
    for (int i = 0; i < 4; i++) if (on[nt][i]) out[idx[nt][i]] = val[nt][i];
}
