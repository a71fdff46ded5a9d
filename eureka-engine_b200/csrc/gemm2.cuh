// gemm2.cuh -- second-generation skinny GEMM for the 4/5-bit K-quants (Q4_K, Q5_K), the formats that
// carry most of a Q4_K_M model's bytes.  Same arithmetic as gemm.cuh (integer codes as fp16
// subnormals into mma.m16n8k16, scales applied to fp32 partial sums); what changes is everything
// around the MMAs, driven by the first kernel's profile (issue-bound at 670 instructions per
// 16-row x 256-column tile-super-block, activation loads waiting on L1/L2):
//
//  * a CTA owns ONE K-slice and stages that slice of the activation planes in shared memory once;
//    all B-fragment reads are then conflict-free LDS.128 (column stride = 64 mod 128 bytes);
//  * 16 warps per SM, one-super-block stages, three-deep private cp.async rings
//    (row stride 160 / 224 bytes = 32 / 96 mod 128: conflict-free 8-byte A-fragment reads);
//  * the copy issue loop has no division and no per-piece address arithmetic beyond one add;
//  * the Q4_K "min" term  dmin * sum_b m_b * sum(x in sub-block b)  is ONE extra MMA per
//    tile-super-block: A = the eight 6-bit mins as fp16 numbers (m against the means' hi halves,
//    m / 2048 against their lo halves), B = the sub-block activation means as fp16 hi/lo pairs
//    prepared with the planes;
//  * first MMAs of a sub-block take a zero C operand instead of zeroing registers.
#pragma once
#include "gemm.cuh"

#ifndef G2_STAGES
#define G2_STAGES 3
#endif
// CTAs per SM.  With 2, two half-size CTAs (8 warps, at most half the shared memory) share an SM, so
// that the CTAs of the next GEMM (programmatic dependent launch) can take the place of draining ones
// and fill their weight rings early.  Measured on the 27B shape: the gate|up GEMM 30.4 us against
// 27.9 us with one CTA, the verify pass 8.08 ms against 7.94 ms -- so the default stays 1.
#ifndef G2_CPSM
#define G2_CPSM 1
#endif
#define G2_SMEM_MAX ((233472 - 1024 * G2_CPSM) / G2_CPSM / 128 * 128)   // 228 KB per SM, 1 KB reserved per CTA

// SB bytes per super-block, RS ring row stride, P 16-byte pieces per row-super-block, WARPS per CTA,
// XPAD: padding of a plane column in shared memory (column stride = 64 mod 128 bytes for the 16-byte
// B reads of Q4_K/Q5_K, 32 mod 128 for the 8-byte ones of Q6_K), AUX: bytes per (super-block, column)
// of the side array (Q4_K/Q5_K: 16 fp16 sub-block means; Q6_K: 16 f32 sums of 16 columns)
template <int FMT> struct G2Traits;
template <> struct G2Traits<LLB_FM_Q4_K> { enum { SB = 144, RS = 160, P = 9, QOFF = 16, WARPS = 16 / G2_CPSM, XPAD = 64, AUX = 32 }; };
template <> struct G2Traits<LLB_FM_Q5_K> { enum { SB = 176, RS = 224, P = 11, QOFF = 48, WARPS = 16 / G2_CPSM, XPAD = 64, AUX = 32 }; };
template <> struct G2Traits<LLB_FM_Q6_K> { enum { SB = 224, RS = 240, P = 14, QOFF = 0, WARPS = 16 / G2_CPSM, XPAD = 32, AUX = 64 }; };
// Q8_0 rows are [K x int8][K/32 x f16]: a "super-block" here is 256 codes plus their 8 scales, which sit K - 256 sb + 16 sb
// bytes further on in the row; piece 16 of a row-super-block is that scale piece (copy plan below).  AUX: 8 f32 sums of 32 columns.
template <> struct G2Traits<LLB_FM_Q8_0> { enum { SB = 256, RS = 304, P = 17, QOFF = 0, WARPS = 8 / G2_CPSM, XPAD = 32, AUX = 32 }; };

// Warps of a CTA: the format's count, but eight at 32 plane columns (16 rows, four n-tiles).  Sixteen warps cap a thread
// at 128 registers, and four n-tiles of accumulators, scale sums and min-term products do not fit in them: the 16-row
// kernel spilled (40 bytes of stores, 120 of loads per thread and super-block) and spent its time waiting on local
// memory (long-scoreboard stalls 1.3 per issue, 830 instructions per tile-super-block against 397 at 4 rows, tensor pipe
// 34 % busy).  Eight warps get 255 registers and a ring half the size, which also leaves the activation slice more room.
// sel: the routed-expert launches at 32 plane columns, which multiply a weight tile with two of the four staged n-tiles
// (g2_phase's NTC = 2) and so need the registers of the two-n-tile kernel only: more warps (the eight-warp launch left its
// schedulers two warps each and half their issue slots empty), two-deep rings so that the 32 staged columns of a whole
// d = 2048 K-slice (139 KB) still fit beside them.
template <int FMT> __host__ __device__ constexpr int g2_warps(int NC, bool sel = false) {
  if (sel && NC >= 32 && G2_CPSM == 1) return FMT == LLB_FM_Q4_K ? 16 : FMT == LLB_FM_Q5_K ? 12 : 8;
  return NC >= 32 && G2Traits<FMT>::WARPS > 8 ? 8 : G2Traits<FMT>::WARPS;
}
template <int FMT> __host__ __device__ constexpr int g2_stages(int NC, bool sel = false) { return sel && NC >= 32 && G2_CPSM == 1 ? 2 : G2_STAGES; }
template <int FMT> __host__ __device__ constexpr int g2_ring_bytes(int NC, bool sel = false) {
  return g2_warps<FMT>(NC, sel) * g2_stages<FMT>(NC, sel) * 16 * G2Traits<FMT>::RS;
}
// bytes of shared memory a K-slice of nsl super-blocks needs for NC activation columns
template <int FMT> __host__ __device__ inline int g2_xp_bytes(int nsl, int NC) {
  return NC * (nsl * 512 + G2Traits<FMT>::XPAD) + nsl * NC * G2Traits<FMT>::AUX;
}
template <int FMT> inline int g2_max_slice_sb(int NC, bool sel = false) {
  int left = G2_SMEM_MAX - g2_ring_bytes<FMT>(NC, sel) - NC * G2Traits<FMT>::XPAD;
  return left / (NC * 512 + NC * G2Traits<FMT>::AUX);
}

// D = A*B with a zero C operand
__device__ __forceinline__ void mma16816_z(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
               : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

// One GEMM launch's work of a CTA (bid of cps * ksplit): fill the ring, call stage(xh_s, xsf_s, CS, sb0, nsl) --
// which waits for whatever produces the activations, puts the CTA's slice of the planes and its side array into
// shared memory and ends with a block-wide barrier --, then stream the CTA's tiles.  Warps beyond the format's
// count and CTAs beyond the launch's only take part in the staging step's barriers.
// Where a launch's row tiles live.  A policy says how many 16-row tiles there are, where tile i's rows and
// the super-blocks of the CTA's K-slice start, and what to do with a finished tile.  G2MatsPlain is the
// launch of up to four matrices that GemmArgs describes; the routed-expert launches (moe.cuh) find their
// matrices through the expert ids an earlier kernel chose.
//   EARLY   the weight addresses depend on no earlier kernel: the ring's prologue is issued before the wait
//   Cur     per-thread cursor of the tile being copied
//   locate  tile -> first row, row count, cursor;  src: row 0 of super-block (sb0 + c) of the slice
template <int FMT> struct G2MatsPlain {
  static constexpr bool EARLY = true;
  const GemmArgs &a;
  struct Cur { const uint8_t *W, *W0; };   // first code of the slice in row 0 of the matrix; the matrix itself
  __device__ __forceinline__ int ntiles() const { return a.tile0[a.nmat]; }
  __device__ __forceinline__ size_t row_bytes() const { return dev_row_bytes(FMT, a.K); }
  __device__ __forceinline__ void locate(int tile, int sb0, Cur &c, int &row0, int &rows) const {
    int m = 0;
    while (m + 1 < a.nmat && tile >= a.tile0[m + 1]) m++;
    row0 = (tile - a.tile0[m]) * 16; rows = a.m[m].rows;
    c.W0 = a.m[m].W;
    c.W = c.W0 + (size_t)sb0 * G2Traits<FMT>::SB;
  }
  __device__ __forceinline__ const uint8_t *src(const Cur &c, int sb0, int pc) const { return c.W + (size_t)pc * G2Traits<FMT>::SB; }
  template <int NT> __device__ __forceinline__ void epilogue(int ks, int tile, float (&acc)[NT][4], int lane) const {
    int m = 0;
    while (m + 1 < a.nmat && tile >= a.tile0[m + 1]) m++;
    gemm_epilogue<NT>(a, a.m[m], ks, tile, (tile - a.tile0[m]) * 16, acc, lane);
  }
};

// NTC < NT (the routed-expert launches at 16 rows): a weight tile is multiplied with NTC = 2 of the NT staged n-tiles only,
// the hi and lo tiles of the eight rows its own row is among (Mats::col0(tile) = first plane column of the hi tile; the
// lo tile is NC / 2 columns on), since the epilogue keeps one row of the tile.
template <int FMT, int NT, class Stage, class Mats, int NTC = NT>
__device__ __forceinline__ void g2_phase(const GemmArgs &a, const int cps, const int bid, uint8_t *smem, Stage stage, const Mats mats) {
  using TR = G2Traits<FMT>;
  constexpr int NC = 8 * NT, RS = TR::RS, SB = TR::SB, P = TR::P, NIT = (16 * P + 31) / 32, G2_WARPS = g2_warps<FMT>(8 * NT, NTC != NT), ST = g2_stages<FMT>(8 * NT, NTC != NT);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, gid = lane >> 2, j = lane & 3;
  const bool live = bid < cps * a.ksplit && warp < G2_WARPS;
  const int ks = bid % a.ksplit, ci = bid / a.ksplit;
  const int sb0 = (int)(((long long)ks * a.nsb) / a.ksplit), nsl = (int)(((long long)(ks + 1) * a.nsb) / a.ksplit) - sb0;
  const int CS = nsl * 512 + TR::XPAD;
  uint8_t *xh_s = smem, *xsf_s = smem + NC * CS, *ring = xsf_s + nsl * NC * TR::AUX + (size_t)warp * ST * 16 * RS;
  const uint32_t ring_s = smem_u32(ring);
  int ntiles = live && Mats::EARLY ? mats.ntiles() : 0;   // a warp that is not live sees no tiles
  const int nws = cps * G2_WARPS;
  const size_t rb = mats.row_bytes();

  // per-lane copy plan: piece i = lane + 32*it of the 16 x P sixteen-byte pieces of a stage
  uint32_t dst_rel[NIT], row_of[NIT], pc_of[NIT];
  bool is_sc[NIT];
#pragma unroll
  for (int it = 0; it < NIT; it++) {
    is_sc[it] = false;
    const int i = lane + 32 * it, r = i / P, p = i - r * P;
    row_of[it] = r; pc_of[it] = p * 16; dst_rel[it] = i < 16 * P ? r * RS + p * 16 : 0xffffffffu;
    // Q8_0: the scale piece comes from the row's scale area (K bytes into the row) and advances 16 bytes per
    // super-block, not 256; its source is taken from the row start, not from the slice's first code
    if (FMT == LLB_FM_Q8_0 && p == P - 1) { pc_of[it] = (uint32_t)a.K + (uint32_t)sb0 * 16; is_sc[it] = true; }
  }
  // producer cursor
  // tile of (CTA ci, warp w, round n) = (n * WARPS + w) * cps + ci: consecutive tiles go to different SMs, so the
  // SMs' tile counts differ by one at most (the kernel is issue-bound per SM: time follows the fullest SM)
  int p_tile = warp * cps + ci, p_c = 0;
  typename Mats::Cur p_cur;
  uint32_t p_off[NIT];
  auto plan_tile = [&](int tile) {
    if (tile >= ntiles) return;
    int row0, rows;
    mats.locate(tile, sb0, p_cur, row0, rows);
#pragma unroll
    for (int it = 0; it < NIT; it++) p_off[it] = (uint32_t)min(row0 + (int)row_of[it], rows - 1) * (uint32_t)rb + pc_of[it];
  };
  auto issue = [&](int stage) {
    if (p_tile < ntiles) {
      const uint8_t *src = mats.src(p_cur, sb0, p_c);
      const uint32_t dst = ring_s + stage * 16 * RS;
#pragma unroll
      for (int it = 0; it < NIT; it++)
        if (dst_rel[it] != 0xffffffffu) {
          if constexpr (FMT == LLB_FM_Q8_0) {
            if (is_sc[it]) { cp_async16(dst + dst_rel[it], p_cur.W0 + (size_t)p_c * 16 + p_off[it]); continue; }
          }
          cp_async16(dst + dst_rel[it], src + p_off[it]);
        }
      if (++p_c == nsl) { p_c = 0; p_tile += nws; plan_tile(p_tile); }
    }
    cp_async_commit();
  };
  if constexpr (Mats::EARLY) {
    plan_tile(p_tile);
    // weights first: the ring's prologue is in flight while the producer of the activations still
    // runs (weights depend on no kernel), and while the activation slice is staged
#pragma unroll 1
    for (int s = 0; s < ST - 1; s++) issue(s);
    stage(xh_s, xsf_s, CS, sb0, nsl);
  } else {
    // the weight addresses come from an earlier kernel's choice: the wait (inside stage) comes first
    stage(xh_s, xsf_s, CS, sb0, nsl);
    ntiles = live ? mats.ntiles() : 0;
    plan_tile(p_tile);
#pragma unroll 1
    for (int s = 0; s < ST - 1; s++) issue(s);
  }
  // the XP group sits between prologue groups and later ones; from here on group accounting is per
  // warp again: ST-1 chunks are complete, none pending
  int pstage = ST - 1, cstage = 0;
  int c_tile = warp * cps + ci, c_c = 0;
  static_assert(NTC == NT || NTC == 2, "a column selection computes one hi and one lo n-tile");
  constexpr int NTS = NTC == NT ? 8 : NC / 2;            // plane columns from one computed n-tile to the next
  int cb = 0;                                            // first plane column of the computed n-tiles
  float acc[NTC][4];
  const uint8_t *xb = xh_s + gid * CS + 16 * j;          // B fragments of column gid (n-tile 0)
  const uint8_t *xfb = xsf_s + gid * 32 + 8 * j;
  const uint32_t mn_sel = (j & 1) ? 0x4342u : 0x4140u;
#pragma unroll 1
  while (c_tile < ntiles) {
    if (c_c == 0) {
#pragma unroll
      for (int nt = 0; nt < NTC; nt++) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.0f;
      if constexpr (NTC != NT) cb = mats.col0(c_tile);
    }
    issue(pstage);                       // refill the stage consumed last iteration
    pstage = pstage + 1 == ST ? 0 : pstage + 1;
    cp_async_wait<ST - 1>();             // all but the newest ST-1 groups: the stage to consume is in
    __syncwarp();
    if constexpr (FMT == LLB_FM_Q8_0) {
      // eight blocks of 32 codes per super-block, two MMAs each; code (q ^ 0x80) = q + 128 as an fp16 subnormal,
      // the offset taken back through the 32-column sums: d * (2^24 P - 128 sum x)
      const uint8_t *b0 = ring + cstage * 16 * RS + gid * RS, *b1 = b0 + 8 * RS;
      const uint4 sw0 = *(const uint4 *)(b0 + 256), sw1 = *(const uint4 *)(b1 + 256);
      const uint32_t d0w[4] = {sw0.x, sw0.y, sw0.z, sw0.w}, d1w[4] = {sw1.x, sw1.y, sw1.z, sw1.w};
      const uint8_t *xb8 = xh_s + (gid + cb) * CS + 8 * j + (size_t)c_c * 512;
      const float *xs8 = (const float *)xsf_s + (size_t)c_c * 8 * NC + 2 * j + cb;
#pragma unroll
      for (int blk = 0; blk < 8; blk++) {
        float p[NTC][4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int m = 2 * blk + u;
          const uint32_t w0 = *(const uint32_t *)(b0 + 16 * m + 4 * j) ^ 0x80808080u, w1 = *(const uint32_t *)(b1 + 16 * m + 4 * j) ^ 0x80808080u;
          const uint32_t a0 = __byte_perm(w0, 0, 0x4240), a2 = __byte_perm(w0, 0, 0x4341);
          const uint32_t a1 = __byte_perm(w1, 0, 0x4240), a3 = __byte_perm(w1, 0, 0x4341);
#pragma unroll
          for (int nt = 0; nt < NTC; nt++) {
            const uint2 bx = *(const uint2 *)(xb8 + (size_t)nt * NTS * CS + 32 * m);
            if (u == 0) mma16816_z(p[nt], a0, a1, a2, a3, bx.x, bx.y);
            else mma16816(p[nt], a0, a1, a2, a3, bx.x, bx.y);
          }
        }
        const float d0 = h2f_bits((d0w[blk >> 1] >> (16 * (blk & 1))) & 0xffffu), d1 = h2f_bits((d1w[blk >> 1] >> (16 * (blk & 1))) & 0xffffu);
#pragma unroll
        for (int nt = 0; nt < NTC; nt++) {
          const float2 xs = *(const float2 *)(xs8 + (size_t)blk * NC + nt * NTS);
          acc[nt][0] += d0 * (p[nt][0] * TWO24 - 128.0f * xs.x);
          acc[nt][1] += d0 * (p[nt][1] * TWO24 - 128.0f * xs.y);
          acc[nt][2] += d1 * (p[nt][2] * TWO24 - 128.0f * xs.x);
          acc[nt][3] += d1 * (p[nt][3] * TWO24 - 128.0f * xs.y);
        }
      }
    } else if constexpr (FMT == LLB_FM_Q6_K) {
      // 16 scale groups of 16 columns per super-block, one MMA each; code 0..63 as fp16 subnormals
      // (quarters 2, 3 carry the code shifted left by 4), offset -32 through the 16-column sums
      const uint8_t *b0 = ring + cstage * 16 * RS + gid * RS, *b1 = b0 + 8 * RS;
      const float d0 = h2f_bits(*(const unsigned short *)(b0 + 208)), d1 = h2f_bits(*(const unsigned short *)(b1 + 208));
      const uint4 sw0 = *(const uint4 *)(b0 + 192), sw1 = *(const uint4 *)(b1 + 192);
      const uint32_t sc0w[4] = {sw0.x ^ 0x80808080u, sw0.y ^ 0x80808080u, sw0.z ^ 0x80808080u, sw0.w ^ 0x80808080u};
      const uint32_t sc1w[4] = {sw1.x ^ 0x80808080u, sw1.y ^ 0x80808080u, sw1.z ^ 0x80808080u, sw1.w ^ 0x80808080u};
      const uint8_t *xb6 = xh_s + (gid + cb) * CS + 8 * j + (size_t)c_c * 512;
      const float *xs6 = (const float *)xsf_s + (size_t)c_c * 16 * NC + 2 * j + cb;
#pragma unroll
      for (int hf = 0; hf < 2; hf++) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
          const int o = 16 * u + 4 * j;
          const uint32_t la0 = *(const uint32_t *)(b0 + 64 * hf + o), lb0 = *(const uint32_t *)(b0 + 64 * hf + 32 + o);
          const uint32_t la1 = *(const uint32_t *)(b1 + 64 * hf + o), lb1 = *(const uint32_t *)(b1 + 64 * hf + 32 + o);
          const uint32_t hq0 = *(const uint32_t *)(b0 + 128 + 32 * hf + o), hq1 = *(const uint32_t *)(b1 + 128 + 32 * hf + o);
          const uint32_t h0s4 = hq0 << 4, h0s2 = hq0 << 2, h1s4 = hq1 << 4, h1s2 = hq1 << 2;
          const uint32_t h0o4 = (hq0 >> 8) << 4, h0o2 = (hq0 >> 8) << 2, h1o4 = (hq1 >> 8) << 4, h1o2 = (hq1 >> 8) << 2;
#pragma unroll
          for (int qd = 0; qd < 4; qd++) {
            const uint32_t l0 = (qd & 1) ? lb0 : la0, l1 = (qd & 1) ? lb1 : la1;
            const uint32_t nm = qd < 2 ? 0x000f000fu : 0x00f000f0u, hm = qd < 2 ? 0x00300030u : 0x03000300u;
            const uint32_t e0 = (l0 & nm) | (((qd & 1) ? h0s2 : h0s4) & hm), e1 = (l1 & nm) | (((qd & 1) ? h1s2 : h1s4) & hm);
            const uint32_t o0 = ((l0 >> 8) & nm) | (((qd & 1) ? h0o2 : h0o4) & hm), o1 = ((l1 >> 8) & nm) | (((qd & 1) ? h1o2 : h1o4) & hm);
            const float w = qd < 2 ? TWO24 : TWO24 * 0.0625f;
            const int gi = 8 * hf + 2 * qd + u;
            // signed scale: (sc ^ 0x80) is sc + 128 as an unsigned byte
            const float s0 = d0 * (__uint_as_float(__byte_perm(sc0w[gi >> 2], 0x4B000000u, 0x7650u | (gi & 3))) - 8388736.0f);
            const float s1 = d1 * (__uint_as_float(__byte_perm(sc1w[gi >> 2], 0x4B000000u, 0x7650u | (gi & 3))) - 8388736.0f);
            const int kl = 128 * hf + 32 * qd + 16 * u;
#pragma unroll
            for (int nt = 0; nt < NTC; nt++) {
              const uint2 bx = *(const uint2 *)(xb6 + (size_t)nt * NTS * CS + kl * 2);
              float p[4];
              mma16816_z(p, e0, e1, o0, o1, bx.x, bx.y);
              const float2 xs = *(const float2 *)(xs6 + (size_t)(kl >> 4) * NC + nt * NTS);
              acc[nt][0] += s0 * (p[0] * w - 32.0f * xs.x);
              acc[nt][1] += s0 * (p[1] * w - 32.0f * xs.y);
              acc[nt][2] += s1 * (p[2] * w - 32.0f * xs.x);
              acc[nt][3] += s1 * (p[3] * w - 32.0f * xs.y);
            }
          }
        }
      }
    } else {
      const uint8_t *b0 = ring + cstage * 16 * RS + gid * RS, *b1 = b0 + 8 * RS;
      const uint4 h0 = *(const uint4 *)b0, h1 = *(const uint4 *)b1;
      uint32_t scA0, scB0, mnA0, mnB0, scA1, scB1, mnA1, mnB1;
      k4_scales(h0.y, h0.z, h0.w, scA0, scB0, mnA0, mnB0);
      k4_scales(h1.y, h1.z, h1.w, scA1, scB1, mnA1, mnB1);
      // the two mins of this thread's k-pair as fp16 numbers: 0x6400 | m is 1024 + m exactly; one FMA each gives m for
      // the means' hi halves and m / 2048 for their lo halves (which are stored times 2048), both exact
      const uint32_t at0 = __byte_perm(j < 2 ? mnA0 : mnB0, 0, mn_sel) | 0x64006400u, at1 = __byte_perm(j < 2 ? mnA1 : mnB1, 0, mn_sel) | 0x64006400u;
      const uint32_t am0 = g2_hfma2(at0, 0x3c003c00u, 0xe400e400u), am1 = g2_hfma2(at1, 0x3c003c00u, 0xe400e400u);       // * 1 - 1024
      const uint32_t al0 = g2_hfma2(at0, 0x10001000u, 0xb800b800u), al1 = g2_hfma2(at1, 0x10001000u, 0xb800b800u);       // * 2^-11 - 0.5
      uint32_t qh0 = 0, qh0b = 0, qh1 = 0, qh1b = 0;
      if constexpr (FMT == LLB_FM_Q5_K) {
        const uint2 t0 = *(const uint2 *)(b0 + 16 + 8 * j), t1 = *(const uint2 *)(b1 + 16 + 8 * j);
        qh0 = t0.x; qh0b = t0.y; qh1 = t1.x; qh1b = t1.y;
      }
      float sS[NTC][4], pm[NTC][4];
#pragma unroll
      for (int nt = 0; nt < NTC; nt++) {
        const uint2 xf = *(const uint2 *)(xfb + (size_t)c_c * NC * 32 + (nt * NTS + cb) * 32);
        mma16816_z(pm[nt], am0, am1, al0, al1, xf.x, xf.y);
        sS[nt][0] = sS[nt][1] = sS[nt][2] = sS[nt][3] = 0.0f;
      }
#pragma unroll
      for (int g = 0; g < 4; g++) {
        const uint2 a0 = *(const uint2 *)(b0 + TR::QOFF + 32 * g + 8 * j), a1 = *(const uint2 *)(b1 + TR::QOFF + 32 * g + 8 * j);
        uint32_t f0l = 0, f0h = 0, f1l = 0, f1h = 0, f0lb = 0, f0hb = 0, f1lb = 0, f1hb = 0;
        if constexpr (FMT == LLB_FM_Q5_K) {
          f0l = (qh0 >> (2 * g)) & 0x01010101u; f0h = (qh0 >> (2 * g + 1)) & 0x01010101u;
          f1l = (qh1 >> (2 * g)) & 0x01010101u; f1h = (qh1 >> (2 * g + 1)) & 0x01010101u;
          f0lb = (qh0b >> (2 * g)) & 0x01010101u; f0hb = (qh0b >> (2 * g + 1)) & 0x01010101u;
          f1lb = (qh1b >> (2 * g)) & 0x01010101u; f1hb = (qh1b >> (2 * g + 1)) & 0x01010101u;
        }
        const uint32_t s0 = g < 2 ? scA0 : scB0, s1 = g < 2 ? scA1 : scB1;
        const float sc0l = byte_f(s0, (2 * g) & 3), sc0h = byte_f_scaled(s0, (2 * g + 1) & 3, 0.0625f);
        const float sc1l = byte_f(s1, (2 * g) & 3), sc1h = byte_f_scaled(s1, (2 * g + 1) & 3, 0.0625f);
        const uint32_t a0x8 = a0.x >> 8, a0y8 = a0.y >> 8, a1x8 = a1.x >> 8, a1y8 = a1.y >> 8;
#pragma unroll
        for (int nt = 0; nt < NTC; nt++) {
          const uint8_t *xr = xb + (size_t)(nt * NTS + cb) * CS + ((size_t)c_c * 256 + 64 * g) * 2;
          const uint4 bl = *(const uint4 *)xr, bh = *(const uint4 *)(xr + 64);
          float pl[4], ph[4];
          mma16816_z(pl, (a0.x & 0x000f000fu) | ((f0l & 0x00010001u) << 4), (a1.x & 0x000f000fu) | ((f1l & 0x00010001u) << 4),
                     (a0x8 & 0x000f000fu) | (((f0l >> 8) & 0x00010001u) << 4), (a1x8 & 0x000f000fu) | (((f1l >> 8) & 0x00010001u) << 4), bl.x, bl.y);
          mma16816(pl, (a0.y & 0x000f000fu) | ((f0lb & 0x00010001u) << 4), (a1.y & 0x000f000fu) | ((f1lb & 0x00010001u) << 4),
                   (a0y8 & 0x000f000fu) | (((f0lb >> 8) & 0x00010001u) << 4), (a1y8 & 0x000f000fu) | (((f1lb >> 8) & 0x00010001u) << 4), bl.z, bl.w);
          mma16816_z(ph, (a0.x & 0x00f000f0u) | ((f0h & 0x00010001u) << 8), (a1.x & 0x00f000f0u) | ((f1h & 0x00010001u) << 8),
                     (a0x8 & 0x00f000f0u) | (((f0h >> 8) & 0x00010001u) << 8), (a1x8 & 0x00f000f0u) | (((f1h >> 8) & 0x00010001u) << 8), bh.x, bh.y);
          mma16816(ph, (a0.y & 0x00f000f0u) | ((f0hb & 0x00010001u) << 8), (a1.y & 0x00f000f0u) | ((f1hb & 0x00010001u) << 8),
                   (a0y8 & 0x00f000f0u) | (((f0hb >> 8) & 0x00010001u) << 8), (a1y8 & 0x00f000f0u) | (((f1hb >> 8) & 0x00010001u) << 8), bh.z, bh.w);
          sS[nt][0] += sc0l * pl[0] + sc0h * ph[0];
          sS[nt][1] += sc0l * pl[1] + sc0h * ph[1];
          sS[nt][2] += sc1l * pl[2] + sc1h * ph[2];
          sS[nt][3] += sc1l * pl[3] + sc1h * ph[3];
        }
      }
      const float d0 = h2f_bits(h0.x & 0xffffu) * TWO24, dm0 = h2f_bits(h0.x >> 16) * 32.0f;
      const float d1 = h2f_bits(h1.x & 0xffffu) * TWO24, dm1 = h2f_bits(h1.x >> 16) * 32.0f;
#pragma unroll
      for (int nt = 0; nt < NTC; nt++) {
        acc[nt][0] += d0 * sS[nt][0] - dm0 * pm[nt][0];
        acc[nt][1] += d0 * sS[nt][1] - dm0 * pm[nt][1];
        acc[nt][2] += d1 * sS[nt][2] - dm1 * pm[nt][2];
        acc[nt][3] += d1 * sS[nt][3] - dm1 * pm[nt][3];
      }
    }
    __syncwarp();
    cstage = cstage + 1 == ST ? 0 : cstage + 1;
    if (++c_c == nsl) {
      mats.template epilogue<NTC>(ks, c_tile, acc, lane);
      c_c = 0;
      c_tile += nws;
    }
  }
  cp_async_wait<0>();
}

// the activation slice from the planes in global memory: cp.async, one wait, one barrier
template <int FMT, int NT> struct G2StagePlanes {
  const GemmArgs &a;
  __device__ __forceinline__ void operator()(uint8_t *xh_s, uint8_t *xsf_s, int CS, int sb0, int nsl) const {
    using TR = G2Traits<FMT>;
    constexpr int NC = 8 * NT;
    pdl_wait();
    const int per_col = nsl * 32;   // 16-byte pieces of one column's slice
    for (int i = threadIdx.x; i < NC * per_col; i += blockDim.x) {
      const int c = i / per_col, p = i - c * per_col;
      cp_async16(smem_u32(xh_s + c * CS + p * 16), (const uint8_t *)(a.xp.xh + (size_t)c * a.K + (size_t)sb0 * 256) + p * 16);
    }
    // the side array of the slice: contiguous in global memory for all kinds
    const uint8_t *xf = FMT == LLB_FM_Q6_K   ? (const uint8_t *)(a.xp.xs16 + (size_t)sb0 * 16 * NC)
                        : FMT == LLB_FM_Q8_0 ? (const uint8_t *)(a.xp.xs32 + (size_t)sb0 * 8 * NC)
                                             : (const uint8_t *)(a.xp.xsf + (size_t)sb0 * NC * 16);
    for (int i = threadIdx.x; i < nsl * NC * (TR::AUX / 16); i += blockDim.x) cp_async16(smem_u32(xsf_s + i * 16), xf + i * 16);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
  }
};

template <int FMT, int NT>
__global__ void __launch_bounds__(g2_warps<FMT>(8 * NT) * 32, G2_CPSM) k_gemm2(const GemmArgs a, const int cps) {
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_trigger();
  g2_phase<FMT, NT>(a, cps, (int)blockIdx.x, smem, G2StagePlanes<FMT, NT>{a}, G2MatsPlain<FMT>{a});
}
