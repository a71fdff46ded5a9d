// attention.cu -- split-K GQA attention of the T query rows over the KV cache, on tensor cores.
// (llb_t_attn4 computes one block per (head, row) with no split, tools/payload-spec2.patch:208-315; the
// reference's own split-K form is llb_attn4_sk8, tools/payload-sk8add.patch:16-93; the arithmetic is
// full_attn of the CPU engine, tools/qwen35_engine.c:667-726.)
//
// The cache holds every K and V value as two fp16 numbers, hi = fp16(x) and lo = fp16((x - hi) * 2048)
// (the same bytes as one f32, about 22 bits of it), written that way by k_qkrope.  A block owns one kv
// head and one slice of the context and streams its K and V rows ONCE, 32 positions at a time through a
// two-stage cp.async ring, for all NQ = (H / KV) * T queries of that head:
//   scores  S[pos][q] = K_hi q_hi + (K_hi q_lo + K_lo q_hi) / 2048       mma.m16n8k16, warps split (16 positions, 8 queries)
//   softmax online per query (running max and sum), warps split the queries, lane = position
//   output  O[d][q] += V_hi^T (P_hi + P_lo) + V_lo^T P_hi / 2048        warps split the head dimension
// Per (query, slice) it leaves a running max, a sum and an unnormalised accumulator for k_attn_comb.
// The scalar-FMA kernel this replaces spent 2400 warp instructions per 32 positions and warp; this one about 350.
#include "host.cuh"
#include "model.cuh"

#define ATT_PT 32
#define ATT_PS 40   // halves per row of the probability tiles: 80-byte rows keep ldmatrix conflict-free

__device__ __forceinline__ float aw_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
__device__ __forceinline__ float aw_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(addr));
}

// bytes of shared memory for NQG groups of 8 queries
template <int HD> static size_t att_smem(int nqg) {
  const size_t rsk = (size_t)(HD + 8) * 2, nqp = (size_t)nqg * 8;
  return 2 * nqp * rsk + 2 * 4 * ATT_PT * rsk + nqp * 33 * 4 + 2 * nqp * ATT_PS * 2 + 2 * nqp * 4 + 128;
}

template <int HD, int NQG>
__global__ void __launch_bounds__(256) k_attn_mma(const float *__restrict__ q, const __half *__restrict__ Kc, const __half *__restrict__ Vc,
                                                  AttnShape sh, int Tmax, float *__restrict__ pm, float *__restrict__ pl,
                                                  float *__restrict__ po, const RowSet *rs) {
  // blockIdx.z: one of several row groups -- the groups of a prompt chunk, which share a cache, or the streams of a pass,
  // each with its own -- each with its own row set, Tmax query rows and partial results
  {
    const size_t z = blockIdx.z, per = (size_t)sh.H * Tmax * gridDim.y;
    rs = (const RowSet *)((uintptr_t)rs + z * sh.rs_stride);
    q += z * Tmax * sh.H * HD; pm += z * per; pl += z * per; po += z * per * HD;
    Kc += z * sh.kv_group; Vc += z * sh.kv_group;
  }
  int rs_n, rs_p0;
  rs = rs_begin(rs, rs_n, rs_p0);
  extern __shared__ __align__(128) uint8_t sm[];
  constexpr int RSK = HD + 8, NQP = 8 * NQG, MTW = HD / 128, KSTEPS = HD / 16;
  constexpr int TILE_B = ATT_PT * RSK * 2;   // bytes of one staged array (32 rows)
  __half *qh = (__half *)sm, *ql = qh + NQP * RSK;
  uint8_t *kv = (uint8_t *)(ql + NQP * RSK);                  // [stage][Kh, Kl, Vh, Vl][32][RSK]
  float *Ssm = (float *)(kv + 2 * 4 * TILE_B);                // [NQP][33]
  __half *Ph = (__half *)(Ssm + NQP * 33), *Pl = Ph + NQP * ATT_PS;
  float *corr = (float *)(Pl + NQP * ATT_PS), *mfin = corr + NQP;
  const int kvh = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gid = lane >> 2, j = lane & 3, lr = lane & 7, mi = lane >> 3;
  const int G = sh.H / sh.KV, NQ = G * Tmax, n = rs_n, pos0 = rs_p0, total = pos0 + n, kvd = sh.KV * HD;
  // slices of whole 32-position tiles, at least min_per positions: short contexts use the first few blocks only
  const int per = max(sh.min_per, ((total + nsplit - 1) / nsplit + 31) & ~31), s0 = split * per, s1 = min(total, s0 + per);
  const int ntiles = s1 > s0 ? (s1 - s0 + ATT_PT - 1) / ATT_PT : 0;
  const uint32_t kv_s = smem_u32(kv);

  auto load_tile = [&](int it) {
    if (it < ntiles) {
      const int p0 = s0 + it * ATT_PT;
      const uint32_t dst0 = kv_s + (uint32_t)(it & 1) * 4 * TILE_B;
      // 4 arrays x 32 rows x HD/8 sixteen-byte pieces
      for (int i = tid; i < 4 * ATT_PT * (HD / 8); i += 256) {
        const int arr = i / (ATT_PT * (HD / 8)), rem = i - arr * (ATT_PT * (HD / 8)), row = rem / (HD / 8), pc = rem - row * (HD / 8);
        const int p = min(p0 + row, s1 - 1);   // rows past the slice repeat its last row; their scores are masked
        const __half *src = ((arr < 2) ? Kc : Vc) + (size_t)(arr & 1) * sh.kv_plane + (size_t)p * kvd + kvh * HD + pc * 8;
        cp_async16(dst0 + arr * TILE_B + (row * RSK + pc * 8) * 2, src);
      }
    }
    cp_async_commit();
  };
  load_tile(0);
  // the queries of this kv head as hi / lo planes: local query g * Tmax + r is head kvh * G + g, row r
  for (int i = tid; i < NQP * (HD / 2); i += 256) {
    const int qi = i / (HD / 2), dd = 2 * (i - qi * (HD / 2)), g = qi / Tmax, r = qi - g * Tmax;
    float2 v = make_float2(0.f, 0.f);
    if (qi < NQ && r < n) v = __ldcg((const float2 *)(q + ((size_t)r * sh.H + kvh * G + g) * HD + dd));
    const __half2 h = __floats2half2_rn(v.x, v.y);
    const float2 hf = __half22float2(h);
    *(__half2 *)(qh + qi * RSK + dd) = h;
    *(__half2 *)(ql + qi * RSK + dd) = __floats2half2_rn((v.x - hf.x) * XP_LO_SCALE, (v.y - hf.y) * XP_LO_SCALE);
  }
  float m_r[NQG], l_r[NQG];      // running max and sum of query warp + 8 i (the same in every lane)
  float acc[MTW][NQG][4], acl[MTW][NQG][4];
#pragma unroll
  for (int i = 0; i < NQG; i++) { m_r[i] = -INFINITY; l_r[i] = 0.0f; }
#pragma unroll
  for (int a = 0; a < MTW; a++)
#pragma unroll
    for (int b = 0; b < NQG; b++)
#pragma unroll
      for (int c = 0; c < 4; c++) { acc[a][b][c] = 0.0f; acl[a][b][c] = 0.0f; }
  const float scale = 1.0f / sqrtf((float)HD);
  const uint32_t qh_s = smem_u32(qh), ql_s = smem_u32(ql), ph_s = smem_u32(Ph), pl_s = smem_u32(Pl);

  for (int it = 0; it < ntiles; it++) {
    load_tile(it + 1);
    cp_async_wait<1>();
    __syncthreads();
    const int p0 = s0 + it * ATT_PT;
    const uint32_t st_s = kv_s + (uint32_t)(it & 1) * 4 * TILE_B;
    // ---- scores: work item = (16 positions, 8 queries) ----
    for (int item = warp; item < 2 * NQG; item += 8) {
      const int mt = item & 1, qg = item >> 1;
      float hh[4] = {0.f, 0.f, 0.f, 0.f}, hl[4] = {0.f, 0.f, 0.f, 0.f}, lh[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t a_off = (uint32_t)((16 * mt + lr + ((mi & 1) ? 8 : 0)) * RSK + ((mi & 2) ? 8 : 0)) * 2;
      const uint32_t b_off = (uint32_t)((8 * qg + lr) * RSK + ((mi & 1) ? 8 : 0)) * 2;
#pragma unroll 4
      for (int ks = 0; ks < KSTEPS; ks++) {
        uint32_t ah[4], al[4], bh[2], bl[2];
        ldsm_x4(ah, st_s + a_off + ks * 32);
        ldsm_x4(al, st_s + TILE_B + a_off + ks * 32);
        ldsm_x2(bh, qh_s + b_off + ks * 32);
        ldsm_x2(bl, ql_s + b_off + ks * 32);
        mma16816(hh, ah[0], ah[1], ah[2], ah[3], bh[0], bh[1]);
        mma16816(hl, ah[0], ah[1], ah[2], ah[3], bl[0], bl[1]);
        mma16816(lh, al[0], al[1], al[2], al[3], bh[0], bh[1]);
      }
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int prow = 16 * mt + gid + ((c & 2) ? 8 : 0), qi = 8 * qg + 2 * j + (c & 1), r = qi % Tmax, p = p0 + prow;
        const float s = (hh[c] + (hl[c] + lh[c]) * XP_LO_INV) * scale;
        Ssm[qi * 33 + prow] = (qi < NQ && r < n && p < s1 && p <= pos0 + r) ? s : -INFINITY;
      }
    }
    __syncthreads();
    // ---- online softmax: warp w owns queries w, w + 8, ..; lane = position ----
#pragma unroll
    for (int i = 0; i < NQG; i++) {
      const int qi = warp + 8 * i;
      const float s = Ssm[qi * 33 + lane];
      const float mt = aw_max(s);
      float e = 0.0f, cf = 1.0f;
      if (mt != -INFINITY) {            // (a fully masked tile leaves the query's state alone)
        const float mn = fmaxf(m_r[i], mt);
        cf = expf(m_r[i] - mn);         // exp(-inf) = 0 on the first tile
        e = expf(s - mn);
        l_r[i] = l_r[i] * cf + aw_sum(e);
        m_r[i] = mn;
      }
      const __half eh = __float2half_rn(e);
      Ph[qi * ATT_PS + lane] = eh;
      Pl[qi * ATT_PS + lane] = __float2half_rn(e - __half2float(eh));
      if (lane == 0) corr[qi] = cf;
    }
    __syncthreads();
    // ---- output: warp w owns dims 16 MTW w .. + 16 MTW - 1 of every query ----
#pragma unroll
    for (int nt = 0; nt < NQG; nt++) {
      const float c0 = corr[8 * nt + 2 * j], c1 = corr[8 * nt + 2 * j + 1];
#pragma unroll
      for (int a = 0; a < MTW; a++) {
        acc[a][nt][0] *= c0; acc[a][nt][1] *= c1; acc[a][nt][2] *= c0; acc[a][nt][3] *= c1;
        acl[a][nt][0] *= c0; acl[a][nt][1] *= c1; acl[a][nt][2] *= c0; acl[a][nt][3] *= c1;
      }
    }
#pragma unroll
    for (int ks = 0; ks < ATT_PT / 16; ks++) {
      uint32_t bph[NQG][2], bpl[NQG][2];
#pragma unroll
      for (int nt = 0; nt < NQG; nt++) {
        const uint32_t off = (uint32_t)((8 * nt + lr) * ATT_PS + 16 * ks + ((mi & 1) ? 8 : 0)) * 2;
        ldsm_x2(bph[nt], ph_s + off);
        ldsm_x2(bpl[nt], pl_s + off);
      }
#pragma unroll
      for (int a = 0; a < MTW; a++) {
        const int d0 = 16 * (MTW * warp + a);
        const uint32_t v_off = (uint32_t)((16 * ks + lr + ((mi & 2) ? 8 : 0)) * RSK + d0 + ((mi & 1) ? 8 : 0)) * 2;
        uint32_t vh[4], vl[4];
        ldsm_x4_t(vh, st_s + 2 * TILE_B + v_off);
        ldsm_x4_t(vl, st_s + 3 * TILE_B + v_off);
#pragma unroll
        for (int nt = 0; nt < NQG; nt++) {
          mma16816(acc[a][nt], vh[0], vh[1], vh[2], vh[3], bph[nt][0], bph[nt][1]);
          mma16816(acc[a][nt], vh[0], vh[1], vh[2], vh[3], bpl[nt][0], bpl[nt][1]);
          mma16816(acl[a][nt], vl[0], vl[1], vl[2], vl[3], bph[nt][0], bph[nt][1]);
        }
      }
    }
    __syncthreads();   // the stage and the probability tiles are free again
  }
  cp_async_wait<0>();
  // ---- per (query, slice): running max, sum, unnormalised output ----
#pragma unroll
  for (int i = 0; i < NQG; i++) {
    const int qi = warp + 8 * i, g = qi / Tmax, r = qi - g * Tmax;
    if (lane == 0) {
      mfin[qi] = m_r[i];
      if (qi < NQ && r < n) {
        const size_t o = ((size_t)(kvh * G + g) * Tmax + r) * nsplit + split;
        pm[o] = m_r[i]; pl[o] = l_r[i];
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int nt = 0; nt < NQG; nt++)
#pragma unroll
    for (int c = 0; c < 4; c++) {
      const int qi = 8 * nt + 2 * j + (c & 1), g = qi / Tmax, r = qi - g * Tmax;
      if (qi >= NQ || r >= n || mfin[qi] == -INFINITY) continue;   // an empty slice: the merge skips it on m alone
      const size_t o = ((size_t)(kvh * G + g) * Tmax + r) * nsplit + split;
#pragma unroll
      for (int a = 0; a < MTW; a++) {
        const int d = 16 * (MTW * warp + a) + gid + ((c & 2) ? 8 : 0);
        po[o * HD + d] = acc[a][nt][c] + acl[a][nt][c] * XP_LO_INV;
      }
    }
}

// merge the splits, normalise, apply the sigmoid output gate, write the planes of attn_output's input
// (llb_attn4_combine + llb_t_ogq, tools/payload-sk8add.patch, tools/payload-spec2.patch:149-156)
// block = (head, row); thread (sg, i4): split group sg, dims 4*i4 .. 4*i4+3
__global__ void __launch_bounds__(256) k_attn_comb(const float *__restrict__ pm, const float *__restrict__ pl, const float *__restrict__ po, PartIn qg,
                                                   AttnShape sh, int nsplit, int Tmax, XPlanes xp, const RowSet *rs, __half *__restrict__ kg, int kg_row0) {
  {
    const size_t z = blockIdx.z, per = (size_t)sh.H * Tmax * nsplit;
    rs = (const RowSet *)((uintptr_t)rs + z * sh.rs_stride);
    pm += z * per; pl += z * per; po += z * per * sh.hd;
    qg.p += z * Tmax * 2 * sh.H * sh.hd;
    kg_row0 += (int)z * Tmax;
  }
  const int xrow0 = blockIdx.z * Tmax;   // the group's rows in the planes
  int rs_n, rs_p0;
  rs = rs_begin(rs, rs_n, rs_p0);
  __shared__ float wsm[128];
  __shared__ float red[32];
  __shared__ __align__(16) float osm[1024];   // [split group][hd]
  const int h = blockIdx.x, t = blockIdx.y, i = threadIdx.x, hd = sh.hd, lane = threadIdx.x & 31;
  if (t >= rs_n) return;
  const size_t qb = ((size_t)h * Tmax + t) * nsplit;
  // slices in use at this context length (the partial kernel's split rule)
  const int total = rs_p0 + rs_n;
  const int per = max(sh.min_per, ((total + nsplit - 1) / nsplit + 31) & ~31), nact = min(nsplit, (total + per - 1) / per);
  float m = -INFINITY, l = 0.0f;
  if (i < nact) { m = __ldcg(pm + qb + i); l = __ldcg(pl + qb + i); }
  float M = aw_max(m);
  __syncthreads();
  if (lane == 0) red[i >> 5] = M;
  __syncthreads();
  M = red[0];
  for (int k = 1; k < (blockDim.x >> 5); k++) M = fmaxf(M, red[k]);
  const float wgt = (i < nact && m != -INFINITY) ? expf(m - M) : 0.0f;
  if (i < 128) wsm[i] = wgt;
  float L = aw_sum(l * wgt);
  __syncthreads();
  if (lane == 0) red[i >> 5] = L;
  __syncthreads();   // (wsm is visible after it too)
  L = 0.0f;
  for (int k = 0; k < (blockDim.x >> 5); k++) L += red[k];
  const int hd4 = hd >> 2, ng = blockDim.x / hd4, sg = i / hd4, i4 = i - sg * hd4;   // ng split groups of hd/4 threads
  float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
  if (sg < ng) {
    // split s = sg + ng*j: four loads in flight per trip, added in split order within the group
    for (int s0 = sg; s0 < nact; s0 += 4 * ng) {
      float4 v[4];
      float ws[4];
#pragma unroll
      for (int jj = 0; jj < 4; jj++) {
        const int s = s0 + jj * ng;
        ws[jj] = s < nact ? wsm[s] : 0.0f;
        v[jj] = ws[jj] != 0.0f ? __ldcg((const float4 *)(po + (qb + s) * hd + 4 * i4)) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int jj = 0; jj < 4; jj++) { o.x += v[jj].x * ws[jj]; o.y += v[jj].y * ws[jj]; o.z += v[jj].z * ws[jj]; o.w += v[jj].w * ws[jj]; }
    }
    *(float4 *)&osm[sg * hd + 4 * i4] = o;
  }
  __syncthreads();
  if (i < hd4) {   // a multiple of 8 threads: eight lanes per 32 dims
    float4 a = *(const float4 *)&osm[4 * i];
    for (int g = 1; g < ng; g++) { const float4 b = *(const float4 *)&osm[g * hd + 4 * i]; a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w; }
    const float4 gate = part_get4(qg, (size_t)t * 2 * sh.H * hd + (size_t)h * 2 * hd + hd + 4 * i);
    const float hv[4] = {(a.x / L) / (1.0f + expf(-gate.x)), (a.y / L) / (1.0f + expf(-gate.y)), (a.z / L) / (1.0f + expf(-gate.z)),
                         (a.w / L) / (1.0f + expf(-gate.w))};
    // the prompt path takes the rows as fp16 in the dense GEMM's k-group-major order instead of the T-row planes
    if (kg) pf_kg_store4(kg, sh.H * hd, kg_row0 + t, h * hd + 4 * i, hv[0], hv[1], hv[2], hv[3]);
    else xp_store4(xp, xrow0 + t, 2, h * hd + 4 * i, hv, lane, true);
  }
}

template <int HD, int NQG> static int att_go(cudaStream_t s, dim3 grid, const float *q, const __half *Kc, const __half *Vc, AttnShape sh, int Tmax,
                                             float *pm, float *pl, float *po, const RowSet *rs) {
  CU_OK(llb_launch(k_attn_mma<HD, NQG>, grid, dim3(256), att_smem<HD>(NQG), s, q, Kc, Vc, sh, Tmax, pm, pl, po, rs));
  return 0;
}
template <int HD> static int att_hd(cudaStream_t s, int nqg, dim3 grid, const float *q, const __half *Kc, const __half *Vc, AttnShape sh, int Tmax,
                                    float *pm, float *pl, float *po, const RowSet *rs) {
  switch (nqg) {
    case 1: return att_go<HD, 1>(s, grid, q, Kc, Vc, sh, Tmax, pm, pl, po, rs);
    case 2: return att_go<HD, 2>(s, grid, q, Kc, Vc, sh, Tmax, pm, pl, po, rs);
    case 3: return att_go<HD, 3>(s, grid, q, Kc, Vc, sh, Tmax, pm, pl, po, rs);
    case 4: return att_go<HD, 4>(s, grid, q, Kc, Vc, sh, Tmax, pm, pl, po, rs);
    case 5: return att_go<HD, 5>(s, grid, q, Kc, Vc, sh, Tmax, pm, pl, po, rs);
    case 6: return att_go<HD, 6>(s, grid, q, Kc, Vc, sh, Tmax, pm, pl, po, rs);
  }
  return llb_fail("attention: %d queries per kv head", nqg * 8);
}

int op_attention(cudaStream_t s, const float *q, const float *Kc, const float *Vc, PartIn qg, AttnShape sh, int nsplit,
                 float *pm, float *pl, float *po, XPlanes xp, const RowSet *rs, int Tmax, __half *kg, int kg_row0, int nz) {
  const int G = sh.H / sh.KV, NQ = G * Tmax, nqg = (NQ + 7) / 8;
  dim3 grid(sh.KV, nsplit, nz);
  int rc;
  if (sh.hd == 128) rc = att_hd<128>(s, nqg, grid, q, (const __half *)Kc, (const __half *)Vc, sh, Tmax, pm, pl, po, rs);
  else if (sh.hd == 256) rc = att_hd<256>(s, nqg, grid, q, (const __half *)Kc, (const __half *)Vc, sh, Tmax, pm, pl, po, rs);
  else return llb_fail("attention: head_dim %d", sh.hd);
  if (rc) return rc;
  CU_OK(cudaGetLastError());
  CU_OK(llb_launch(k_attn_comb, dim3(sh.H, Tmax, nz), dim3(256), (size_t)(0), s, pm, pl, po, qg, sh, nsplit, Tmax, xp, rs, kg, kg_row0));
  CU_OK(cudaGetLastError());
  return 0;
}

template <int HD, int NQG> static int att_attr() {
  CU_OK(cudaFuncSetAttribute(k_attn_mma<HD, NQG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)att_smem<HD>(NQG)));
  return 0;
}
int ops_model_setup(void) {
  if (att_attr<128, 1>() || att_attr<128, 2>() || att_attr<128, 3>() || att_attr<128, 4>() || att_attr<128, 5>() || att_attr<128, 6>()) return -1;
  if (att_attr<256, 1>() || att_attr<256, 2>() || att_attr<256, 3>() || att_attr<256, 4>() || att_attr<256, 5>() || att_attr<256, 6>()) return -1;
  return 0;
}
