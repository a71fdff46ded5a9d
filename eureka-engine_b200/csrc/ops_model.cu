// ops_model.cu -- the non-GEMM device ops of the verify / draft passes, T rows per launch.
// Each kernel restates one or more of the reference's llb_t_* row kernels
// (tools/payload-spec2.patch:35-483); the arithmetic follows the CPU engine
// (tools/qwen35_engine.c:510-778), which is what parity is judged against.
#include <cooperative_groups.h>

#include "model.cuh"
namespace cg = cooperative_groups;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, m));
  return v;
}
// sum over the block; every thread gets the result (red: >= 32 floats of shared memory)
__device__ __forceinline__ float block_sum(float v, float *red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.0f;
  for (int i = 0; i < nw; i++) t += red[i];
  return t;
}
static Streams g_streams = {1 << 30, 0};
void ops_set_streams(int per, int stride) { g_streams.per = per > 0 ? per : 1 << 30; g_streams.stride = stride; }
Streams ops_streams(void) { return g_streams; }

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// ---- embedding rows (llb_embedk, tools/payload-kpair.patch:526) ---------------------------------
__global__ void k_embed(int fmt, const uint8_t *__restrict__ W, int d, const RowSet *rs, Streams sg, float *__restrict__ x) {
  int rs_n, rs_p0, tl;
  const int t = blockIdx.y;
  rs = rs_begin_row(rs, sg, t, rs_n, rs_p0, tl);
  if (tl >= rs_n) return;
  const uint8_t *row = W + (size_t)rs->tok[tl] * dev_row_bytes(fmt, d);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < d; c += gridDim.x * blockDim.x) x[(size_t)t * d + c] = deq_elem(fmt, row, d, c);
}
int op_embed(cudaStream_t s, int fmt, const uint8_t *W, int d, const RowSet *rs, int Tmax, float *x) {
  CU_OK(llb_launch(k_embed, dim3((d + 255) / 256, Tmax), dim3(256), (size_t)(0), s, fmt, W, d, rs, g_streams, x));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- residual add + RMSNorm -> activation planes (llb_t_rnaddq / llb_t_rnormq,
// tools/payload-spec2.patch:35-112; rms_norm tools/qwen35_engine.c:510-515) ----------------------
// v = xin + sum(partials); xout = v (optional); h = (v * s) * w, s = 1/sqrt(mean(v^2) + eps);
// h goes to the planes at column offset xp_col0 and, optionally, to hn_out as f32.
// One block per row; a thread holds NI groups of four consecutive columns (float4 loads and stores), so a
// row of 5120 columns costs each of 640 threads a handful of instructions instead of one SM 13k.
#define NORM_MAXT 1024
template <int NI>
__global__ void __launch_bounds__(NORM_MAXT) k_norm_xp(const float *__restrict__ xin, PartIn add, const float *__restrict__ w, float eps, int d,
                                                       float *__restrict__ xout, XPlanes xp, int xp_col0, float *__restrict__ hn_out,
                                                       const RowSet *rs, Streams sg, int zero_if_pos0) {
  // the norm weights depend on no kernel: their trip to DRAM overlaps the wait on the producer
  float4 wv[NI];
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);
    wv[i] = c < d ? *(const float4 *)(w + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  int rs_n, rs_p0, tl;
  const int t = blockIdx.x;
  rs = rs_begin_row(rs, sg, t, rs_n, rs_p0, tl);
  __shared__ float red[32];
  if (tl >= rs_n) return;
  const bool zero = zero_if_pos0 && (rs_p0 + tl == 0);
  const size_t row = (size_t)t * d;
  // every load of a trip is issued before the first use: one round trip to L2 per four slices
  float4 v[NI];
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);
    v[i] = (c < d && xin && !zero) ? *(const float4 *)(xin + row + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (add.p && !zero) {
    for (int k = 0; k < add.ns; k += 4) {
      const float *pk = add.p + (size_t)k * add.stride + row;
      const int nk = add.ns - k;
      float4 l[4][NI];
#pragma unroll
      for (int q = 0; q < 4; q++)
#pragma unroll
        for (int i = 0; i < NI; i++) {
          const int c = 4 * (threadIdx.x + i * blockDim.x);
          l[q][i] = (c < d && q < nk) ? *(const float4 *)(pk + (size_t)q * add.stride + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
      for (int q = 0; q < 4; q++)   // added in slice order
#pragma unroll
        for (int i = 0; i < NI; i++) { v[i].x += l[q][i].x; v[i].y += l[q][i].y; v[i].z += l[q][i].z; v[i].w += l[q][i].w; }
    }
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);
    if (c < d) {
      if (xout) *(float4 *)(xout + row + c) = v[i];
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = block_sum(ss, red);
  const float sc = 1.0f / sqrtf(ss / (float)d + eps);
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);   // eight lanes hold 32 consecutive columns
    const float h[4] = {v[i].x * sc * wv[i].x, v[i].y * sc * wv[i].y, v[i].z * sc * wv[i].z, v[i].w * sc * wv[i].w};
    if (c < d && hn_out) *(float4 *)(hn_out + row + c) = make_float4(h[0], h[1], h[2], h[3]);
    xp_store4(xp, t, 2, xp_col0 + c, h, lane, c < d);
  }
}
int op_norm_xp(cudaStream_t s, const float *xin, PartIn add, const float *w, float eps, int d, float *xout, XPlanes xp,
               int xp_col0, float *hn_out, const RowSet *rs, int Tmax, int zero_if_pos0) {
  if (d % 32 || xp_col0 % 32 || d > 4 * 4 * NORM_MAXT) return llb_fail("norm: d %d at column %d", d, xp_col0);
  const int d4 = d / 4, ni = (d4 + NORM_MAXT - 1) / NORM_MAXT;
  const int threads = (((d4 + ni - 1) / ni) + 31) & ~31;
#define NORM_GO(NI) CU_OK(llb_launch(k_norm_xp<NI>, dim3(Tmax), dim3(threads), (size_t)(0), s, xin, add, w, eps, d, xout, xp, xp_col0, hn_out, rs, g_streams, zero_if_pos0))
  switch (ni) {
    case 1: NORM_GO(1); break;
    case 2: NORM_GO(2); break;
    case 3: NORM_GO(3); break;
    default: NORM_GO(4); break;
  }
#undef NORM_GO
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- silu(gate) * up -> planes (llb_t_siluq, tools/payload-spec2.patch:114-124) -----------------
// scale (optional): the product of row t, columns [j seg, (j+1) seg) is multiplied by scale[t * (f / seg) + j]
// (the routed experts' weights, folded into the activations the down matrices see)
__global__ void __launch_bounds__(256) k_silu_xp(PartIn g, PartIn u, int f, XPlanes xp, const RowSet *rs, Streams sg, const float *__restrict__ scale, int seg) {
  int rs_n, rs_p0, tl;
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  rs = rs_begin_row(rs, sg, t, rs_n, rs_p0, tl);
  if (tl >= rs_n) return;
  const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);   // four columns per thread, eight lanes per 32-column group
  const bool on = c < f;
  float h[4] = {0.f, 0.f, 0.f, 0.f};
  if (on) {
    const size_t i = (size_t)t * f + c;
    const float4 gv = part_get4(g, i), uv = part_get4(u, i);
    h[0] = silu_f(gv.x) * uv.x; h[1] = silu_f(gv.y) * uv.y; h[2] = silu_f(gv.z) * uv.z; h[3] = silu_f(gv.w) * uv.w;
    if (scale) {
      const float w = scale[(size_t)t * (f / seg) + c / seg];
      h[0] *= w; h[1] *= w; h[2] *= w; h[3] *= w;
    }
  }
  xp_store4(xp, t, 2, c, h, lane, on);
}
int op_silu_xp(cudaStream_t s, PartIn g, PartIn u, int f, XPlanes xp, const RowSet *rs, int Tmax) {
  if (f % 32) return llb_fail("silu: f %d", f);
  CU_OK(llb_launch(k_silu_xp, dim3((f / 4 + 255) / 256, Tmax), dim3(256), (size_t)(0), s, g, u, f, xp, rs, g_streams, (const float *)nullptr, f));
  CU_OK(cudaGetLastError());
  return 0;
}
int op_silu_scaled_xp(cudaStream_t s, PartIn g, PartIn u, int f, XPlanes xp, const RowSet *rs, int Tmax, const float *scale, int seg) {
  if (f % 32 || seg % 4 || f % seg) return llb_fail("silu: f %d, segments of %d", f, seg);
  CU_OK(llb_launch(k_silu_xp, dim3((f / 4 + 255) / 256, Tmax), dim3(256), (size_t)(0), s, g, u, f, xp, rs, g_streams, scale, seg));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- the router of a routed-expert layer (host/llb_host.c:622-724; llb_moe_topk of tools/payload-moeany.patch) ----
// One warp per row of the pass: softmax over the ne logits, the k largest probabilities in descending order with
// ties to the lower index, their weights divided by their sum clamped at 6.103515625e-5; slot k is the shared
// expert (id ne) with weight sigmoid(its gate logit).
template <int NQ> __device__ __forceinline__ void moe_route_row(const float *l, int ne, int nk, int *ids, float *wt, int lane) {
  float p[NQ];   // experts lane, lane + 32, ...: ne <= 32 NQ
  float mx = -INFINITY;
#pragma unroll
  for (int q = 0; q < NQ; q++) {
    const int e = lane + 32 * q;
    p[q] = e < ne ? __ldcg(l + e) : -INFINITY;
    mx = fmaxf(mx, p[q]);
  }
  mx = warp_max(mx);
  float sm = 0.0f;
#pragma unroll
  for (int q = 0; q < NQ; q++) {
    const int e = lane + 32 * q;
    if (e < ne) { p[q] = expf(p[q] - mx); sm += p[q]; }
    else p[q] = -1.0f;
  }
  sm = warp_sum(sm);
  const float inv = 1.0f / sm;
#pragma unroll
  for (int q = 0; q < NQ; q++)
    if (p[q] >= 0.0f) p[q] *= inv;
  float s = 0.0f, mine_w = 0.0f;   // lane j keeps the weight of rank j
  int mine_id = 0;
  for (int j = 0; j < nk; j++) {
    float bv = -1.0f;
    int bi = 0x7fffffff;
#pragma unroll
    for (int q = 0; q < NQ; q++)
      if (p[q] > bv) { bv = p[q]; bi = lane + 32 * q; }   // ascending q: the lane's lowest index among equals
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((bi & 31) == lane) {
#pragma unroll
      for (int q = 0; q < NQ; q++)
        if (q == (bi >> 5)) p[q] = -2.0f;
    }
    s += bv;
    if (j == lane) { mine_w = bv; mine_id = bi; }
  }
  s = s < 6.103515625e-5f ? 6.103515625e-5f : s;
  if (lane < nk) { ids[lane] = mine_id; wt[lane] = mine_w / s; }
  if (lane == 0) {
    ids[nk] = ne;
    wt[nk] = 1.0f / (1.0f + expf(-__ldcg(l + ne)));
  }
}
// Router logits lg[t][r] = W[r] . h[t] for the ne router rows and the shared expert's gate row (row ne): F32
// weights, a block per row (every load of the row in flight at once), all rows of the pass.  The block that
// finishes last (a counter, no waiting) then routes: its warp t takes row t of the pass.
#define MOE_MAXROWS 16   // rows of a pass the router takes (several streams of k + 1 rows)
template <int NQ, int MR>   // MR: the most rows of a pass (8 or 16); two resident blocks a multiprocessor, so that the ne + 1 blocks are one wave
__global__ void __launch_bounds__(256, 2) k_moe_router(const float *__restrict__ W, const float *__restrict__ h, int d, int ne, int nk, float *__restrict__ lg,
                                                    int *__restrict__ ids, float *__restrict__ wt, unsigned int *__restrict__ ctr, const RowSet *rs, int n_all) {
  int rs_n, rs_p0;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, r = blockIdx.x, nrows = ne + 1;
  __shared__ float red[8][MR];
  __shared__ unsigned int last;
  // the row's weights depend on no kernel: fetched before the wait (two float4 per thread cover d <= 2048)
  const float4 *wr = (const float4 *)(W + (size_t)r * d);
  const int c0 = threadIdx.x, c1 = threadIdx.x + 256, nc = d / 4;
  const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const float4 w0 = c0 < nc ? __ldg(wr + c0) : z4, w1 = c1 < nc ? __ldg(wr + c1) : z4;
  rs = rs_begin(rs, rs_n, rs_p0);
  if (n_all > 0) rs_n = n_all;   // a pass over several streams: every row of the pass (a stream's idle rows cost nothing that matters)
  float acc[MR];
#pragma unroll
  for (int t = 0; t < MR; t++) {
    acc[t] = 0.0f;
    if (t < rs_n) {
      const float4 *x = (const float4 *)(h + (size_t)t * d);
      if (c0 < nc) { const float4 v = x[c0]; acc[t] += (w0.x * v.x + w0.y * v.y) + (w0.z * v.z + w0.w * v.w); }
      if (c1 < nc) { const float4 v = x[c1]; acc[t] += (w1.x * v.x + w1.y * v.y) + (w1.z * v.z + w1.w * v.w); }
      for (int c = threadIdx.x + 512; c < nc; c += 256) {
        const float4 w = __ldg(wr + c), v = x[c];
        acc[t] += (w.x * v.x + w.y * v.y) + (w.z * v.z + w.w * v.w);
      }
    }
  }
#pragma unroll
  for (int t = 0; t < MR; t++) {
    if (t < rs_n) {   // the same for every thread of the launch
      const float v = warp_sum(acc[t]);
      if (lane == 0) red[warp][t] = v;
    }
  }
  __syncthreads();
  if (threadIdx.x < rs_n) {
    float v = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; w++) v += red[w][threadIdx.x];
    lg[(size_t)threadIdx.x * nrows + r] = v;
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) last = atomicAdd(ctr, 1u);
  __syncthreads();
  if (last != gridDim.x - 1) return;
  __threadfence();
  if (threadIdx.x == 0) *ctr = 0;   // ready for the next launch (launches of one stream do not overlap here)
  for (int t = warp; t < rs_n; t += 8) moe_route_row<NQ>(lg + (size_t)t * nrows, ne, nk, ids + (size_t)t * (nk + 1), wt + (size_t)t * (nk + 1), lane);
}
static unsigned int *g_moe_ctr = nullptr;
int op_moe_route(cudaStream_t s, const float *Wr, const float *h, int d, int ne, int nk, float *lg, int *ids, float *wt, const RowSet *rs, int Tmax) {
  const int n_all = g_streams.stride ? Tmax : 0;
  if (Tmax > MOE_MAXROWS) return llb_fail("moe route: %d rows in a pass (at most %d)", Tmax, MOE_MAXROWS);
  if (ne < 1 || ne > 1024 || nk < 1 || nk > 32 || nk > ne || d % 4) return llb_fail("moe route: %d experts, top %d, d %d", ne, nk, d);
  if (!g_moe_ctr) {
    CU_OK(cudaMalloc(&g_moe_ctr, 4));
    CU_OK(cudaMemset(g_moe_ctr, 0, 4));
  }
#define ROUTE_GO(NQ, MR) CU_OK(llb_launch(k_moe_router<NQ, MR>, dim3(ne + 1), dim3(256), (size_t)(0), s, Wr, h, d, ne, nk, lg, ids, wt, g_moe_ctr, rs, n_all))
  if (ne <= 256) { if (Tmax <= 8) ROUTE_GO(8, 8); else ROUTE_GO(8, MOE_MAXROWS); }
  else { if (Tmax <= 8) ROUTE_GO(32, 8); else ROUTE_GO(32, MOE_MAXROWS); }
#undef ROUTE_GO
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- per-head QK RMSNorm + partial NEOX RoPE; K and V rows straight into their cache slots
// (llb_t_qkr, tools/payload-spec2.patch:159-204; tools/qwen35_engine.c:523-533, 667-690) ----------
// grid (H + 2 KV, Tmax), block hd.  q input rows are [H][q(hd) | gate(hd)].  The cache keeps a value as two
// fp16 numbers in two planes kv_plane halves apart, hi = fp16(x) and lo = fp16((x - hi) * 2048): the bytes
// of the f32, in the form the attention kernel's tensor-core operands take.
__device__ __forceinline__ void kv_put(__half *c, long long plane, size_t i, float x) {
  const __half h = __float2half_rn(x);
  c[i] = h;
  c[plane + i] = __float2half_rn((x - __half2float(h)) * XP_LO_SCALE);
}
__global__ void k_qkrope(PartIn q, PartIn k, PartIn v, const float *__restrict__ qn_w, const float *__restrict__ kn_w,
                         const double *__restrict__ invfreq, AttnShape sh, float *__restrict__ qout, __half *__restrict__ Kc,
                         __half *__restrict__ Vc, const RowSet *rs, Streams sg, int blk0) {
  int rs_n, rs_p0, tl;
  const int t = blockIdx.y, b = blockIdx.x + blk0, i = threadIdx.x, hd = sh.hd;
  rs = rs_begin_row(rs, sg, t, rs_n, rs_p0, tl);
  extern __shared__ float hv[];
  __shared__ float red[32];
  if (tl >= rs_n) return;
  const int pos = rs_p0 + tl, kvd = sh.KV * hd;
  Kc += (size_t)(t / sg.per) * sh.kv_group; Vc += (size_t)(t / sg.per) * sh.kv_group;   // the row's stream has its own cache
  if (b >= sh.H + sh.KV) {  // V row: copied
    const int g = b - sh.H - sh.KV;
    kv_put(Vc, sh.kv_plane, (size_t)pos * kvd + g * hd + i, part_get(v, (size_t)t * kvd + g * hd + i));
    return;
  }
  float x;
  const float *nw;
  float *dst = nullptr;
  size_t kdst = 0;
  if (b < sh.H) {
    x = part_get(q, (size_t)t * 2 * sh.H * hd + (size_t)b * 2 * hd + i);
    nw = qn_w;
    dst = qout + ((size_t)t * sh.H + b) * hd;
  } else {
    const int g = b - sh.H;
    x = part_get(k, (size_t)t * kvd + g * hd + i);
    nw = kn_w;
    kdst = (size_t)pos * kvd + g * hd;
  }
  const float ss = block_sum(x * x, red);
  const float sc = 1.0f / sqrtf(ss / (float)hd + sh.eps);
  const float y = x * sc * nw[i];
  hv[i] = y;
  __syncthreads();
  float out = y;
  const int half = sh.rope_dim >> 1;
  if (i < sh.rope_dim) {
    const int pi = i < half ? i : i - half;
    const float th = (float)((double)pos * invfreq[pi]);
    const float c = (float)cos((double)th), sn = (float)sin((double)th);
    const float a = hv[pi], bb = hv[pi + half];
    out = i < half ? __fsub_rn(__fmul_rn(a, c), __fmul_rn(bb, sn)) : __fadd_rn(__fmul_rn(a, sn), __fmul_rn(bb, c));
  }
  if (dst) dst[i] = out;
  else kv_put(Kc, sh.kv_plane, kdst + i, out);
}
int op_qkrope(cudaStream_t s, PartIn q, PartIn k, PartIn v, const float *qn_w, const float *kn_w, const double *invfreq,
              AttnShape sh, float *qout, float *Kc, float *Vc, const RowSet *rs, int Tmax, bool kv_only) {
  // blocks 0 .. H-1 are the query heads, then KV key heads, then KV value heads
  const int blk0 = kv_only ? sh.H : 0;
  CU_OK(llb_launch(k_qkrope, dim3(sh.H + 2 * sh.KV - blk0, Tmax), dim3(sh.hd), (size_t)((size_t)sh.hd * 4), s, q, k, v, qn_w, kn_w, invfreq, sh, qout,
                   (__half *)Kc, (__half *)Vc, rs, g_streams, blk0));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- gated DeltaNet ------------------------------------------------------------------------------
// conv1d + SiLU over the position-indexed ring, and the per-head gates
// (llb_t_midconv, tools/payload-spec2.patch:319-350; tools/qwen35_engine.c:589-602).
// grid (ceil(convd/256) + 1, Tmax): the last block computes beta = sigmoid(b), decay = exp(softplus(a + dt) * ssm_a).
__global__ void k_delta_conv(PartIn ring, const float *__restrict__ cw, PartIn bp, PartIn ap,
                             const float *__restrict__ dt, const float *__restrict__ sa, DeltaShape sh, float *__restrict__ y,
                             float *__restrict__ beta, float *__restrict__ decay, const RowSet *rs, Streams sg) {
  int rs_n, rs_p0, tl;
  const int t = blockIdx.y;
  rs = rs_begin_row(rs, sg, t, rs_n, rs_p0, tl);
  if (tl >= rs_n) return;
  if (blockIdx.x == gridDim.x - 1) {
    for (int h = threadIdx.x; h < sh.TR; h += blockDim.x) {
      const float b = part_get(bp, (size_t)t * sh.TR + h), a = part_get(ap, (size_t)t * sh.TR + h);
      beta[t * sh.TR + h] = 1.0f / (1.0f + (float)exp((double)-b));
      const float x = a + dt[h];
      const float sp = x > 20.0f ? x : (float)log1p((double)(float)exp((double)(x < 88.0f ? x : 88.0f)));
      decay[t * sh.TR + h] = (float)exp((double)(sp * sa[h]));
    }
    return;
  }
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= sh.convd) return;
  const int pos = rs_p0 + tl, slot0 = (t / sg.per) * ring.ns * CONV_RING;   // a stream's ring: [K-slice][CONV_RING slots], the streams' rings one after the other
  float acc = 0.0f;
  for (int k = 0; k < sh.KC; k++) {  // tap KC-1 is the current token (tools/qwen35_engine.c:599-600)
    const int slot = slot0 + ((pos - (sh.KC - 1) + k) & (CONV_RING - 1));
    acc = __fadd_rn(acc, __fmul_rn(part_get(ring, (size_t)slot * sh.convd + c), cw[c * sh.KC + k]));
  }
  y[(size_t)t * sh.convd + c] = silu_f(acc);
}
int op_delta_conv(cudaStream_t s, PartIn ring, const float *cw, PartIn bp, PartIn ap, const float *dt, const float *sa,
                  DeltaShape sh, float *y, float *beta, float *decay, const RowSet *rs, int Tmax) {
  if (sh.KC > CONV_RING / 2) return llb_fail("conv kernel %d", sh.KC);
  CU_OK(llb_launch(k_delta_conv, dim3((sh.convd + 255) / 256 + 1, Tmax), dim3(256), (size_t)(0), s, ring, cw, bp, ap, dt, sa, sh, y, beta, decay, rs, g_streams));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- DeltaNet scan + gated RMSNorm as one kernel ------------------------------------------------
// The recurrent scan over the T rows with per-row state checkpoints (llb_t_l2qk + llb_t_gdl,
// tools/payload-spec2.patch:353-410; tools/qwen35_engine.c:610-646), then the gated RMSNorm of each head's
// output into the planes of ssm_out's input (llb_t_grn, tools/payload-spec2.patch:413-447;
// tools/qwen35_engine.c:648-654).  grid (TR, 4) in clusters of four blocks = one value head, 128 threads:
// block (hh, jq) owns state rows j = 32 jq .. 32 jq + 31 of head hh, 32 registers of state per thread
// (thread = row jr, column quarter cq); the RMSNorm's sum of squares over the head's 128 outputs is
// exchanged through distributed shared memory.  The state is read from ring slot sc and the state after
// row r is written to slot (sc + r + 1) % R, so rejecting rows costs nothing: the next cycle simply
// starts from the slot of the last served row.
// (Folding the conv in as well was measured and dropped: every block has to redo the conv of its whole
// q/k group from the four partial-sum slices of the ring, 12x the loads, 65 us against 29 us for three kernels.)
__global__ void __cluster_dims__(1, 4, 1) __launch_bounds__(128)
k_delta_fused(float *__restrict__ S, const SpecCtl *__restrict__ ctl, const float *__restrict__ y, const float *__restrict__ beta,
              const float *__restrict__ decay, PartIn z, const float *__restrict__ nw, DeltaShape sh, XPlanes xp,
              const RowSet *rs, Streams sg, long long s_group) {
  __shared__ __align__(16) float qs[SPEC_MAXT][128], ks[SPEC_MAXT][128];
  __shared__ float vs[SPEC_MAXT][32], db[SPEC_MAXT][2], os[SPEC_MAXT][32], ssq[SPEC_MAXT], tot[SPEC_MAXT];
  __shared__ float red[2 * SPEC_MAXT][4];
  cg::cluster_group cl = cg::this_cluster();
  const int hh = blockIdx.x, jq = blockIdx.y, tid = threadIdx.x, lane = tid & 31, wp = tid >> 5;
  const int g = hh % sh.GK;
  const int jr = tid >> 2, cq = tid & 3;
  const size_t head_sz = 128 * 128, slot_sz = (size_t)sh.TR * head_sz;
  const size_t off = (size_t)hh * head_sz + (size_t)(32 * jq + jr) * 128 + 4 * cq;
  // The committed state (ring slot sc) was written by an earlier pass and sc by that pass's accept kernel: neither
  // depends on the kernel in front, so the 16 KB a block reads from HBM are requested before the dependency wait.
  pdl_trigger();
  {
    // blockIdx.z: the stream -- its control block, its state ring, its rows of the pass
    const size_t zz = blockIdx.z;
    ctl = (const SpecCtl *)((const char *)ctl + zz * sg.stride);
    rs = (const RowSet *)((uintptr_t)rs + zz * sg.stride);
    S += zz * s_group;
    const size_t r0 = sg.stride ? zz * sg.per : 0;
    y += r0 * sh.convd; beta += r0 * sh.TR; decay += r0 * sh.TR; z.p += r0 * sh.vdc;
  }
  const int row0 = sg.stride ? blockIdx.z * sg.per : 0;
  const int R = *(const volatile int *)&ctl->R, sc = *(const volatile int *)&ctl->sc;
  float st[32];
  {
    const float4 *src = (const float4 *)(S + (size_t)sc * slot_sz + off);
#pragma unroll
    for (int i = 0; i < 8; i++) { float4 v = __ldcg(src + 4 * i); st[4 * i] = v.x; st[4 * i + 1] = v.y; st[4 * i + 2] = v.z; st[4 * i + 3] = v.w; }
  }
  const float nwv = nw[32 * jq + lane];
  pdl_wait();
  rs = (const RowSet *)((uintptr_t)rs & ~(uintptr_t)1);
  const int n = rs->n;
  if (n < 1) return;   // every block of every cluster takes the same exit
  float qv[SPEC_MAXT], kv[SPEC_MAXT];
#pragma unroll
  for (int t = 0; t < SPEC_MAXT; t++) {
    qv[t] = t < n ? y[(size_t)t * sh.convd + g * 128 + tid] : 0.0f;
    kv[t] = t < n ? y[(size_t)t * sh.convd + sh.kdc + g * 128 + tid] : 0.0f;
  }
  if (tid < 32) {
#pragma unroll
    for (int t = 0; t < SPEC_MAXT; t++) if (t < n) vs[t][tid] = y[(size_t)t * sh.convd + 2 * sh.kdc + hh * 128 + 32 * jq + tid];
  }
  if (tid < 2 * SPEC_MAXT && (tid >> 1) < n) db[tid >> 1][tid & 1] = (tid & 1) ? beta[(tid >> 1) * sh.TR + hh] : decay[(tid >> 1) * sh.TR + hh];
#pragma unroll
  for (int t = 0; t < SPEC_MAXT; t++) {
    const float a = warp_sum(qv[t] * qv[t]), b = warp_sum(kv[t] * kv[t]);
    if (lane == 0) { red[2 * t][wp] = a; red[2 * t + 1][wp] = b; }
  }
  __syncthreads();
#pragma unroll
  for (int t = 0; t < SPEC_MAXT; t++) {
    if (t < n) {
      const float sq = red[2 * t][0] + red[2 * t][1] + red[2 * t][2] + red[2 * t][3];
      const float sk = red[2 * t + 1][0] + red[2 * t + 1][1] + red[2 * t + 1][2] + red[2 * t + 1][3];
      const float nq = sqrtf(sq), nk = sqrtf(sk);
      const float iq = (1.0f / (nq > sh.eps ? nq : sh.eps)) / sqrtf(128.0f), ik = 1.0f / (nk > sh.eps ? nk : sh.eps);
      qs[t][tid] = qv[t] * iq;
      ks[t][tid] = kv[t] * ik;
    }
  }
  __syncthreads();
  for (int t = 0; t < n; t++) {
    const float dec = db[t][0], bt = db[t][1];
    float kq[32];
#pragma unroll
    for (int i = 0; i < 8; i++) { const float4 v = *(const float4 *)&ks[t][16 * i + 4 * cq]; kq[4 * i] = v.x; kq[4 * i + 1] = v.y; kq[4 * i + 2] = v.z; kq[4 * i + 3] = v.w; }
    float ka[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; i++) { st[i] *= dec; ka[i & 3] += st[i] * kq[i]; }
    float kvacc = (ka[0] + ka[1]) + (ka[2] + ka[3]);
    kvacc += __shfl_xor_sync(0xffffffffu, kvacc, 1);
    kvacc += __shfl_xor_sync(0xffffffffu, kvacc, 2);
    const float delta = (vs[t][jr] - kvacc) * bt;
#pragma unroll
    for (int i = 0; i < 32; i++) st[i] += kq[i] * delta;
#pragma unroll
    for (int i = 0; i < 8; i++) { const float4 v = *(const float4 *)&qs[t][16 * i + 4 * cq]; kq[4 * i] = v.x; kq[4 * i + 1] = v.y; kq[4 * i + 2] = v.z; kq[4 * i + 3] = v.w; }
    float oa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 32; i++) oa[i & 3] += st[i] * kq[i];
    float oacc = (oa[0] + oa[1]) + (oa[2] + oa[3]);
    oacc += __shfl_xor_sync(0xffffffffu, oacc, 1);
    oacc += __shfl_xor_sync(0xffffffffu, oacc, 2);
    if (cq == 0) os[t][jr] = oacc;
    float4 *dst = (float4 *)(S + (size_t)((sc + t + 1) % R) * slot_sz + off);
#pragma unroll
    for (int i = 0; i < 8; i++) dst[4 * i] = make_float4(st[4 * i], st[4 * i + 1], st[4 * i + 2], st[4 * i + 3]);
  }
  __syncthreads();
  if (wp == 0) {
    for (int t = 0; t < n; t++) {
      const float v = os[t][lane], s2 = warp_sum(v * v);
      if (lane == 0) ssq[t] = s2;
    }
  }
  cl.sync();                                   // every block's partial sums of squares are in place
  if (tid < n) {
    float s2 = 0.0f;
    for (unsigned r = 0; r < 4; r++) s2 += *cl.map_shared_rank(&ssq[tid], r);   // rank order: the same sum in all four blocks
    tot[tid] = s2;
  }
  cl.sync();                                   // nobody leaves while a peer still reads its shared memory
  for (int t = wp; t < n; t += 4) {
    const float r = 1.0f / sqrtf(tot[t] / 128.0f + sh.eps);
    const int col = hh * 128 + 32 * jq;
    const float zz = part_get(z, (size_t)t * sh.vdc + col + lane);
    xp_store32(xp, row0 + t, 2, col, os[t][lane] * r * nwv * silu_f(zz), lane);
  }
}
int op_delta_fused(cudaStream_t s, float *S, const SpecCtl *ctl, const float *y, const float *beta, const float *decay, PartIn z,
                   const float *nw, DeltaShape sh, XPlanes xp, const RowSet *rs, int nz, long long s_group) {
  if (sh.SZ != 128) return llb_fail("DeltaNet state size %d (only 128, as host/llb_host.c:1608)", sh.SZ);
  CU_OK(llb_launch(k_delta_fused, dim3(sh.TR, 4, nz), dim3(128), (size_t)0, s, S, ctl, y, beta, decay, z, nw, sh, xp, rs, g_streams, s_group));
  return 0;
}

// ---- top-2 over the logits (llb_t_amaxp / llb_t_amax, tools/payload-spec2.patch:450-483) ---------
// Order: larger value first, lower id on equal values (tools/qwen35_engine.c:763-778).
struct Top2 { float v1; int i1; float v2; int i2; };
__device__ __forceinline__ bool t2_before(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }
__device__ __forceinline__ void t2_push(Top2 &a, float v, int i) {
  if (i < 0) return;
  if (a.i1 < 0 || t2_before(v, i, a.v1, a.i1)) { a.v2 = a.v1; a.i2 = a.i1; a.v1 = v; a.i1 = i; }
  else if (a.i2 < 0 || t2_before(v, i, a.v2, a.i2)) { a.v2 = v; a.i2 = i; }
}
__device__ __forceinline__ Top2 t2_warp(Top2 a) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    float v1 = __shfl_xor_sync(0xffffffffu, a.v1, m), v2 = __shfl_xor_sync(0xffffffffu, a.v2, m);
    int i1 = __shfl_xor_sync(0xffffffffu, a.i1, m), i2 = __shfl_xor_sync(0xffffffffu, a.i2, m);
    t2_push(a, v1, i1);
    t2_push(a, v2, i2);
  }
  return a;
}
__global__ void __launch_bounds__(256) k_top2_part(PartIn logits, int V, long long row_stride,
                                                   float *__restrict__ part, const RowSet *rs, Streams sg) {
  int rs_n, rs_p0, tl;
  const int t = blockIdx.y;
  rs = rs_begin_row(rs, sg, t, rs_n, rs_p0, tl);
  __shared__ Top2 sh[8];
  if (tl >= rs_n) return;
  const size_t z0 = (size_t)t * row_stride;
  const int per = (V + gridDim.x - 1) / gridDim.x, i0 = blockIdx.x * per, i1 = min(V, i0 + per);
  Top2 a = {0.f, -1, 0.f, -1};
  for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) t2_push(a, part_get(logits, z0 + i), i);
  a = t2_warp(a);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x < 32) {
    Top2 b = threadIdx.x < 8 ? sh[threadIdx.x] : Top2{0.f, -1, 0.f, -1};
    b = t2_warp(b);
    if (threadIdx.x == 0) {
      float *p = part + ((size_t)t * gridDim.x + blockIdx.x) * 4;
      p[0] = b.v1; p[1] = __int_as_float(b.i1); p[2] = b.v2; p[3] = __int_as_float(b.i2);
    }
  }
}
int op_top2_part(cudaStream_t s, PartIn logits, int V, long long row_stride, float *part, const RowSet *rs, int Tmax) {
  CU_OK(llb_launch(k_top2_part, dim3(TOP2_NB, Tmax), dim3(256), (size_t)(0), s, logits, V, row_stride, part, rs, g_streams));
  CU_OK(cudaGetLastError());
  return 0;
}
__device__ __forceinline__ Top2 t2_final(const float *part, int t, int lane) {
  Top2 a = {0.f, -1, 0.f, -1};
  for (int b = lane; b < TOP2_NB; b += 32) {
    const float *p = part + ((size_t)t * TOP2_NB + b) * 4;
    t2_push(a, p[0], __float_as_int(p[1]));
    t2_push(a, p[2], __float_as_int(p[3]));
  }
  return t2_warp(a);
}

// ---- fused argmax + accept/reject + commit -------------------------------------------------------
// The reference serves row r while the caller's next token equals the row's input
// (host/llb_host.c:1911) and advances the state ring by the rows served (:1932); under greedy
// sampling that is "accept while argmax(row j) == draft j+1" (host/llb_sampler_impl.h:400-405).
// Here the whole decision runs on the device and also prepares the next cycle: new p0, ring slot,
// committed token, and the drafter's catch-up rows (host/llb_host.c:1815).
__global__ void k_accept(const float *__restrict__ part, SpecCtl *__restrict__ ctl, SpecResult *__restrict__ ring, int ring_n, int per,
                         const int *__restrict__ smp_tok, const float *__restrict__ smp_val) {
  pdl_trigger();
  pdl_wait();
  __shared__ Top2 rows[SPEC_MAXT];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one block per stream: its control block, its result ring, its rows of the pass
  ctl += blockIdx.x; ring += (size_t)blockIdx.x * ring_n;
  const int row0 = blockIdx.x * per;
  const int T = ctl->verify.n;
  if (T < 1) return;   // an empty pass (the sizing run at open, a stream that is not running) decides nothing
  if (warp < T) {
    Top2 a = t2_final(part, row0 + warp, lane);
    // sampling mode: the row's emitted token is the sampler's (llb_smp_verify / llb_smp_sample), not the argmax; the
    // argmax's runner-up stays in the record's third and fourth words
    if (smp_tok) { if (a.i1 != smp_tok[row0 + warp]) { a.i2 = a.i1; a.v2 = a.v1; } a.i1 = smp_tok[row0 + warp]; a.v1 = smp_val[row0 + warp]; }
    if (lane == 0) rows[warp] = a;
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int p0 = ctl->verify.pos0;
  SpecResult *res = ring + (ctl->seq % (unsigned long long)ring_n);
  int served = 1;
  if (ctl->forced > 0) served = T;
  else while (served < T && rows[served - 1].i1 == ctl->verify.tok[served]) served++;
  res->p0 = p0; res->T = T; res->served = served;
  res->pad = (ctl->chk_on && (ctl->chk_pos != p0 || ctl->chk_tok != ctl->verify.tok[0])) ? 1 : 0;
  ctl->chk_on = 0;
  for (int r = 0; r < SPEC_MAXT; r++) {
    res->tin[r] = r < T ? ctl->verify.tok[r] : -1;
    res->ids[r] = r < T ? rows[r].i1 : -1;
    res->top2[r][0] = r < T ? (unsigned)rows[r].i1 : 0u;
    res->top2[r][1] = r < T ? __float_as_uint(rows[r].v1) : 0u;
    res->top2[r][2] = r < T ? (unsigned)rows[r].i2 : 0u;
    res->top2[r][3] = r < T ? __float_as_uint(rows[r].v2) : 0u;
  }
  // commit: the state after the last served row becomes the committed state
  ctl->sc = (ctl->sc + served) % ctl->R;
  const int np0 = p0 + served;
  // the drafter catches up over the served positions p0+1 .. p0+served, whose tokens are the
  // emitted ids (or the given prompt tokens), paired with the trunk's normed hidden rows 0..served-1
  ctl->catchup.n = served;
  ctl->catchup.pos0 = p0 + 1;
  for (int r = 0; r < served; r++) ctl->catchup.tok[r] = ctl->forced > 0 ? ctl->next_tok[r] : rows[r].i1;
  const int tok0 = ctl->catchup.tok[served - 1];
  if (ctl->hist)   // the prompt-lookup drafter searches the whole token history
    for (int r = 0; r < served; r++) ctl->hist[p0 + 1 + r] = ctl->catchup.tok[r];
  int Tn = ctl->k + 1;
  if (np0 + Tn > ctl->max_pos) Tn = ctl->max_pos - np0 > 0 ? ctl->max_pos - np0 : 1;
  ctl->verify.n = Tn;
  ctl->verify.pos0 = np0;
  ctl->verify.tok[0] = tok0;
  for (int r = 0; r < SPEC_MAXT; r++) ctl->verify.slot[r] = (np0 + r) & (CONV_RING - 1);
  ctl->forced = 0;
  __threadfence_system();
  res->seq = ctl->seq + 1;   // written last: the host polls it
  ctl->seq += 1;
}
int op_accept(cudaStream_t s, const float *part, SpecCtl *ctl, SpecResult *ring, int ring_n, int Tmax, int nz, int per, const int *smp_tok,
              const float *smp_val) {
  CU_OK(llb_launch(k_accept, dim3(nz), dim3(32 * (nz > 1 ? per : Tmax)), (size_t)(0), s, part, ctl, ring, ring_n, per, smp_tok, smp_val));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- prompt-lookup drafter (spec_draft, host/llb_host.c:1655-1676) --------------------------------
// The reference scans the token history on the host every cycle: the LATEST earlier position j whose last
// L = 3, 2, 1 tokens equal the history's last L, longest L first; the up-to-k tokens after j are the drafts.
// Here one block scans the device copy of the history right after the accept kernel, so the next cycle's
// rows are complete before its graph is launched.  Each thread keeps the latest match per L of its stride.
__global__ void __launch_bounds__(256) k_lookup_draft(SpecCtl *__restrict__ ctl) {
  pdl_trigger();
  pdl_wait();
  __shared__ int best[3];
  ctl += blockIdx.x;   // one block per stream
  const int *hist = ctl->hist;
  const int pos = ctl->verify.pos0;
  if (!hist || ctl->verify.n < 1) return;
  if (threadIdx.x < 3) best[threadIdx.x] = -1;
  __syncthreads();
  const int t0 = hist[pos], t1 = pos >= 1 ? hist[pos - 1] : -1, t2 = pos >= 2 ? hist[pos - 2] : -1;
  int b1 = -1, b2 = -1, b3 = -1;
  for (int j = pos - 1 - (int)threadIdx.x; j >= 0; j -= blockDim.x) {
    if (hist[j] != t0) continue;
    if (b1 < 0) b1 = j;
    if (j >= 1 && pos >= 2 && hist[j - 1] == t1) {
      if (b2 < 0) b2 = j;
      if (j >= 2 && pos >= 3 && hist[j - 2] == t2) { if (b3 < 0) b3 = j; }
    }
    if (b3 >= 0) break;   // later iterations only see smaller j
  }
  if (b1 >= 0) atomicMax(&best[0], b1);
  if (b2 >= 0) atomicMax(&best[1], b2);
  if (b3 >= 0) atomicMax(&best[2], b3);
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int j = best[2] >= 0 ? best[2] : best[1] >= 0 ? best[1] : best[0];
  int n = 0;
  if (j >= 0) {
    const int room = ctl->verify.n - 1;   // the accept kernel already clipped the rows to the context
    while (n < ctl->k && n < room && j + 1 + n <= pos) { ctl->verify.tok[1 + n] = hist[j + 1 + n]; n++; }
  }
  ctl->verify.n = 1 + n;
}
int op_lookup_draft(cudaStream_t s, SpecCtl *ctl, int nz) {
  CU_OK(llb_launch(k_lookup_draft, dim3(nz), dim3(256), (size_t)(0), s, ctl));
  CU_OK(cudaGetLastError());
  return 0;
}

// After a drafter pass: the head argmax of its last row is draft j (mapped through the draft-vocab ids,
// host/llb_host.c:1800-1807); it becomes verify input j and the token of the next chained row, whose hidden
// is the drafter's own normed hidden of that last row (host/llb_host.c:1824-1827).
__global__ void k_draft_pick(const float *__restrict__ part, const int *__restrict__ ids, SpecCtl *__restrict__ ctl,
                             int from_chain, int j, const float *__restrict__ mt_hn, float *__restrict__ chain_h, int d, int per) {
  pdl_trigger();
  pdl_wait();
  __shared__ int s_tok;
  // one block per stream: its control block and its rows of the drafter pass; the chained row is the stream's row 0
  ctl += blockIdx.x;
  const size_t row0 = (size_t)blockIdx.x * per;
  part += row0 * TOP2_NB * 4; mt_hn += row0 * d; chain_h += row0 * d;
  const RowSet *rs = from_chain ? &ctl->chain : &ctl->catchup;
  const int last = rs->n - 1;
  if (last < 0) return;
  if (threadIdx.x < 32) {
    Top2 a = t2_final(part, last, threadIdx.x);
    if (threadIdx.x == 0) s_tok = a.i1 < 0 ? 0 : ids ? ids[a.i1] : a.i1;
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) chain_h[c] = mt_hn[(size_t)last * d + c];
  if (threadIdx.x == 0) {
    const int p = ctl->verify.pos0;
    if (j < ctl->verify.n) ctl->verify.tok[j] = s_tok;
    ctl->chain.n = 1;
    ctl->chain.pos0 = p + j;
    ctl->chain.tok[0] = s_tok;
    ctl->chain.slot[0] = 0;
  }
}
int op_draft_pick(cudaStream_t s, const float *part, const int *ids, SpecCtl *ctl, int from_chain, int j, const float *mt_hn,
                  float *chain_h, int d, int nz, int per) {
  CU_OK(llb_launch(k_draft_pick, dim3(nz), dim3(256), (size_t)(0), s, part, ids, ctl, from_chain, j, mt_hn, chain_h, d, per));
  CU_OK(cudaGetLastError());
  return 0;
}
