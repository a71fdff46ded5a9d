// pf.cu -- the prompt path: a chunk of up to PF_RMAX = 256 prompt rows per pass, dense GEMMs on tcgen05 (pfmm.cuh) and
// row-batched small ops.  It stands where the reference has its fast prefill tier (host/llb_pf.h:551 pf_take; kernels
// tools/pf27/pfmm.cuh, host/llb_pf.cuh; hand-off into the speculative state host/llb_host.c:1831-1899 spec_pf /
// spec_take): the trunk's K/V rows, conv history and DeltaNet state after the chunk, the drafter's K/V rows for the
// chunk's positions (k and v only: no drafter attention, FFN or head), and the normed hidden row it continues from.
// The arithmetic follows the CPU engine (tools/qwen35_engine.c:510-761) like the T-row kernels of ops_model.cu; what
// differs is the GEMM operand precision (fp16, see pfmm.cuh) and that a DeltaNet layer scans the chunk's rows in one
// kernel with the state in registers, writing the state once.
#include "pfmm.cuh"
#include "model.cuh"
#include "pf.cuh"

static unsigned int *g_pf_err = nullptr;   // device word: a bounded wait of k_pfmm ran out

template <int FMT> static int pf_attr() {
  CU_OK(cudaFuncSetAttribute(k_pfmm<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, PF_SMEM));
  return 0;
}
int pf_setup(void) {
  if (pf_attr<LLB_FM_Q4_K>() || pf_attr<LLB_FM_Q5_K>() || pf_attr<LLB_FM_Q6_K>() || pf_attr<LLB_FM_Q8_0>()) return -1;
  if (!g_pf_err) {
    CU_OK(cudaMalloc(&g_pf_err, 4));
    CU_OK(cudaMemset(g_pf_err, 0, 4));
  }
  return 0;
}
int pf_wait_errors(void) {
  unsigned int v = 0;
  if (g_pf_err && cudaMemcpy(&v, g_pf_err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)v;
}
int pf_wait_errors_clear(void) {
  if (g_pf_err) CU_OK(cudaMemset(g_pf_err, 0, 4));
  return 0;
}

// K-slices of a dense launch: whole waves of (tile, slice) units over the SMs, each unit costing its slice's
// super-blocks plus about two super-blocks' worth of pipeline fill and epilogue; slices are whole super-blocks.
int pf_pick_ksplit(int ntiles, int nsb, int sms) {
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= 8 && ks <= nsb; ks++) {
    const long long units = (long long)ntiles * ks, waves = (units + sms - 1) / sms;
    const double cost = (double)waves * ((nsb + ks - 1) / ks + 2.0) * (1.0 + 0.03 * (ks - 1));   // the longest slice sets the pace
    if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
  }
  return best;
}

// fills the tile table; K-slices are whole super-blocks, as equal as they come
int pf_gemm(cudaStream_t s, int fmt, PfArgs &a) {
  if (a.nmat < 1 || a.nmat > PF_MAXMAT) return llb_fail("pf gemm: nmat %d", a.nmat);
  if (a.K % 256 || a.ksplit < 1 || a.ksplit > a.K / 256) return llb_fail("pf gemm: K %d in %d slices", a.K, a.ksplit);
  if (a.R < 1 || a.R > PF_RMAX) return llb_fail("pf gemm: %d rows", a.R);
  a.t128[0] = 0;
  for (int i = 0; i < PF_MAXMAT; i++) a.t128[i + 1] = a.t128[i] + (i < a.nmat ? (a.m[i].rows + 127) / 128 : 0);
  a.err = g_pf_err;
  const int units = a.t128[a.nmat] * a.ksplit;
  if (units < 1) return 0;
  const int grid = units < g_llb.sms ? units : g_llb.sms;
  cudaError_t e;
  switch (fmt) {
    case LLB_FM_Q4_K: e = llb_launch(k_pfmm<LLB_FM_Q4_K>, dim3(grid), dim3(PF_THREADS), (size_t)PF_SMEM, s, a); break;
    case LLB_FM_Q5_K: e = llb_launch(k_pfmm<LLB_FM_Q5_K>, dim3(grid), dim3(PF_THREADS), (size_t)PF_SMEM, s, a); break;
    case LLB_FM_Q6_K: e = llb_launch(k_pfmm<LLB_FM_Q6_K>, dim3(grid), dim3(PF_THREADS), (size_t)PF_SMEM, s, a); break;
    case LLB_FM_Q8_0: e = llb_launch(k_pfmm<LLB_FM_Q8_0>, dim3(grid), dim3(PF_THREADS), (size_t)PF_SMEM, s, a); break;
    default: return llb_fail("pf gemm: format %d has no kernel", fmt);
  }
  if (e != cudaSuccess) return llb_fail("k_pfmm launch: %s", cudaGetErrorString(e));
  return 0;
}

// ---- row-batched small ops: one launch covers the R rows of the chunk --------------------------------
// Every kernel triggers its dependents first and waits for its producer before it touches a buffer another kernel writes.
// Those buffers are reused by every layer and the chain of resident, waiting kernels can be a dozen launches deep (the scan
// of a chunk is long), so loads of them bypass L1 (__ldcg / part_get): an SM's L1 may still hold what an earlier layer put
// in the same buffer.  Found the hard way: with plain loads the third DeltaNet layer of a chunk read the second one's rows.
__device__ __forceinline__ float pf_warp_sum(float v) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}
__device__ __forceinline__ float pf_block_sum(float v, float *red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = pf_warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.0f;
  for (int i = 0; i < nw; i++) t += red[i];
  return t;
}
__device__ __forceinline__ float pf_silu(float x) { return x / (1.0f + expf(-x)); }

// embedding rows of the chunk's tokens (llb_embedk; bit-exact dequantisation)
__global__ void k_pf_embed(int fmt, const uint8_t *__restrict__ W, int d, const int *__restrict__ ids, float *__restrict__ x) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y;
  const uint8_t *row = W + (size_t)ids[t] * dev_row_bytes(fmt, d);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < d; c += gridDim.x * blockDim.x) x[(size_t)t * d + c] = deq_elem(fmt, row, d, c);
}
int op_pf_embed(cudaStream_t s, int fmt, const uint8_t *W, int d, const int *ids, int R, float *x) {
  CU_OK(llb_launch(k_pf_embed, dim3((d + 255) / 256, R), dim3(256), (size_t)0, s, fmt, W, d, ids, x));
  return 0;
}

// v = xin + sum(partials); xout = v (optional); h = (v * s) * w with s = 1 / sqrt(mean(v^2) + eps) (rms_norm,
// tools/qwen35_engine.c:510-515); h goes to the k-group-major fp16 activations at column kg_col0 and, optionally,
// to hn_out as f32.  One block per row, as k_norm_xp.
#define PF_NORM_MAXT 1024
template <int NI>
__global__ void __launch_bounds__(PF_NORM_MAXT) k_pf_norm(const float *__restrict__ xin, PartIn add, const float *__restrict__ w, float eps, int d,
                                                          float *__restrict__ xout, __half *__restrict__ kg, int kg_K, int kg_col0, float *__restrict__ hn_out) {
  float4 wv[NI];
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);
    wv[i] = c < d ? *(const float4 *)(w + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int t = blockIdx.x;
  const size_t row = (size_t)t * d;
  float4 v[NI];
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);
    v[i] = (c < d && xin) ? __ldcg((const float4 *)(xin + row + c)) : make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < d && add.p) { const float4 p = part_get4(add, row + c); v[i].x += p.x; v[i].y += p.y; v[i].z += p.z; v[i].w += p.w; }
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
  ss = pf_block_sum(ss, red);
  const float sc = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
  for (int i = 0; i < NI; i++) {
    const int c = 4 * (threadIdx.x + i * blockDim.x);
    if (c >= d) continue;
    const float h0 = v[i].x * sc * wv[i].x, h1 = v[i].y * sc * wv[i].y, h2 = v[i].z * sc * wv[i].z, h3 = v[i].w * sc * wv[i].w;
    if (hn_out) *(float4 *)(hn_out + row + c) = make_float4(h0, h1, h2, h3);
    if (kg) pf_kg_store4(kg, kg_K, t, kg_col0 + c, h0, h1, h2, h3);
  }
}
int op_pf_norm(cudaStream_t s, const float *xin, PartIn add, const float *w, float eps, int d, float *xout, __half *kg, int kg_K, int kg_col0, float *hn_out, int R) {
  if (d % 8 || kg_col0 % 8 || d > 4 * 4 * PF_NORM_MAXT) return llb_fail("pf norm: d %d at column %d", d, kg_col0);
  const int d4 = d / 4, ni = (d4 + PF_NORM_MAXT - 1) / PF_NORM_MAXT;
  const int threads = (((d4 + ni - 1) / ni) + 31) & ~31;
#define PF_NORM_GO(NI) CU_OK(llb_launch(k_pf_norm<NI>, dim3(R), dim3(threads), (size_t)0, s, xin, add, w, eps, d, xout, kg, kg_K, kg_col0, hn_out))
  switch (ni) {
    case 1: PF_NORM_GO(1); break;
    case 2: PF_NORM_GO(2); break;
    case 3: PF_NORM_GO(3); break;
    default: PF_NORM_GO(4); break;
  }
#undef PF_NORM_GO
  return 0;
}

// silu(gate) * up -> activations of ffn_down (llb_t_siluq)
__global__ void __launch_bounds__(256) k_pf_silu(PartIn g, PartIn u, int f, __half *__restrict__ kg) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= f) return;
  const size_t i = (size_t)t * f + c;
  const float4 gv = part_get4(g, i), uv = part_get4(u, i);
  pf_kg_store4(kg, f, t, c, pf_silu(gv.x) * uv.x, pf_silu(gv.y) * uv.y, pf_silu(gv.z) * uv.z, pf_silu(gv.w) * uv.w);
}
int op_pf_silu(cudaStream_t s, PartIn g, PartIn u, int f, __half *kg, int R) {
  CU_OK(llb_launch(k_pf_silu, dim3((f / 4 + 255) / 256, R), dim3(256), (size_t)0, s, g, u, f, kg));
  return 0;
}

// ---- gated DeltaNet over a chunk (tools/qwen35_engine.c:581-662) -----------------------------------
// beta = sigmoid(b), decay = exp(softplus(a + dt) * ssm_a) for every (row, head); transcendentals through double as the
// T-row kernel k_delta_conv and the CPU engine do
__global__ void k_pf_gates(PartIn bp, PartIn ap, const float *__restrict__ dt, const float *__restrict__ sa, int TR, float *__restrict__ beta,
                           float *__restrict__ decay) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  for (int h = threadIdx.x; h < TR; h += blockDim.x) {
    const float b = part_get(bp, (size_t)t * TR + h), a = part_get(ap, (size_t)t * TR + h);
    beta[t * TR + h] = 1.0f / (1.0f + (float)exp((double)-b));
    const float x = a + dt[h];
    const float sp = x > 20.0f ? x : (float)log1p((double)(float)exp((double)(x < 88.0f ? x : 88.0f)));
    decay[t * TR + h] = (float)exp((double)(sp * sa[h]));
  }
}
// conv1d + SiLU: row t of the chunk (position p0 + t) reads its KC - 1 predecessors from the chunk's own raw rows or,
// before the chunk's first row, from the position-indexed ring (tap KC - 1 is the current token, :599-600)
__global__ void k_pf_conv(PartIn qkv, PartIn ring, const float *__restrict__ cw, int convd, int KC, int p0, float *__restrict__ y) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= convd) return;
  float acc = 0.0f;
  for (int k = 0; k < KC; k++) {
    const int tt = t - (KC - 1) + k;
    const float x = tt >= 0 ? part_get(qkv, (size_t)tt * convd + c) : part_get(ring, (size_t)((p0 + tt) & (CONV_RING - 1)) * convd + c);
    acc = __fadd_rn(acc, __fmul_rn(x, cw[c * KC + k]));
  }
  y[(size_t)t * convd + c] = pf_silu(acc);
}
// the chunk's last rows become the ring's history: whole values into slice 0, zeros into the other K-slices
__global__ void k_pf_ring(PartIn qkv, float *__restrict__ ring, int ring_ks, long long ring_stride, int convd, int p0, int t0) {
  pdl_trigger();
  pdl_wait();
  const int t = t0 + blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= convd) return;
  const size_t dst = (size_t)((p0 + t) & (CONV_RING - 1)) * convd + c;
  ring[dst] = part_get(qkv, (size_t)t * convd + c);
  for (int k = 1; k < ring_ks; k++) ring[(size_t)k * ring_stride + dst] = 0.0f;
}
// per row and q/k group: q / max(|q|, eps) / sqrt(128), k / max(|k|, eps), in place (no eps inside the root, :613-620)
__global__ void __launch_bounds__(128) k_pf_l2(float *__restrict__ y, int convd, int kdc, float eps) {
  pdl_trigger();
  pdl_wait();
  __shared__ float red[32];
  const int g = blockIdx.x, t = blockIdx.y, i = threadIdx.x;
  float *q = y + (size_t)t * convd + g * 128 + i, *k = q + kdc;
  const float qv = __ldcg(q), kv = __ldcg(k);
  const float nq = sqrtf(pf_block_sum(qv * qv, red)), nk = sqrtf(pf_block_sum(kv * kv, red));
  *q = qv * ((1.0f / (nq > eps ? nq : eps)) / sqrtf(128.0f));
  *k = kv * (1.0f / (nk > eps ? nk : eps));
}

// The recurrence over the chunk's R rows.  grid (TR, 4), 128 threads, as k_delta_fused: block (hh, jq) keeps state rows
// 32 jq .. 32 jq + 31 of value head hh in registers (thread = row jr, column quarter cq) from the first row of the chunk
// to the last and writes the state back once.  Rows come in batches of eight through double-buffered shared memory:
// the next batch's q, k, v, beta and decay are requested before the current batch is computed.  Per row and state
// row j: S_j *= decay; delta = (v_j - S_j . k) * beta; S_j += k * delta; o_j = S_j . q   (:630-646)
#define PF_SCAN_B 8
__global__ void __launch_bounds__(128) k_pf_scan(float *__restrict__ S, const SpecCtl *__restrict__ ctl, const float *__restrict__ y,
                                                 const float *__restrict__ beta, const float *__restrict__ decay, DeltaShape sh, float *__restrict__ o, int R) {
  __shared__ __align__(16) float qs[2][PF_SCAN_B][128], ks[2][PF_SCAN_B][128];
  __shared__ float vs[2][PF_SCAN_B][32], db[2][PF_SCAN_B][2];
  const int hh = blockIdx.x, jq = blockIdx.y, tid = threadIdx.x, g = hh % sh.GK, jr = tid >> 2, cq = tid & 3;
  const size_t head_sz = 128 * 128, slot_sz = (size_t)sh.TR * head_sz;
  const size_t off = (size_t)hh * head_sz + (size_t)(32 * jq + jr) * 128 + 4 * cq;
  pdl_trigger();
  float4 *Sp = (float4 *)(S + (size_t)(*(const volatile int *)&ctl->sc) * slot_sz + off);   // the committed slot: stable during the pass
  float st[32];
#pragma unroll
  for (int i = 0; i < 8; i++) { const float4 v = __ldcg(Sp + 4 * i); st[4 * i] = v.x; st[4 * i + 1] = v.y; st[4 * i + 2] = v.z; st[4 * i + 3] = v.w; }
  pdl_wait();
  float rq[PF_SCAN_B], rk[PF_SCAN_B], rv[PF_SCAN_B], rd = 0.0f;
  auto fetch = [&](int b) {
#pragma unroll
    for (int u = 0; u < PF_SCAN_B; u++) {
      const int t = b * PF_SCAN_B + u;
      const float *row = y + (size_t)min(t, R - 1) * sh.convd;
      rq[u] = __ldcg(row + g * 128 + tid);
      rk[u] = __ldcg(row + sh.kdc + g * 128 + tid);
      rv[u] = tid < 32 ? __ldcg(row + 2 * sh.kdc + hh * 128 + 32 * jq + tid) : 0.0f;
    }
    if (tid < 2 * PF_SCAN_B) { const int t = min(b * PF_SCAN_B + (tid >> 1), R - 1); rd = __ldcg((tid & 1) ? beta + t * sh.TR + hh : decay + t * sh.TR + hh); }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int u = 0; u < PF_SCAN_B; u++) { qs[buf][u][tid] = rq[u]; ks[buf][u][tid] = rk[u]; if (tid < 32) vs[buf][u][tid] = rv[u]; }
    if (tid < 2 * PF_SCAN_B) db[buf][tid >> 1][tid & 1] = rd;
  };
  const int nb = (R + PF_SCAN_B - 1) / PF_SCAN_B;
  fetch(0);
  stash(0);
  __syncthreads();
  for (int b = 0; b < nb; b++) {
    const int buf = b & 1;
    if (b + 1 < nb) fetch(b + 1);
    const int n = min(PF_SCAN_B, R - b * PF_SCAN_B);
    for (int u = 0; u < n; u++) {
      const float dec = db[buf][u][0], bt = db[buf][u][1];
      float kq[32];
#pragma unroll
      for (int i = 0; i < 8; i++) { const float4 v = *(const float4 *)&ks[buf][u][16 * i + 4 * cq]; kq[4 * i] = v.x; kq[4 * i + 1] = v.y; kq[4 * i + 2] = v.z; kq[4 * i + 3] = v.w; }
      float ka[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 32; i++) { st[i] *= dec; ka[i & 3] += st[i] * kq[i]; }
      float kvacc = (ka[0] + ka[1]) + (ka[2] + ka[3]);
      kvacc += __shfl_xor_sync(0xffffffffu, kvacc, 1);
      kvacc += __shfl_xor_sync(0xffffffffu, kvacc, 2);
      const float delta = (vs[buf][u][jr] - kvacc) * bt;
#pragma unroll
      for (int i = 0; i < 32; i++) st[i] += kq[i] * delta;
#pragma unroll
      for (int i = 0; i < 8; i++) { const float4 v = *(const float4 *)&qs[buf][u][16 * i + 4 * cq]; kq[4 * i] = v.x; kq[4 * i + 1] = v.y; kq[4 * i + 2] = v.z; kq[4 * i + 3] = v.w; }
      float oa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 32; i++) oa[i & 3] += st[i] * kq[i];
      float oacc = (oa[0] + oa[1]) + (oa[2] + oa[3]);
      oacc += __shfl_xor_sync(0xffffffffu, oacc, 1);
      oacc += __shfl_xor_sync(0xffffffffu, oacc, 2);
      if (cq == 0) o[(size_t)(b * PF_SCAN_B + u) * sh.vdc + hh * 128 + 32 * jq + jr] = oacc;
    }
    if (b + 1 < nb) stash(buf ^ 1);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 8; i++) Sp[4 * i] = make_float4(st[4 * i], st[4 * i + 1], st[4 * i + 2], st[4 * i + 3]);
}
// gated RMSNorm of each head's output -> activations of ssm_out (:648-654); a warp per (head, row)
__global__ void __launch_bounds__(32) k_pf_gnorm(const float *__restrict__ o, PartIn z, const float *__restrict__ nw, int vdc, float eps, __half *__restrict__ kg) {
  pdl_trigger();
  pdl_wait();
  const int hh = blockIdx.x, t = blockIdx.y, i = threadIdx.x;
  const size_t idx = (size_t)t * vdc + hh * 128 + 4 * i;
  const float4 v = __ldcg((const float4 *)(o + idx)), zz = part_get4(z, idx), w = *(const float4 *)(nw + 4 * i);
  const float r = 1.0f / sqrtf(pf_warp_sum(v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w) / 128.0f + eps);
  pf_kg_store4(kg, vdc, t, hh * 128 + 4 * i, v.x * r * w.x * pf_silu(zz.x), v.y * r * w.y * pf_silu(zz.y), v.z * r * w.z * pf_silu(zz.z), v.w * r * w.w * pf_silu(zz.w));
}

// One DeltaNet layer's ops between its input GEMM (qkv | z | beta | alpha) and its output GEMM, for R rows at p0 ...
int op_pf_delta(cudaStream_t s, PartIn qkv, PartIn z, PartIn bp, PartIn ap, float *ring, int ring_ks, const float *cw, const float *dt, const float *sa,
                const float *nw, DeltaShape sh, float *S, const SpecCtl *ctl, float *y, float *beta, float *decay, float *o, __half *kg, int p0, int R) {
  if (sh.SZ != 128 || sh.KC > CONV_RING / 2) return llb_fail("pf delta: state size %d, conv kernel %d", sh.SZ, sh.KC);
  const long long rstride = (long long)CONV_RING * sh.convd;
  CU_OK(llb_launch(k_pf_gates, dim3(R), dim3(64), (size_t)0, s, bp, ap, dt, sa, sh.TR, beta, decay));
  CU_OK(llb_launch(k_pf_conv, dim3((sh.convd + 255) / 256, R), dim3(256), (size_t)0, s, qkv, PartIn{ring, ring_ks, rstride}, cw, sh.convd, sh.KC, p0, y));
  const int nr = R < CONV_RING ? R : CONV_RING;
  CU_OK(llb_launch(k_pf_ring, dim3((sh.convd + 255) / 256, nr), dim3(256), (size_t)0, s, qkv, ring, ring_ks, rstride, sh.convd, p0, R - nr));
  CU_OK(llb_launch(k_pf_l2, dim3(sh.GK, R), dim3(128), (size_t)0, s, y, sh.convd, sh.kdc, sh.eps));
  CU_OK(llb_launch(k_pf_scan, dim3(sh.TR, 4), dim3(128), (size_t)0, s, S, ctl, (const float *)y, (const float *)beta, (const float *)decay, sh, o, R));
  CU_OK(llb_launch(k_pf_gnorm, dim3(sh.TR, R), dim3(32), (size_t)0, s, (const float *)o, z, nw, sh.vdc, sh.eps, kg));
  return 0;
}

// ---- operator entry point: the dense GEMM alone ------------------------------------------------------
// f32 rows [R][K] -> fp16, k-group major
__global__ void __launch_bounds__(256) k_pf_pack(const float *__restrict__ x, int K, __half *__restrict__ kg) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
  if (c >= K) return;
  const float4 v = __ldcg((const float4 *)(x + (size_t)t * K + c));
  pf_kg_store4(kg, K, t, c, v.x, v.y, v.z, v.w);
}
int op_pf_pack(cudaStream_t s, const float *x, int K, int R, __half *kg) {
  CU_OK(llb_launch(k_pf_pack, dim3((K / 4 + 255) / 256, R), dim3(256), (size_t)0, s, x, K, kg));
  return 0;
}

extern "C" __attribute__((visibility("default")))
int llb_b200_pf_gemm(int fmt, unsigned long long w, int rows, int K, unsigned long long x_f32, int R, unsigned long long out_f32, int ksplit) {
  if (!g_llb.stream) return llb_fail("llb_b200_init has not been called");
  if (K < 256 || K % 256 || rows < 1 || R < 1 || R > PF_RMAX) return llb_fail("pf_gemm: rows %d, K %d, R %d (K a multiple of 256, R up to %d)", rows, K, R, PF_RMAX);
  if (!dev_row_bytes(fmt, K) || fmt == LLB_FM_F32) return llb_fail("pf_gemm: format %d has no kernel", fmt);
  if (pf_setup()) return -1;
  const int nsb = K / 256;
  if (ksplit <= 0) ksplit = pf_pick_ksplit((rows + 127) / 128, nsb, g_llb.sms);
  if (ksplit > nsb) return llb_fail("pf_gemm: %d K-slices of %d super-blocks", ksplit, nsb);
  __half *kg = nullptr;
  float *parts = nullptr;
  CU_OK(cudaMalloc(&kg, 2 * pf_kg_halves(K) * 2));      // two units of 128 rows
  CU_OK(cudaMemsetAsync(kg, 0, 2 * pf_kg_halves(K) * 2, g_llb.stream));
  if (ksplit > 1) CU_OK(cudaMalloc(&parts, (size_t)ksplit * R * rows * 4));
  int rc = op_pf_pack(g_llb.stream, (const float *)(uintptr_t)x_f32, K, R, kg);
  PfArgs a;
  memset(&a, 0, sizeof a);
  a.nmat = 1; a.K = K; a.ksplit = ksplit; a.R = R; a.x = kg;
  a.m[0].W = (const uint8_t *)(uintptr_t)w; a.m[0].rows = rows; a.m[0].ostride = rows;
  a.m[0].out = ksplit > 1 ? parts : (float *)(uintptr_t)out_f32; a.m[0].split_stride = (long long)R * rows;
  if (!rc) rc = pf_gemm(g_llb.stream, fmt, a);
  if (!rc && ksplit > 1) rc = ops_sum_parts(g_llb.stream, parts, ksplit, (long long)R * rows, R * rows, (float *)(uintptr_t)out_f32);
  cudaStreamSynchronize(g_llb.stream);
  cudaFree(kg);
  if (parts) cudaFree(parts);
  if (!rc && cudaGetLastError() != cudaSuccess) rc = llb_fail("pf_gemm: a kernel failed");
  return rc;
}
