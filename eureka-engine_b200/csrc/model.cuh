// model.cuh -- device-side control block and kernel launchers of the verify / draft passes.
#pragma once
#include <stdint.h>
#include "host.cuh"

#define SPEC_MAXT 8      // rows per pass (k + 1 <= 8, host/llb_host.c:1608 limits k to 0..7)
#define CONV_RING 16     // conv history slots, indexed by position & 15 (host/llb_host.c:1630)
#define TOP2_NB 64       // blocks of the first argmax stage

// A set of rows a pass works on: n rows at positions pos0 .. pos0+n-1 with input tokens tok[].
struct RowSet {
  int n;
  int pos0;
  int tok[SPEC_MAXT];
  int slot[SPEC_MAXT];   // conv ring slot of each row, (pos0 + t) & 15
};

// Everything a cycle needs lives on the device, so a cycle is one CUDA graph replay with no host
// decision inside (the reference makes them on the host: host/llb_host.c:1902-1950).
struct SpecCtl {
  RowSet verify;         // rows of the (k+1)-token verify pass
  RowSet catchup;        // drafter rows over the positions the last cycle served (host/llb_host.c:1815)
  RowSet chain;          // the drafter's single chained row (host/llb_host.c:1824-1827)
  int sc;                // DeltaNet state-ring slot holding the committed state
  int R;                 // ring slots, k + 2 (host/llb_host.c:1621)
  int k;                 // drafts per cycle
  int forced;            // > 0: a prompt chunk; the rows and their successors are given, all are served
  int next_tok[SPEC_MAXT];
  int max_pos;           // exclusive bound on positions (context capacity)
  int chk_on, chk_pos, chk_tok;   // the caller's (pos, tok) for this cycle, checked against the committed state
  int err;               // sticky device-side error word (0 = none)
  int *hist;             // prompt-lookup drafter only: the token at every position up to the committed one, else null
  unsigned long long seq;
};

// What one cycle reports to the host (written to a pinned ring by the accept kernel).
struct SpecResult {
  unsigned long long seq;
  int p0, T, served, pad;
  int tin[SPEC_MAXT];            // verify inputs: tin[0] the committed token, then the drafts
  int ids[SPEC_MAXT];            // argmax of each row; ids[0..served-1] are emitted
  unsigned int top2[SPEC_MAXT][4];  // id1, bits(v1), id2, bits(v2) per row (tools/qwen35_engine.c:985)
};

// a tensor that may be split into K-slice partial sums: value(i) = sum_k p[k*stride + i]
struct PartIn {
  const float *p;
  int ns;
  long long stride;
};
// (the slices are added in index order; four loads are in flight at a time so that a value split
// seven ways costs two round trips to L2, not seven)
// four consecutive values (i a multiple of 4, strides multiples of 4): all slices of a trip in flight at once
// (loads of another kernel's output go to L2, ld.global.cg: under programmatic dependent launch a consumer kernel can be
// resident on an SM long before its producer runs, and that SM's L1 may still hold the buffer's previous contents)
__device__ __forceinline__ float4 part_get4(const PartIn &a, size_t i) {
  float4 v = __ldcg((const float4 *)(a.p + i));
  for (int k = 1; k < a.ns; k += 4) {
    const float *p = a.p + (size_t)k * a.stride + i;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    const float4 l0 = __ldcg((const float4 *)p);
    const float4 l1 = k + 1 < a.ns ? __ldcg((const float4 *)(p + a.stride)) : z;
    const float4 l2 = k + 2 < a.ns ? __ldcg((const float4 *)(p + 2 * a.stride)) : z;
    const float4 l3 = k + 3 < a.ns ? __ldcg((const float4 *)(p + 3 * a.stride)) : z;
    v.x += l0.x; v.y += l0.y; v.z += l0.z; v.w += l0.w;
    v.x += l1.x; v.y += l1.y; v.z += l1.z; v.w += l1.w;
    v.x += l2.x; v.y += l2.y; v.z += l2.z; v.w += l2.w;
    v.x += l3.x; v.y += l3.y; v.z += l3.z; v.w += l3.w;
  }
  return v;
}
__device__ __forceinline__ float part_get(const PartIn &a, size_t i) {
  float v = __ldcg(a.p + i);
  for (int k = 1; k < a.ns; k += 4) {
    const float *p = a.p + (size_t)k * a.stride + i;
    const float l0 = __ldcg(p);
    const float l1 = k + 1 < a.ns ? __ldcg(p + a.stride) : 0.0f;
    const float l2 = k + 2 < a.ns ? __ldcg(p + 2 * a.stride) : 0.0f;
    const float l3 = k + 3 < a.ns ? __ldcg(p + 3 * a.stride) : 0.0f;
    v += l0; v += l1; v += l2; v += l3;
  }
  return v;
}

// Several streams in one pass: row t of the pass is row t % per of stream t / per, whose row sets (and the rest of its
// control block) lie `stride` bytes after the previous stream's.  One stream: per is larger than any row index.
struct Streams { int per; int stride; };
// the geometry the launchers below hand to their kernels; the engine sets it before it enqueues a pass
void ops_set_streams(int per, int stride);
Streams ops_streams(void);

// min_per: fewest cache positions a split-K attention block takes (a multiple of 32)
// kv_plane: halves between the hi and the lo plane of a K or V cache (max_ctx * KV * hd)
// rs_stride: bytes between the row sets of consecutive row groups (grid z of the attention kernels)
// kv_group: halves between the caches of consecutive row groups (0: all groups read one cache, as a prompt chunk's do)
struct AttnShape { int H, KV, hd, rope_dim; float eps; int min_per; long long kv_plane; int rs_stride; long long kv_group; };
struct DeltaShape { int TR, GK, SZ, KC, convd, kdc, vdc; float eps; };

// launchers (ops_model.cu); a stream has SPEC_MAXT rows at most, a kernel ignores rows >= its stream's rs->n
int op_embed(cudaStream_t s, int fmt, const uint8_t *W, int d, const RowSet *rs, int Tmax, float *x);
int op_norm_xp(cudaStream_t s, const float *xin, PartIn add, const float *w, float eps, int d, float *xout, XPlanes xp,
               int xp_col0, float *hn_out, const RowSet *rs, int Tmax, int zero_if_pos0);
int op_silu_xp(cudaStream_t s, PartIn g, PartIn u, int f, XPlanes xp, const RowSet *rs, int Tmax);
int op_silu_scaled_xp(cudaStream_t s, PartIn g, PartIn u, int f, XPlanes xp, const RowSet *rs, int Tmax, const float *scale, int seg);
// router logits (ne rows + the shared gate row of Wr, F32) on the normed rows h[T][d], then ids / wt [T][nk + 1]
int op_moe_route(cudaStream_t s, const float *Wr, const float *h, int d, int ne, int nk, float *lg, int *ids, float *wt, const RowSet *rs, int Tmax);
// kv_only: only the K and V rows (the drafter's cache fill of the prompt path: no query rows)
int op_qkrope(cudaStream_t s, PartIn q, PartIn k, PartIn v, const float *qn_w, const float *kn_w, const double *invfreq,
              AttnShape sh, float *qout, float *Kc, float *Vc, const RowSet *rs, int Tmax, bool kv_only = false);
// kg != null: the gated rows go out as fp16 rows kg_row0 .. of a k-group-major chunk buffer (pf.cu) instead of the planes
// nz > 1: that many consecutive groups of Tmax rows in one launch (rs, q, qg, pm / pl / po and the output rows advance
// by one group per grid z)
int op_attention(cudaStream_t s, const float *q, const float *Kc, const float *Vc, PartIn qg, AttnShape sh, int nsplit,
                 float *pm, float *pl, float *po, XPlanes xp, const RowSet *rs, int Tmax, __half *kg = nullptr, int kg_row0 = 0, int nz = 1);
int op_delta_conv(cudaStream_t s, PartIn ring, const float *cw, PartIn bp, PartIn ap, const float *dt, const float *sa,
                  DeltaShape sh, float *y, float *beta, float *decay, const RowSet *rs, int Tmax);
// S: the streams' state rings one after the other (s_group floats apart); nz streams
int op_delta_fused(cudaStream_t s, float *S, const SpecCtl *ctl, const float *y, const float *beta, const float *decay, PartIn z,
                   const float *nw, DeltaShape sh, XPlanes xp, const RowSet *rs, int nz = 1, long long s_group = 0);
// A row set that no kernel of the pass in flight writes (the verify rows: k_accept sets them at the end
// of the previous cycle) may be read before the wait on the preceding kernel, which takes one trip to L2
// off every small kernel's critical path.  The host says so by setting bit 0 of the pointer it passes.
static inline const RowSet *rs_stable(const RowSet *rs) { return (const RowSet *)((uintptr_t)rs | 1u); }
#ifdef __CUDACC__
// Opens every row-set kernel: trigger the dependents, read n and pos0 (early if tagged), wait.
__device__ __forceinline__ const RowSet *rs_begin(const RowSet *rs, int &n, int &pos0) {
  pdl_trigger();
  const bool early = ((uintptr_t)rs & 1u) != 0;
  rs = (const RowSet *)((uintptr_t)rs & ~(uintptr_t)1);
  if (early) { n = *(const volatile int *)&rs->n; pos0 = *(const volatile int *)&rs->pos0; }
  pdl_wait();
  if (!early) { n = rs->n; pos0 = rs->pos0; }
  return rs;
}
// The same for row t of a pass over several streams: the row set of the row's stream, and tl, the row's index in it.
__device__ __forceinline__ const RowSet *rs_begin_row(const RowSet *rs, Streams sg, int t, int &n, int &pos0, int &tl) {
  const int z = t / sg.per;
  tl = t - z * sg.per;
  return rs_begin((const RowSet *)((uintptr_t)rs + (size_t)z * (size_t)sg.stride), n, pos0);
}
#endif
int op_lookup_draft(cudaStream_t s, SpecCtl *ctl, int nz = 1);
int op_top2_part(cudaStream_t s, PartIn logits, int V, long long row_stride, float *part, const RowSet *rs, int Tmax);
// nz streams: control blocks consecutive, result rings ring_n records apart, rows of the pass `per` apart
// smp_tok / smp_val (sampling mode): the emitted token of every row and its raw logit, in place of the argmax
int op_accept(cudaStream_t s, const float *part, SpecCtl *ctl, SpecResult *ring, int ring_n, int Tmax, int nz = 1, int per = 0,
              const int *smp_tok = nullptr, const float *smp_val = nullptr);
int op_draft_pick(cudaStream_t s, const float *part, const int *ids, SpecCtl *ctl, int from_chain, int j, const float *mt_hn,
                  float *chain_h, int d, int nz = 1, int per = 0);
int ops_model_setup(void);
