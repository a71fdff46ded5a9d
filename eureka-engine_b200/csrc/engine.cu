// engine.cu -- the speculative-decoding engine: weights on the device, per-sequence state, and the
// draft -> verify -> accept -> commit cycle as one CUDA graph.
//
// It replaces, for this path, the reference's host chain host/llb_host.c:1474-1950 (spec_init,
// mtp_load, spec_mdraft / mtp_rows, spec_rows, spec_attn, spec_ffn, spec_pass).  Differences that
// are design, not omission:
//   * every decision of a cycle (argmax, accept length, ring advance, the drafter's catch-up rows,
//     the next cycle's inputs) is taken on the device (k_accept / k_draft_pick), so a cycle is one
//     graph launch and one small result record, instead of k blocking reads plus one host round
//     trip per served row;
//   * the prompt is fed through the same T-row pass in chunks of k+1 given tokens.
#include <math.h>
#include <stdlib.h>

#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/llb_b200.h"
#include "model.cuh"
#include "gguf.cuh"
#include "pf.cuh"
#include "tp.cuh"
#include "sampler.cuh"

struct DevMat { uint8_t *w = nullptr; int rows = 0, cols = 0, fmt = -1; };
struct OutBuf { float *p = nullptr; int ns = 1; long long stride = 0; size_t cap = 0; };   // K-slice partial sums of one matrix (cap: floats allocated)
static PartIn as_in(const OutBuf &o) { return PartIn{o.p, o.ns, o.stride}; }

struct AttnW { DevMat q, k, v, o; float *qn = nullptr, *kn = nullptr; };
// moe: the layer's FFN is the routed-expert one (host/llb_host.c:622-724).  router: [ne + 1][d] F32, the ne
// router rows and then the shared expert's gate row; gu / dn: the expert stacks in the layout of moe.cuh, the
// shared expert being block ne; gate / up / down are unused then.
struct FfnW { DevMat gate, up, down; float *post = nullptr; bool moe = false; float *router = nullptr; uint8_t *gu = nullptr, *dn = nullptr;
              long long es_gu = 0, es_dn = 0; int fmt_gu = -1, fmt_dn = -1; };
struct DeltaW { DevMat qkv, z, beta, alpha, out; float *dt = nullptr, *a = nullptr, *conv = nullptr, *norm = nullptr; };
struct LayerW { bool full = false; float *attn_norm = nullptr; AttnW at; DeltaW dn; FfnW ffn; };

// blocked: Q8_0 in GGUF's [f16 d][32 x int8] blocks (host memory only), re-sliced to the row-split layout at upload
struct TensorRec { uint64_t off, bytes; int rows, cols, fmt; bool blocked = false; };

// Buffers of the prompt path (pf.cu), allocated at the first fast prefill: residual rows, fp16 activations in the
// dense GEMM's k-group-major order, GEMM outputs as K-slice partial sums of PF_RMAX rows, and the row sets of the chunk.
struct PfState {
  bool ready = false;
  float *x = nullptr, *x1 = nullptr, *hn = nullptr, *e = nullptr, *qn = nullptr, *y = nullptr, *beta = nullptr, *decay = nullptr, *o = nullptr;
  __half *kg_d = nullptr, *kg_f = nullptr, *kg_qa = nullptr, *kg_v = nullptr, *kg_2d = nullptr;
  OutBuf q, k, v, qkv, z, bp, ap, a, g, u, dn, eh;
  float *pm = nullptr, *pl = nullptr, *po = nullptr;   // split-K attention partials of every row group of a chunk
  RowSet *rs = nullptr;    // [0] the whole chunk, [1 + i] its i-th group of attention rows
  int *ids = nullptr;      // the chunk's tokens
};

// host mirror of one stream (sequence): where it is, what it reported last, and its statistics
struct SeqHost {
  unsigned long long seq = 0;
  int pos = 0;            // position of the next cycle's row 0
  int last_tok = -1;      // the committed token of the next cycle
  bool primed = false;    // prefill done
  // reference-shaped row serving (llb_spec_pass)
  SpecResult last;
  int last_served_idx = 0;
  bool have_last = false;
  // statistics, as the reference's "spec:" line (host/llb_host.c:1513-1523)
  unsigned long long cycles = 0, rows = 0, served = 0, drafted[8] = {0}, accepted[8] = {0};
};

struct llb_spec {
  // configuration (index.tsv #cfg keys, tools/qwen35_engine.c:386-409)
  int L = 0, d = 0, H = 0, KV = 0, hd = 0, f = 0, V = 0, interval = 4, KC = 4, SZ = 128, GK = 0, TR = 0, vdc = 0, kdc = 0,
      convd = 0, rope_dim = 64;
  float rope_base = 1e7f, eps = 1e-6f;
  int ne = 0, nk = 0, ef = 0, sf = 0;   // routed experts, experts per token, expert width, shared expert width (ne = 0: dense FFN)
  float *moe_lg = nullptr, *moe_wt = nullptr, *moe_g = nullptr, *moe_u = nullptr, *hn2 = nullptr;
  int *moe_ids = nullptr;
  XPlanes xp_e;
  size_t pack_bytes = 0;   // size of the pack the index describes: every tensor range is checked against it
  int k = 0, Tmax = 1, R = 2, max_ctx = 0, NC = 8;   // Tmax / NC: rows and plane columns of the pass being enqueued
  // Several streams (sequences) per engine share every weight read: a pass has B x per rows, row t belonging to stream
  // t / per; every piece of per-sequence state below is B copies one after the other, and the control blocks, result
  // rings and host mirrors are arrays of B.  B = 1: per = the pass's width, as before.
  int B = 1, per = 1;
  long long kv_group = 0, s_group = 0, ring_group_unit = 0;   // halves between the streams' K (V) caches; floats between their state rings
  int *const_rows = nullptr;   // device word holding B x per (the routed-expert launches' row count in a multi-stream pass)
  // A speculative pass has k + 1 rows; a prompt chunk has Tpf rows (8 where the attention kernel's query budget allows:
  // the weights stream once per pass whatever its rows, so a wider chunk halves the prompt's time).  The two widths
  // share every buffer; the planes have one view per column count.
  int Tspec = 1, Tpf = 1;
  XPlanes xpv[3][6];   // [NC 8 / 16 / 32][xp_d, xp_f, xp_qa, xp_v, xp_2d, xp_e]
  // weights
  std::vector<void *> allocs;
  // An engine opened by llb_spec_open_sibling uses the weights of the engine it names (`share`) and owns only its
  // sequence state: its open replays the first engine's, taking that engine's weight allocations (wlist, in order)
  // where the first one allocated and uploaded.  What the replay needs is kept by the first engine: the index text, the
  // drafter image's header and size, the layer count asked for.
  llb_spec *share = nullptr;
  int sharers = 0;         // siblings open on this engine's weights
  bool closed = false;     // closed by its owner while siblings were open: freed with the last of them
  std::vector<std::pair<void *, size_t>> wlist;
  size_t wnext = 0;
  std::string index_copy;
  std::vector<uint8_t> mtp_hdr;
  size_t mtp_total = 0;
  int layers_arg = 0;
  std::vector<LayerW> layer;
  DevMat embd, head;
  float *out_norm = nullptr;
  double *invfreq = nullptr;
  // drafter
  bool has_mtp = false;
  bool lookup = false;                // no drafter image and k > 0: the prompt-lookup drafter (host/llb_host.c:1936)
  int *hist = nullptr;                // its token history on the device
  float *mt_enorm = nullptr, *mt_hnorm = nullptr, *mt_attn_norm = nullptr, *mt_shn = nullptr;
  DevMat mt_eh, mt_head;
  AttnW mt_at;
  FfnW mt_ffn;
  int *mt_ids = nullptr;
  int mt_nv = 0;
  // per-sequence state
  std::vector<float *> Kc, Vc, ring, S;   // per layer (null where not applicable)
  // K-slices of the attn_qkv launch of each DeltaNet layer.  The conv ring keeps a row as that many partial sums and
  // every later pass adds them up again, so the split is fixed at open and is the same at both pass widths.
  std::vector<int> ring_ks;
  float *mt_Kc = nullptr, *mt_Vc = nullptr;
  SpecCtl *ctl = nullptr;
  SpecResult *res_host = nullptr, *res_dev = nullptr;
  int res_n = 256;
  // activations
  float *x = nullptr, *x1 = nullptr, *hn = nullptr, *e = nullptr, *qn = nullptr, *y = nullptr, *beta = nullptr, *decay = nullptr,
        *logits = nullptr, *t2part = nullptr, *pm = nullptr, *pl = nullptr, *po = nullptr;
  float *mt_x = nullptr, *mt_hn = nullptr, *chain_h = nullptr, *mt_logits = nullptr;
  XPlanes xp_d, xp_f, xp_qa, xp_v, xp_2d;
  OutBuf b_q, b_k, b_v, b_z, b_bp, b_ap, b_a, b_g, b_u, b_dn, b_eh, b_lg, b_mlg, b_ring;
  int att_split = 1;
  int att_min = 96;                   // fewest positions per attention block (three 32-position tiles)
  // tensor parallel (tp.cu): the dimensions above are this rank's share once the model is open; the full ones are kept
  // for slicing.  r_a / r_dn: the out-projections' [T, d] tiles summed over K-slices and ranks.
  TpPlan tp = {0, 1, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
  int Hf = 0, KVf = 0, ff = 0, GKf = 0, TRf = 0, kdcf = 0, vdcf = 0, convdf = 0;
  OutBuf r_a, r_dn;
  PfState pf;
  int prefill_mode = 0;   // 0: every prompt row through the T-row pass; 1: chunks of PF_R rows through the dense path (LLB_PREFILL=fast)
  double pf_rows = 0;     // prompt rows the dense path has processed since the engine was opened
  // graphs
  cudaGraphExec_t g_spec = nullptr, g_prefill = nullptr, g_verify = nullptr;
  size_t n_spec_nodes = 0, n_verify_nodes = 0;
  std::vector<SeqHost> sq;   // one per stream
  // sampling-mode verify (sampler.cu): off while the parameters leave the argmax untouched
  bool smp_on = false;
  SmpDev smp;
  float *smp_adj = nullptr, *smp_val = nullptr;   // biased / penalised logits of every row; the emitted tokens' raw logits
  int *smp_tok = nullptr;
  unsigned int *smp_err = nullptr;
};
// the streams' copies of per-sequence device state
static inline SpecCtl *ctl_of(const llb_spec *m, int b) { return m->ctl + b; }
static inline float *kc_of(const llb_spec *m, float *base, int b) { return base ? (float *)((__half *)base + (size_t)b * m->kv_group) : nullptr; }
static inline float *ring_of(const llb_spec *m, int il, int b) { return m->ring[il] + (size_t)b * m->ring_ks[il] * CONV_RING * m->convd; }
static inline float *state_of(const llb_spec *m, int il, int b) { return m->S[il] + (size_t)b * m->s_group; }
static inline int *hist_of(const llb_spec *m, int b) { return m->hist ? m->hist + (size_t)b * (m->max_ctx + 16) : nullptr; }
// the launchers' stream geometry while this engine enqueues (engines of different shapes may coexist)
struct StreamScope {
  Streams was;
  explicit StreamScope(const llb_spec *m, bool single = false) : was(ops_streams()) {
    if (m->B > 1 && !single) ops_set_streams(m->Tspec, (int)sizeof(SpecCtl)); else ops_set_streams(0, 0);
  }
  ~StreamScope() { ops_set_streams(was.per, was.stride); }
};

#define CK(call) do { if ((call)) return -1; } while (0)

// Optional per-op timing of an eager (not captured) pass: an event after every op.
struct ProfRec { const char *name; cudaEvent_t ev; };
static std::vector<ProfRec> g_prof;
static bool g_prof_on = false;
static void prof_mark(const char *name) {
  if (!g_prof_on) return;
  cudaEvent_t e;
  cudaEventCreate(&e);
  cudaEventRecord(e, g_llb.stream);
  g_prof.push_back({name, e});
}
#define PK(name, call) do { if ((call)) return -1; prof_mark(name); } while (0)
#define RING_MAXSPLIT 8   // most K-slices a conv ring keeps per row
static float bits_float(unsigned int u) { float f; memcpy(&f, &u, 4); return f; }

static void *dalloc(llb_spec *m, size_t bytes) {
  void *p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes ? bytes : 256);
  if (e != cudaSuccess) { llb_fail("cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e)); cudaGetLastError(); return nullptr; }
  cudaMemsetAsync(p, 0, bytes, g_llb.stream);
  m->allocs.push_back(p);
  return p;
}
static float *falloc(llb_spec *m, size_t n) { return (float *)dalloc(m, n * 4); }
// storage of a weight: allocated (fresh: the caller uploads into it), or, in a sibling, the first engine's
static void *walloc(llb_spec *m, size_t bytes, bool *fresh) {
  if (!m->share) {
    void *p = dalloc(m, bytes);
    if (p) m->wlist.push_back({p, bytes});
    *fresh = true;
    return p;
  }
  *fresh = false;
  const std::vector<std::pair<void *, size_t>> &wl = m->share->wlist;
  if (m->wnext >= wl.size() || wl[m->wnext].second != bytes) {
    llb_fail("sibling: weight %zu of %zu bytes is not what the first engine loaded there (a drafter it was opened without?)", m->wnext, bytes);
    return nullptr;
  }
  return wl[m->wnext++].first;
}
// plane columns of a pass of T rows (hi and lo halves): 8, 16 or 32
static int nc_of(int T) { return T <= 4 ? 8 : T <= 8 ? 16 : 32; }
static int rows_cap(const llb_spec *m) { const int a = m->B * m->Tspec, b = m->Tpf; return a > b ? a : b; }
static int xp_alloc(llb_spec *m, int which, int K) {
  const int ncmax = nc_of(rows_cap(m));
  void *b = dalloc(m, xp_bytes(K, ncmax));
  if (!b) return -1;
  m->xpv[0][which] = xp_carve(b, K, 8);
  m->xpv[1][which] = xp_carve(b, K, ncmax < 16 ? ncmax : 16);
  m->xpv[2][which] = xp_carve(b, K, ncmax);
  return 0;
}
// the width of the passes enqueued from here on: T rows in all, `per` of them to a stream
static void set_width(llb_spec *m, int T) {
  m->Tmax = T; m->NC = nc_of(T);
  m->per = m->B > 1 ? m->Tspec : T;
  const XPlanes *v = m->xpv[m->NC == 8 ? 0 : m->NC == 16 ? 1 : 2];
  m->xp_d = v[0]; m->xp_f = v[1]; m->xp_qa = v[2]; m->xp_v = v[3]; m->xp_2d = v[4]; m->xp_e = v[5];
}

static int fmt_of(const std::string &ty) {
  if (ty == "F32") return LLB_FM_F32;
  if (ty == "Q8_0") return LLB_FM_Q8_0;
  if (ty == "Q4_K") return LLB_FM_Q4_K;
  if (ty == "Q6_K") return LLB_FM_Q6_K;
  if (ty == "Q5_K") return LLB_FM_Q5_K;
  return -1;
}

// index.tsv: "#cfg\tKEY\tVALUE" lines, then name off bytes rows cols TYPE [row_bytes fmt]
// (tools/qwen35_engine.c:379-433)
static int parse_index(llb_spec *m, const char *text, std::unordered_map<std::string, TensorRec> &tab) {
  const char *p = text;
  while (*p) {
    const char *e = strchr(p, '\n');
    std::string line(p, e ? (size_t)(e - p) : strlen(p));
    p = e ? e + 1 : p + line.size();
    if (line.rfind("#cfg\t", 0) == 0) {
      size_t t = line.find('\t', 5);
      if (t == std::string::npos) continue;
      std::string key = line.substr(5, t - 5), val = line.substr(t + 1);
      struct { const char *k; int *v; } im[] = {
        {"n_layers", &m->L}, {"n_heads", &m->H}, {"n_kv_heads", &m->KV}, {"d_model", &m->d}, {"head_dim", &m->hd},
        {"d_ff", &m->f}, {"vocab_size", &m->V}, {"full_attention_interval", &m->interval}, {"ssm_conv_kernel", &m->KC},
        {"ssm_state_size", &m->SZ}, {"ssm_group_count", &m->GK}, {"ssm_time_step_rank", &m->TR}, {"ssm_inner_size", &m->vdc},
        {"linear_key_dim", &m->kdc}, {"linear_conv_dim", &m->convd}, {"rope_dim", &m->rope_dim}, {"expert_count", &m->ne},
        {"expert_used_count", &m->nk}, {"expert_feed_forward_length", &m->ef}, {"expert_shared_feed_forward_length", &m->sf}};
      for (auto &kv : im) if (key == kv.k) *kv.v = atoi(val.c_str());
      if (key == "rope_freq_base") m->rope_base = strtof(val.c_str(), nullptr);
      if (key == "rms_norm_eps") m->eps = strtof(val.c_str(), nullptr);
      continue;
    }
    if (line.empty() || line[0] == '#') continue;
    char name[128], ty[32];
    unsigned long long off, nb;
    int rows, cols;
    if (sscanf(line.c_str(), "%127[^\t]\t%llu\t%llu\t%d\t%d\t%31[^\t\n]", name, &off, &nb, &rows, &cols, ty) != 6) continue;
    const bool blocked = !strcmp(ty, "Q8_0G");
    int fm = blocked ? LLB_FM_Q8_0 : fmt_of(ty);
    if (fm < 0) return llb_fail("index: tensor %s has unsupported type %s", name, ty);
    TensorRec tr{off, nb, rows, cols, fm};
    tr.blocked = blocked;
    tab[name] = tr;
  }
  return 0;
}

static bool in_range(uint64_t off, uint64_t bytes, size_t src_bytes);
static size_t rec_bytes(const TensorRec &t);
// The configuration values every later division, modulo and allocation relies on (a stale or zeroed index must be an
// error message, not a SIGFPE or a wild allocation), then every tensor record against the pack's size.
static int validate_index(const llb_spec *m, const std::unordered_map<std::string, TensorRec> &tab, size_t pack_bytes) {
  struct { const char *k; int v; } pos[] = {{"n_layers", m->L}, {"n_heads", m->H}, {"n_kv_heads", m->KV}, {"d_model", m->d}, {"head_dim", m->hd},
    {"vocab_size", m->V}, {"full_attention_interval", m->interval}, {"ssm_conv_kernel", m->KC}, {"ssm_state_size", m->SZ},
    {"ssm_group_count", m->GK}, {"ssm_time_step_rank", m->TR}, {"ssm_inner_size", m->vdc}, {"linear_key_dim", m->kdc},
    {"linear_conv_dim", m->convd}, {"rope_dim", m->rope_dim}};
  for (auto &p : pos) if (p.v < 1) return llb_fail("index: #cfg %s is %d (missing or not positive)", p.k, p.v);
  if (m->ne == 0 && m->f < 1) return llb_fail("index: #cfg d_ff is %d (missing or not positive)", m->f);
  if (m->ne < 0 || m->nk < 0 || m->ef < 0 || m->sf < 0) return llb_fail("index: negative expert configuration");
  if (m->L > 4096 || m->V > (1 << 24) || m->d > (1 << 16)) return llb_fail("index: n_layers %d / vocab_size %d / d_model %d out of range", m->L, m->V, m->d);
  if (m->rope_dim > m->hd || (m->rope_dim & 1)) return llb_fail("index: rope_dim %d with head_dim %d", m->rope_dim, m->hd);
  if (m->convd != 2 * m->kdc + m->vdc) return llb_fail("index: linear_conv_dim %d is not 2 x %d + %d", m->convd, m->kdc, m->vdc);
  if (m->kdc != m->GK * m->SZ || m->vdc != m->TR * m->SZ) return llb_fail("index: DeltaNet widths %d / %d do not match %d groups, %d heads of %d", m->kdc, m->vdc, m->GK, m->TR, m->SZ);
  if (!(m->eps > 0.0f) || !(m->rope_base > 0.0f)) return llb_fail("index: rms_norm_eps / rope_freq_base must be positive");
  for (const auto &kv : tab) {
    const TensorRec &t = kv.second;
    if (t.rows < 1 || t.cols < 1) return llb_fail("index: tensor %s is [%d x %d]", kv.first.c_str(), t.rows, t.cols);
    if (t.fmt != LLB_FM_F32 && t.cols % (t.fmt == LLB_FM_Q8_0 ? 32 : 256)) return llb_fail("index: tensor %s has %d columns, not whole blocks of its format", kv.first.c_str(), t.cols);
    if (rec_bytes(t) != t.bytes) return llb_fail("index: tensor %s has %llu bytes, its shape needs %zu", kv.first.c_str(), (unsigned long long)t.bytes, rec_bytes(t));
    if (!in_range(t.off, t.bytes, pack_bytes))
      return llb_fail("index: tensor %s (offset %llu, %llu bytes) reaches past the end of the pack (%zu bytes): truncated pack or stale index",
                      kv.first.c_str(), (unsigned long long)t.off, (unsigned long long)t.bytes, pack_bytes);
  }
  return 0;
}

// one tensor from pack bytes into its device layout; `dedupe` shares the copy of aliased tensors
// does [off, off + bytes) lie inside a source of src_bytes bytes?  (no overflow: the two sides are compared separately)
static bool in_range(uint64_t off, uint64_t bytes, size_t src_bytes) { return off <= src_bytes && bytes <= src_bytes - off; }
// bytes a tensor record occupies in its source (GGUF-blocked Q8_0 has the same size as the row-split layout)
static size_t rec_bytes(const TensorRec &t) { return (size_t)t.rows * pack_row_bytes(t.fmt, t.cols); }

static int load_tensor(llb_spec *m, const TensorRec &t, const uint8_t *pack, size_t src_bytes, int on_device, void **out,
                       std::unordered_map<uint64_t, void *> &dedupe) {
  auto it = dedupe.find(t.off);
  if (it != dedupe.end()) { *out = it->second; return 0; }
  const size_t want = rec_bytes(t);
  if (want != t.bytes) return llb_fail("index: tensor at %llu has %llu bytes, its shape needs %zu", (unsigned long long)t.off,
                                       (unsigned long long)t.bytes, want);
  if (!in_range(t.off, t.bytes, src_bytes)) return llb_fail("index: tensor at %llu (%llu bytes) reaches past the end of its source (%zu bytes)",
                                                             (unsigned long long)t.off, (unsigned long long)t.bytes, src_bytes);
  bool fresh;
  void *dst = walloc(m, (size_t)t.rows * dev_row_bytes(t.fmt, t.cols), &fresh);
  if (!dst) return -1;
  if (!fresh) { dedupe[t.off] = dst; *out = dst; return 0; }
  if (t.blocked) {
    // [f16 d][32 q] x cols/32 per row -> [cols q][cols/32 f16 d] per row (tools/gguf2pack.c:25-27), 4096 rows at a time
    if (on_device) return llb_fail("index: blocked Q8_0 tensors are read from host memory only");
    const size_t rb = (size_t)t.cols + (size_t)t.cols / 16, nb = (size_t)t.cols / 32;
    std::vector<uint8_t> tmp;
    for (int r0 = 0; r0 < t.rows; r0 += 4096) {
      const int nr = t.rows - r0 < 4096 ? t.rows - r0 : 4096;
      tmp.resize((size_t)nr * rb);
      for (int r = 0; r < nr; r++) {
        const uint8_t *src = pack + t.off + (size_t)(r0 + r) * rb;
        uint8_t *q = tmp.data() + (size_t)r * rb, *sc = q + t.cols;
        for (size_t b = 0; b < nb; b++) { memcpy(sc + 2 * b, src + 34 * b, 2); memcpy(q + 32 * b, src + 34 * b + 2, 32); }
      }
      CK(llb_b200_weight_upload(t.fmt, nr, t.cols, tmp.data(), 0, (llb_b200_dptr)(uintptr_t)((uint8_t *)dst + (size_t)r0 * dev_row_bytes(t.fmt, t.cols))));
    }
    dedupe[t.off] = dst;
    *out = dst;
    return 0;
  }
  CK(llb_b200_weight_upload(t.fmt, t.rows, t.cols, pack + t.off, on_device, (llb_b200_dptr)(uintptr_t)dst));
  dedupe[t.off] = dst;
  *out = dst;
  return 0;
}

// rows / cols (either may be null = all) of a tensor into a matrix of its own in the device layout: the whole tensor goes
// to a temporary first, then strided device copies pick the ranges (columns of a quantised row are whole super-blocks)
static int load_sliced(llb_spec *m, const TensorRec &t, const uint8_t *pack, size_t src_bytes, int on_device, const TpSel *rows, const TpSel *cols,
                       DevMat &out) {
  std::unordered_map<uint64_t, void *> none;
  void *full = nullptr;
  CK(load_tensor(m, t, pack, src_bytes, on_device, &full, none));
  m->allocs.pop_back();                                    // the temporary is freed below, not at close
  m->wlist.pop_back();
  TpSel allr, allc;
  allr.add(0, t.rows); allc.add(0, t.cols);
  if (!rows) rows = &allr;
  if (!cols) cols = &allc;
  const int lr = rows->total(), lc = cols->total();
  const size_t frb = dev_row_bytes(t.fmt, t.cols), lrb = dev_row_bytes(t.fmt, lc);
  int rc = 0;
  uint8_t *dst = (uint8_t *)dalloc(m, (size_t)lr * lrb);
  if (!dst) rc = -1;
  const int unit = t.fmt == LLB_FM_F32 ? 1 : t.fmt == LLB_FM_Q8_0 ? 32 : 256;
  int drow = 0;
  for (int i = 0; i < rows->n && !rc; i++) {
    int dcol = 0;
    for (int j = 0; j < cols->n && !rc; j++) {
      const int c0 = cols->start[j], cn = cols->count[j];
      if (c0 % unit || cn % unit) { rc = llb_fail("tensor slice: columns %d + %d are not whole blocks", c0, cn); break; }
      const uint8_t *src = (const uint8_t *)full + (size_t)rows->start[i] * frb;
      cudaError_t e;
      if (t.fmt == LLB_FM_Q8_0) {   // [cols x int8][cols / 32 x f16]: the codes and the scales are two column ranges
        e = cudaMemcpy2DAsync(dst + (size_t)drow * lrb + dcol, lrb, src + c0, frb, cn, rows->count[i], cudaMemcpyDeviceToDevice, g_llb.stream);
        if (e == cudaSuccess)
          e = cudaMemcpy2DAsync(dst + (size_t)drow * lrb + lc + dcol / 16, lrb, src + t.cols + c0 / 16, frb, cn / 16, rows->count[i], cudaMemcpyDeviceToDevice, g_llb.stream);
      } else {
        e = cudaMemcpy2DAsync(dst + (size_t)drow * lrb + dev_row_bytes(t.fmt, dcol), lrb, src + dev_row_bytes(t.fmt, c0), frb, dev_row_bytes(t.fmt, cn),
                              rows->count[i], cudaMemcpyDeviceToDevice, g_llb.stream);
      }
      if (e != cudaSuccess) rc = llb_fail("tensor slice: %s", cudaGetErrorString(e));
      dcol += cn;
    }
    drow += rows->count[i];
  }
  cudaStreamSynchronize(g_llb.stream);
  cudaFree(full);
  if (rc) return rc;
  out.w = dst; out.rows = lr; out.cols = lc; out.fmt = t.fmt;
  return 0;
}

// The routed experts of one layer: the router and the shared gate row into one F32 matrix, the expert
// stacks (GGUF tensors ffn_gate_exps / ffn_up_exps [ne * ef][d], ffn_down_exps [ne * d][ef]) and the shared
// expert re-laid as blocks [gate rows | up rows] and [down rows], the shared expert last.
static int load_moe(llb_spec *m, FfnW &w, const std::string &p, const std::unordered_map<std::string, TensorRec> &tab, const uint8_t *pack,
                    int on_device) {
  const int d = m->d, ne = m->ne, ef = m->ef;
  auto rec = [&](const char *leaf, int rows, int cols, TensorRec &out) -> int {
    auto it = tab.find(p + leaf);
    if (it == tab.end()) return llb_fail("pack has no tensor %s%s", p.c_str(), leaf);
    out = it->second;
    if (out.rows != rows || out.cols != cols) return llb_fail("%s%s is [%d x %d], the configuration needs [%d x %d]", p.c_str(), leaf, out.rows, out.cols, rows, cols);
    if ((size_t)rows * pack_row_bytes(out.fmt, cols) != out.bytes) return llb_fail("%s%s: %llu bytes do not match its shape", p.c_str(), leaf, (unsigned long long)out.bytes);
    if (!in_range(out.off, out.bytes, m->pack_bytes)) return llb_fail("%s%s reaches past the end of the pack (%zu bytes)", p.c_str(), leaf, m->pack_bytes);
    return 0;
  };
  TensorRec r_in, r_sh, eg, eu, ed, sg, su, sd;
  CK(rec("ffn_gate_inp.weight", ne, d, r_in)); CK(rec("ffn_gate_inp_shexp.weight", 1, d, r_sh));
  // the experts' gate and up either as two stacks or as one of [gate rows | up rows] per expert (ffn_gate_up_exps,
  // host/llb_host.c:629 "fz")
  const bool fused = tab.count(p + "ffn_gate_up_exps.weight") != 0;
  size_t gu_stride = (size_t)ef;   // rows between consecutive experts in the gate (and up) source
  if (fused) {
    CK(rec("ffn_gate_up_exps.weight", ne * 2 * ef, d, eg));
    eu = eg; eu.off += (uint64_t)ef * pack_row_bytes(eg.fmt, d);
    gu_stride = 2 * (size_t)ef;
  } else {
    CK(rec("ffn_gate_exps.weight", ne * ef, d, eg)); CK(rec("ffn_up_exps.weight", ne * ef, d, eu));
  }
  CK(rec("ffn_down_exps.weight", ne * d, ef, ed));
  CK(rec("ffn_gate_shexp.weight", ef, d, sg)); CK(rec("ffn_up_shexp.weight", ef, d, su)); CK(rec("ffn_down_shexp.weight", d, ef, sd));
  for (const TensorRec *t : {&eg, &eu, &ed, &sg, &su, &sd}) if (t->blocked) return llb_fail("%s: blocked Q8_0 expert stacks have no kernel", p.c_str());
  if (r_in.fmt != LLB_FM_F32 || r_sh.fmt != LLB_FM_F32) return llb_fail("%sffn_gate_inp must be F32", p.c_str());
  if (eg.fmt != eu.fmt || sg.fmt != eg.fmt || su.fmt != eg.fmt || sd.fmt != ed.fmt)
    return llb_fail("%s: the shared expert and the expert stacks must share their formats (gate/up %d %d %d %d, down %d %d)", p.c_str(), eg.fmt, eu.fmt, sg.fmt,
                    su.fmt, ed.fmt, sd.fmt);
  for (int fm : {eg.fmt, ed.fmt})
    if (fm != LLB_FM_Q4_K && fm != LLB_FM_Q5_K && fm != LLB_FM_Q6_K) return llb_fail("%s: expert stacks of format %d have no kernel (Q4_K, Q5_K, Q6_K do)", p.c_str(), fm);
  w.moe = true; w.fmt_gu = eg.fmt; w.fmt_dn = ed.fmt;
  bool fresh;
  w.router = (float *)walloc(m, (size_t)(ne + 1) * d * 4, &fresh);
  if (!w.router) return -1;
  const size_t rb_gu0 = dev_row_bytes(eg.fmt, d), rb_dn0 = dev_row_bytes(ed.fmt, ef);
  if (!fresh) {
    w.es_gu = (long long)(2 * ef * rb_gu0); w.es_dn = (long long)(d * rb_dn0);
    w.gu = (uint8_t *)walloc(m, (size_t)(ne + 1) * w.es_gu, &fresh);
    w.dn = (uint8_t *)walloc(m, (size_t)(ne + 1) * w.es_dn, &fresh);
    return w.gu && w.dn ? 0 : -1;
  }
  const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
  CU_OK(cudaMemcpyAsync(w.router, pack + r_in.off, (size_t)ne * d * 4, kind, g_llb.stream));
  CU_OK(cudaMemcpyAsync(w.router + (size_t)ne * d, pack + r_sh.off, (size_t)d * 4, kind, g_llb.stream));
  const size_t rb_gu = dev_row_bytes(eg.fmt, d), rb_dn = dev_row_bytes(ed.fmt, ef);
  const size_t pb_gu = pack_row_bytes(eg.fmt, d), pb_dn = pack_row_bytes(ed.fmt, ef);
  w.es_gu = (long long)(2 * ef * rb_gu); w.es_dn = (long long)(d * rb_dn);
  w.gu = (uint8_t *)walloc(m, (size_t)(ne + 1) * w.es_gu, &fresh);
  w.dn = (uint8_t *)walloc(m, (size_t)(ne + 1) * w.es_dn, &fresh);
  if (!w.gu || !w.dn) return -1;
  for (int e = 0; e <= ne; e++) {
    const uint8_t *g = e < ne ? pack + eg.off + (size_t)e * gu_stride * pb_gu : pack + sg.off;
    const uint8_t *u = e < ne ? pack + eu.off + (size_t)e * gu_stride * pb_gu : pack + su.off;
    const uint8_t *dn = e < ne ? pack + ed.off + (size_t)e * d * pb_dn : pack + sd.off;
    CK(llb_b200_weight_upload(eg.fmt, ef, d, g, on_device, (llb_b200_dptr)(uintptr_t)(w.gu + (size_t)e * w.es_gu)));
    CK(llb_b200_weight_upload(eg.fmt, ef, d, u, on_device, (llb_b200_dptr)(uintptr_t)(w.gu + (size_t)e * w.es_gu + (size_t)ef * rb_gu)));
    CK(llb_b200_weight_upload(ed.fmt, d, ef, dn, on_device, (llb_b200_dptr)(uintptr_t)(w.dn + (size_t)e * w.es_dn)));
  }
  return 0;
}

static int check_k(const DevMat &w, int rows, int cols, const char *what) {
  if (w.rows != rows || w.cols != cols) return llb_fail("%s is [%d x %d], the configuration needs [%d x %d]", what, w.rows, w.cols, rows, cols);
  if (w.fmt == LLB_FM_F32) return llb_fail("%s: F32 matrices have no GEMM kernel", what);
  if (cols % 256) return llb_fail("%s: %d columns is not a multiple of 256", what, cols);
  return 0;
}

// ---- GEMM sites ---------------------------------------------------------------------------------
// direct: the matrix writes into caller-owned storage (the conv ring) laid out [direct_splits][slots][direct_stride];
// `out` then only records how many K-slices the launch used
// force_ks > 0: the K-split of the launch this matrix lands in (all matrices of one format share a launch)
struct SiteMat { const DevMat *w; OutBuf *out; const int *tok_slot; float *direct; int direct_stride; long long direct_split_stride = 0; int direct_splits = 1; int force_ks = 0; };

// Allocate (at init) or reuse the partial-sum buffer of one matrix and record its split.
static int out_prepare(llb_spec *m, OutBuf &o, int rows, int ks) {
  const size_t need = (size_t)ks * m->Tmax * rows;
  if (!o.p || o.cap < need) {
    o.p = falloc(m, need);
    if (!o.p) return -1;
    o.cap = need;
  }
  o.ns = ks; o.stride = (long long)m->Tmax * rows;
  return 0;
}

// Enqueue the GEMMs of one site: matrices sharing the activation planes, grouped by format.
static int site_gemm(llb_spec *m, std::vector<SiteMat> mats, const XPlanes &xp, int force_ks) {
  std::vector<bool> done(mats.size(), false);
  for (size_t i = 0; i < mats.size(); i++) {
    if (done[i]) continue;
    GemmArgs a;
    memset(&a, 0, sizeof a);
    a.K = mats[i].w->cols; a.xp = xp; a.planes = 2; a.T = m->Tmax;
    int ntiles = 0;
    std::vector<size_t> grp;
    for (size_t j = i; j < mats.size() && grp.size() < GEMM_MAXMAT; j++)
      if (!done[j] && mats[j].w->fmt == mats[i].w->fmt) { grp.push_back(j); ntiles += (mats[j].w->rows + 15) / 16; }
    int fk = force_ks;
    for (size_t j : grp) if (mats[j].force_ks > 0) fk = mats[j].force_ks;
    int ks = gemm_fix_ksplit(mats[i].w->fmt, xp.NC, a.K / 256,
                             fk > 0 ? fk : gemm_pick_ksplit(mats[i].w->fmt, xp.NC, ntiles, a.K / 256, g_llb.sms));
    if (fk > 0 && ks != fk) return llb_fail("gemm site: the fixed K-split %d is not valid at %d plane columns (%d)", fk, xp.NC, ks);
    a.ksplit = ks;
    a.nmat = (int)grp.size();
    for (size_t g = 0; g < grp.size(); g++) {
      SiteMat &sm = mats[grp[g]];
      a.m[g].W = sm.w->w; a.m[g].rows = sm.w->rows; a.m[g].tok_slot = sm.tok_slot;
      if (sm.tok_slot && m->B > 1) {   // every stream's rows go to that stream's ring, by that stream's slot numbers
        a.m[g].tok_per = m->per; a.m[g].tok_stride = (int)(sizeof(SpecCtl) / 4); a.m[g].tok_add = sm.direct_splits * CONV_RING;
      }
      if (sm.direct) {
        if (ks > sm.direct_splits) return llb_fail("gemm site: %d K-slices, the direct output holds %d", ks, sm.direct_splits);
        a.m[g].out = sm.direct; a.m[g].ostride = sm.direct_stride; a.m[g].split_stride = sm.direct_split_stride;
        if (sm.out) { sm.out->p = sm.direct; sm.out->ns = ks; sm.out->stride = sm.direct_split_stride; }
      }
      else {
        CK(out_prepare(m, *sm.out, sm.w->rows, ks));
        a.m[g].out = sm.out->p; a.m[g].ostride = sm.w->rows; a.m[g].split_stride = sm.out->stride;
      }
      done[grp[g]] = true;
    }
    CK(gemm_launch(g_llb.stream, mats[i].w->fmt, a));
  }
  return 0;
}

// Tensor parallel: a row-split projection leaves, on every rank, partial sums over its share of the columns (and over
// its K-slices).  Add the K-slices, sum over the ranks (NCCL all-reduce on the library's stream, captured into the graph
// like a kernel), and hand the consumer one complete [T, d] tile.  One rank: the consumer adds the K-slices itself.
static int tp_reduce(llb_spec *m, const OutBuf &part, OutBuf &whole) {
  if (m->tp.size <= 1) return 0;
  const size_t n = (size_t)m->Tmax * m->d;
  if (!whole.p || whole.cap < n) {
    whole.p = falloc(m, n);
    if (!whole.p) return -1;
    whole.cap = n;
  }
  whole.ns = 1; whole.stride = 0;
  // peer buffers open: one kernel adds the K-slices, stores the tile into every peer and adds what the peers stored here
  if (tp_peer_ready()) return tp_allreduce_parts(part.p, part.ns, part.stride, n, whole.p);
  CK(ops_sum_parts(g_llb.stream, part.p, part.ns, part.stride, (int)n, whole.p));
  return tp_allreduce(whole.p, n);
}
static PartIn in_a(const llb_spec *m) { return m->tp.size > 1 ? as_in(m->r_a) : as_in(m->b_a); }
static PartIn in_dn(const llb_spec *m) { return m->tp.size > 1 ? as_in(m->r_dn) : as_in(m->b_dn); }

// ---- blocks -------------------------------------------------------------------------------------
// full attention block on rows `rs`: planes xp_d hold the normed input; result partial sums in b_a
static int enq_attn(llb_spec *m, const AttnW &w, float *Kc, float *Vc, const RowSet *rs) {
  cudaStream_t s = g_llb.stream;
  AttnShape sh{m->H, m->KV, m->hd, m->rope_dim, m->eps, m->att_min, (long long)m->max_ctx * m->KV * m->hd,
               m->B > 1 ? (int)sizeof(SpecCtl) : 0, m->B > 1 ? m->kv_group : 0};
  PK("gemm qkv", site_gemm(m, {{&w.q, &m->b_q, nullptr, nullptr, 0}, {&w.k, &m->b_k, nullptr, nullptr, 0}, {&w.v, &m->b_v, nullptr, nullptr, 0}}, m->xp_d, 0));
  PK("qkrope", op_qkrope(s, as_in(m->b_q), as_in(m->b_k), as_in(m->b_v), w.qn, w.kn, m->invfreq, sh, m->qn, Kc, Vc, rs, m->Tmax));
  PK("attention", op_attention(s, m->qn, Kc, Vc, as_in(m->b_q), sh, m->att_split, m->pm, m->pl, m->po, m->xp_qa, rs, m->per, nullptr, 0, m->B));
  PK("gemm attn_out", site_gemm(m, {{&w.o, &m->b_a, nullptr, nullptr, 0}}, m->xp_qa, 0));
  PK("all-reduce", tp_reduce(m, m->b_a, m->r_a));
  return 0;
}

// x1 = xin + sum(b_a); h = rms(x1) * post -> planes; x1 + down(silu(gate h) * up h) stays split in b_dn
// The routed-expert FFN: router logits and top k on the normed rows, gate|up of every (row, slot), the slots'
// weights folded into silu(gate) * up, and one down launch per pass whose accumulation order is the rank order;
// like the dense FFN it leaves x1 + (its output) as x1 and K-slice partial sums in b_dn.
static int enq_moe_core(llb_spec *m, const FfnW &w, const RowSet *rs);
static int enq_moe_ffn(llb_spec *m, const FfnW &w, const float *xin, float *x1, const RowSet *rs) {
  cudaStream_t s = g_llb.stream;
  PK("norm post", op_norm_xp(s, xin, in_a(m), w.post, m->eps, m->d, x1, m->xp_d, 0, m->hn2, rs, m->Tmax, 0));
  return enq_moe_core(m, w, rs);
}
// ... from the normed rows on: planes in xp_d, the same rows as F32 in hn2
static int enq_moe_core(llb_spec *m, const FfnW &w, const RowSet *rs) {
  cudaStream_t s = g_llb.stream;
  const int ns = m->nk + 1, fe = ns * m->ef;
  const int *n_rows = m->B > 1 ? m->const_rows : &((const RowSet *)((uintptr_t)rs & ~(uintptr_t)1))->n;
  PK("moe route", op_moe_route(s, w.router, m->hn2, m->d, m->ne, m->nk, m->moe_lg, m->moe_ids, m->moe_wt, rs, m->Tmax));
  MoeArgs a;
  memset(&a, 0, sizeof a);
  a.ids = m->moe_ids; a.nslot = ns; a.ne = m->ne; a.ef = m->ef; a.d = m->d; a.T = m->Tmax; a.n_rows = n_rows;
  a.W = w.gu; a.es = w.es_gu; a.g = m->moe_g; a.u = m->moe_u;
  int one = 1;
  PK("moe gate|up", gemm_launch_moe(s, w.fmt_gu, false, m->xp_d, a, &one, nullptr));
  const bool silu_in_down = m->NC == 8;
  if (!silu_in_down) PK("moe silu", op_silu_scaled_xp(s, PartIn{m->moe_g, 1, 0}, PartIn{m->moe_u, 1, 0}, fe, m->xp_e, rs, m->Tmax, m->moe_wt, m->ef));
  const bool sel = m->NC >= 32;
  int ks = gemm_fix_ksplit(w.fmt_dn, m->NC, fe / 256, gemm_pick_ksplit(w.fmt_dn, m->NC, m->Tmax * (m->d / 16), fe / 256, g_llb.sms, sel), sel);
  CK(out_prepare(m, m->b_dn, m->d, ks));
  a.W = w.dn; a.es = w.es_dn; a.out = m->b_dn.p; a.split_stride = m->b_dn.stride;
  PK("moe down", gemm_launch_moe(s, w.fmt_dn, true, m->xp_e, a, &ks, silu_in_down ? m->moe_wt : nullptr));
  return 0;
}

static int enq_ffn(llb_spec *m, const FfnW &w, const float *xin, float *x1, const RowSet *rs) {
  cudaStream_t s = g_llb.stream;
  if (w.moe) return enq_moe_ffn(m, w, xin, x1, rs);
  PK("norm post", op_norm_xp(s, xin, in_a(m), w.post, m->eps, m->d, x1, m->xp_d, 0, nullptr, rs, m->Tmax, 0));
  if (w.gate.fmt == w.up.fmt && gemm_ffn_fusable(w.gate.fmt, w.down.fmt, m->NC, m->d) && m->tp.size <= 1) {
    // one launch: gate|up in one K-slice, a grid barrier, silu(gate) * up built in shared memory, down
    GemmArgs a1, a2;
    memset(&a1, 0, sizeof a1); memset(&a2, 0, sizeof a2);
    a1.K = m->d; a1.xp = m->xp_d; a1.planes = 2; a1.T = m->Tmax; a1.nmat = 2; a1.ksplit = 1;
    CK(out_prepare(m, m->b_g, w.gate.rows, 1)); CK(out_prepare(m, m->b_u, w.up.rows, 1));
    a1.m[0].W = w.gate.w; a1.m[0].rows = w.gate.rows; a1.m[0].out = m->b_g.p; a1.m[0].ostride = w.gate.rows; a1.m[0].split_stride = m->b_g.stride;
    a1.m[1].W = w.up.w; a1.m[1].rows = w.up.rows; a1.m[1].out = m->b_u.p; a1.m[1].ostride = w.up.rows; a1.m[1].split_stride = m->b_u.stride;
    const int ks2 = gemm_fix_ksplit(w.down.fmt, m->NC, m->f / 256, gemm_pick_ksplit(w.down.fmt, m->NC, (w.down.rows + 15) / 16, m->f / 256, g_llb.sms));
    a2.K = m->f; a2.xp = m->xp_f; a2.planes = 2; a2.T = m->Tmax; a2.nmat = 1; a2.ksplit = ks2;
    CK(out_prepare(m, m->b_dn, w.down.rows, ks2));
    a2.m[0].W = w.down.w; a2.m[0].rows = w.down.rows; a2.m[0].out = m->b_dn.p; a2.m[0].ostride = w.down.rows; a2.m[0].split_stride = m->b_dn.stride;
    PK("ffn fused", gemm_launch_ffn(s, a1, w.down.fmt, a2));
    return 0;
  }
  PK("gemm gate|up", site_gemm(m, {{&w.gate, &m->b_g, nullptr, nullptr, 0}, {&w.up, &m->b_u, nullptr, nullptr, 0}}, m->xp_d, 0));
  PK("silu", op_silu_xp(s, as_in(m->b_g), as_in(m->b_u), m->f, m->xp_f, rs, m->Tmax));
  PK("gemm down", site_gemm(m, {{&w.down, &m->b_dn, nullptr, nullptr, 0}}, m->xp_f, 0));
  PK("all-reduce", tp_reduce(m, m->b_dn, m->r_dn));
  return 0;
}

static int enq_delta(llb_spec *m, const DeltaW &w, float *ring, int ring_ks, float *S, const RowSet *rs) {
  cudaStream_t s = g_llb.stream;
  DeltaShape sh{m->TR, m->GK, m->SZ, m->KC, m->convd, m->kdc, m->vdc, m->eps};
  // raw qkv rows go straight into the conv ring slot of their position (host/llb_host.c:1747-1749)
  // (the ring keeps the K-slice partial sums of each row; the conv kernel adds them as it reads -- rows of earlier
  // passes too, whatever their width was, hence the split fixed per layer at open)
  PK("gemm qkv|z|b|a", site_gemm(m, {{&w.qkv, &m->b_ring, &m->ctl->verify.slot[0], ring, m->convd, (long long)CONV_RING * m->convd, ring_ks, ring_ks},
                   {&w.z, &m->b_z, nullptr, nullptr, 0}, {&w.beta, &m->b_bp, nullptr, nullptr, 0}, {&w.alpha, &m->b_ap, nullptr, nullptr, 0}},
               m->xp_d, 0));
  PK("delta conv", op_delta_conv(s, as_in(m->b_ring), w.conv, as_in(m->b_bp), as_in(m->b_ap), w.dt, w.a, sh, m->y, m->beta, m->decay, rs, m->Tmax));
  PK("delta scan+gnorm", op_delta_fused(s, S, m->ctl, m->y, m->beta, m->decay, as_in(m->b_z), w.norm, sh, m->xp_v, rs, m->B, m->s_group));
  PK("gemm ssm_out", site_gemm(m, {{&w.out, &m->b_a, nullptr, nullptr, 0}}, m->xp_v, 0));
  PK("all-reduce", tp_reduce(m, m->b_a, m->r_a));
  return 0;
}

// the (k+1)-row verify pass (spec_rows, host/llb_host.c:1714-1769)
static int enq_verify(llb_spec *m) {
  cudaStream_t s = g_llb.stream;
  // the verify rows were set before this pass began (k_accept of the previous cycle, or the host for a
  // prompt chunk): kernels may read them ahead of their wait
  const RowSet *rs = rs_stable(&m->ctl->verify);
  PK("embed", op_embed(s, m->embd.fmt, m->embd.w, m->d, rs, m->Tmax, m->x));
  PartIn none{nullptr, 0, 0};
  for (int il = 0; il < m->L; il++) {
    const LayerW &l = m->layer[il];
    // x += previous layer's FFN output (kept as partial sums), h = rms(x) * attn_norm
    PK("norm attn", op_norm_xp(s, il ? m->x1 : m->x, il ? in_dn(m) : none, l.attn_norm, m->eps, m->d, m->x, m->xp_d, 0, nullptr, rs,
                  m->Tmax, 0));
    if (l.full) CK(enq_attn(m, l.at, m->Kc[il], m->Vc[il], rs));
    else CK(enq_delta(m, l.dn, m->ring[il], m->ring_ks[il], m->S[il], rs));
    CK(enq_ffn(m, l.ffn, m->x, m->x1, rs));
  }
  PK("norm out", op_norm_xp(s, m->x1, in_dn(m), m->out_norm, m->eps, m->d, m->x, m->xp_d, 0, m->hn, rs, m->Tmax, 0));
  PK("gemm head", site_gemm(m, {{&m->head, &m->b_lg, nullptr, nullptr, 0}}, m->xp_d, 0));
  PK("top2", op_top2_part(s, as_in(m->b_lg), m->V, m->V, m->t2part, rs, m->Tmax));
  return 0;
}

// where the drafter's top-2 partials start in t2part (the trunk's come first)
static size_t t2_mtp(const llb_spec *m) { const int r = rows_cap(m); return (size_t)(r > SPEC_MAXT ? r : SPEC_MAXT) * TOP2_NB * 4; }
// the drafter's NextN block over rows `rs` with hidden rows `h` (mtp_rows, host/llb_host.c:1775-1808)
static int enq_mtp(llb_spec *m, const RowSet *rs, const float *h, bool with_head, int zero_h_at_pos0) {
  cudaStream_t s = g_llb.stream;
  PartIn none{nullptr, 0, 0};
  CK(op_embed(s, m->embd.fmt, m->embd.w, m->d, rs, m->Tmax, m->e));
  CK(op_norm_xp(s, m->e, none, m->mt_enorm, m->eps, m->d, nullptr, m->xp_2d, 0, nullptr, rs, m->Tmax, 0));
  CK(op_norm_xp(s, h, none, m->mt_hnorm, m->eps, m->d, nullptr, m->xp_2d, m->d, nullptr, rs, m->Tmax, zero_h_at_pos0));
  CK(site_gemm(m, {{&m->mt_eh, &m->b_eh, nullptr, nullptr, 0}}, m->xp_2d, 0));
  // x = eh_proj [e ; h]; normed by attn_norm into the planes; x itself kept in mt_x
  CK(op_norm_xp(s, nullptr, as_in(m->b_eh), m->mt_attn_norm, m->eps, m->d, m->mt_x, m->xp_d, 0, nullptr, rs, m->Tmax, 0));
  CK(enq_attn(m, m->mt_at, m->mt_Kc, m->mt_Vc, rs));
  CK(enq_ffn(m, m->mt_ffn, m->mt_x, m->x1, rs));
  CK(op_norm_xp(s, m->x1, in_dn(m), m->mt_shn, m->eps, m->d, nullptr, m->xp_d, 0, m->mt_hn, rs, m->Tmax, 0));
  if (with_head) {
    CK(site_gemm(m, {{&m->mt_head, &m->b_mlg, nullptr, nullptr, 0}}, m->xp_d, 0));
    CK(op_top2_part(s, as_in(m->b_mlg), m->mt_nv, m->mt_nv, m->t2part + t2_mtp(m), rs, m->Tmax));
  }
  return 0;
}

static int enq_cycle(llb_spec *m, bool spec) {
  cudaStream_t s = g_llb.stream;
  if (m->has_mtp) {
    // catch-up over the rows the previous cycle served; the hidden at position 0 is zero
    // (host/llb_host.c:1815-1817); in a speculative cycle its last row's head gives draft 1
    CK(enq_mtp(m, &m->ctl->catchup, m->hn, spec && m->k > 0, 0));
    if (spec) {
      for (int j = 1; j <= m->k; j++) {
        CK(op_draft_pick(s, m->t2part + t2_mtp(m), m->mt_ids, m->ctl, j > 1, j, m->mt_hn, m->chain_h, m->d, m->B, m->B > 1 ? m->per : 0));
        if (j < m->k) CK(enq_mtp(m, &m->ctl->chain, m->chain_h, true, 0));
      }
    }
  }
  CK(enq_verify(m));
  // sampling mode (speculative cycles only: a prompt chunk's rows are given): every row's emitted token from its logits
  const bool smp = spec && m->smp_on;
  if (smp) CK(op_smp_rows(s, m->smp, as_in(m->b_lg), m->V, m->smp_adj, m->ctl, m->Tmax, nullptr, nullptr, nullptr, nullptr, m->smp_tok, m->smp_val, nullptr,
                          m->smp_err));
  CK(op_accept(s, m->t2part, m->ctl, m->res_dev, m->res_n, m->Tmax, m->B, m->B > 1 ? m->per : 0, smp ? m->smp_tok : nullptr, smp ? m->smp_val : nullptr));
  if (m->lookup) CK(op_lookup_draft(s, m->ctl, m->B));   // the next cycle's drafts, from the history the accept kernel extended
  return 0;
}

// which: 0 the speculative cycle, 1 a prompt chunk, 2 the verify pass alone (no accept: replaying
// it changes nothing that is committed, so it can be timed in place)
static int capture(llb_spec *m, int which, cudaGraphExec_t *out, size_t *nodes) {
  cudaStream_t s = g_llb.stream;
  cudaGraph_t g = nullptr;
  CU_OK(cudaStreamSynchronize(s));
  StreamScope scope(m);
  CU_OK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  int rc = which == 2 ? enq_verify(m) : enq_cycle(m, which == 0);
  cudaError_t e = cudaStreamEndCapture(s, &g);
  if (rc) { if (g) cudaGraphDestroy(g); return -1; }
  if (e != cudaSuccess) return llb_fail("graph capture: %s", cudaGetErrorString(e));
  if (nodes) cudaGraphGetNodes(g, nullptr, nodes);
  e = cudaGraphInstantiate(out, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return llb_fail("graph instantiate: %s", cudaGetErrorString(e));
  return 0;
}

// ---- open ---------------------------------------------------------------------------------------
static int open_impl(llb_spec *m, const char *index_text, const uint8_t *pack, int on_device, const uint8_t *mtp, size_t mtp_bytes,
                     int mtp_on_device, int k, int max_ctx, int layers, int tp_n, int nstreams) {
  std::unordered_map<std::string, TensorRec> tab;
  CK(parse_index(m, index_text, tab));
  CK(validate_index(m, tab, m->pack_bytes));
  if (!m->share) { m->index_copy = index_text; m->layers_arg = layers; }
  const int L_index = m->L;   // the trunk's length in the index: a nextn (MTP) block, if the index has one, is block L_index
  if (layers > 0 && layers < m->L) m->L = layers;
  if (k < 0 || k > 7) return llb_fail("k = %d: the path takes 0..7 drafts (host/llb_host.c:1608)", k);
  if (max_ctx < 1 || max_ctx > (1 << 24)) return llb_fail("max_ctx = %d: a context of 1 .. 16777216 positions", max_ctx);
  if (m->SZ != 128 || m->KC < 2) return llb_fail("ssm_state_size %d / conv kernel %d unsupported", m->SZ, m->KC);
  if (m->hd != 128 && m->hd != 256) return llb_fail("head_dim %d unsupported", m->hd);
  if (m->ne > 0 && (m->sf != m->ef || m->ef % 256 || m->nk < 1 || m->nk > 32 || m->nk > m->ne || m->ne > 1024))
    return llb_fail("routed experts: %d experts, top %d, widths %d / %d (the shared expert must be as wide as the others, a multiple of 256; at most 1024 experts, top 32)",
                    m->ne, m->nk, m->ef, m->sf);
  if (m->d % 256 || m->f % 256 || m->vdc % 256 || (m->H * m->hd) % 256) return llb_fail("model widths must be multiples of 256");
  if (m->TR % m->GK || m->H % m->KV) return llb_fail("head counts do not divide");
  // ---- tensor parallel: this rank's share of the projections (tp.cuh).  Column split (rows of the matrix): attn_q by
  // query head, attn_k / attn_v by kv head, attn_qkv / attn_gate / ssm_beta / ssm_alpha by DeltaNet group and the value
  // heads that read it, ffn_gate / ffn_up by FFN column; row split (columns of the matrix, summed over the ranks by an
  // all-reduce): attn_output, ssm_out, ffn_down.  Embedding, head and norms are replicated: every rank computes the
  // same logits and takes the same accept decision, so no token ever has to be exchanged.
  m->Hf = m->H; m->KVf = m->KV; m->ff = m->f; m->GKf = m->GK; m->TRf = m->TR; m->kdcf = m->kdc; m->vdcf = m->vdc; m->convdf = m->convd;
  TpSel s_q, s_kv, s_o, s_f, s_qkv, s_vrow, s_head;   // rows of attn_q; of attn_k / v; columns of attn_output; FFN; rows of attn_qkv; value rows x 128; value heads
  const bool tp_on = tp_n > 1;
  if (tp_on) {
    if (tp_size() != tp_n) return llb_fail("llb_spec_open_tp: %d ranks asked for, llb_b200_tp_init joined %d", tp_n, tp_size());
    if (m->ne > 0) return llb_fail("tensor parallel: models with routed experts are not split");
    CK(tp_plan(tp_rank(), tp_n, m->H, m->KV, m->f, m->GK, m->TR, &m->tp));
    const TpPlan &t = m->tp;
    s_q.add(t.h0 * 2 * m->hd, t.H_l * 2 * m->hd);
    s_kv.add(t.kv0 * m->hd, t.KV_l * m->hd);
    s_o.add(t.h0 * m->hd, t.H_l * m->hd);
    s_f.add(t.f0, t.f_l);
    s_qkv.add(t.g0 * m->SZ, t.GK_l * m->SZ);
    s_qkv.add(m->kdc + t.g0 * m->SZ, t.GK_l * m->SZ);
    if (t.reps + 2 > 8) return llb_fail("tensor parallel: %d value heads per q/k group", t.reps);
    for (int r = 0; r < t.reps; r++) {
      s_qkv.add(2 * m->kdc + (r * m->GK + t.g0) * m->SZ, t.GK_l * m->SZ);
      s_vrow.add((r * m->GK + t.g0) * m->SZ, t.GK_l * m->SZ);
      s_head.add(r * m->GK + t.g0, t.GK_l);
    }
    m->H = t.H_l; m->KV = t.KV_l; m->f = t.f_l; m->GK = t.GK_l; m->TR = t.TR_l;
    m->kdc = m->GK * m->SZ; m->vdc = m->TR * m->SZ; m->convd = 2 * m->kdc + m->vdc;
    if (m->vdc % 256 || (m->H * m->hd) % 256) return llb_fail("tensor parallel: a rank's share (%d value columns, %d attention columns) is not whole super-blocks", m->vdc, m->H * m->hd);
  }
  // which rows / columns of a tensor this rank keeps, by the tensor's leaf name (trunk layers, a nextn block and the
  // drafter image use the same names)
  auto tp_sel = [&](const std::string &leaf, const TpSel *&rows, const TpSel *&cols) {
    rows = cols = nullptr;
    if (!tp_on) return;
    if (leaf == "attn_q") rows = &s_q;
    else if (leaf == "attn_k" || leaf == "attn_v") rows = &s_kv;
    else if (leaf == "attn_output") cols = &s_o;
    else if (leaf == "ffn_gate" || leaf == "ffn_up") rows = &s_f;
    else if (leaf == "ffn_down") cols = &s_f;
    else if (leaf == "attn_qkv" || leaf == "ssm_conv1d") rows = &s_qkv;
    else if (leaf == "attn_gate") rows = &s_vrow;
    else if (leaf == "ssm_beta" || leaf == "ssm_alpha") rows = &s_head;
    else if (leaf == "ssm_out") cols = &s_vrow;
    else if (leaf == "ssm_dt" || leaf == "ssm_a") cols = &s_head;
  };
  auto leaf_of = [](const std::string &name) {
    std::string n = name;
    for (const char *suf : {".weight", ".bias"}) { const size_t l = strlen(suf); if (n.size() > l && n.compare(n.size() - l, l, suf) == 0) n.resize(n.size() - l); }
    const size_t dot = n.rfind('.');
    return dot == std::string::npos ? n : n.substr(dot + 1);
  };
  { const char *e = getenv("LLB_PREFILL"); m->prefill_mode = e && !strcmp(e, "fast"); }   // the reference's switch (host/llb_host.c:206)
  m->k = k; m->Tspec = k + 1; m->max_ctx = max_ctx;
  if (nstreams < 1 || nstreams > 16) return llb_fail("streams: %d (1..16 per engine)", nstreams);
  m->B = nstreams;
  if (m->B > 1) {
    // the rows of all streams go through every GEMM together: 16 rows at most (32 plane columns)
    const int cap = 16;
    if (m->B * m->Tspec > cap) return llb_fail("streams: %d streams of k + 1 = %d rows are %d rows a pass, the limit is %d", m->B, m->Tspec, m->B * m->Tspec, cap);
    if (tp_on) return llb_fail("streams: a tensor-parallel engine runs one stream");
  }
  m->sq.assign(m->B, SeqHost());
  {
    // rows of a prompt chunk: 8, fewer where (H / KV) x rows would pass the attention kernel's 48 queries per kv head
    int pf = 8;
    const char *e = getenv("LLB_PREFILL_ROWS");
    if (e && atoi(e) >= 1 && atoi(e) <= SPEC_MAXT) pf = atoi(e);
    if (pf > 48 / (m->H / m->KV)) pf = 48 / (m->H / m->KV);
    m->Tpf = pf > m->Tspec ? pf : m->Tspec;
    if (m->B > 1) m->Tpf = m->Tspec;     // several streams: a stream's prompt chunk is as wide as its speculative pass
  }
  m->per = m->Tpf;
  m->Tmax = rows_cap(m);                 // buffers are sized for the widest pass
  m->R = m->Tpf + 1;                     // state-ring slots: a stream's rows + 1 (k + 2 in the reference, host/llb_host.c:1621)
  m->NC = nc_of(m->Tmax);
  const int d = m->d, qa = m->H * m->hd, kvd = m->KV * m->hd, T = m->Tmax, B = m->B;
  m->kv_group = 2LL * max_ctx * kvd;
  m->s_group = (long long)m->R * m->TR * m->SZ * m->SZ;
  std::unordered_map<uint64_t, void *> dedupe;
  auto mat = [&](const std::string &name, DevMat &w) -> int {
    auto it = tab.find(name);
    if (it == tab.end()) return llb_fail("pack has no tensor %s", name.c_str());
    const TpSel *rsel, *csel;
    tp_sel(leaf_of(name), rsel, csel);
    if (rsel || csel) return load_sliced(m, it->second, pack, m->pack_bytes, on_device, rsel, csel, w);
    void *p;
    CK(load_tensor(m, it->second, pack, m->pack_bytes, on_device, &p, dedupe));
    w.w = (uint8_t *)p; w.rows = it->second.rows; w.cols = it->second.cols; w.fmt = it->second.fmt;
    return 0;
  };
  auto vec = [&](const std::string &name, float **v, int n) -> int {
    DevMat w;
    CK(mat(name, w));
    if (w.fmt != LLB_FM_F32 || w.rows * w.cols != n) return llb_fail("%s must be %d F32 values", name.c_str(), n);
    *v = (float *)w.w;
    return 0;
  };
  CK(mat("token_embd.weight", m->embd));
  CK(mat("output.weight", m->head));
  CK(check_k(m->head, m->V, d, "output.weight"));
  if (m->embd.rows != m->V || m->embd.cols != d) return llb_fail("token_embd.weight shape");
  CK(vec("output_norm.weight", &m->out_norm, d));
  m->layer.resize(m->L);
  m->Kc.assign(m->L, nullptr); m->Vc.assign(m->L, nullptr); m->ring.assign(m->L, nullptr); m->S.assign(m->L, nullptr); m->ring_ks.assign(m->L, 1);
  for (int il = 0; il < m->L; il++) {
    LayerW &l = m->layer[il];
    std::string p = "blk." + std::to_string(il) + ".";
    l.full = (il + 1) % m->interval == 0;
    CK(vec(p + "attn_norm.weight", &l.attn_norm, d));
    if (l.full) {
      CK(mat(p + "attn_q.weight", l.at.q)); CK(check_k(l.at.q, 2 * qa, d, "attn_q"));
      CK(mat(p + "attn_k.weight", l.at.k)); CK(check_k(l.at.k, kvd, d, "attn_k"));
      CK(mat(p + "attn_v.weight", l.at.v)); CK(check_k(l.at.v, kvd, d, "attn_v"));
      CK(mat(p + "attn_output.weight", l.at.o)); CK(check_k(l.at.o, d, qa, "attn_output"));
      CK(vec(p + "attn_q_norm.weight", &l.at.qn, m->hd));
      CK(vec(p + "attn_k_norm.weight", &l.at.kn, m->hd));
      m->Kc[il] = falloc(m, (size_t)B * max_ctx * kvd); m->Vc[il] = falloc(m, (size_t)B * max_ctx * kvd);
      if (!m->Kc[il] || !m->Vc[il]) return -1;
    } else {
      CK(mat(p + "attn_qkv.weight", l.dn.qkv)); CK(check_k(l.dn.qkv, m->convd, d, "attn_qkv"));
      CK(mat(p + "attn_gate.weight", l.dn.z)); CK(check_k(l.dn.z, m->vdc, d, "attn_gate"));
      CK(mat(p + "ssm_beta.weight", l.dn.beta)); CK(check_k(l.dn.beta, m->TR, d, "ssm_beta"));
      CK(mat(p + "ssm_alpha.weight", l.dn.alpha)); CK(check_k(l.dn.alpha, m->TR, d, "ssm_alpha"));
      CK(mat(p + "ssm_out.weight", l.dn.out)); CK(check_k(l.dn.out, d, m->vdc, "ssm_out"));
      CK(vec(p + "ssm_dt.bias", &l.dn.dt, m->TR));
      CK(vec(p + "ssm_a", &l.dn.a, m->TR));
      CK(vec(p + "ssm_conv1d.weight", &l.dn.conv, m->convd * m->KC));
      CK(vec(p + "ssm_norm.weight", &l.dn.norm, m->SZ));
      {
        // the launch attn_qkv lands in: the matrices of its format among qkv | z | beta | alpha
        int ntiles = 0;
        for (const DevMat *w : {&l.dn.qkv, &l.dn.z, &l.dn.beta, &l.dn.alpha}) if (w->fmt == l.dn.qkv.fmt) ntiles += (w->rows + 15) / 16;
        const int ks = gemm_ring_ksplit(l.dn.qkv.fmt, d / 256, ntiles, nc_of(B * m->Tspec), nc_of(B > 1 ? B * m->Tspec : m->Tpf), g_llb.sms, RING_MAXSPLIT);
        if (ks < 1) return llb_fail("blk.%d.attn_qkv: %d columns need more than %d K-slices at a pass width in use", il, d, RING_MAXSPLIT);
        m->ring_ks[il] = ks;
      }
      m->ring[il] = falloc(m, (size_t)B * m->ring_ks[il] * CONV_RING * m->convd);
      m->S[il] = falloc(m, (size_t)B * m->s_group);
      if (!m->ring[il] || !m->S[il]) return -1;
    }
    CK(vec(p + "post_attention_norm.weight", &l.ffn.post, d));
    if (m->ne > 0) { CK(load_moe(m, l.ffn, p, tab, pack, on_device)); continue; }
    CK(mat(p + "ffn_gate.weight", l.ffn.gate)); CK(check_k(l.ffn.gate, m->f, d, "ffn_gate"));
    CK(mat(p + "ffn_up.weight", l.ffn.up)); CK(check_k(l.ffn.up, m->f, d, "ffn_up"));
    CK(mat(p + "ffn_down.weight", l.ffn.down)); CK(check_k(l.ffn.down, d, m->f, "ffn_down"));
  }
  // rope inverse frequencies in double, as the reference computes the angle (tools/qwen35_engine.c:527)
  {
    std::vector<double> f(m->rope_dim / 2);
    for (int i = 0; i < m->rope_dim / 2; i++) f[i] = pow((double)m->rope_base, -2.0 * i / m->rope_dim);
    m->invfreq = (double *)dalloc(m, f.size() * 8);
    if (!m->invfreq) return -1;
    CU_OK(cudaMemcpyAsync(m->invfreq, f.data(), f.size() * 8, cudaMemcpyHostToDevice, g_llb.stream));
    CU_OK(cudaStreamSynchronize(g_llb.stream));
  }
  // drafter: AUX1 named container (host/llb_host.c:1543-1570) or positional MTP1 (:1539-1542)
  if (mtp && mtp_bytes >= 16) {
    static const char *names[17] = {"nextn.enorm", "nextn.hnorm", "nextn.eh_proj", "attn_norm", "attn_q", "attn_k", "attn_v",
                                    "attn_q_norm", "attn_k_norm", "attn_output", "post_attention_norm", "ffn_gate", "ffn_up", "ffn_down",
                                    "nextn.shared_head_norm", "mtp.head_slice", "mtp.ids"};
    std::vector<uint8_t> hdr(16 + 72 * 64);
    size_t hb = mtp_bytes < hdr.size() ? mtp_bytes : hdr.size();
    if (mtp_on_device) CU_OK(cudaMemcpy(hdr.data(), mtp, hb, cudaMemcpyDeviceToHost)); else memcpy(hdr.data(), mtp, hb);
    if (!m->share) { m->mtp_hdr.assign(hdr.begin(), hdr.begin() + hb); m->mtp_total = mtp_bytes; }
    uint64_t off[17], nb[17];
    int fm[17];
    bool got[17] = {false};
    const int mtp1_fmt[17] = {0, 0, LLB_FM_Q4_K, 0, LLB_FM_Q6_K, LLB_FM_Q6_K, LLB_FM_Q6_K, 0, 0, LLB_FM_Q6_K, 0, LLB_FM_Q4_K, LLB_FM_Q4_K,
                              LLB_FM_Q4_K, 0, LLB_FM_Q6_K, 0};
    if (!memcmp(hdr.data(), "MTP1", 4)) {
      uint32_t n; memcpy(&n, hdr.data() + 4, 4);
      if (n != 17) return llb_fail("MTP1: %u entries, 17 expected", n);
      for (int j = 0; j < 17; j++) { memcpy(&off[j], hdr.data() + 8 + 16 * j, 8); memcpy(&nb[j], hdr.data() + 16 + 16 * j, 8); fm[j] = mtp1_fmt[j]; got[j] = true; }
    } else if (!memcmp(hdr.data(), "AUX1", 4)) {
      uint32_t n; memcpy(&n, hdr.data() + 8, 4);
      if (n < 17 || n > 64) return llb_fail("AUX1: %u entries", n);
      for (uint32_t i = 0; i < n; i++) {
        const uint8_t *e = hdr.data() + 16 + 72 * (size_t)i;
        char nm[33]; memcpy(nm, e, 32); nm[32] = 0;
        for (int j = 0; j < 17; j++) if (!strcmp(nm, names[j])) {
          if (got[j]) return llb_fail("AUX1: duplicate entry %s", nm);
          uint32_t dt; memcpy(&dt, e + 32, 4); memcpy(&off[j], e + 56, 8); memcpy(&nb[j], e + 64, 8);
          fm[j] = dt == 0 ? LLB_FM_F32 : dt == 2 ? LLB_FM_Q8_0 : dt == 3 ? LLB_FM_Q4_K : dt == 4 ? LLB_FM_Q6_K : dt == 7 ? LLB_FM_Q5_K : j == 16 ? 0 : -1;
          got[j] = true;
        }
      }
    } else return llb_fail("drafter image is neither AUX1 nor MTP1");
    for (int j = 0; j < 17; j++) if (!got[j] || fm[j] < 0 || off[j] + nb[j] > mtp_bytes) return llb_fail("drafter image: entry %s missing or out of range", names[j]);
    const int nv = (int)(nb[16] / 4);
    // shapes in the image are the whole model's; a tensor-parallel rank keeps its share of the attention and FFN matrices
    const int qaf = m->Hf * m->hd, kvdf = m->KVf * m->hd;
    int rows[17] = {1, 1, d, 1, 2 * qaf, kvdf, kvdf, 1, 1, d, 1, m->ff, m->ff, d, 1, nv, 1};
    int cols[17] = {d, d, 2 * d, d, d, d, d, m->hd, m->hd, qaf, d, d, d, m->ff, d, d, nv};
    std::unordered_map<uint64_t, void *> dd;
    void *ptr[17];
    for (int j = 0; j < 17; j++) {
      TensorRec t{off[j], nb[j], rows[j], cols[j], j == 16 ? LLB_FM_F32 : fm[j]};
      const TpSel *rsel, *csel;
      tp_sel(names[j], rsel, csel);
      if (rsel || csel) {
        DevMat w;
        CK(load_sliced(m, t, mtp, mtp_bytes, mtp_on_device, rsel, csel, w));
        ptr[j] = w.w; rows[j] = w.rows; cols[j] = w.cols;
      } else {
        CK(load_tensor(m, t, mtp, mtp_bytes, mtp_on_device, &ptr[j], dd));
      }
    }
    auto MM = [&](int j) { DevMat w; w.w = (uint8_t *)ptr[j]; w.rows = rows[j]; w.cols = cols[j]; w.fmt = fm[j]; return w; };
    m->mt_enorm = (float *)ptr[0]; m->mt_hnorm = (float *)ptr[1]; m->mt_eh = MM(2); m->mt_attn_norm = (float *)ptr[3];
    m->mt_at.q = MM(4); m->mt_at.k = MM(5); m->mt_at.v = MM(6); m->mt_at.qn = (float *)ptr[7]; m->mt_at.kn = (float *)ptr[8];
    m->mt_at.o = MM(9); m->mt_ffn.post = (float *)ptr[10]; m->mt_ffn.gate = MM(11); m->mt_ffn.up = MM(12); m->mt_ffn.down = MM(13);
    m->mt_shn = (float *)ptr[14]; m->mt_head = MM(15); m->mt_ids = (int *)ptr[16]; m->mt_nv = nv;
    CK(check_k(m->mt_eh, d, 2 * d, "nextn.eh_proj")); CK(check_k(m->mt_head, nv, d, "mtp.head_slice"));
    m->mt_Kc = falloc(m, (size_t)B * max_ctx * kvd); m->mt_Vc = falloc(m, (size_t)B * max_ctx * kvd);
    if (!m->mt_Kc || !m->mt_Vc) return -1;
    m->has_mtp = true;
  } else if (k > 0 && m->ne == 0 && tab.count("blk." + std::to_string(L_index) + ".nextn.eh_proj.weight")) {
    // no image, but the index holds the model's own nextn block after the trunk (a GGUF with nextn_predict_layers,
    // reports/cuda-moe/scripts/gen_moe.py:116-118): the same 15 tensors by their GGUF names, the trunk's head and the
    // whole vocabulary (no draft-vocabulary slice, ids = identity)
    const std::string p = "blk." + std::to_string(L_index) + ".";
    CK(vec(p + "nextn.enorm.weight", &m->mt_enorm, d)); CK(vec(p + "nextn.hnorm.weight", &m->mt_hnorm, d));
    CK(mat(p + "nextn.eh_proj.weight", m->mt_eh)); CK(check_k(m->mt_eh, d, 2 * d, "nextn.eh_proj"));
    CK(vec(p + "attn_norm.weight", &m->mt_attn_norm, d));
    CK(mat(p + "attn_q.weight", m->mt_at.q)); CK(check_k(m->mt_at.q, 2 * qa, d, "nextn attn_q"));
    CK(mat(p + "attn_k.weight", m->mt_at.k)); CK(check_k(m->mt_at.k, kvd, d, "nextn attn_k"));
    CK(mat(p + "attn_v.weight", m->mt_at.v)); CK(check_k(m->mt_at.v, kvd, d, "nextn attn_v"));
    CK(mat(p + "attn_output.weight", m->mt_at.o)); CK(check_k(m->mt_at.o, d, qa, "nextn attn_output"));
    CK(vec(p + "attn_q_norm.weight", &m->mt_at.qn, m->hd)); CK(vec(p + "attn_k_norm.weight", &m->mt_at.kn, m->hd));
    CK(vec(p + "post_attention_norm.weight", &m->mt_ffn.post, d));
    CK(mat(p + "ffn_gate.weight", m->mt_ffn.gate)); CK(check_k(m->mt_ffn.gate, m->f, d, "nextn ffn_gate"));
    CK(mat(p + "ffn_up.weight", m->mt_ffn.up)); CK(check_k(m->mt_ffn.up, m->f, d, "nextn ffn_up"));
    CK(mat(p + "ffn_down.weight", m->mt_ffn.down)); CK(check_k(m->mt_ffn.down, d, m->f, "nextn ffn_down"));
    CK(vec(p + "nextn.shared_head_norm.weight", &m->mt_shn, d));
    m->mt_head = m->head; m->mt_ids = nullptr; m->mt_nv = m->V;
    m->mt_Kc = falloc(m, (size_t)B * max_ctx * kvd); m->mt_Vc = falloc(m, (size_t)B * max_ctx * kvd);
    if (!m->mt_Kc || !m->mt_Vc) return -1;
    m->has_mtp = true;
  } else if (k > 0) {
    // no MTP image: the reference's other drafter, prompt lookup over the token history
    m->lookup = true;
  }
  // every stream's token history on the device: the lookup drafter searches it, the sampler's penalties read its tail
  m->hist = (int *)dalloc(m, (size_t)B * ((size_t)max_ctx + 16) * 4);
  if (!m->hist) return -1;

  // activations
  int big = m->f > m->convd ? m->f : m->convd;
  const int Tc = T > SPEC_MAXT ? T : SPEC_MAXT;
  m->x = falloc(m, (size_t)T * d); m->x1 = falloc(m, (size_t)T * d); m->hn = falloc(m, (size_t)Tc * d); m->e = falloc(m, (size_t)T * d);
  m->qn = falloc(m, (size_t)T * qa); m->y = falloc(m, (size_t)T * big); m->beta = falloc(m, (size_t)T * m->TR); m->decay = falloc(m, (size_t)T * m->TR);
  m->t2part = falloc(m, (size_t)2 * Tc * TOP2_NB * 4);
  m->mt_x = falloc(m, (size_t)T * d); m->mt_hn = falloc(m, (size_t)T * d); m->chain_h = falloc(m, (size_t)T * d);
  m->att_split = g_llb.sms / (m->KV * B);   // one wave of blocks: the kernel takes a whole SM's shared memory
  if (m->att_split < 1) m->att_split = 1;
  if (m->att_split > 128) m->att_split = 128;
  m->pm = falloc(m, (size_t)m->H * T * m->att_split); m->pl = falloc(m, (size_t)m->H * T * m->att_split);
  m->po = falloc(m, (size_t)m->H * T * m->att_split * m->hd);
  CK(xp_alloc(m, 0, d)); CK(xp_alloc(m, 1, m->f)); CK(xp_alloc(m, 2, qa)); CK(xp_alloc(m, 3, m->vdc));
  CK(xp_alloc(m, 4, 2 * d));
  for (int v = 0; v < 3; v++) m->xpv[v][5] = m->xpv[v][0];   // placeholder where there are no routed experts
  if (m->ne > 0) {
    const int ns = m->nk + 1;
    m->moe_lg = falloc(m, (size_t)T * (m->ne + 1)); m->moe_wt = falloc(m, (size_t)T * ns); m->moe_ids = (int *)dalloc(m, (size_t)T * ns * 4);
    m->moe_g = falloc(m, (size_t)T * ns * m->ef); m->moe_u = falloc(m, (size_t)T * ns * m->ef); m->hn2 = falloc(m, (size_t)T * d);
    CK(xp_alloc(m, 5, ns * m->ef));
    if (!m->moe_lg || !m->moe_wt || !m->moe_ids || !m->moe_g || !m->moe_u || !m->hn2) return -1;
  }
  m->ctl = (SpecCtl *)dalloc(m, sizeof(SpecCtl) * B);
  m->const_rows = (int *)dalloc(m, 4);
  if (!m->x || !m->po || !m->ctl || !m->const_rows) return -1;
  { const int rows = B * m->Tspec; CU_OK(cudaMemcpyAsync(m->const_rows, &rows, 4, cudaMemcpyHostToDevice, g_llb.stream)); CU_OK(cudaStreamSynchronize(g_llb.stream)); }
  CU_OK(cudaHostAlloc((void **)&m->res_host, sizeof(SpecResult) * m->res_n * B, cudaHostAllocMapped));
  memset(m->res_host, 0, sizeof(SpecResult) * m->res_n * B);
  CU_OK(cudaHostGetDevicePointer((void **)&m->res_dev, m->res_host, 0));
  CK(ops_model_setup());
  set_width(m, B * m->Tspec);
  return 0;
}

// ---- the prompt path: chunks of up to PF_RMAX rows through dense tcgen05 GEMMs (pf.cu) ----------------------------
#define PF_GROUPS (PF_RMAX + 1)
static int pf_alloc(llb_spec *m) {
  PfState &f = m->pf;
  if (f.ready) return 0;
  CK(pf_setup());
  const int d = m->d, qa = m->H * m->hd;
  auto kg = [&](int K) { return (__half *)dalloc(m, (PF_RMAX / PF_R) * pf_kg_halves(K) * 2); };   // the chunk's units one after the other
  f.x = falloc(m, (size_t)PF_RMAX * d); f.x1 = falloc(m, (size_t)PF_RMAX * d); f.hn = falloc(m, (size_t)(PF_RMAX + 1) * d); f.e = falloc(m, (size_t)PF_RMAX * d);
  f.qn = falloc(m, (size_t)PF_RMAX * qa); f.y = falloc(m, (size_t)PF_RMAX * m->convd); f.beta = falloc(m, (size_t)PF_RMAX * m->TR);
  f.decay = falloc(m, (size_t)PF_RMAX * m->TR); f.o = falloc(m, (size_t)PF_RMAX * m->vdc);
  f.kg_d = kg(d); f.kg_f = kg(m->f); f.kg_qa = kg(qa); f.kg_v = kg(m->vdc); f.kg_2d = kg(2 * d);
  {
    const size_t ng = (PF_RMAX + m->Tpf - 1) / m->Tpf, per = (size_t)m->H * m->Tpf * m->att_split;
    f.pm = falloc(m, ng * per); f.pl = falloc(m, ng * per); f.po = falloc(m, ng * per * m->hd);
    if (!f.pm || !f.pl || !f.po) return -1;
  }
  f.rs = (RowSet *)dalloc(m, sizeof(RowSet) * (1 + PF_GROUPS));
  f.ids = (int *)dalloc(m, (size_t)(PF_RMAX + 1) * 4);
  if (!f.x || !f.x1 || !f.hn || !f.e || !f.qn || !f.y || !f.beta || !f.decay || !f.o || !f.kg_d || !f.kg_f || !f.kg_qa || !f.kg_v || !f.kg_2d ||
      !f.rs || !f.ids) return -1;
  f.ready = true;
  return 0;
}

// LLB_PF_MS=1 (the reference's switch for timing a fast-prefill chunk, host/llb_backend_cuda.h:215): device time of a
// prompt's dense path by kind of op, printed to stderr when the prompt is done
struct PfProf { const char *name; cudaEvent_t a, b; };
static std::vector<PfProf> g_pfprof;
static int pf_prof_on() { static int v = -1; if (v < 0) { const char *e = getenv("LLB_PF_MS"); v = e && e[0] == '1'; } return v; }
struct PfTimer {
  PfProf r; bool on;
  PfTimer(const char *name) : on(pf_prof_on() != 0) { if (on) { r.name = name; cudaEventCreate(&r.a); cudaEventCreate(&r.b); cudaEventRecord(r.a, g_llb.stream); } }
  ~PfTimer() { if (on) { cudaEventRecord(r.b, g_llb.stream); g_pfprof.push_back(r); } }
};
static void pf_prof_report(int rows, double wall_ms) {
  if (!pf_prof_on()) return;
  cudaStreamSynchronize(g_llb.stream);
  std::vector<std::string> names; std::vector<double> tot; std::vector<int> cnt;
  for (auto &r : g_pfprof) {
    float ms = 0; cudaEventElapsedTime(&ms, r.a, r.b);
    size_t k = 0;
    for (; k < names.size(); k++) if (names[k] == r.name) break;
    if (k == names.size()) { names.push_back(r.name); tot.push_back(0); cnt.push_back(0); }
    tot[k] += ms; cnt[k]++;
    cudaEventDestroy(r.a); cudaEventDestroy(r.b);
  }
  g_pfprof.clear();
  fprintf(stderr, "pf: %d rows in %.1f ms:", rows, wall_ms);
  for (size_t k = 0; k < names.size(); k++) fprintf(stderr, " %s %.2f ms / %d;", names[k].c_str(), tot[k], cnt[k]);
  fprintf(stderr, "\n");
}
#define PFK(name, call) do { PfTimer t_(name); if ((call)) return -1; } while (0)

struct PfSiteMat { const DevMat *w; OutBuf *out; };
// the dense GEMMs of one site: matrices sharing the activations `kg` of K columns, one launch per format
static int pf_site(llb_spec *m, std::vector<PfSiteMat> mats, const __half *kg, int K, int R) {
  std::vector<bool> done(mats.size(), false);
  for (size_t i = 0; i < mats.size(); i++) {
    if (done[i]) continue;
    PfArgs a;
    memset(&a, 0, sizeof a);
    a.K = K; a.R = R; a.x = kg;
    int ntiles = 0;
    std::vector<size_t> grp;
    for (size_t j = i; j < mats.size() && grp.size() < PF_MAXMAT; j++)
      if (!done[j] && mats[j].w->fmt == mats[i].w->fmt) { grp.push_back(j); ntiles += (mats[j].w->rows + 127) / 128; }
    a.ksplit = pf_pick_ksplit(ntiles, K / 256, g_llb.sms);
    a.nmat = (int)grp.size();
    for (size_t g = 0; g < grp.size(); g++) {
      const PfSiteMat &sm = mats[grp[g]];
      OutBuf &o = *sm.out;
      const size_t need = (size_t)a.ksplit * PF_RMAX * sm.w->rows;
      if (!o.p || o.cap < need) {
        o.p = falloc(m, need);
        if (!o.p) return -1;
        o.cap = need;
      }
      o.ns = a.ksplit; o.stride = (long long)PF_RMAX * sm.w->rows;
      a.m[g].W = sm.w->w; a.m[g].rows = sm.w->rows; a.m[g].ostride = sm.w->rows; a.m[g].out = o.p; a.m[g].split_stride = o.stride;
      done[grp[g]] = true;
    }
    CK(pf_gemm(g_llb.stream, mats[i].w->fmt, a));
  }
  return 0;
}

// One chunk: rows of positions p0 .. p0 + R - 1 with the given tokens through every layer.  Leaves the trunk's K/V rows,
// conv rings and DeltaNet states as the T-row pass would have (the state written back into the committed slot), the
// drafter's K/V rows of the same positions, and in pf.hn row 0 the normed hidden of the chunk's last row.
static int pf_chunk(llb_spec *m, int b, const int *ids, int p0, int R) {
  PfState &f = m->pf;
  cudaStream_t s = g_llb.stream;
  StreamScope scope(m, true);   // the chunk's kernels see one stream: stream b's state is handed to them directly
  const int d = m->d, qa = m->H * m->hd, gsz = m->Tpf, ngrp = (R + gsz - 1) / gsz;
  std::vector<RowSet> rs(1 + ngrp);
  memset(rs.data(), 0, rs.size() * sizeof(RowSet));
  rs[0].n = R; rs[0].pos0 = p0;
  for (int g = 0; g < ngrp; g++) { rs[1 + g].n = R - g * gsz < gsz ? R - g * gsz : gsz; rs[1 + g].pos0 = p0 + g * gsz; }
  CU_OK(cudaMemcpyAsync(f.rs, rs.data(), rs.size() * sizeof(RowSet), cudaMemcpyHostToDevice, s));
  CU_OK(cudaMemcpyAsync(f.ids, ids + p0, (size_t)R * 4, cudaMemcpyHostToDevice, s));
  CU_OK(cudaStreamSynchronize(s));   // rs is a local: the copy must have read it before it goes
  PartIn none{nullptr, 0, 0};
  AttnShape ash{m->H, m->KV, m->hd, m->rope_dim, m->eps, m->att_min, (long long)m->max_ctx * m->KV * m->hd, (int)sizeof(RowSet), 0};
  DeltaShape dsh{m->TR, m->GK, m->SZ, m->KC, m->convd, m->kdc, m->vdc, m->eps};
  PFK("embed", op_pf_embed(s, m->embd.fmt, m->embd.w, d, f.ids, R, f.x));
  for (int il = 0; il < m->L; il++) {
    const LayerW &l = m->layer[il];
    PFK("norm", op_pf_norm(s, il ? f.x1 : f.x, il ? as_in(f.dn) : none, l.attn_norm, m->eps, d, f.x, f.kg_d, d, 0, nullptr, R));
    if (l.full) {
      PFK("gemm qkv", pf_site(m, {{&l.at.q, &f.q}, {&l.at.k, &f.k}, {&l.at.v, &f.v}}, f.kg_d, d, R));
      PFK("qkrope", op_qkrope(s, as_in(f.q), as_in(f.k), as_in(f.v), l.at.qn, l.at.kn, m->invfreq, ash, f.qn, kc_of(m, m->Kc[il], b), kc_of(m, m->Vc[il], b), &f.rs[0], R));
      // every group of gsz rows in one launch (grid z): each streams the K/V rows up to its own last position
      PFK("attention", op_attention(s, f.qn, kc_of(m, m->Kc[il], b), kc_of(m, m->Vc[il], b), as_in(f.q), ash, m->att_split, f.pm, f.pl, f.po, m->xp_qa, &f.rs[1], gsz, f.kg_qa, 0, ngrp));
      PFK("gemm attn_out", pf_site(m, {{&l.at.o, &f.a}}, f.kg_qa, qa, R));
    } else {
      PFK("gemm qkv|z|b|a", pf_site(m, {{&l.dn.qkv, &f.qkv}, {&l.dn.z, &f.z}, {&l.dn.beta, &f.bp}, {&l.dn.alpha, &f.ap}}, f.kg_d, d, R));
      PFK("delta", op_pf_delta(s, as_in(f.qkv), as_in(f.z), as_in(f.bp), as_in(f.ap), ring_of(m, il, b), m->ring_ks[il], l.dn.conv, l.dn.dt, l.dn.a, l.dn.norm, dsh,
                     state_of(m, il, b), ctl_of(m, b), f.y, f.beta, f.decay, f.o, f.kg_v, p0, R));
      PFK("gemm ssm_out", pf_site(m, {{&l.dn.out, &f.a}}, f.kg_v, m->vdc, R));
    }
    PFK("norm", op_pf_norm(s, f.x, as_in(f.a), l.ffn.post, m->eps, d, f.x1, f.kg_d, d, 0, nullptr, R));
    PFK("gemm gate|up", pf_site(m, {{&l.ffn.gate, &f.g}, {&l.ffn.up, &f.u}}, f.kg_d, d, R));
    PFK("silu", op_pf_silu(s, as_in(f.g), as_in(f.u), m->f, f.kg_f, R));
    PFK("gemm down", pf_site(m, {{&l.ffn.down, &f.dn}}, f.kg_f, m->f, R));
  }
  // the trunk's output-normed rows: row r of the chunk into pf.hn row r + 1 (row 0 holds the row before the chunk)
  CK(op_pf_norm(s, f.x1, as_in(f.dn), m->out_norm, m->eps, d, nullptr, nullptr, 0, 0, f.hn + d, R));
  if (m->has_mtp) {
    // the drafter's row at position p pairs token p with the trunk's normed hidden of position p - 1
    // (host/llb_host.c:1775-1808); a prompt chunk only needs its K and V rows (:1831-1876)
    CK(op_pf_embed(s, m->embd.fmt, m->embd.w, d, f.ids, R, f.e));
    CK(op_pf_norm(s, f.e, none, m->mt_enorm, m->eps, d, nullptr, f.kg_2d, 2 * d, 0, nullptr, R));
    CK(op_pf_norm(s, f.hn, none, m->mt_hnorm, m->eps, d, nullptr, f.kg_2d, 2 * d, d, nullptr, R));
    CK(pf_site(m, {{&m->mt_eh, &f.eh}}, f.kg_2d, 2 * d, R));
    CK(op_pf_norm(s, nullptr, as_in(f.eh), m->mt_attn_norm, m->eps, d, nullptr, f.kg_d, d, 0, nullptr, R));
    CK(pf_site(m, {{&m->mt_at.k, &f.k}, {&m->mt_at.v, &f.v}}, f.kg_d, d, R));
    CK(op_qkrope(s, none, as_in(f.k), as_in(f.v), m->mt_at.qn, m->mt_at.kn, m->invfreq, ash, f.qn, kc_of(m, m->mt_Kc, b), kc_of(m, m->mt_Vc, b), &f.rs[0], R, true));
  }
  CU_OK(cudaMemcpyAsync(f.hn, f.hn + (size_t)R * d, (size_t)d * 4, cudaMemcpyDeviceToDevice, s));
  m->pf_rows += R;
  return 0;
}

// The fast part of a prompt: whole chunks from position 0 while more than `keep` rows remain for the T-row pass.
// Returns the position the T-row pass continues from; the drafter's row there is left pending as a one-row catch-up
// whose hidden (the normed row of the position before) is put where the catch-up reads it.
static int pf_prefill(llb_spec *m, int b, const int *ids, int n_rows, int keep, int *p_out) {
  CK(pf_alloc(m));
  PfState &f = m->pf;
  CU_OK(cudaMemsetAsync(f.hn, 0, (size_t)m->d * 4, g_llb.stream));   // the hidden before position 0 is zero (host/llb_host.c:1816)
  int p = 0;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (pf_prof_on()) { cudaEventCreate(&e0); cudaEventCreate(&e1); cudaEventRecord(e0, g_llb.stream); }
  while (n_rows - p > keep) {
    const int R = n_rows - p - keep < PF_RMAX ? n_rows - p - keep : PF_RMAX;
    CK(pf_chunk(m, b, ids, p, R));
    p += R;
  }
  if (e0) {
    float ms = 0;
    cudaEventRecord(e1, g_llb.stream); cudaEventSynchronize(e1); cudaEventElapsedTime(&ms, e0, e1);
    pf_prof_report(p, ms);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
  }
  if (p > 0) {
    // the stream's first row of the trunk's normed hidden rows: what the pending catch-up row pairs with
    CU_OK(cudaMemcpyAsync(m->hn + (size_t)(m->B > 1 ? b * m->per : 0) * m->d, f.hn, (size_t)m->d * 4, cudaMemcpyDeviceToDevice, g_llb.stream));
    struct { int n, pos0, tok[SPEC_MAXT], slot[SPEC_MAXT]; } c;
    memset(&c, 0, sizeof c);
    c.n = m->has_mtp ? 1 : 0; c.pos0 = p; c.tok[0] = ids[p];
    CU_OK(cudaMemcpyAsync(&ctl_of(m, b)->catchup, &c, sizeof c, cudaMemcpyHostToDevice, g_llb.stream));
    CU_OK(cudaStreamSynchronize(g_llb.stream));
  }
  *p_out = p;
  return 0;
}

static int ctl_write(llb_spec *m, int b, const SpecCtl &c) {
  CU_OK(cudaMemcpyAsync(ctl_of(m, b), &c, sizeof c, cudaMemcpyHostToDevice, g_llb.stream));
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  return 0;
}
// a fresh control block of stream b
static SpecCtl ctl_fresh(const llb_spec *m, int b) {
  SpecCtl c;
  memset(&c, 0, sizeof c);
  c.R = m->R; c.k = m->k; c.max_pos = m->max_ctx; c.seq = m->sq[b].seq; c.hist = hist_of(m, b);
  return c;
}

static int wait_result(llb_spec *m, int b, SpecResult *out) {
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  SeqHost &q = m->sq[b];
  const SpecResult *r = &m->res_host[(size_t)b * m->res_n + q.seq % (unsigned long long)m->res_n];
  if (r->seq != q.seq + 1) return llb_fail("cycle %llu of stream %d did not report (device error word set?)", q.seq, b);
  *out = *r;
  q.seq += 1;
  return 0;
}
// the host mirror of stream b after a cycle that reported r
static void note_cycle(llb_spec *m, int b, const SpecResult &r, int served_idx) {
  SeqHost &q = m->sq[b];
  q.pos += r.served;
  q.last_tok = r.ids[r.served - 1];
  q.cycles += 1; q.rows += (unsigned long long)r.T; q.served += (unsigned long long)r.served;
  for (int j = 1; j < r.T; j++) { q.drafted[j] += 1; q.accepted[j] += r.served > j; }
  q.last = r; q.have_last = true; q.last_served_idx = served_idx;
}

extern "C" {

LLB_API llb_spec *llb_spec_open(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp,
                                size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers) {
  return llb_spec_open_tp(index_text, pack, pack_bytes, pack_on_device, mtp, mtp_bytes, mtp_on_device, k, max_ctx, layers, 1);
}

// The engine as rank tp_rank of tp_size tensor-parallel ranks (llb_b200_tp_init first): this rank loads its share of every
// projection and the passes exchange one all-reduce after each row-split projection.  Every rank must make the same calls
// in the same order (the collectives inside a cycle pair up across the ranks); all of them return the same tokens.
static llb_spec *open_any(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp, size_t mtp_bytes,
                          int mtp_on_device, int k, int max_ctx, int layers, int tp_n, int nstreams);
static llb_spec *open_finish(llb_spec *m);
LLB_API llb_spec *llb_spec_open_tp(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp,
                                   size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers, int tp_n) {
  return open_any(index_text, pack, pack_bytes, pack_on_device, mtp, mtp_bytes, mtp_on_device, k, max_ctx, layers, tp_n, 1);
}
// The engine with `streams` independent sequences that share every weight read: a pass carries the k + 1 rows of every
// stream through each GEMM together (streams x (k + 1) <= 16 rows), attention, the DeltaNet
// scan, the drafter and the accept step run per stream in the same launches.  A stream's tokens are those of the
// same stream alone in such an engine, bit for bit (a row's GEMM result does not depend on its neighbours).
LLB_API llb_spec *llb_spec_open_streams(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp,
                                        size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers, int streams) {
  return open_any(index_text, pack, pack_bytes, pack_on_device, mtp, mtp_bytes, mtp_on_device, k, max_ctx, layers, 1, streams);
}
static llb_spec *open_any(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp, size_t mtp_bytes,
                          int mtp_on_device, int k, int max_ctx, int layers, int tp_n, int nstreams) {
  if (!g_llb.stream) { llb_fail("llb_b200_init has not been called"); return nullptr; }
  if (!index_text || !pack) { llb_fail("llb_spec_open: no index or no pack"); return nullptr; }
  llb_spec *m = new llb_spec();
  m->pack_bytes = pack_bytes;
  if (open_impl(m, index_text, (const uint8_t *)pack, pack_on_device, (const uint8_t *)mtp, mtp_bytes, mtp_on_device, k, max_ctx, layers, tp_n, nstreams)) {
    llb_spec_close(m);
    return nullptr;
  }
  return open_finish(m);
}
// Another engine on the weights `first` has on the device: its own k, context, streams, sequence state and graphs, no
// second copy of the model.  Streams beyond the 16 rows of a pass go into siblings: their passes run one after the
// other, each streaming the weights once.  Tokens are those of an engine opened the usual way with the same k and
// streams, bit for bit.  `first` may be closed before its siblings; the weights are freed with the last of them.
// Refused: tensor-parallel engines; k > 0 with a drafter the first engine did not load.
LLB_API llb_spec *llb_spec_open_sibling(llb_spec *first, int k, int max_ctx, int streams) {
  if (!first) { llb_fail("llb_spec_open_sibling: no engine"); return nullptr; }
  if (first->share) first = first->share;
  if (first->tp.size > 1) { llb_fail("llb_spec_open_sibling: a tensor-parallel engine has no siblings"); return nullptr; }
  llb_spec *m = new llb_spec();
  m->pack_bytes = first->pack_bytes;
  m->share = first;
  first->sharers += 1;
  const uint8_t *mtp = first->mtp_hdr.empty() ? nullptr : first->mtp_hdr.data();
  if (open_impl(m, first->index_copy.c_str(), nullptr, 0, mtp, first->mtp_total, 0, k, max_ctx, first->layers_arg, 1, streams)) {
    llb_spec_close(m);
    return nullptr;
  }
  return open_finish(m);
}
// bytes of weights this engine allocated itself: 0 for a sibling
LLB_API size_t llb_spec_weight_bytes(const llb_spec *m) {
  size_t n = 0;
  if (m && !m->share) for (const auto &w : m->wlist) n += w.second;
  return n;
}
static llb_spec *open_finish(llb_spec *m) {
  // One eager pass with empty row sets sizes and allocates every partial-sum buffer, so that the
  // captures below allocate nothing.  Then the graphs are captured once; everything that changes
  // between cycles lives in device memory.
  // (an eager pass at either width first: a K-split, and so a buffer's size, may differ between them)
  bool bad = false;
  const int w_spec = m->B * m->Tspec, w_pf = m->B > 1 ? w_spec : m->Tpf;
  if (m->tp.size > 1 && tp_host_barrier()) { llb_spec_close(m); return nullptr; }   // the ranks finished loading at different times
  {
    StreamScope scope(m);
    set_width(m, w_pf);
    bad = bad || llb_spec_reset(m) || enq_cycle(m, false);
    set_width(m, w_spec);
    bad = bad || llb_spec_reset(m) || enq_cycle(m, true) || llb_spec_reset(m);
  }
  bad = bad || capture(m, 0, &m->g_spec, &m->n_spec_nodes);
  set_width(m, w_pf);
  bad = bad || capture(m, 1, &m->g_prefill, nullptr);
  set_width(m, w_spec);
  bad = bad || capture(m, 2, &m->g_verify, &m->n_verify_nodes) || llb_spec_reset(m);
  if (bad) {
    llb_spec_close(m);
    return nullptr;
  }
  return m;
}

// The checks llb_spec_open makes before it touches the GPU, alone (needs no device): the index parses, its
// configuration is complete and consistent, and every tensor lies inside a pack of pack_bytes bytes.
LLB_API int llb_spec_check_index(const char *index_text, size_t pack_bytes) {
  if (!index_text) return llb_fail("check_index: no index");
  llb_spec m;
  std::unordered_map<std::string, TensorRec> tab;
  if (parse_index(&m, index_text, tab)) return -1;
  return validate_index(&m, tab, pack_bytes);
}

// The same engine from a GGUF file (qwen35 / qwen35moe): the header gives the index, the mapped file is the pack.
LLB_API llb_spec *llb_spec_open_gguf(const char *path, const void *mtp, size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers) {
  GgufFile g;
  if (gguf_map(path, g)) return nullptr;
  llb_spec *m = llb_spec_open(g.index.c_str(), g.map, g.size, 0, mtp, mtp_bytes, mtp_on_device, k, max_ctx, layers);
  gguf_unmap(g);   // every tensor now lives on the device
  return m;
}
// The index text llb_spec_open_gguf derives from a file's header (no GPU needed): returns its length, or -1.
LLB_API int llb_b200_gguf_index(const char *path, char *buf, int cap) {
  GgufFile g;
  if (gguf_map(path, g)) return -1;
  const int n = (int)g.index.size();
  if (buf && cap > 0) { const int c = n < cap - 1 ? n : cap - 1; memcpy(buf, g.index.data(), (size_t)c); buf[c] = 0; }
  gguf_unmap(g);
  return n;
}

LLB_API void llb_spec_close(llb_spec *m) {
  if (!m) return;
  cudaStreamSynchronize(g_llb.stream);
  if (m->sharers > 0) { m->closed = true; return; }   // its weights are in use: freed when the last sibling closes
  if (llb_spec *first = m->share) {
    m->share = nullptr;
    first->sharers -= 1;
    if (first->sharers == 0 && first->closed) llb_spec_close(first);
  }
  if (m->g_spec) cudaGraphExecDestroy(m->g_spec);
  if (m->g_prefill) cudaGraphExecDestroy(m->g_prefill);
  if (m->g_verify) cudaGraphExecDestroy(m->g_verify);
  for (void *p : m->allocs) cudaFree(p);
  if (m->res_host) cudaFreeHost(m->res_host);
  delete m;
}

// zero the sequence state of stream b (host/llb_host.c:1915-1928): KV rows are overwritten before they are
// read, so only the conv rings and the committed DeltaNet slot need clearing
static int reset_stream(llb_spec *m, int b) {
  for (int il = 0; il < m->L; il++) {
    if (m->ring[il]) CU_OK(cudaMemsetAsync(ring_of(m, il, b), 0, (size_t)m->ring_ks[il] * CONV_RING * m->convd * 4, g_llb.stream));
    if (m->S[il]) CU_OK(cudaMemsetAsync(state_of(m, il, b), 0, (size_t)m->s_group * 4, g_llb.stream));
  }
  // the trunk's normed hidden rows the drafter pairs with (the stream's rows of the widest pass)
  const int rows = m->B > 1 ? m->Tspec : (m->Tpf > SPEC_MAXT ? m->Tpf : SPEC_MAXT);
  CU_OK(cudaMemsetAsync(m->hn + (size_t)b * rows * m->d, 0, (size_t)rows * m->d * 4, g_llb.stream));
  CK(ctl_write(m, b, ctl_fresh(m, b)));
  SeqHost &q = m->sq[b];
  q.pos = 0; q.primed = false; q.have_last = false;
  q.cycles = q.rows = q.served = 0;
  memset(q.drafted, 0, sizeof q.drafted); memset(q.accepted, 0, sizeof q.accepted);
  return 0;
}
LLB_API int llb_spec_reset(llb_spec *m) {
  for (int b = 0; b < m->B; b++) CK(reset_stream(m, b));
  return 0;
}

// The prompts of nb streams (bs[i] gets ids[i][0 .. ns[i]-1]) through the same prompt passes: every stream feeds its own
// rows of a pass, so prompts that arrive together share each pass's weight read; a stream whose prompt is through sits
// the remaining passes out.
static int prefill_many(llb_spec *m, int nb, const int *bs, const int *const *ids, const int *ns) {
  if (nb < 1 || nb > m->B) return llb_fail("prefill: %d prompts for %d streams", nb, m->B);
  std::vector<char> in_set(m->B, 0);
  for (int i = 0; i < nb; i++) {
    const int b = bs[i], n = ns[i];
    if (b < 0 || b >= m->B) return llb_fail("prefill: stream %d of %d", b, m->B);
    if (in_set[b]) return llb_fail("prefill: stream %d given twice", b);
    in_set[b] = 1;
    if (n < 1) return llb_fail("prefill: empty prompt");
    if (n + m->Tpf + 1 > m->max_ctx) return llb_fail("prefill: %d tokens do not fit a context of %d", n, m->max_ctx);
    for (int j = 0; j < n; j++) if (ids[i][j] < 0 || ids[i][j] >= m->V) return llb_fail("prefill: token %d out of range", ids[i][j]);
  }
  for (int i = 0; i < nb; i++) CK(reset_stream(m, bs[i]));
  if (m->tp.size > 1) CK(tp_host_barrier());
  // a stream that takes no part in a pass sits it out: with no rows in its control block every kernel skips it, and the
  // accept kernel neither decides nor reports for it; its block is put back at the end
  std::vector<SpecCtl> keep(m->B);
  std::vector<char> kept(m->B, 0);
  auto park = [&](int o) -> int {
    CU_OK(cudaMemcpy(&keep[o], ctl_of(m, o), sizeof(SpecCtl), cudaMemcpyDeviceToHost));
    kept[o] = 1;
    SpecCtl c = keep[o];
    c.verify.n = 0; c.catchup.n = 0; c.chain.n = 0;
    return ctl_write(m, o, c);
  };
  for (int o = 0; o < m->B; o++) if (!in_set[o] && m->sq[o].primed) CK(park(o));
  std::vector<int> p(nb, 0);
  for (int i = 0; i < nb; i++) {
    const int b = bs[i];
    SpecCtl c = ctl_fresh(m, b);
    CU_OK(cudaMemcpyAsync(hist_of(m, b), ids[i], (size_t)ns[i] * 4, cudaMemcpyHostToDevice, g_llb.stream));
    // the drafter's row for position 0 pairs token 0 with a zero hidden (host/llb_host.c:1815-1817)
    c.catchup.n = 1; c.catchup.pos0 = 0; c.catchup.tok[0] = ids[i][0];
    c.verify.n = m->lookup ? 1 : m->per;   // nothing to look up at position 0
    c.verify.pos0 = 0; c.verify.tok[0] = ids[i][0];
    for (int r = 0; r < SPEC_MAXT; r++) c.verify.slot[r] = r & (CONV_RING - 1);
    CK(ctl_write(m, b, c));
  }
  // LLB_PREFILL=fast: everything but the last k + 1 rows in chunks of PF_RMAX rows through the dense path (dense FFN only),
  // one stream after the other (a chunk fills the tensor cores by itself)
  for (int i = 0; i < nb; i++)
    if (m->prefill_mode == 1 && m->ne == 0 && m->tp.size <= 1 && ns[i] - 1 >= m->Tspec + 32) CK(pf_prefill(m, bs[i], ids[i], ns[i] - 1, m->Tspec, &p[i]));
  for (int i = 0; i < nb; i++) if (nb > 1 && p[i] >= ns[i] - 1) CK(park(bs[i]));   // a one-token prompt: nothing to run
  for (;;) {
    std::vector<int> rows_of(nb, 0);
    int live = 0;
    for (int i = 0; i < nb; i++) {
      const int b = bs[i], n = ns[i];
      if (p[i] >= n - 1) continue;
      live++;
      // wide chunks, except that the last one has at most k + 1 rows: the first speculative cycle's drafter catches up
      // over the rows of the last chunk, and that cycle's kernels cover k + 1 rows
      const int rem = n - 1 - p[i];
      const int rows = rem <= m->Tspec ? rem : (rem - m->Tspec < m->Tpf ? rem - m->Tspec : m->Tpf);
      rows_of[i] = rows;
      // rows and their successors are given; only these fields of the control block change
      struct { int n, pos0, tok[SPEC_MAXT], slot[SPEC_MAXT]; } v;
      v.n = rows; v.pos0 = p[i];
      for (int r = 0; r < SPEC_MAXT; r++) { v.tok[r] = r < rows ? ids[i][p[i] + r] : 0; v.slot[r] = (p[i] + r) & (CONV_RING - 1); }
      int tail[1 + SPEC_MAXT];
      tail[0] = rows;  // forced
      for (int r = 0; r < SPEC_MAXT; r++) tail[1 + r] = r < rows ? ids[i][p[i] + r + 1] : 0;
      // pageable sources: the copies have taken their bytes when the calls return
      CU_OK(cudaMemcpyAsync(&ctl_of(m, b)->verify, &v, sizeof v, cudaMemcpyHostToDevice, g_llb.stream));
      CU_OK(cudaMemcpyAsync(&ctl_of(m, b)->forced, tail, sizeof tail, cudaMemcpyHostToDevice, g_llb.stream));
    }
    if (!live) break;
    CU_OK(cudaGraphLaunch(m->g_prefill, g_llb.stream));
    for (int i = 0; i < nb; i++) {
      if (!rows_of[i]) continue;
      SpecResult r;
      CK(wait_result(m, bs[i], &r));
      if (r.served != rows_of[i]) return llb_fail("prefill: chunk at %d of stream %d served %d of %d rows", p[i], bs[i], r.served, rows_of[i]);
      p[i] += rows_of[i];
      if (p[i] >= ns[i] - 1 && live > 1) CK(park(bs[i]));   // through, while others still have rows to feed
    }
  }
  for (int o = 0; o < m->B; o++) if (kept[o]) CK(ctl_write(m, o, keep[o]));
  for (int i = 0; i < nb; i++) {
    SeqHost &q = m->sq[bs[i]];
    q.pos = ns[i] - 1;        // n == 1: nothing ran, the first cycle starts at position 0 with the single prompt token
    q.last_tok = ids[i][ns[i] - 1];
    q.primed = true;
    q.have_last = false;
  }
  return 0;
}
static int prefill_stream(llb_spec *m, int b, const int *ids, int n) { return prefill_many(m, 1, &b, &ids, &n); }
// Feed the prompt.  Positions 0 .. n-2 run through the verify pass in chunks of given rows (or, for long prompts with
// LLB_PREFILL=fast, through the dense path); the last prompt token becomes the first speculative cycle's committed
// input, exactly where the reference's first cycle after a prompt starts (host/llb_host.c:1911, pos = n-1).
LLB_API int llb_spec_prefill(llb_spec *m, const int *ids, int n) { return prefill_stream(m, 0, ids, n); }
// The same for stream b of an engine opened with llb_spec_open_streams; the other streams keep their state.
LLB_API int llb_spec_prefill_stream(llb_spec *m, int stream, const int *ids, int n) { return prefill_stream(m, stream, ids, n); }
// Several streams' prompts at once (streams[i] gets ids[i][0 .. n[i]-1]): the prompts' rows share the prompt passes, each
// stream feeding its own k + 1 rows of a pass; results are those of llb_spec_prefill_stream on each stream in turn.
LLB_API int llb_spec_prefill_streams(llb_spec *m, int n_prompts, const int *streams, const int *const *ids, const int *n) {
  if (!m || !streams || !ids || !n) return llb_fail("llb_spec_prefill_streams: null argument");
  return prefill_many(m, n_prompts, streams, ids, n);
}

// One speculative cycle.  ids_out[0..*n_out-1] are the emitted tokens; top2_out (may be null) gets
// [id1, bits1, id2, bits2] of each emitted row.
LLB_API int llb_spec_cycle(llb_spec *m, int *ids_out, int *n_out, uint32_t *top2_out) {
  if (m->B > 1) return llb_fail("llb_spec_cycle: the engine has %d streams, use llb_spec_cycle_streams", m->B);
  SeqHost &q = m->sq[0];
  if (!q.primed) return llb_fail("llb_spec_cycle before llb_spec_prefill");
  // every row of the cycle, and the drafter's chained rows, must fit: no clipped cycles
  if (q.pos + m->Tmax >= m->max_ctx) return llb_fail("context of %d positions is full", m->max_ctx);
  if (m->tp.size > 1) CK(tp_host_barrier());
  CU_OK(cudaGraphLaunch(m->g_spec, g_llb.stream));
  SpecResult r;
  CK(wait_result(m, 0, &r));
  if (r.p0 != q.pos) return llb_fail("cycle ran at position %d, host expected %d", r.p0, q.pos);
  for (int i = 0; i < r.served; i++) {
    ids_out[i] = r.ids[i];
    if (top2_out) memcpy(top2_out + 4 * i, r.top2[i], 16);
  }
  *n_out = r.served;
  note_cycle(m, 0, r, 0);
  return 0;
}

// One cycle of every stream that has a prompt, as ONE graph launch.  ids_out[b][0 .. n_out[b]-1] (rows of SPEC_MAXT
// ints) are stream b's emitted tokens, n_out[b] = 0 for a stream without a prompt; top2_out (may be null) rows of
// SPEC_MAXT x 4 words.
LLB_API int llb_spec_cycle_streams(llb_spec *m, int *ids_out, int *n_out, uint32_t *top2_out) {
  int live = 0;
  for (int b = 0; b < m->B; b++) {
    const SeqHost &q = m->sq[b];
    if (!q.primed) continue;
    if (q.pos + m->per >= m->max_ctx) return llb_fail("stream %d: context of %d positions is full", b, m->max_ctx);
    live++;
  }
  if (!live) return llb_fail("llb_spec_cycle_streams: no stream has a prompt");
  CU_OK(cudaGraphLaunch(m->g_spec, g_llb.stream));
  for (int b = 0; b < m->B; b++) {
    n_out[b] = 0;
    SeqHost &q = m->sq[b];
    if (!q.primed) continue;
    SpecResult r;
    CK(wait_result(m, b, &r));
    if (r.p0 != q.pos) return llb_fail("stream %d: cycle ran at position %d, host expected %d", b, r.p0, q.pos);
    for (int i = 0; i < r.served; i++) {
      ids_out[b * SPEC_MAXT + i] = r.ids[i];
      if (top2_out) memcpy(top2_out + ((size_t)b * SPEC_MAXT + i) * 4, r.top2[i], 16);
    }
    n_out[b] = r.served;
    note_cycle(m, b, r, r.served);
  }
  return 0;
}

// `n` cycles of every stream back to back with no host round trip between them; tokens[b] = tokens stream b emitted.
LLB_API int llb_spec_run_cycles_streams(llb_spec *m, int n, int *tokens) {
  if (n > m->res_n) return llb_fail("at most %d cycles per call", m->res_n);
  for (int b = 0; b < m->B; b++) {
    tokens[b] = 0;
    const SeqHost &q = m->sq[b];
    if (q.primed && q.pos + n * m->per >= m->max_ctx) return llb_fail("stream %d: context of %d positions cannot take %d more cycles", b, m->max_ctx, n);
  }
  for (int i = 0; i < n; i++) CU_OK(cudaGraphLaunch(m->g_spec, g_llb.stream));
  for (int i = 0; i < n; i++)
    for (int b = 0; b < m->B; b++) {
      SeqHost &q = m->sq[b];
      if (!q.primed) continue;
      SpecResult r;
      CK(wait_result(m, b, &r));
      if (r.p0 != q.pos) return llb_fail("stream %d: cycle ran at position %d, host expected %d", b, r.p0, q.pos);
      tokens[b] += r.served;
      note_cycle(m, b, r, r.served);
    }
  return 0;
}

// Generate `steps` tokens after the prompt (greedy).  Returns the number written (== steps).
LLB_API int llb_spec_generate(llb_spec *m, int steps, int *ids, uint32_t *top2) {
  int out = 0;
  while (out < steps) {
    int got[SPEC_MAXT], n = 0;
    uint32_t t2[SPEC_MAXT * 4];
    CK(llb_spec_cycle(m, got, &n, t2));
    for (int i = 0; i < n && out < steps; i++, out++) {
      ids[out] = got[i];
      if (top2) memcpy(top2 + 4 * out, t2 + 4 * i, 16);
    }
  }
  return out;
}

// The reference's per-token entry (spec_pass, host/llb_host.c:1902-1950): the caller hands in
// (pos, tok) and gets the row's four words y = [v1, id1, v2, id2] (ids as floats, as the device
// argmax writes them).  Rows of the running cycle are served while (pos, tok) follows the cycle;
// otherwise a new cycle starts there.  Because acceptance is committed on the device under the
// greedy rule, a caller that leaves the greedy stream gets "a step out of order", the reference's
// own error for that case (host/llb_host.c:1929-1930).
LLB_API int llb_spec_pass(llb_spec *m, int pos, int tok, float *y) {
  SeqHost &q = m->sq[0];
  if (q.have_last && q.last_served_idx < q.last.served && pos == q.last.p0 + q.last_served_idx &&
      (q.last_served_idx == 0 || tok == q.last.ids[q.last_served_idx - 1])) {
    const int r = q.last_served_idx++;
    y[0] = bits_float(q.last.top2[r][1]); y[1] = (float)q.last.top2[r][0];
    y[2] = bits_float(q.last.top2[r][3]); y[3] = (float)q.last.top2[r][2];
    return 0;
  }
  if (q.primed && pos == q.pos && tok == q.last_tok) {
    // a new cycle at (pos, tok): the pair crosses to the device and the accept kernel checks it
    // against the state it committed itself
    int chk[3] = {1, pos, tok};
    CU_OK(cudaMemcpyAsync(&m->ctl->chk_on, chk, sizeof chk, cudaMemcpyHostToDevice, g_llb.stream));
    int ids[SPEC_MAXT], n = 0;
    CK(llb_spec_cycle(m, ids, &n, nullptr));
    if (q.last.pad) return llb_fail("LLB_SPEC: the device's committed (pos, tok) differs from the caller's");
    return llb_spec_pass(m, pos, tok, y);
  }
  return llb_fail("LLB_SPEC: a step out of order");
}

// Enqueue `n` cycles back to back with no host round trip between them (nothing a cycle needs comes
// from the host), then collect what they emitted.  ids (may be null) receives the tokens in order,
// at most cap of them; returns the number of tokens emitted by the n cycles.
LLB_API int llb_spec_run_cycles(llb_spec *m, int n, int *ids, int cap) {
  if (m->B > 1) return llb_fail("llb_spec_run_cycles: the engine has %d streams, use llb_spec_run_cycles_streams", m->B);
  SeqHost &q = m->sq[0];
  if (!q.primed) return llb_fail("llb_spec_run_cycles before llb_spec_prefill");
  if (n > m->res_n) return llb_fail("at most %d cycles per call", m->res_n);
  if (q.pos + n * m->Tmax >= m->max_ctx) return llb_fail("context of %d positions cannot take %d more cycles", m->max_ctx, n);
  if (m->tp.size > 1) CK(tp_host_barrier());
  for (int i = 0; i < n; i++) CU_OK(cudaGraphLaunch(m->g_spec, g_llb.stream));
  int total = 0;
  for (int i = 0; i < n; i++) {
    SpecResult r;
    CK(wait_result(m, 0, &r));
    if (r.p0 != q.pos) return llb_fail("cycle ran at position %d, host expected %d", r.p0, q.pos);
    for (int j = 0; j < r.served; j++, total++) if (ids && total < cap) ids[total] = r.ids[j];
    note_cycle(m, 0, r, r.served);
  }
  return total;
}

// Device time of the verify pass alone at the current position: `iters` replays, CUDA events on the
// library's stream.  Replaying commits nothing (no accept kernel), so the sequence is unchanged.
LLB_API int llb_spec_time_verify(llb_spec *m, int iters, float *ms_per_pass) {
  if (m->tp.size > 1) CK(tp_host_barrier());
  cudaEvent_t a, b;
  CU_OK(cudaEventCreate(&a)); CU_OK(cudaEventCreate(&b));
  CU_OK(cudaGraphLaunch(m->g_verify, g_llb.stream));
  CU_OK(cudaEventRecord(a, g_llb.stream));
  for (int i = 0; i < iters; i++) CU_OK(cudaGraphLaunch(m->g_verify, g_llb.stream));
  CU_OK(cudaEventRecord(b, g_llb.stream));
  CU_OK(cudaEventSynchronize(b));
  float ms = 0;
  CU_OK(cudaEventElapsedTime(&ms, a, b));
  *ms_per_pass = ms / iters;
  cudaEventDestroy(a); cudaEventDestroy(b);
  return 0;
}

// The same with the pass forced to `rows` rows (1 .. k + 1): a drafter that found fewer drafts leaves a shorter
// pass in the control block; for timing, the missing rows repeat the pass's first token at the following
// positions.  The control block is restored afterwards, but the rows' KV / conv / state-ring slots have been
// overwritten with the forced rows' values: call it after the tokens that matter have been generated.
LLB_API int llb_spec_time_verify_rows(llb_spec *m, int iters, int rows, float *ms_per_pass) {
  if (m->B > 1) return llb_fail("time_verify_rows: a one-stream engine's entry");
  if (rows < 1 || rows > m->Tmax) return llb_fail("time_verify_rows: %d rows, the engine was opened for %d", rows, m->Tmax);
  SpecCtl c, keep;
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  CU_OK(cudaMemcpy(&c, m->ctl, sizeof c, cudaMemcpyDeviceToHost));
  keep = c;
  if (c.verify.pos0 + rows + 1 > m->max_ctx) return llb_fail("time_verify_rows: the context is full");
  for (int t = c.verify.n > 0 ? c.verify.n : 1; t < rows; t++) { c.verify.tok[t] = c.verify.tok[0]; c.verify.slot[t] = (c.verify.pos0 + t) & (CONV_RING - 1); }
  c.verify.n = rows;
  CU_OK(cudaMemcpy(m->ctl, &c, sizeof c, cudaMemcpyHostToDevice));
  const int rc = llb_spec_time_verify(m, iters, ms_per_pass);
  CU_OK(cudaMemcpy(m->ctl, &keep, sizeof keep, cudaMemcpyHostToDevice));
  return rc;
}

// Device time per launch of the FFN gate|up GEMM (the largest launch of the pass), cycling over the
// layers so that every launch streams weights that are not in L2.  bytes_per_launch = the two
// matrices' stored bytes plus the activation planes and the outputs.
LLB_API int llb_spec_time_gemm(llb_spec *m, int iters, float *us_per_launch, double *bytes_per_launch) {
  cudaEvent_t a, b;
  CU_OK(cudaEventCreate(&a)); CU_OK(cudaEventCreate(&b));
  auto go = [&](int il) { const FfnW &w = m->layer[il % m->L].ffn;
    return site_gemm(m, {{&w.gate, &m->b_g, nullptr, nullptr, 0}, {&w.up, &m->b_u, nullptr, nullptr, 0}}, m->xp_d, 0); };
  for (int i = 0; i < 4; i++) CK(go(i));
  CU_OK(cudaEventRecord(a, g_llb.stream));
  for (int i = 0; i < iters; i++) CK(go(4 + i));
  CU_OK(cudaEventRecord(b, g_llb.stream));
  CU_OK(cudaEventSynchronize(b));
  float ms = 0;
  CU_OK(cudaEventElapsedTime(&ms, a, b));
  *us_per_launch = ms * 1000.0f / iters;
  const FfnW &w0 = m->layer[0].ffn;
  *bytes_per_launch = (double)w0.gate.rows * pack_row_bytes(w0.gate.fmt, m->d) + (double)w0.up.rows * pack_row_bytes(w0.up.fmt, m->d) +
                      (double)m->NC * m->d * 2 + 2.0 * m->Tmax * m->f * 4;
  cudaEventDestroy(a); cudaEventDestroy(b);
  return 0;
}

// One eager verify pass with an event after every op; writes "name count total_us" lines into buf.
LLB_API int llb_spec_profile_verify(llb_spec *m, char *buf, int cap) {
  if (m->tp.size > 1) CK(tp_host_barrier());
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  for (int rep = 0; rep < 2; rep++) {      // the second pass is the one reported (warm)
    for (auto &r : g_prof) cudaEventDestroy(r.ev);
    g_prof.clear();
    g_prof_on = true;
    prof_mark("start");
    StreamScope scope(m);
    int rc = enq_verify(m);
    g_prof_on = false;
    if (rc) return -1;
    CU_OK(cudaStreamSynchronize(g_llb.stream));
  }
  std::vector<std::string> names;
  std::vector<double> tot;
  std::vector<int> cnt;
  for (size_t i = 1; i < g_prof.size(); i++) {
    float ms = 0;
    cudaEventElapsedTime(&ms, g_prof[i - 1].ev, g_prof[i].ev);
    size_t k = 0;
    for (; k < names.size(); k++) if (names[k] == g_prof[i].name) break;
    if (k == names.size()) { names.push_back(g_prof[i].name); tot.push_back(0); cnt.push_back(0); }
    tot[k] += ms * 1000.0; cnt[k] += 1;
  }
  int off = 0;
  for (size_t k = 0; k < names.size() && off < cap - 80; k++) off += snprintf(buf + off, cap - off, "%s\t%d\t%.1f\n", names[k].c_str(), cnt[k], tot[k]);
  return off;
}

// kernels per replay of the cycle graph (which = 0) or of the verify pass (which = 2)
LLB_API int llb_spec_graph_nodes(const llb_spec *m, int which) { return (int)(which == 2 ? m->n_verify_nodes : m->n_spec_nodes); }

// Sampling parameters of the cycles from now on (set before llb_spec_prefill): the cycle graph is captured again with or
// without the sampler's kernel in it.
LLB_API int llb_spec_set_sampler(llb_spec *m, const llb_smp_params *p) {
  if (!p) return llb_fail("set_sampler: no parameters");
  for (int b = 0; b < m->B; b++) if (m->sq[b].primed) return llb_fail("set_sampler: set the sampler before the prompt goes in (stream %d has one)", b);
  SmpDev d;
  bool argmax_only = false;
  CK(smp_prepare(p, &d, &argmax_only));
  if (m->tp.size > 1 && !argmax_only) return llb_fail("set_sampler: a tensor-parallel engine decodes greedily");
  const int rows = m->B * m->Tspec;
  if (!argmax_only && !m->smp_adj) {
    m->smp_adj = falloc(m, (size_t)rows * m->V); m->smp_val = falloc(m, rows); m->smp_tok = (int *)dalloc(m, (size_t)rows * 4);
    m->smp_err = (unsigned int *)dalloc(m, 4);
    if (!m->smp_adj || !m->smp_val || !m->smp_tok || !m->smp_err) return -1;
  }
  m->smp = d;
  m->smp_on = !argmax_only;
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  if (m->g_spec) { cudaGraphExecDestroy(m->g_spec); m->g_spec = nullptr; }
  set_width(m, rows);
  CK(llb_spec_reset(m));
  return capture(m, 0, &m->g_spec, &m->n_spec_nodes);
}
// 0, or the device sampler's error word: 2 min_keep above what min_p kept, 3 a token out of range
LLB_API int llb_spec_sampler_errors(llb_spec *m) {
  if (!m->smp_err) return 0;
  unsigned int v = 0;
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  CU_OK(cudaMemcpy(&v, m->smp_err, 4, cudaMemcpyDeviceToHost));
  return (int)v;
}

// The result record of a stream's last cycle as 3 + 8 + 8 + 32 words: p0, T, served, the verify inputs tin[8] (the
// committed token, then the drafts), the rows' emitted ids[8], and [id1, bits1, id2, bits2] of each row.
LLB_API int llb_spec_last_record(const llb_spec *m, int stream, unsigned int *out51) {
  if (stream < 0 || stream >= m->B || !m->sq[stream].have_last) return llb_fail("last_record: stream %d has not run a cycle", stream);
  const SpecResult &r = m->sq[stream].last;
  out51[0] = (unsigned)r.p0; out51[1] = (unsigned)r.T; out51[2] = (unsigned)r.served;
  for (int i = 0; i < SPEC_MAXT; i++) { out51[3 + i] = (unsigned)r.tin[i]; out51[11 + i] = (unsigned)r.ids[i]; memcpy(out51 + 19 + 4 * i, r.top2[i], 16); }
  return 0;
}
LLB_API int llb_spec_position(const llb_spec *m) { return m->sq[0].pos; }
LLB_API int llb_spec_position_stream(const llb_spec *m, int stream) { return stream >= 0 && stream < m->B ? m->sq[stream].pos : -1; }
LLB_API int llb_spec_streams(const llb_spec *m) { return m->B; }

// mode 1: prompts go through the dense tcgen05 path in chunks of 128 rows (all but their last k + 1 rows); mode 0: every
// row through the T-row pass.  Returns the previous mode.
LLB_API int llb_spec_set_prefill(llb_spec *m, int mode) {
  const int was = m->prefill_mode;
  m->prefill_mode = mode == 1;
  return was;
}
LLB_API double llb_spec_fast_rows(const llb_spec *m) { return m->pf_rows; }

LLB_API int llb_spec_stats_stream(const llb_spec *m, int stream, unsigned long long *out /* cycles, rows, served, drafted[8], accepted[8] */) {
  if (stream < 0 || stream >= m->B) return llb_fail("stats: stream %d of %d", stream, m->B);
  const SeqHost &q = m->sq[stream];
  out[0] = q.cycles; out[1] = q.rows; out[2] = q.served;
  for (int j = 0; j < 8; j++) { out[3 + j] = q.drafted[j]; out[11 + j] = q.accepted[j]; }
  return 0;
}
LLB_API int llb_spec_stats(const llb_spec *m, unsigned long long *out) { return llb_spec_stats_stream(m, 0, out); }

// State read-back for parity checks: what = 0 committed DeltaNet state of layer il [TR][128][128],
// 1 the K row and 2 the V row of position `pos` in layer il, 3 the conv ring row of position `pos`,
// 4 the trunk's output-normed hidden row `pos` (0..k) of the last pass, 5 the drafter's K row, 6 the output-normed
// hidden of row `pos` of the last chunk the dense prompt path processed.
LLB_API int llb_spec_read_state_stream(llb_spec *m, int stream, int what, int il, int pos, float *out, size_t n);
LLB_API int llb_spec_read_state(llb_spec *m, int what, int il, int pos, float *out, size_t n) { return llb_spec_read_state_stream(m, 0, what, il, pos, out, n); }
// ... of stream `stream` (what = 4: `pos` is the row within the stream's rows of the pass)
LLB_API int llb_spec_read_state_stream(llb_spec *m, int stream, int what, int il, int pos, float *out, size_t n) {
  if (stream < 0 || stream >= m->B) return llb_fail("read_state: stream %d of %d", stream, m->B);
  const int b = stream;
  if (il < 0 || pos < 0 || ((what == 1 || what == 2 || what == 5) && pos >= m->max_ctx)) return llb_fail("read_state: layer %d, position %d", il, pos);
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  const float *src = nullptr;
  size_t have = 0;
  const int kvd = m->KV * m->hd;
  if (what == 0 && il < m->L && m->S[il]) {
    SpecCtl c;
    CU_OK(cudaMemcpy(&c, ctl_of(m, b), sizeof c, cudaMemcpyDeviceToHost));
    have = (size_t)m->TR * m->SZ * m->SZ; src = state_of(m, il, b) + (size_t)c.sc * have;
  } else if ((what == 1 || what == 2 || what == 5) && (what == 5 ? m->mt_Kc != nullptr : (il < m->L && m->Kc[il]))) {
    // a cache row is kept as two fp16 planes, hi and lo * 2048
    const __half *c = (const __half *)kc_of(m, what == 5 ? m->mt_Kc : what == 1 ? m->Kc[il] : m->Vc[il], b);
    have = kvd;
    if (n < have) return llb_fail("read_state: buffer of %zu floats, %zu needed", n, have);
    std::vector<__half> hi(have), lo(have);
    CU_OK(cudaMemcpy(hi.data(), c + (size_t)pos * kvd, have * 2, cudaMemcpyDeviceToHost));
    CU_OK(cudaMemcpy(lo.data(), c + (size_t)m->max_ctx * kvd + (size_t)pos * kvd, have * 2, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < have; i++) out[i] = __half2float(hi[i]) + __half2float(lo[i]) * XP_LO_INV;
    return (int)have;
  }
  else if (what == 3 && il < m->L && m->ring[il]) {
    have = m->convd;
    if (n < have) return llb_fail("read_state: buffer of %zu floats, %zu needed", n, have);
    std::vector<float> tmp(have);
    for (size_t i = 0; i < have; i++) out[i] = 0.0f;
    for (int k = 0; k < m->ring_ks[il]; k++) {
      CU_OK(cudaMemcpy(tmp.data(), ring_of(m, il, b) + (size_t)k * CONV_RING * m->convd + (size_t)(pos & (CONV_RING - 1)) * m->convd, have * 4,
                       cudaMemcpyDeviceToHost));
      for (size_t i = 0; i < have; i++) out[i] += tmp[i];
    }
    return (int)have;
  }
  else if (what == 4 && pos < (m->B > 1 ? m->Tspec : SPEC_MAXT)) { have = m->d; src = m->hn + (size_t)((m->B > 1 ? b * m->Tspec : 0) + pos) * m->d; }
  else if (what == 6 && m->pf.ready && pos >= 0 && pos < PF_RMAX) { have = m->d; src = m->pf.hn + (size_t)(pos + 1) * m->d; }   // dense path: normed hidden of row `pos` of its last chunk
  else return llb_fail("read_state: nothing of kind %d in layer %d", what, il);
  if (n < have) return llb_fail("read_state: buffer of %zu floats, %zu needed", n, have);
  CU_OK(cudaMemcpy(out, src, have * 4, cudaMemcpyDeviceToHost));
  return (int)have;
}

// The logits of verify row r of the last pass (f32 [V]), for the logit-tolerance parity check.
// Test entry: the routed-expert FFN of layer il alone on T given normed rows (host memory, [T][d]); out[T][d]
// is its output without the residual, ids / wt [T][k + 1] the chosen experts and weights (slot k: the shared
// expert and its gate).  Resets the sequence state: call it before llb_spec_prefill, not between cycles.
LLB_API int llb_spec_moe_ffn(llb_spec *m, int il, int T, const float *h2, float *out, int *ids, float *wt) {
  if (il < 0 || il >= m->L || !m->layer[il].ffn.moe) return llb_fail("moe_ffn: layer %d has no routed experts", il);
  if (T < 1 || T > m->Tmax) return llb_fail("moe_ffn: %d rows, the engine was opened for %d", T, m->Tmax);
  CK(llb_spec_reset(m));
  // rows in pass order: with several streams, row t is row t % (k + 1) of stream t / (k + 1)
  for (int b = 0; b < m->B; b++) {
    SpecCtl c = ctl_fresh(m, b);
    const int left = T - b * m->per;
    c.verify.n = left < 0 ? 0 : left > m->per ? m->per : left;
    CK(ctl_write(m, b, c));
  }
  StreamScope scope(m);
  cudaStream_t s = g_llb.stream;
  CU_OK(cudaMemcpyAsync(m->hn2, h2, (size_t)T * m->d * 4, cudaMemcpyHostToDevice, s));
  CK(ops_xp_from_f32(s, m->hn2, T, 2, m->xp_d));
  CK(enq_moe_core(m, m->layer[il].ffn, &m->ctl->verify));
  CU_OK(cudaStreamSynchronize(s));
  const int ns = m->nk + 1;
  std::vector<float> tmp((size_t)T * m->d);
  for (size_t i = 0; i < tmp.size(); i++) out[i] = 0.0f;
  for (int k = 0; k < m->b_dn.ns; k++) {
    CU_OK(cudaMemcpy(tmp.data(), m->b_dn.p + (size_t)k * m->b_dn.stride, tmp.size() * 4, cudaMemcpyDeviceToHost));
    for (size_t i = 0; i < tmp.size(); i++) out[i] += tmp[i];
  }
  if (ids) CU_OK(cudaMemcpy(ids, m->moe_ids, (size_t)T * ns * 4, cudaMemcpyDeviceToHost));
  if (wt) CU_OK(cudaMemcpy(wt, m->moe_wt, (size_t)T * ns * 4, cudaMemcpyDeviceToHost));
  return llb_spec_reset(m);
}

LLB_API int llb_spec_read_logits(llb_spec *m, int r, float *out) {
  if (r < 0 || r >= m->Tmax || !m->b_lg.p) return llb_fail("read_logits: row %d of a pass of %d rows", r, m->Tmax);
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  std::vector<float> tmp(m->V);
  for (int i = 0; i < m->V; i++) out[i] = 0.0f;
  for (int k = 0; k < m->b_lg.ns; k++) {
    CU_OK(cudaMemcpy(tmp.data(), m->b_lg.p + (size_t)k * m->b_lg.stride + (size_t)r * m->V, (size_t)m->V * 4, cudaMemcpyDeviceToHost));
    for (int i = 0; i < m->V; i++) out[i] += tmp[i];
  }
  return 0;
}

}  // extern "C"
