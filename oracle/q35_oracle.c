/* oracle/q35_oracle.c -- TEST INFRASTRUCTURE ONLY (see q35_oracle.h).
 *
 * Plain-C restatement of the reference CPU engine's arithmetic for the Qwen3.5 hybrid model,
 * plus the two pieces the reference only has on its GPU host: the MTP drafter and the greedy
 * speculative cycle.  All float math is F32 with the reference's evaluation order (serial
 * accumulation per row, transcendentals through double and rounded once), so that a build with
 * -ffp-contract=off is bit-identical to the reference engine on the trunk.
 */
#include "q35_oracle.h"

#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define API __attribute__((visibility("default")))
enum { FM_F32 = 0, FM_Q8_0 = 1, FM_Q4_K = 3, FM_Q6_K = 4, FM_Q5_K = 9 }; /* host/llb_formats.h:4-15 */

static int g_threads = 0;
API void q35_threads(int n) { g_threads = n; }

/* ---- scalar helpers: tools/qwen35_engine.c:45-56 (through double, one rounding) ------------- */
static float f_exp(float x) { return (float)exp((double)x); }
static float f_sqrt(float x) { return (float)sqrt((double)x); }
API float q35_exp(float x) { return f_exp(x); }
API float q35_sigmoid(float x) { return 1.0f / (1.0f + f_exp(-x)); }
API float q35_silu(float x) { return x / (1.0f + f_exp(-x)); }
API float q35_softplus(float x) {
  if (x > 20.0f) return x;
  return (float)log1p((double)f_exp(x < 88.0f ? x : 88.0f));
}

/* IEEE binary16 -> binary32, every class of value (tools/qwen35_engine.c:329-347) */
API float q35_half(uint16_t h) {
  uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 31u, m = h & 1023u, bits;
  if (e == 31u) bits = s | 0x7f800000u | (m << 13);
  else if (e != 0u) bits = s | ((e + 112u) << 23) | (m << 13);
  else if (m == 0u) bits = s;
  else {
    int sh = 0;
    while (!(m & 1024u)) { m <<= 1; sh++; }
    bits = s | ((uint32_t)(113 - sh) << 23) | ((m & 1023u) << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
static float rd16(const uint8_t *p) { return q35_half((uint16_t)(p[0] | (p[1] << 8))); }

/* six-bit (scale, min) pair j of a Q4_K / Q5_K block (tools/qwen35_engine.c:66-72) */
static void scale_min(const uint8_t *s, int j, int *sc, int *mn) {
  if (j < 4) { *sc = s[j] & 63; *mn = s[j + 4] & 63; return; }
  *sc = (s[j + 4] & 15) | ((s[j - 4] >> 6) << 4);
  *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
}

/* One decoder per format writes the 256 (or 32) weights of a block in column order; the dot and
 * the row dequantiser both go through it, so they cannot disagree.  Values follow
 * tools/qwen35_engine.c:233-307 operation for operation. */
static void blk_q4k(const uint8_t *b, float *o, int five) {
  float d = rd16(b), dm = rd16(b + 2);
  const uint8_t *qh = b + 16, *qs = b + (five ? 48 : 16);
  for (int g = 0; g < 4; g++) {
    int s0, m0, s1, m1;
    scale_min(b + 4, 2 * g, &s0, &m0);
    scale_min(b + 4, 2 * g + 1, &s1, &m1);
    float d0 = d * (float)s0, n0 = dm * (float)m0, d1 = d * (float)s1, n1 = dm * (float)m1;
    for (int l = 0; l < 32; l++) {
      int lo = qs[32 * g + l] & 15, hi = qs[32 * g + l] >> 4;
      if (five) { lo += ((qh[l] >> (2 * g)) & 1) * 16; hi += ((qh[l] >> (2 * g + 1)) & 1) * 16; }
      o[64 * g + l] = d0 * (float)lo - n0;
      o[64 * g + 32 + l] = d1 * (float)hi - n1;
    }
  }
}
static void blk_q6k(const uint8_t *b, float *o) {
  const int8_t *sc = (const int8_t *)(b + 192);
  float d = rd16(b + 208);
  for (int hf = 0; hf < 2; hf++)
    for (int qd = 0; qd < 4; qd++)
      for (int l = 0; l < 32; l++) {
        uint8_t lq = b[64 * hf + 32 * (qd & 1) + l];
        int nib = qd < 2 ? (lq & 15) : (lq >> 4);
        int code = (nib | (((b[128 + 32 * hf + l] >> (2 * qd)) & 3) << 4)) - 32;
        o[128 * hf + 32 * qd + l] = (d * (float)sc[8 * hf + 2 * qd + (l >> 4)]) * (float)code;
      }
}

API void q35_deq_row(int fmt, const uint8_t *row, int cols, float *out) {
  if (fmt == FM_F32) { memcpy(out, row, (size_t)cols * 4); return; }
  if (fmt == FM_Q8_0) {
    const int8_t *q = (const int8_t *)row;
    for (int b = 0; b < cols / 32; b++) {
      float d = rd16(row + cols + 2 * b);
      for (int j = 0; j < 32; j++) out[32 * b + j] = (float)q[32 * b + j] * d;
    }
    return;
  }
  for (int b = 0; b < cols / 256; b++) {
    if (fmt == FM_Q4_K) blk_q4k(row + (size_t)b * 144, out + 256 * b, 0);
    else if (fmt == FM_Q5_K) blk_q4k(row + (size_t)b * 176, out + 256 * b, 1);
    else if (fmt == FM_Q6_K) blk_q6k(row + (size_t)b * 210, out + 256 * b);
  }
}

/* serial dot in column order: acc += w * x, one block of weights at a time
 * (tools/qwen35_engine.c:74-216) */
API float q35_dot(int fmt, const uint8_t *row, int cols, const float *x) {
  float acc = 0.0f, w[256];
  if (fmt == FM_F32) {
    const float *m = (const float *)row;
    for (int c = 0; c < cols; c++) acc += m[c] * x[c];
    return acc;
  }
  if (fmt == FM_Q8_0) {
    for (int b = 0; b < cols / 32; b++) {
      float d = rd16(row + cols + 2 * b);
      for (int j = 0; j < 32; j++) acc += ((float)((const int8_t *)row)[32 * b + j] * d) * x[32 * b + j];
    }
    return acc;
  }
  int bb = fmt == FM_Q4_K ? 144 : fmt == FM_Q5_K ? 176 : 210;
  for (int b = 0; b < cols / 256; b++) {
    if (fmt == FM_Q6_K) blk_q6k(row + (size_t)b * bb, w);
    else blk_q4k(row + (size_t)b * bb, w, fmt == FM_Q5_K);
    for (int c = 0; c < 256; c++) acc += w[c] * x[256 * b + c];
  }
  return acc;
}

API void q35_gemv(int fmt, const uint8_t *W, int rb, int rows, int cols, const float *x, float *y) {
  if (fmt == FM_F32) rb = cols * 4;
#ifdef _OPENMP
  int nt = g_threads > 0 ? g_threads : omp_get_max_threads();
  if (rows < 64) nt = 1;
#pragma omp parallel for schedule(static) num_threads(nt)
#endif
  for (int r = 0; r < rows; r++) y[r] = q35_dot(fmt, W + (size_t)r * rb, cols, x);
}

/* ---- model ---------------------------------------------------------------------------------- */
typedef struct { const uint8_t *w; int rows, cols, fmt, rb; } Mat;
typedef struct { char name[64]; uint64_t off, bytes; int rows, cols, fmt, rb; } Tensor;

typedef struct { /* one full-attention block's weights (trunk layer or the drafter) */
  Mat q, k, v, o;
  const float *qn, *kn;
} AttnW;
/* moe != 0: router [ne x d] and sh_inp [d] F32; gate/up/down are the shared expert; eg/eu [ne*ef x d] and
 * ed [ne*d x ef] the expert stacks (GGUF tensors ffn_gate_exps, ffn_up_exps, ffn_down_exps) */
typedef struct { Mat gate, up, down; const float *post; int moe; Mat router, eg, eu, ed; const float *sh_inp; } FfnW;
typedef struct {
  Mat qkv, z, beta, alpha, out;
  const float *dt, *a, *conv, *norm;
} DeltaW;
typedef struct { int full; const float *attn_norm; AttnW at; DeltaW dn; FfnW ffn; } Layer;

struct Q35 {
  Q35Cfg c;
  Tensor *t;
  int nt, cap, owns_pack;
  const uint8_t *pack;
  Layer *layer;
  Mat embd, head;
  const float *out_norm;
  /* state */
  float *S, *conv, *K, *V;
  /* scratch */
  float *x, *h, *a, *qkv, *z, *y, *qg, *qn, *kb, *vb, *att, *prob, *qt, *kt, *f1, *f2, *o128, *logits, *hn, *moe_p, *moe_o;
  /* drafter */
  int has_mtp, mt_nv;
  uint8_t *mt_img;
  const float *mt_enorm, *mt_hnorm, *mt_attn_norm, *mt_shn;
  Mat mt_eh, mt_head;
  AttnW mt_at;
  FfnW mt_ffn;
  const uint32_t *mt_ids;
  float *mt_K, *mt_V, *mt_cat, *mt_logits;
};

static const Tensor *find(const Q35 *m, const char *name) {
  for (int i = 0; i < m->nt; i++) if (!strcmp(m->t[i].name, name)) return &m->t[i];
  return NULL;
}
static Mat mat_of(const Q35 *m, const char *fmt, int il, const char *leaf) {
  char nm[96];
  snprintf(nm, sizeof nm, fmt, il, leaf);
  const Tensor *t = find(m, nm);
  Mat r = {0};
  if (!t) { fprintf(stderr, "q35_oracle: missing tensor %s\n", nm); return r; }
  r.w = m->pack + t->off; r.rows = t->rows; r.cols = t->cols; r.fmt = t->fmt;
  r.rb = t->fmt == FM_F32 ? t->cols * 4 : t->rb;
  return r;
}
static const float *vec_of(const Q35 *m, int il, const char *leaf) {
  return (const float *)mat_of(m, "blk.%d.%s", il, leaf).w;
}
static int fmt_of(const char *ty) {
  if (!strcmp(ty, "F32")) return FM_F32;
  if (!strcmp(ty, "Q8_0")) return FM_Q8_0;
  if (!strcmp(ty, "Q4_K")) return FM_Q4_K;
  if (!strcmp(ty, "Q6_K")) return FM_Q6_K;
  if (!strcmp(ty, "Q5_K")) return FM_Q5_K;
  return -1;
}

static int parse_index(Q35 *m, const char *text) {
  int cap = 0;
  const char *p = text;
  while (*p) {
    const char *e = strchr(p, '\n');
    size_t len = e ? (size_t)(e - p) : strlen(p);
    char line[1024];
    if (len >= sizeof line) len = sizeof line - 1;
    memcpy(line, p, len);
    line[len] = 0;
    p = e ? e + 1 : p + len;
    if (!strncmp(line, "#cfg\t", 5)) {
      char key[64], val[128];
      if (sscanf(line + 5, "%63[^\t]\t%127[^\n]", key, val) != 2) continue;
      Q35Cfg *c = &m->c;
      struct { const char *k; int *v; } im[] = {
        {"n_layers", &c->n_layers}, {"n_heads", &c->n_heads}, {"n_kv_heads", &c->n_kv_heads},
        {"d_model", &c->d_model}, {"head_dim", &c->head_dim}, {"d_ff", &c->d_ff}, {"vocab_size", &c->vocab},
        {"full_attention_interval", &c->interval}, {"ssm_conv_kernel", &c->conv_kernel},
        {"ssm_state_size", &c->ssm_state}, {"ssm_group_count", &c->ssm_groups},
        {"ssm_time_step_rank", &c->ssm_heads}, {"ssm_inner_size", &c->vdc}, {"linear_key_dim", &c->kdc},
        {"linear_value_head_dim", &c->vhd}, {"linear_conv_dim", &c->convd}, {"rope_dim", &c->rope_dim},
        {"expert_count", &c->n_experts}, {"expert_used_count", &c->n_used}, {"expert_feed_forward_length", &c->d_expert},
        {"expert_shared_feed_forward_length", &c->d_shared}};
      for (size_t i = 0; i < sizeof im / sizeof *im; i++) if (!strcmp(key, im[i].k)) *im[i].v = atoi(val);
      if (!strcmp(key, "rope_freq_base")) c->rope_base = strtof(val, NULL);
      if (!strcmp(key, "rms_norm_eps")) c->eps = strtof(val, NULL);
      continue;
    }
    if (line[0] == '#' || line[0] == 0) continue;
    Tensor t;
    char ty[16];
    unsigned long off, nb;
    memset(&t, 0, sizeof t);
    int n = sscanf(line, "%63[^\t]\t%lu\t%lu\t%d\t%d\t%15[^\t]\t%d\t%d", t.name, &off, &nb, &t.rows, &t.cols, ty,
                   &t.rb, &t.fmt);
    if (n < 6) continue;
    t.off = off; t.bytes = nb;
    if (n < 7) t.rb = 0;
    t.fmt = fmt_of(ty);
    if (t.fmt < 0) { fprintf(stderr, "q35_oracle: unknown type %s\n", ty); return 1; }
    if (m->nt == cap) { cap = cap ? 2 * cap : 256; m->t = (Tensor *)realloc(m->t, (size_t)cap * sizeof(Tensor)); }
    m->t[m->nt++] = t;
  }
  return 0;
}

static float *fz(size_t n) { return (float *)calloc(n ? n : 1, 4); }

static Q35 *finish_open(Q35 *m, int layers, int cap) {
  Q35Cfg *c = &m->c;
  if (layers > 0 && layers < c->n_layers) c->n_layers = layers;
  m->cap = cap;
  m->layer = (Layer *)calloc((size_t)c->n_layers, sizeof(Layer));
  for (int il = 0; il < c->n_layers; il++) {
    Layer *l = &m->layer[il];
    l->full = (il + 1) % c->interval == 0;
    l->attn_norm = vec_of(m, il, "attn_norm.weight");
    if (l->full) {
      l->at.q = mat_of(m, "blk.%d.%s", il, "attn_q.weight");
      l->at.k = mat_of(m, "blk.%d.%s", il, "attn_k.weight");
      l->at.v = mat_of(m, "blk.%d.%s", il, "attn_v.weight");
      l->at.o = mat_of(m, "blk.%d.%s", il, "attn_output.weight");
      l->at.qn = vec_of(m, il, "attn_q_norm.weight");
      l->at.kn = vec_of(m, il, "attn_k_norm.weight");
    } else {
      l->dn.qkv = mat_of(m, "blk.%d.%s", il, "attn_qkv.weight");
      l->dn.z = mat_of(m, "blk.%d.%s", il, "attn_gate.weight");
      l->dn.beta = mat_of(m, "blk.%d.%s", il, "ssm_beta.weight");
      l->dn.alpha = mat_of(m, "blk.%d.%s", il, "ssm_alpha.weight");
      l->dn.out = mat_of(m, "blk.%d.%s", il, "ssm_out.weight");
      l->dn.dt = vec_of(m, il, "ssm_dt.bias");
      l->dn.a = vec_of(m, il, "ssm_a");
      l->dn.conv = vec_of(m, il, "ssm_conv1d.weight");
      l->dn.norm = vec_of(m, il, "ssm_norm.weight");
    }
    l->ffn.post = vec_of(m, il, "post_attention_norm.weight");
    if (c->n_experts > 0) {
      l->ffn.moe = 1;
      l->ffn.router = mat_of(m, "blk.%d.%s", il, "ffn_gate_inp.weight");
      l->ffn.sh_inp = vec_of(m, il, "ffn_gate_inp_shexp.weight");
      l->ffn.eg = mat_of(m, "blk.%d.%s", il, "ffn_gate_exps.weight");
      l->ffn.eu = mat_of(m, "blk.%d.%s", il, "ffn_up_exps.weight");
      l->ffn.ed = mat_of(m, "blk.%d.%s", il, "ffn_down_exps.weight");
      l->ffn.gate = mat_of(m, "blk.%d.%s", il, "ffn_gate_shexp.weight");
      l->ffn.up = mat_of(m, "blk.%d.%s", il, "ffn_up_shexp.weight");
      l->ffn.down = mat_of(m, "blk.%d.%s", il, "ffn_down_shexp.weight");
      continue;
    }
    l->ffn.gate = mat_of(m, "blk.%d.%s", il, "ffn_gate.weight");
    l->ffn.up = mat_of(m, "blk.%d.%s", il, "ffn_up.weight");
    l->ffn.down = mat_of(m, "blk.%d.%s", il, "ffn_down.weight");
  }
  m->embd = mat_of(m, "%.0d%s", 0, "token_embd.weight");
  m->head = mat_of(m, "%.0d%s", 0, "output.weight");
  m->out_norm = (const float *)mat_of(m, "%.0d%s", 0, "output_norm.weight").w;
  int L = c->n_layers, d = c->d_model, kvd = c->n_kv_heads * c->head_dim, qa = c->n_heads * c->head_dim;
  m->S = fz((size_t)L * c->ssm_heads * c->ssm_state * c->ssm_state);
  m->conv = fz((size_t)L * (c->conv_kernel - 1) * c->convd);
  m->K = fz((size_t)L * cap * kvd);
  m->V = fz((size_t)L * cap * kvd);
  int big = c->d_ff > c->convd ? c->d_ff : c->convd;
  if (d > big) big = d;
  if (c->d_expert > big) big = c->d_expert;
  if (c->d_shared > big) big = c->d_shared;
  if (c->n_experts > 0) { m->moe_p = fz(c->n_experts); m->moe_o = fz(d); }
  if (c->vdc > big) big = c->vdc;
  m->x = fz(d); m->h = fz(d); m->a = fz(big); m->qkv = fz(c->convd); m->z = fz(c->vdc); m->y = fz(big);
  m->qg = fz(2 * qa); m->qn = fz(qa); m->kb = fz(kvd); m->vb = fz(kvd); m->att = fz(qa); m->prob = fz(cap);
  m->qt = fz(c->vdc); m->kt = fz(c->vdc); m->f1 = fz(big); m->f2 = fz(big); m->o128 = fz(c->ssm_state);
  m->logits = fz(c->vocab); m->hn = fz(d);
  return m;
}

API Q35 *q35_open_mem(const char *index_text, const uint8_t *pack, size_t pack_bytes, int layers, int cap) {
  (void)pack_bytes;
  Q35 *m = (Q35 *)calloc(1, sizeof(Q35));
  m->pack = pack;
  if (parse_index(m, index_text)) { free(m); return NULL; }
  return finish_open(m, layers, cap);
}

static uint8_t *slurp(const char *path, size_t *n) {
  FILE *f = fopen(path, "rb");
  if (!f) return NULL;
  fseek(f, 0, SEEK_END);
  long sz = ftell(f);
  fseek(f, 0, SEEK_SET);
  uint8_t *b = (uint8_t *)malloc((size_t)sz + 1);
  if (!b || fread(b, 1, (size_t)sz, f) != (size_t)sz) { fclose(f); free(b); return NULL; }
  fclose(f);
  b[sz] = 0;
  *n = (size_t)sz;
  return b;
}

API Q35 *q35_open_dir(const char *dir, int layers, int cap) {
  char p[4096];
  size_t ni, np;
  snprintf(p, sizeof p, "%s/index.tsv", dir);
  uint8_t *idx = slurp(p, &ni);
  snprintf(p, sizeof p, "%s/pack.bin", dir);
  uint8_t *pk = idx ? slurp(p, &np) : NULL;
  if (!idx || !pk) { free(idx); return NULL; }
  Q35 *m = q35_open_mem((const char *)idx, pk, np, layers, cap);
  free(idx);
  if (m) m->owns_pack = 1; else free(pk);
  return m;
}

API void q35_close(Q35 *m) {
  if (!m) return;
  float *bufs[] = {m->S, m->conv, m->K, m->V, m->x, m->h, m->a, m->qkv, m->z, m->y, m->qg, m->qn, m->kb, m->vb,
                   m->att, m->prob, m->qt, m->kt, m->f1, m->f2, m->o128, m->logits, m->hn, m->mt_K, m->mt_V,
                   m->mt_cat, m->mt_logits, m->moe_p, m->moe_o};
  for (size_t i = 0; i < sizeof bufs / sizeof *bufs; i++) free(bufs[i]);
  if (m->owns_pack) free((void *)m->pack);
  free(m->mt_img); free(m->layer); free(m->t); free(m);
}
API void q35_cfg(const Q35 *m, Q35Cfg *out) { *out = m->c; }
API void q35_reset(Q35 *m) {
  const Q35Cfg *c = &m->c;
  memset(m->S, 0, (size_t)c->n_layers * c->ssm_heads * c->ssm_state * c->ssm_state * 4);
  memset(m->conv, 0, (size_t)c->n_layers * (c->conv_kernel - 1) * c->convd * 4);
}

/* ---- ops ------------------------------------------------------------------------------------ */
static void gemv(const Mat *w, const float *x, float *y) { q35_gemv(w->fmt, w->w, w->rb, w->rows, w->cols, x, y); }

/* h = (x * s) * w, s = 1/sqrt(mean(x^2) + eps)   (tools/qwen35_engine.c:510-515) */
static void rms_norm(float *h, const float *x, const float *w, int n, float eps) {
  float ss = 0.0f;
  for (int i = 0; i < n; i++) ss += x[i] * x[i];
  float s = 1.0f / f_sqrt(ss / (float)n + eps);
  for (int i = 0; i < n; i++) h[i] = x[i] * s * w[i];
}

/* partial NEOX rotation of the first nd dims, pairs (i, i + nd/2), angle through double
 * (tools/qwen35_engine.c:523-533) */
API void q35_rope(float *x, int pos, int nd, float base) {
  int half = nd / 2;
  for (int i = 0; i < half; i++) {
    float th = (float)((double)pos * pow((double)base, -2.0 * i / nd));
    float c = (float)cos((double)th), s = (float)sin((double)th), a = x[i], b = x[i + half];
    x[i] = a * c - b * s;
    x[i + half] = a * s + b * c;
  }
}

/* gated full attention with per-head QK RMSNorm and output gate over a KV cache laid out
 * [pos][kv head][head_dim]; writes the block output (before the residual add) to out[d]
 * (tools/qwen35_engine.c:664-724) */
static void attn_block(Q35 *m, const AttnW *w, float *Kc, float *Vc, const float *h, int pos, float *out) {
  const Q35Cfg *c = &m->c;
  int H = c->n_heads, KV = c->n_kv_heads, hd = c->head_dim, kvd = KV * hd;
  gemv(&w->q, h, m->qg);
  for (int hh = 0; hh < H; hh++) {
    rms_norm(m->qn + hh * hd, m->qg + 2 * hh * hd, w->qn, hd, c->eps);
    q35_rope(m->qn + hh * hd, pos, c->rope_dim, c->rope_base);
  }
  gemv(&w->k, h, m->kb);
  float *krow = Kc + (size_t)pos * kvd, *vrow = Vc + (size_t)pos * kvd;
  for (int g = 0; g < KV; g++) {
    rms_norm(krow + g * hd, m->kb + g * hd, w->kn, hd, c->eps);
    q35_rope(krow + g * hd, pos, c->rope_dim, c->rope_base);
  }
  gemv(&w->v, h, m->vb);
  memcpy(vrow, m->vb, (size_t)kvd * 4);
  int grp = H / KV;
  float scale = 1.0f / f_sqrt((float)hd);
  for (int hh = 0; hh < H; hh++) {
    int g = hh / grp;
    const float *q = m->qn + hh * hd;
    float mx = -INFINITY;
    for (int t = 0; t <= pos; t++) {
      const float *kk = Kc + (size_t)t * kvd + g * hd;
      float s = 0.0f;
      for (int i = 0; i < hd; i++) s += kk[i] * q[i];
      s *= scale;
      m->prob[t] = s;
      if (s > mx) mx = s;
    }
    float sum = 0.0f;
    for (int t = 0; t <= pos; t++) { float e = f_exp(m->prob[t] - mx); m->prob[t] = e; sum += e; }
    for (int i = 0; i < hd; i++) {
      float acc = 0.0f;
      for (int t = 0; t <= pos; t++) acc += (m->prob[t] / sum) * Vc[(size_t)t * kvd + g * hd + i];
      m->att[hh * hd + i] = acc;
    }
  }
  for (int hh = 0; hh < H; hh++)
    for (int i = 0; i < hd; i++) m->att[hh * hd + i] *= q35_sigmoid(m->qg[2 * hh * hd + hd + i]);
  gemv(&w->o, m->att, out);
}

/* gated DeltaNet mixer for one token (tools/qwen35_engine.c:581-662) */
static void delta_block(Q35 *m, const DeltaW *w, float *S, float *cs, const float *h, float *out) {
  const Q35Cfg *c = &m->c;
  int TR = c->ssm_heads, GK = c->ssm_groups, SZ = c->ssm_state, KC = c->conv_kernel, CD = c->convd, kd = c->kdc;
  float *beta = m->f1, *gpre = m->f1 + TR, *y = m->y;
  gemv(&w->qkv, h, m->qkv);
  gemv(&w->z, h, m->z);
  gemv(&w->beta, h, m->f2);
  for (int i = 0; i < TR; i++) beta[i] = q35_sigmoid(m->f2[i]);
  gemv(&w->alpha, h, m->f2);
  for (int i = 0; i < TR; i++) gpre[i] = q35_softplus(m->f2[i] + w->dt[i]) * w->a[i];
  for (int ch = 0; ch < CD; ch++) {
    float acc = 0.0f;
    for (int k = 0; k < KC - 1; k++) acc += cs[k * CD + ch] * w->conv[ch * KC + k];
    acc += m->qkv[ch] * w->conv[ch * KC + KC - 1];
    y[ch] = q35_silu(acc);
  }
  for (int ch = 0; ch < CD; ch++) {
    for (int k = 0; k < KC - 2; k++) cs[k * CD + ch] = cs[(k + 1) * CD + ch];
    cs[(KC - 2) * CD + ch] = m->qkv[ch];
  }
  const float *yq = y, *yk = y + kd, *yv = y + 2 * kd;
  for (int hh = 0; hh < TR; hh++) {       /* value head hh reads key group hh % GK (tile) */
    const float *qg = yq + (hh % GK) * SZ, *kg = yk + (hh % GK) * SZ;
    float sq = 0.0f, sk = 0.0f;
    for (int i = 0; i < SZ; i++) { sq += qg[i] * qg[i]; sk += kg[i] * kg[i]; }
    float nq = f_sqrt(sq), nk = f_sqrt(sk);
    float iq = (1.0f / (nq > c->eps ? nq : c->eps)) / f_sqrt((float)SZ), ik = 1.0f / (nk > c->eps ? nk : c->eps);
    for (int i = 0; i < SZ; i++) { m->qt[hh * SZ + i] = qg[i] * iq; m->kt[hh * SZ + i] = kg[i] * ik; }
  }
  for (int hh = 0; hh < TR; hh++) {
    float *Sh = S + (size_t)hh * SZ * SZ;
    const float *q = m->qt + hh * SZ, *k = m->kt + hh * SZ, *v = yv + hh * c->vhd;
    float decay = f_exp(gpre[hh]), b = beta[hh];
    for (int j = 0; j < SZ; j++) {
      float *row = Sh + j * SZ, kv = 0.0f, o = 0.0f;
      for (int i = 0; i < SZ; i++) { row[i] *= decay; kv += row[i] * k[i]; }
      float delta = (v[j] - kv) * b;
      for (int i = 0; i < SZ; i++) row[i] += k[i] * delta;
      for (int i = 0; i < SZ; i++) o += row[i] * q[i];
      m->o128[j] = o;
    }
    float ss = 0.0f;
    for (int i = 0; i < SZ; i++) ss += m->o128[i] * m->o128[i];
    float r = 1.0f / f_sqrt(ss / (float)SZ + c->eps);
    for (int i = 0; i < SZ; i++)
      m->a[hh * c->vhd + i] = m->o128[i] * r * w->norm[i] * q35_silu(m->z[hh * c->vhd + i]);
  }
  gemv(&w->out, m->a, out);
}

/* The routed-expert FFN on one normed row h2[d]: out[d] = sum_j wt_j * down_{e_j}(silu(gate_{e_j} h2) * up_{e_j} h2)
 * in rank order, plus sigmoid(sh_inp . h2) * shared(h2); no residual.  Routing as host/llb_host.c:622-724 with
 * tools/payload-moeany.patch (llb_moe_topk, llb_moe_gu, llb_moe_dn): softmax over every expert's logit (exp
 * through double), the k largest probabilities with ties to the lower index, their weights divided by their sum
 * clamped at 6.103515625e-5.  ids[k], wts[k + 1] (the last is the shared gate) may be NULL. */
static void moe_rows(Q35 *m, const FfnW *w, const float *h2, float *out, int *ids, float *wts) {
  const Q35Cfg *c = &m->c;
  int d = c->d_model, ne = c->n_experts, nk = c->n_used, ef = c->d_expert, sf = c->d_shared;
  float *p = m->moe_p, mx = -INFINITY, sum = 0.0f;
  gemv(&w->router, h2, p);
  for (int e = 0; e < ne; e++) if (p[e] > mx) mx = p[e];
  for (int e = 0; e < ne; e++) { p[e] = f_exp(p[e] - mx); sum += p[e]; }
  float inv = 1.0f / sum;
  for (int e = 0; e < ne; e++) p[e] *= inv;
  int id[64];
  float wt[65], s = 0.0f;
  if (nk > 64) nk = 64;
  for (int j = 0; j < nk; j++) {
    int b = -1;
    float bv = -1.0f;
    for (int e = 0; e < ne; e++) if (p[e] > bv) { bv = p[e]; b = e; }   /* strict: the lower index wins a tie */
    id[j] = b; wt[j] = bv; p[b] = -2.0f;
    s += bv;
  }
  if (s < 6.103515625e-5f) s = 6.103515625e-5f;
  for (int j = 0; j < nk; j++) wt[j] = wt[j] / s;
  float sg = 0.0f;
  for (int i = 0; i < d; i++) sg += w->sh_inp[i] * h2[i];
  wt[nk] = 1.0f / (1.0f + f_exp(-sg));
  for (int i = 0; i < d; i++) out[i] = 0.0f;
  for (int j = 0; j < nk; j++) {
    Mat g = w->eg, u = w->eu, dn = w->ed;
    g.w += (size_t)id[j] * ef * g.rb; g.rows = ef;
    u.w += (size_t)id[j] * ef * u.rb; u.rows = ef;
    dn.w += (size_t)id[j] * d * dn.rb; dn.rows = d;
    gemv(&g, h2, m->f1);
    gemv(&u, h2, m->f2);
    for (int i = 0; i < ef; i++) m->f1[i] = q35_silu(m->f1[i]) * m->f2[i];
    gemv(&dn, m->f1, m->f2);
    for (int i = 0; i < d; i++) out[i] = j == 0 ? m->f2[i] * wt[0] : out[i] + m->f2[i] * wt[j];
  }
  gemv(&w->gate, h2, m->f1);
  gemv(&w->up, h2, m->f2);
  for (int i = 0; i < sf; i++) m->f1[i] = q35_silu(m->f1[i]) * m->f2[i];
  gemv(&w->down, m->f1, m->f2);
  for (int i = 0; i < d; i++) out[i] = out[i] + m->f2[i] * wt[nk];
  if (ids) memcpy(ids, id, (size_t)nk * sizeof(int));
  if (wts) memcpy(wts, wt, (size_t)(nk + 1) * sizeof(float));
}
API int q35_moe_ffn(Q35 *m, int il, const float *h2, float *out, int *ids, float *wts) {
  if (il < 0 || il >= m->c.n_layers || !m->layer[il].ffn.moe) return 1;
  moe_rows(m, &m->layer[il].ffn, h2, out, ids, wts);
  return 0;
}

/* x += down(silu(gate h2) * (up h2)), h2 = rms(x) * post   (tools/qwen35_engine.c:741-746) */
static void ffn_block(Q35 *m, const FfnW *w, float *x) {
  const Q35Cfg *c = &m->c;
  rms_norm(m->h, x, w->post, c->d_model, c->eps);
  if (w->moe) {   /* (moe_out + shared) + residual, llb_moe_dn's last line */
    moe_rows(m, w, m->h, m->moe_o, NULL, NULL);
    for (int i = 0; i < c->d_model; i++) x[i] = m->moe_o[i] + x[i];
    return;
  }
  gemv(&w->gate, m->h, m->f1);
  gemv(&w->up, m->h, m->f2);
  for (int i = 0; i < c->d_ff; i++) m->f1[i] = q35_silu(m->f1[i]) * m->f2[i];
  gemv(&w->down, m->f1, m->f2);
  for (int i = 0; i < c->d_model; i++) x[i] += m->f2[i];
}

API void q35_forward(Q35 *m, int tok, int pos) {
  const Q35Cfg *c = &m->c;
  int d = c->d_model, kvd = c->n_kv_heads * c->head_dim;
  q35_deq_row(m->embd.fmt, m->embd.w + (size_t)tok * m->embd.rb, d, m->x);
  for (int il = 0; il < c->n_layers; il++) {
    Layer *l = &m->layer[il];
    rms_norm(m->h, m->x, l->attn_norm, d, c->eps);
    if (l->full)
      attn_block(m, &l->at, m->K + (size_t)il * m->cap * kvd, m->V + (size_t)il * m->cap * kvd, m->h, pos, m->y);
    else
      delta_block(m, &l->dn, m->S + (size_t)il * c->ssm_heads * c->ssm_state * c->ssm_state,
                  m->conv + (size_t)il * (c->conv_kernel - 1) * c->convd, m->h, m->y);
    for (int i = 0; i < d; i++) m->x[i] += m->y[i];
    ffn_block(m, &l->ffn, m->x);
  }
}

API const float *q35_logits(Q35 *m) {
  rms_norm(m->hn, m->x, m->out_norm, m->c.d_model, m->c.eps);
  gemv(&m->head, m->hn, m->logits);
  return m->logits;
}
API const float *q35_residual(const Q35 *m) { return m->x; }
API const float *q35_hnorm(const Q35 *m) { return m->hn; }
API const float *q35_state_S(const Q35 *m, int il) {
  return m->S + (size_t)il * m->c.ssm_heads * m->c.ssm_state * m->c.ssm_state;
}
API const float *q35_state_conv(const Q35 *m, int il) {
  return m->conv + (size_t)il * (m->c.conv_kernel - 1) * m->c.convd;
}
API const float *q35_state_k(const Q35 *m, int il, int pos) {
  return m->K + ((size_t)il * m->cap + pos) * m->c.n_kv_heads * m->c.head_dim;
}
API const float *q35_state_v(const Q35 *m, int il, int pos) {
  return m->V + ((size_t)il * m->cap + pos) * m->c.n_kv_heads * m->c.head_dim;
}

/* first strict maximum wins; second = the same scan with the winner masked
 * (tools/qwen35_engine.c:763-778) */
API void q35_top2(const float *z, int n, int *ids, float *vals) {
  int b = 0, s = -1;
  for (int i = 1; i < n; i++) if (z[i] > z[b]) b = i;
  for (int i = 0; i < n; i++) {
    if (i == b) continue;
    if (s < 0 || z[i] > z[s]) s = i;
  }
  ids[0] = b; vals[0] = z[b];
  ids[1] = s < 0 ? 0 : s; vals[1] = s < 0 ? -INFINITY : z[s];
}

static void put_top2(uint32_t *dst, const float *z, int n) {
  int id[2];
  float v[2];
  q35_top2(z, n, id, v);
  dst[0] = (uint32_t)id[0]; memcpy(&dst[1], &v[0], 4);
  dst[2] = (uint32_t)id[1]; memcpy(&dst[3], &v[1], 4);
}

API int q35_greedy(Q35 *m, const int *prompt, int np, int steps, int *ids, uint32_t *top2) {
  if (np < 1 || np + steps + 1 > m->cap) return -1;
  q35_reset(m);
  for (int t = 0; t < np; t++) q35_forward(m, prompt[t], t);
  for (int s = 0; s < steps; s++) {
    const float *z = q35_logits(m);
    uint32_t w[4];
    put_top2(w, z, m->c.vocab);
    ids[s] = (int)w[0];
    if (top2) memcpy(top2 + 4 * s, w, 16);
    if (s + 1 < steps) q35_forward(m, ids[s], np + s);
  }
  return steps;
}

/* ---- MTP drafter ----------------------------------------------------------------------------- */
static int aux_fmt(uint32_t dt) { /* tools/auxpack/auxpack.py:32 */
  return dt == 0 ? FM_F32 : dt == 2 ? FM_Q8_0 : dt == 3 ? FM_Q4_K : dt == 4 ? FM_Q6_K : dt == 7 ? FM_Q5_K : -1;
}
static int fm_rb(int fmt, int cols) {
  return fmt == FM_F32 ? cols * 4 : fmt == FM_Q8_0 ? cols / 32 * 34 : fmt == FM_Q4_K ? cols / 256 * 144
       : fmt == FM_Q6_K ? cols / 256 * 210 : fmt == FM_Q5_K ? cols / 256 * 176 : 0;
}

API int q35_mtp_load(Q35 *m, const uint8_t *img, size_t bytes) {
  static const char *names[17] = {
    "nextn.enorm", "nextn.hnorm", "nextn.eh_proj", "attn_norm", "attn_q", "attn_k", "attn_v", "attn_q_norm",
    "attn_k_norm", "attn_output", "post_attention_norm", "ffn_gate", "ffn_up", "ffn_down",
    "nextn.shared_head_norm", "mtp.head_slice", "mtp.ids"};
  const Q35Cfg *c = &m->c;
  int d = c->d_model, qa = c->n_heads * c->head_dim, kvd = c->n_kv_heads * c->head_dim, f = c->d_ff;
  uint64_t off[17], nb[17];
  int fmt[17], got[17] = {0};
  /* positional MTP1 fixes the formats (host/llb_host.c:1574-1577) */
  int mtp1_fmt[17] = {0, 0, FM_Q4_K, 0, FM_Q6_K, FM_Q6_K, FM_Q6_K, 0, 0, FM_Q6_K, 0, FM_Q4_K, FM_Q4_K, FM_Q4_K, 0,
                      FM_Q6_K, 0};
  if (bytes < 16) return 1;
  if (!memcmp(img, "MTP1", 4)) {
    uint32_t n;
    memcpy(&n, img + 4, 4);
    if (n != 17) return 2;
    for (int j = 0; j < 17; j++) {
      memcpy(&off[j], img + 8 + 16 * j, 8); memcpy(&nb[j], img + 16 + 16 * j, 8);
      fmt[j] = mtp1_fmt[j]; got[j] = 1;
    }
  } else if (!memcmp(img, "AUX1", 4)) {
    uint32_t n;
    memcpy(&n, img + 8, 4);
    for (uint32_t i = 0; i < n; i++) {
      const uint8_t *e = img + 16 + 72 * (size_t)i;
      char nm[33];
      memcpy(nm, e, 32); nm[32] = 0;
      for (int j = 0; j < 17; j++) if (!strcmp(nm, names[j])) {
        uint32_t dt;
        if (got[j]) return 3;
        memcpy(&dt, e + 32, 4); memcpy(&off[j], e + 56, 8); memcpy(&nb[j], e + 64, 8);
        fmt[j] = j == 16 ? 0 : aux_fmt(dt); got[j] = 1;
      }
    }
  } else return 4;
  for (int j = 0; j < 17; j++) if (!got[j] || fmt[j] < 0 || off[j] + nb[j] > bytes) return 5;
  int nv = (int)(nb[16] / 4);
  int rows[17] = {1, 1, d, 1, 2 * qa, kvd, kvd, 1, 1, d, 1, f, f, d, 1, nv, 1};
  int cols[17] = {d, d, 2 * d, d, d, d, d, c->head_dim, c->head_dim, qa, d, d, d, f, d, d, nv};
  for (int j = 0; j < 16; j++) if (nb[j] != (uint64_t)rows[j] * fm_rb(fmt[j], cols[j])) return 6;
  free(m->mt_img);
  m->mt_img = (uint8_t *)malloc(bytes);
  memcpy(m->mt_img, img, bytes);
  const uint8_t *b = m->mt_img;
#define MAT(j) ((Mat){b + off[j], rows[j], cols[j], fmt[j], fm_rb(fmt[j], cols[j])})
#define VEC(j) ((const float *)(b + off[j]))
  m->mt_enorm = VEC(0); m->mt_hnorm = VEC(1); m->mt_eh = MAT(2); m->mt_attn_norm = VEC(3);
  m->mt_at.q = MAT(4); m->mt_at.k = MAT(5); m->mt_at.v = MAT(6); m->mt_at.qn = VEC(7); m->mt_at.kn = VEC(8);
  m->mt_at.o = MAT(9); m->mt_ffn.post = VEC(10); m->mt_ffn.gate = MAT(11); m->mt_ffn.up = MAT(12);
  m->mt_ffn.down = MAT(13); m->mt_shn = VEC(14); m->mt_head = MAT(15);
  m->mt_ids = (const uint32_t *)(b + off[16]);
#undef MAT
#undef VEC
  m->mt_nv = nv;
  free(m->mt_K); free(m->mt_V); free(m->mt_cat); free(m->mt_logits);
  m->mt_K = fz((size_t)m->cap * kvd); m->mt_V = fz((size_t)m->cap * kvd);
  m->mt_cat = fz(2 * (size_t)d); m->mt_logits = fz(nv);
  m->has_mtp = 1;
  return 0;
}

/* The NextN block for n rows at positions pa .. pa+n-1 (host/llb_host.c:1775-1808): row r pairs
 * token tk[r] with hidden row hs[r] (the output-normed hidden of position pa+r-1):
 *   x = eh_proj [rms(embed) * enorm ; rms(h) * hnorm]; x += attn(rms(x) * attn_norm) on the
 *   drafter's own KV; x += ffn(x); hn = rms(x) * shared_head_norm; the last row's head-slice
 *   argmax, mapped through ids, is the draft. */
API int q35_mtp_rows(Q35 *m, int n, int pa, const int *tk, const float *hs, float *hn_out) {
  const Q35Cfg *c = &m->c;
  int d = c->d_model, draft = -1;
  /* the blocks use the model's scratch (h, f1, f2, y): the row's residual lives in a buffer of its own */
  float *xr = (float *)malloc((size_t)d * 4), *e = (float *)malloc((size_t)d * 4);
  for (int r = 0; r < n; r++) {
    q35_deq_row(m->embd.fmt, m->embd.w + (size_t)tk[r] * m->embd.rb, d, e);
    rms_norm(m->mt_cat, e, m->mt_enorm, d, c->eps);
    rms_norm(m->mt_cat + d, hs + (size_t)r * d, m->mt_hnorm, d, c->eps);
    gemv(&m->mt_eh, m->mt_cat, xr);
    rms_norm(m->h, xr, m->mt_attn_norm, d, c->eps);
    attn_block(m, &m->mt_at, m->mt_K, m->mt_V, m->h, pa + r, m->y);
    for (int i = 0; i < d; i++) xr[i] += m->y[i];
    ffn_block(m, &m->mt_ffn, xr);
    rms_norm(hn_out + (size_t)r * d, xr, m->mt_shn, d, c->eps);
    if (r == n - 1) {
      int id[2];
      float v[2];
      gemv(&m->mt_head, hn_out + (size_t)r * d, m->mt_logits);
      q35_top2(m->mt_logits, m->mt_nv, id, v);
      draft = (int)m->mt_ids[id[0]];
    }
  }
  free(xr); free(e);
  return draft;
}

/* Greedy speculative decoding with the MTP drafter: the cycle of host/llb_host.c:1902-1950 seen
 * from the token stream.  A cycle at (pos, tok) drafts ke tokens (catch-up rows over the positions
 * the previous cycle served, then a chain on the drafter's own hidden, :1814-1829), runs the trunk
 * over tin[0..ke] at positions pos.., and serves row r while every earlier row's argmax equalled
 * the next input (:1911; greedy accept rule host/llb_sampler_impl.h:400-405).  The CPU forward is
 * sequential, so rows after the first mismatch are simply not computed: the layer state is then
 * exactly the state after the last served row, which is what the device ring's rollback yields. */
API int q35_spec_greedy(Q35 *m, const int *prompt, int np, int steps, int k, int *ids, uint32_t *top2,
                        Q35SpecStats *st) {
  const Q35Cfg *c = &m->c;
  int d = c->d_model;
  if (!m->has_mtp || np < 1 || k < 0 || k > 7 || np + steps + k + 2 > m->cap) return -1;
  int *hist = (int *)calloc((size_t)m->cap + 16, 4);
  float *hn = fz((size_t)8 * d), *mhn = fz((size_t)8 * d), *keep = fz(d);
  Q35SpecStats z;
  memset(&z, 0, sizeof z);
  q35_reset(m);
  memset(m->mt_K, 0, (size_t)m->cap * c->n_kv_heads * c->head_dim * 4);
  memset(m->mt_V, 0, (size_t)m->cap * c->n_kv_heads * c->head_dim * 4);
  /* prompt: every position but the last is one served row; its drafter row keeps the drafter's KV
   * in step (the drafts made there are never served unless they match, and their KV rows are
   * overwritten, so they are not computed here) */
  for (int t = 0; t + 1 < np; t++) {
    hist[t] = prompt[t];
    q35_mtp_rows(m, 1, t, &hist[t], hn, mhn);          /* hn row 0 = h of position t-1 (zeros at 0) */
    q35_forward(m, prompt[t], t);
    q35_logits(m);
    memcpy(hn, m->hn, (size_t)d * 4);
  }
  int pos = np - 1, tok = prompt[np - 1], nprev = 1, out = 0;
  while (out < steps) {
    int tin[9], n = pos == 0 ? 1 : nprev, pa = pos + 1 - n, ke = k;
    hist[pos] = tok;
    tin[0] = tok;
    if (pos == 0) memset(hn, 0, (size_t)d * 4);
    if (ke > 0) {
      tin[1] = q35_mtp_rows(m, n, pa, hist + pa, hn, mhn);
      for (int j = 2; j <= ke; j++) {
        /* the chain's hidden is the drafter's own previous output row; copied out because the
         * call below overwrites mhn */
        memcpy(keep, mhn + (size_t)(j == 2 ? n - 1 : 0) * d, (size_t)d * 4);
        tin[j] = q35_mtp_rows(m, 1, pos + j - 1, &tin[j - 1], keep, mhn);
      }
    } else {
      /* k = 0 still keeps the drafter's KV in step */
      q35_mtp_rows(m, n, pa, hist + pa, hn, mhn);
    }
    int T = 1 + ke, nv = 0;
    z.cycles++; z.rows += (uint64_t)T;
    for (int r = 0; r < T; r++) {
      q35_forward(m, tin[r], pos + r);
      const float *lg = q35_logits(m);
      memcpy(hn + (size_t)r * d, m->hn, (size_t)d * 4);
      uint32_t w[4];
      put_top2(w, lg, c->vocab);
      nv = r + 1;
      hist[pos + r + 1] = (int)w[0];
      if (out < steps) {
        ids[out] = (int)w[0];
        if (top2) memcpy(top2 + 4 * out, w, 16);
        out++;
      }
      if (r + 1 < T && (int)w[0] != tin[r + 1]) break;   /* a cycle always runs to its own end */
    }
    for (int j = 1; j < T; j++) { z.drafted[j]++; z.accepted[j] += nv > j; }
    z.served += (uint64_t)nv;
    tok = hist[pos + nv];
    pos += nv;
    nprev = nv;
  }
  if (st) *st = z;
  free(hist); free(hn); free(mhn); free(keep);
  return out;
}

/* Prompt-lookup drafter (host/llb_host.c:1655-1676): the LATEST earlier match of the history's last
 * L = 3, 2, 1 tokens (positions j-L+1..j == pos-L+1..pos, j < pos); the up-to-k tokens that followed
 * it become the drafts.  Returns the count; hist[0..pos] must be valid. */
API int q35_lookup_draft(const int *hist, int pos, int k, int *out) {
  for (int L = 3; L >= 1; L--) {
    for (int j = pos - 1; j >= L - 1; j--) {
      int m = 0;
      while (m < L && hist[j - m] == hist[pos - m]) m++;
      if (m == L) {
        int n = 0;
        while (n < k && j + 1 + n <= pos) { out[n] = hist[j + 1 + n]; n++; }
        return n;
      }
    }
  }
  return 0;
}

/* Greedy generation with the prompt-lookup drafter in place of the MTP head (the reference's path
 * when LLB_SPEC is set without LLB_MTP, host/llb_host.c:1936): T = 1 + drafts rows per cycle, same
 * accept rule.  The prompt positions before the last are plain single rows. */
API int q35_spec_lookup(Q35 *m, const int *prompt, int np, int steps, int k, int *ids, uint32_t *top2, Q35SpecStats *st) {
  const Q35Cfg *c = &m->c;
  if (np < 1 || k < 0 || k > 7 || np + steps + k + 2 > m->cap) return -1;
  int *hist = (int *)calloc((size_t)m->cap + 16, 4);
  Q35SpecStats z;
  memset(&z, 0, sizeof z);
  q35_reset(m);
  for (int t = 0; t + 1 < np; t++) {
    hist[t] = prompt[t];
    q35_forward(m, prompt[t], t);
  }
  int pos = np - 1, tok = prompt[np - 1], out = 0;
  while (out < steps) {
    int tin[9], nv = 0;
    hist[pos] = tok;
    tin[0] = tok;
    const int T = 1 + q35_lookup_draft(hist, pos, k, tin + 1);
    z.cycles++; z.rows += (uint64_t)T;
    for (int r = 0; r < T; r++) {
      q35_forward(m, tin[r], pos + r);
      const float *lg = q35_logits(m);
      uint32_t w[4];
      put_top2(w, lg, c->vocab);
      nv = r + 1;
      hist[pos + r + 1] = (int)w[0];
      if (out < steps) {
        ids[out] = (int)w[0];
        if (top2) memcpy(top2 + 4 * out, w, 16);
        out++;
      }
      if (r + 1 < T && (int)w[0] != tin[r + 1]) break;
    }
    for (int j = 1; j < T; j++) { z.drafted[j]++; z.accepted[j] += nv > j; }
    z.served += (uint64_t)nv;
    tok = hist[pos + nv];
    pos += nv;
  }
  if (st) *st = z;
  free(hist);
  return out;
}
