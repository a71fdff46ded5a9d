// q35_sampler.c -- CPU restatement of the reference's sampler chain and of its speculative verify step.
// TEST INFRASTRUCTURE ONLY: the checker of the device sampler (csrc/sampler.cu); nothing of the product links it.
//
// What it follows (the reference keeps llama.cpp's float arithmetic on purpose, so the order of every float
// operation below is the reference's):
//   chain order bias -> penalties -> top_k -> top_p -> min_p -> temperature   host/llb_sampler_impl.h:322-358
//   counter RNG: splitmix64 of (seed, 4 pos + k + 1), 53 bits                   host/llb_sampler_impl.h:142-155
//   top_k: partial selection of the k largest, earlier candidate wins ties      :170-199
//   top_p: float softmax and float running sum over the sorted prefix           :201-262
//   min_p: filter against max + logf(p); sorted variant keeps min_keep          :264-297
//   probabilities expf(l - max), their sum in double; the walk                  :313-333
//   sample / verify (accept with min(1, p/q), residual max(0, p - q))           :384-444
// Built with -ffp-contract=off like the rest of the oracle (oracle/Makefile), as the reference builds its own.
// Pinned by tests/golden/sampler_vectors.npz, which tests/golden/make_golden_sampler.py draws from the reference's
// own host/llb_sampler.c compiled where it lies (oracle/_ref/libllbsmp.so).
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define Q35_API __attribute__((visibility("default")))
#define SMP_MAX_BIAS 64
#define SMP_SEL 256

typedef struct {
  float temp, top_p, min_p;
  int top_k;
  float repeat_penalty;
  int repeat_last_n;
  float presence, frequency;
  uint64_t seed;
  int min_keep;
  int n_bias;
  int bias_ids[SMP_MAX_BIAS];
  float bias_vals[SMP_MAX_BIAS];
} Q35Smp;

typedef struct { float l; int id; } Cand;

static double draw(uint64_t seed, uint64_t pos, uint32_t k) {
  uint64_t z = seed ^ 0x6A09E667F3BCC909ull;
  z += (pos * 4 + k + 1) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}

// before(a, b): a comes first in the total order "logit descending, then id ascending"
static int before(Cand a, Cand b) { return a.l > b.l || (a.l == b.l && a.id < b.id); }
static int cmp(const void *x, const void *y) {
  const Cand *a = x, *b = y;
  return before(*a, *b) ? -1 : before(*b, *a) ? 1 : 0;
}
static void sort_all(int *ids, float *lg, int n) {
  Cand *c = malloc(sizeof(Cand) * (size_t)n);
  for (int i = 0; i < n; i++) { c[i].l = lg[i]; c[i].id = ids[i]; }
  qsort(c, (size_t)n, sizeof(Cand), cmp);
  for (int i = 0; i < n; i++) { lg[i] = c[i].l; ids[i] = c[i].id; }
  free(c);
}
// the m largest of an unsorted list, sorted descending; among equal logits the earlier list position first
static void select_top(const int *ids, const float *lg, int n, int m, Cand *out) {
  int cnt = 0;
  for (int i = 0; i < n; i++) {
    const float l = lg[i];
    if (cnt == m && !(l > out[m - 1].l)) continue;
    int at = cnt < m ? cnt++ : m - 1;
    while (at > 0 && out[at - 1].l < l) { out[at] = out[at - 1]; at--; }
    out[at].l = l; out[at].id = ids[i];
  }
}

typedef struct { int *ids; float *lg, *p; int n, sorted; } List;

static void st_top_k(List *c, int k) {
  if (k <= 0) return;
  if (k > c->n) k = c->n;
  if (!c->sorted) {
    if (k <= SMP_SEL) {
      Cand top[SMP_SEL];
      select_top(c->ids, c->lg, c->n, k, top);
      for (int i = 0; i < k; i++) { c->ids[i] = top[i].id; c->lg[i] = top[i].l; }
    } else sort_all(c->ids, c->lg, c->n);
    c->sorted = 1;
  }
  c->n = k;
}

static void st_top_p(List *c, float p, int min_keep) {
  if (p >= 1.0f) return;
  const int N = c->n;
  float mx = c->lg[0];
  if (!c->sorted) for (int i = 1; i < N; i++) if (c->lg[i] > mx) mx = c->lg[i];
  float sum = 0.0f;
  for (int i = 0; i < N; i++) sum += expf(c->lg[i] - mx);
  int last = N;
  if (c->sorted) {
    float cum = 0.0f;
    for (int i = 0; i < N; i++) {
      cum += expf(c->lg[i] - mx) / sum;
      if (cum >= p && i + 1 >= min_keep) { last = i + 1; break; }
    }
    c->n = last;
    return;
  }
  const int m = N < SMP_SEL ? N : SMP_SEL;
  Cand top[SMP_SEL];
  select_top(c->ids, c->lg, N, m, top);
  float cum = 0.0f;
  int found = 0;
  for (int i = 0; i < m; i++) {
    cum += expf(top[i].l - mx) / sum;
    if (cum >= p && i + 1 >= min_keep) { last = i + 1; found = 1; break; }
  }
  if (found) {
    for (int i = 0; i < last; i++) { c->ids[i] = top[i].id; c->lg[i] = top[i].l; }
  } else if (m < N) {
    sort_all(c->ids, c->lg, N);
    cum = 0.0f;
    for (int i = 0; i < N; i++) {
      cum += expf(c->lg[i] - mx) / sum;
      if (cum >= p && i + 1 >= min_keep) { last = i + 1; break; }
    }
  } else {
    for (int i = 0; i < N; i++) { c->ids[i] = top[i].id; c->lg[i] = top[i].l; }
  }
  c->n = last;
  c->sorted = 1;
}

static void st_min_p(List *c, float p, int min_keep) {
  if (p <= 0.0f || c->n == 0) return;
  const int N = c->n;
  if (!c->sorted) {
    float mxl = -FLT_MAX;
    for (int i = 0; i < N; i++) if (c->lg[i] > mxl) mxl = c->lg[i];
    const float floor_l = mxl + logf(p);
    int w = 0;
    for (int i = 0; i < N; i++) if (c->lg[i] >= floor_l) w++;
    if (w > 0 && w >= min_keep) {
      w = 0;
      for (int i = 0; i < N; i++) if (c->lg[i] >= floor_l) { c->ids[w] = c->ids[i]; c->lg[w] = c->lg[i]; w++; }
      c->n = w;
      return;
    }
    sort_all(c->ids, c->lg, N);
    c->sorted = 1;
  }
  const float floor_l = c->lg[0] + logf(p);
  int i = 1;
  for (; i < N; i++) if (c->lg[i] < floor_l && i >= min_keep) break;
  c->n = i;
}

static void st_temp(List *c, float t) {
  if (c->n == 0 || t == 1.0f) return;
  for (int i = 0; i < c->n; i++) c->lg[i] /= t;
}

// p[i] = expf(l - max) and their sum in double
static double probs(const List *c) {
  float mx = c->lg[0];
  if (!c->sorted) for (int i = 1; i < c->n; i++) if (c->lg[i] > mx) mx = c->lg[i];
  double sum = 0.0;
  for (int i = 0; i < c->n; i++) { const float e = expf(c->lg[i] - mx); c->p[i] = e; sum += e; }
  return sum;
}
static int walk(const List *c, double rnd) {
  if (c->n <= 0) return -1;
  if (c->n == 1) { c->p[0] = 1.0f; return 0; }
  const double sum = probs(c), tgt = sum * rnd;
  double run = 0.0;
  int sel = -1;
  for (int i = 0; i < c->n; i++) {
    if (sel < 0) { run += c->p[i]; if (run >= tgt) sel = i; }
    c->p[i] = (float)((double)c->p[i] / sum);
  }
  return sel < 0 ? c->n - 1 : sel;
}

static int pen_off(const Q35Smp *P) {
  return P->repeat_last_n <= 0 || (P->repeat_penalty == 1.0f && P->frequency == 0.0f && P->presence == 0.0f);
}

// stages bias, penalties (window = the last repeat_last_n of hist[0..nh)), then top_k .. temp when `full`
static void chain(const Q35Smp *P, const float *logits, int V, const int *hist, int nh, int full, List *c) {
  memcpy(c->lg, logits, sizeof(float) * (size_t)V);
  for (int i = 0; i < V; i++) c->ids[i] = i;
  c->n = V; c->sorted = 0;
  for (int j = 0; j < P->n_bias; j++) {
    const int t = P->bias_ids[j];
    if (t >= 0 && t < V) c->lg[t] += P->bias_vals[j];
  }
  if (!pen_off(P) && hist) {
    const int i0 = nh > P->repeat_last_n ? nh - P->repeat_last_n : 0;
    for (int a = i0; a < nh; a++) {
      const int t = hist[a];
      if (t < 0 || t >= V) continue;
      int seen = 0, cnt = 0;
      for (int b = i0; b < a; b++) if (hist[b] == t) seen = 1;
      if (seen) continue;                                   // once per distinct token
      for (int b = i0; b < nh; b++) if (hist[b] == t) cnt++;
      if (c->lg[t] <= 0) c->lg[t] *= P->repeat_penalty; else c->lg[t] /= P->repeat_penalty;
      c->lg[t] -= (float)cnt * P->frequency + (float)(cnt > 0) * P->presence;
    }
  }
  if (!full) return;
  st_top_k(c, P->top_k);
  st_top_p(c, P->top_p, P->min_keep);
  st_min_p(c, P->min_p, P->min_keep);
  st_temp(c, P->temp);
}

static int argmax_first(const float *v, int n) {
  int bi = 0;
  float bv = v[0];
  for (int i = 1; i < n; i++) if (v[i] > bv) { bv = v[i]; bi = i; }
  return bi;
}

// One row: the token for position `pos` from its logits.  draft >= 0: the speculative verify of the (deterministic)
// drafter's token, *accepted = 1 iff the token returned is the draft; draft < 0: a plain draw.  hist[0..nh): the tokens
// of the positions before `pos` (the penalty window is their tail).  margin (may be null): how far the accept decision
// was from flipping, |u - p(draft)|, or the distance of the walk's target from the nearest step of the running sum,
// relative to the sum: tests use it to excuse a device decision that differs only where the oracle's own was that close.
Q35_API int q35_smp_row(const Q35Smp *P, const float *logits, int V, const int *hist, int nh, int draft, uint64_t pos, int *accepted,
                        double *margin) {
  List c;
  c.ids = malloc(sizeof(int) * (size_t)V); c.lg = malloc(sizeof(float) * (size_t)V); c.p = malloc(sizeof(float) * (size_t)V);
  int tok;
  if (accepted) *accepted = 0;
  if (margin) *margin = 1.0;
  if (P->temp <= 0.0f) {
    chain(P, logits, V, hist, nh, 0, &c);
    tok = argmax_first(c.lg, V);
    if (accepted) *accepted = draft >= 0 && tok == draft;
    goto done;
  }
  chain(P, logits, V, hist, nh, 1, &c);
  if (draft < 0) {
    const double u = draw(P->seed, pos, 0);
    const int sel = walk(&c, u);
    if (margin && c.n > 1) {
      double run = 0.0, best = 1.0;
      for (int i = 0; i < c.n; i++) { run += c.p[i]; const double d = fabs(run - u); if (d < best) best = d; }
      *margin = best;
    }
    tok = c.ids[sel];
    goto done;
  }
  {
    const double sum = probs(&c);
    double pd = 0.0;
    for (int i = 0; i < c.n; i++) if (c.ids[i] == draft) pd = (double)c.p[i] / sum;
    const double u = draw(P->seed, pos, 1);
    if (margin) *margin = fabs(u - pd);
    if (u < pd) { if (accepted) *accepted = 1; tok = draft; goto done; }
    double rs = 0.0;
    for (int i = 0; i < c.n; i++) {
      const double pi = (double)c.p[i] / sum, qi = c.ids[i] == draft ? 1.0 : 0.0;
      const double r = pi > qi ? pi - qi : 0.0;
      c.p[i] = (float)r;
      rs += r;
    }
    const double u2 = draw(P->seed, pos, 2);
    if (!(rs > 0.0)) { tok = c.ids[walk(&c, u2)]; goto done; }
    const double tgt = rs * u2;
    double run = 0.0, best = 1.0;
    int last = -1, hit = -1;
    for (int i = 0; i < c.n; i++) {
      if (c.p[i] <= 0.0f) continue;
      last = i;
      run += c.p[i];
      if (hit < 0 && run >= tgt) hit = i;
      const double d = fabs(run - tgt) / rs;
      if (d < best) best = d;
    }
    if (margin && best < *margin) *margin = best;
    tok = c.ids[hit >= 0 ? hit : last];
  }
done:
  free(c.ids); free(c.lg); free(c.p);
  return tok;
}

Q35_API double q35_smp_draw(uint64_t seed, uint64_t pos, uint32_t k) { return draw(seed, pos, k); }
