// sampler.cu -- sampling-mode verify on the device: for every row of a verify pass, the token the reference's sampler
// pack would emit from that row's logits -- llb_smp_verify for a row that has a draft (accept with probability
// min(1, p / q), q one-hot because both drafters are deterministic; on a reject a draw from the residual
// max(0, p - q)), llb_smp_sample for the row that has none (host/llb_sampler_impl.h:384-444).  The reference reads V
// logits back per served row and decides on the host (smp_pick, host/llb_host.c:1407-1470); here the rows of a pass
// are decided by one kernel inside the cycle's graph and k_accept takes the emitted tokens from it instead of the
// argmax, so a sampled cycle is still one graph launch and one result record.
//
// The chain (host/llb_sampler_impl.h:322-358): logit bias -> repeat / frequency / presence penalties over the last
// repeat_last_n tokens -> top_k -> top_p -> min_p -> temperature -> probabilities expf(l - max) with their sum in
// double.  The reference keeps llama.cpp's float arithmetic on purpose; where the order of float operations decides
// a result (the float running sums of top_p, the penalty expression) one thread does them in the reference's order
// with no fused multiply-add.  exp is taken in double and rounded (the host's expf is within half an ulp of that).
//   top_k in 1..256: the k largest by rounds of a block-wide argmax under the order "logit descending, id ascending"
//     (the reference's partial selection, ties to the earlier candidate), then the short sorted list goes through
//     top_p, min_p, temperature and the draw sequentially -- the reference's own arithmetic, operation for operation.
//   top_k off: the whole vocabulary in id order; min_p is a mask, the probabilities' sum and the walk's running sums
//     are block-wide reductions and scans in double (they differ from the sequential double sums in the last bits only).
//   top_p without top_k needs the reference's float sum over the whole vocabulary in id order and is refused by
//     llb_spec_set_sampler, as are top_k > 256 and a penalty window longer than 256.
// Random numbers: the reference's counter RNG, splitmix64 of (seed, 4 pos + k + 1) (host/llb_sampler_impl.h:142-155):
// draw 1 decides accept, draw 2 the residual, draw 0 a plain sample; pos = the position the token will occupy.
#include "model.cuh"
#include "sampler.cuh"

#define SMP_THREADS 1024

__device__ __forceinline__ double smp_draw(unsigned long long seed, unsigned long long pos, unsigned int k) {
  unsigned long long z = seed ^ 0x6A09E667F3BCC909ull;
  z += (pos * 4ull + k + 1ull) * 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  z ^= z >> 31;
  return (double)(z >> 11) * (1.0 / 9007199254740992.0);
}
__device__ __forceinline__ float smp_expf(float x) { return (float)exp((double)x); }
// a comes before b: logit descending, then id ascending
__device__ __forceinline__ bool smp_before(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

struct SmpShared {
  int win[SMP_MAX_WIN];
  float cv[SMP_MAX_TOPK];
  int ci[SMP_MAX_TOPK];
  float cp[SMP_MAX_TOPK];
  float rv[32];
  int ri[32];
  double rd[32];
  float bv;
  int bi;
  double bd;
  int hit_lo, hit_hi;
};

// block-wide best (v, i) under smp_before; every thread gets it.  i < 0: no candidate.
__device__ __forceinline__ void smp_block_best(float &v, int &i, SmpShared &sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, m);
    const int oi = __shfl_xor_sync(0xffffffffu, i, m);
    if (oi >= 0 && (i < 0 || smp_before(ov, oi, v, i))) { v = ov; i = oi; }
  }
  __syncthreads();
  if (lane == 0) { sh.rv[w] = v; sh.ri[w] = i; }
  __syncthreads();
  if (w == 0) {
    v = sh.rv[lane]; i = sh.ri[lane];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, m);
      const int oi = __shfl_xor_sync(0xffffffffu, i, m);
      if (oi >= 0 && (i < 0 || smp_before(ov, oi, v, i))) { v = ov; i = oi; }
    }
    if (lane == 0) { sh.bv = v; sh.bi = i; }
  }
  __syncthreads();
  v = sh.bv; i = sh.bi;
}
// block-wide sum in double; every thread gets it
__device__ __forceinline__ double smp_block_sum(double x, SmpShared &sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  __syncthreads();
  if (lane == 0) sh.rd[w] = x;
  __syncthreads();
  if (w == 0) {
    x = sh.rd[lane];
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
    if (lane == 0) sh.bd = x;
  }
  __syncthreads();
  return sh.bd;
}
// exclusive prefix over the threads of the block (thread order), in double
__device__ __forceinline__ double smp_block_excl(double x, SmpShared &sh) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  double inc = x;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) { const double o = __shfl_up_sync(0xffffffffu, inc, m); if (lane >= m) inc += o; }
  __syncthreads();
  if (lane == 31) sh.rd[w] = inc;
  __syncthreads();
  if (w == 0) {
    double t = sh.rd[lane], ti = t;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) { const double o = __shfl_up_sync(0xffffffffu, ti, m); if (lane >= m) ti += o; }
    sh.rd[lane] = ti - t;
  }
  __syncthreads();
  return sh.rd[w] + inc - x;
}

// The walk over the whole vocabulary in id order: the first id whose running sum of val(i) reaches tgt, else the last id
// with val > 0.  Every thread owns a run of consecutive ids.
template <class F> __device__ __forceinline__ int smp_walk_all(int V, double tgt, F val, SmpShared &sh) {
  const int per = (V + SMP_THREADS - 1) / SMP_THREADS, i0 = threadIdx.x * per, i1 = min(V, i0 + per);
  double mine = 0.0;
  int last = -1;
  for (int i = i0; i < i1; i++) { const float p = val(i); if (p > 0.0f) { mine += (double)p; last = i; } }
  const double before = smp_block_excl(mine, sh);
  if (threadIdx.x == 0) { sh.hit_lo = 0x7fffffff; sh.hit_hi = -1; }
  __syncthreads();
  if (last >= 0) atomicMax(&sh.hit_hi, last);
  if (mine > 0.0 && before + mine >= tgt) {
    double run = before;
    for (int i = i0; i < i1; i++) {
      const float p = val(i);
      if (p <= 0.0f) continue;
      run += (double)p;
      if (run >= tgt) { atomicMin(&sh.hit_lo, i); break; }
    }
  }
  __syncthreads();
  return sh.hit_lo != 0x7fffffff ? sh.hit_lo : sh.hit_hi;
}

// One block per row of the pass.  Engine mode (ctl != null): the row's stream, position, draft and penalty window come
// from the control block; test mode: from the explicit arrays.
__global__ void __launch_bounds__(SMP_THREADS) k_smp_rows(SmpDev P, PartIn lg, int V, float *__restrict__ adj, const SpecCtl *__restrict__ ctl, Streams sg,
                                                           const int *__restrict__ t_draft, const long long *__restrict__ t_pos, const int *__restrict__ t_win,
                                                           const int *__restrict__ t_nwin, int *__restrict__ tok_out, float *__restrict__ val_out,
                                                           int *__restrict__ acc_out, unsigned int *__restrict__ err) {
  __shared__ SmpShared sh;
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x, tid = threadIdx.x;
  int draft, nwin = 0;
  unsigned long long pos;   // the position the emitted token will occupy
  if (ctl) {
    const int z = t / sg.per, tl = t - z * sg.per;
    const SpecCtl *c = (const SpecCtl *)((const char *)ctl + (size_t)z * sg.stride);
    const RowSet &rs = c->verify;
    if (tl >= rs.n) return;
    const int prow = rs.pos0 + tl;
    pos = (unsigned long long)prow + 1ull;
    draft = tl + 1 < rs.n ? rs.tok[tl + 1] : -1;
    if (P.pen_on) {
      // the tokens at positions prow + 1 - N .. prow: history up to the pass's first row, then the pass's own inputs
      const int N = P.repeat_last_n, q0 = prow + 1 - N > 0 ? prow + 1 - N : 0;
      nwin = prow + 1 - q0;
      for (int a = tid; a < nwin; a += SMP_THREADS) { const int q = q0 + a; sh.win[a] = q <= rs.pos0 ? (q == rs.pos0 ? rs.tok[0] : (c->hist ? c->hist[q] : -1)) : rs.tok[q - rs.pos0]; }
    }
  } else {
    draft = t_draft[t]; pos = (unsigned long long)t_pos[t];
    if (P.pen_on) { nwin = t_nwin[t]; for (int a = tid; a < nwin; a += SMP_THREADS) sh.win[a] = t_win[(size_t)t * SMP_MAX_WIN + a]; }
  }
  float *row = adj + (size_t)t * V;
  const size_t l0 = (size_t)t * V;
  // ---- bias, then penalties -------------------------------------------------------------------------------------
  for (int i = tid; i < V; i += SMP_THREADS) {
    float v = part_get(lg, l0 + i);
    for (int j = 0; j < P.n_bias; j++) if (P.bias_ids[j] == i) v = __fadd_rn(v, P.bias_vals[j]);
    row[i] = v;
  }
  __syncthreads();
  if (P.pen_on && tid < nwin) {
    const int tk = sh.win[tid];
    if (tk >= 0 && tk < V) {
      bool first = true;
      int cnt = 0;
      for (int b = 0; b < nwin; b++) { if (sh.win[b] == tk) { cnt++; if (b < tid) first = false; } }
      if (first) {   // once per distinct token of the window
        float x = row[tk];
        x = x <= 0.0f ? __fmul_rn(x, P.repeat_penalty) : __fdiv_rn(x, P.repeat_penalty);
        x = __fsub_rn(x, __fadd_rn(__fmul_rn((float)cnt, P.frequency), P.presence));
        row[tk] = x;
      }
    }
  }
  __syncthreads();
  int tok = 0, accepted = 0;
  // ---- the block-wide first maximum (greedy; also the top of every other path) -------------------------------------
  float bv = -INFINITY;
  int bi = -1;
  for (int i = tid; i < V; i += SMP_THREADS) { const float v = row[i]; if (bi < 0 || v > bv) { bv = v; bi = i; } }
  smp_block_best(bv, bi, sh);
  const float top_v = bv;
  const int top_i = bi;
  if (P.temp <= 0.0f) {
    tok = top_i; accepted = draft >= 0 && tok == draft;
  } else if (P.top_k > 0) {
    // ---- the k largest, then the sorted list through top_p, min_p, temperature and the draw, sequentially ----------
    const int K = P.top_k < V ? P.top_k : V;
    float lv = top_v;
    int li = top_i;
    if (tid == 0) { sh.cv[0] = lv; sh.ci[0] = li; }
    for (int r = 1; r < K; r++) {
      float v = -INFINITY;
      int i = -1;
      for (int a = tid; a < V; a += SMP_THREADS) {
        const float x = row[a];
        if (smp_before(lv, li, x, a) && (i < 0 || smp_before(x, a, v, i))) { v = x; i = a; }   // strictly after the last pick
      }
      smp_block_best(v, i, sh);
      lv = v; li = i;
      if (tid == 0) { sh.cv[r] = v; sh.ci[r] = i; }
    }
    __syncthreads();
    if (tid == 0) {
      int n = K;
      float *l = sh.cv, *p = sh.cp;
      const int *id = sh.ci;
      if (P.top_p < 1.0f) {                                  // llama's top_p over a sorted list: float softmax, float running sum
        const float mx = l[0];
        float sum = 0.0f;
        for (int i = 0; i < n; i++) sum = __fadd_rn(sum, smp_expf(__fsub_rn(l[i], mx)));
        float cum = 0.0f;
        int last = n;
        for (int i = 0; i < n; i++) {
          cum = __fadd_rn(cum, __fdiv_rn(smp_expf(__fsub_rn(l[i], mx)), sum));
          if (cum >= P.top_p && i + 1 >= P.min_keep) { last = i + 1; break; }
        }
        n = last;
      }
      if (P.min_p > 0.0f && n > 0) {                          // sorted min_p
        const float floor_l = __fadd_rn(l[0], P.log_min_p);
        int i = 1;
        for (; i < n; i++) if (l[i] < floor_l && i >= P.min_keep) break;
        n = i;
      }
      if (P.temp != 1.0f) for (int i = 0; i < n; i++) l[i] = __fdiv_rn(l[i], P.temp);
      const float mx = l[0];
      double sum = 0.0;
      for (int i = 0; i < n; i++) { const float e = smp_expf(__fsub_rn(l[i], mx)); p[i] = e; sum += (double)e; }
      if (draft < 0) {                                        // a plain draw: walk the unnormalised p against sum * u
        int sel = -1;
        if (n == 1) sel = 0;
        else {
          const double tgt = sum * smp_draw(P.seed, pos, 0);
          double run = 0.0;
          for (int i = 0; i < n && sel < 0; i++) { run += (double)p[i]; if (run >= tgt) sel = i; }
          if (sel < 0) sel = n - 1;
        }
        tok = id[sel];
      } else {
        double pd = 0.0;
        for (int i = 0; i < n; i++) if (id[i] == draft) pd = (double)p[i] / sum;
        if (smp_draw(P.seed, pos, 1) < pd) { tok = draft; accepted = 1; }
        else {
          double rs = 0.0;
          for (int i = 0; i < n; i++) {
            const double pi = (double)p[i] / sum, qi = id[i] == draft ? 1.0 : 0.0, r = pi > qi ? pi - qi : 0.0;
            p[i] = (float)r;
            rs += r;
          }
          const double u2 = smp_draw(P.seed, pos, 2);
          int sel = -1, last = -1;
          if (!(rs > 0.0)) {                                  // p == q exactly: the reference falls back to a draw from p
            const float mx2 = l[0];
            double s2 = 0.0;
            for (int i = 0; i < n; i++) { p[i] = smp_expf(__fsub_rn(l[i], mx2)); s2 += (double)p[i]; }
            const double tgt = s2 * u2;
            double run = 0.0;
            for (int i = 0; i < n && sel < 0; i++) { run += (double)p[i]; if (run >= tgt) sel = i; }
            if (sel < 0) sel = n - 1;
          } else {
            const double tgt = rs * u2;
            double run = 0.0;
            for (int i = 0; i < n && sel < 0; i++) {
              if (p[i] <= 0.0f) continue;
              last = i;
              run += (double)p[i];
              if (run >= tgt) sel = i;
            }
            if (sel < 0) sel = last;
          }
          tok = id[sel];
        }
      }
      sh.bi = tok; sh.hit_hi = accepted;
    }
    __syncthreads();
    tok = sh.bi; accepted = sh.hit_hi;
  } else {
    // ---- the whole vocabulary in id order: min_p as a mask, sums and walks as block-wide reductions ----------------
    const float floor_l = P.min_p > 0.0f ? __fadd_rn(top_v, P.log_min_p) : -INFINITY;
    const float T = P.temp, mx = T != 1.0f ? __fdiv_rn(top_v, T) : top_v;
    auto e_of = [&](int i) -> float {
      const float v = row[i];
      if (!(v >= floor_l)) return 0.0f;
      return smp_expf(__fsub_rn(T != 1.0f ? __fdiv_rn(v, T) : v, mx));
    };
    double part = 0.0;
    int kept = 0;
    {
      const int per = (V + SMP_THREADS - 1) / SMP_THREADS, i0 = tid * per, i1 = min(V, i0 + per);
      for (int i = i0; i < i1; i++) { const float e = e_of(i); part += (double)e; kept += row[i] >= floor_l; }
    }
    const double sum = smp_block_sum(part, sh);
    if (P.min_p > 0.0f && P.min_keep > 1) {
      const int w = (int)(smp_block_sum((double)kept, sh) + 0.5);
      if (w < P.min_keep && tid == 0) atomicExch(err, 2u);   // the reference sorts and keeps min_keep here: not built
    }
    if (draft < 0) {
      tok = smp_walk_all(V, sum * smp_draw(P.seed, pos, 0), e_of, sh);
    } else {
      const double pd = (draft >= 0 && draft < V) ? (double)e_of(draft) / sum : 0.0;
      if (smp_draw(P.seed, pos, 1) < pd) { tok = draft; accepted = 1; }
      else {
        auto r_of = [&](int i) -> float {
          if (i == draft) return 0.0f;                        // max(0, p - 1)
          return (float)((double)e_of(i) / sum);
        };
        double rpart = 0.0;
        {
          const int per = (V + SMP_THREADS - 1) / SMP_THREADS, i0 = tid * per, i1 = min(V, i0 + per);
          for (int i = i0; i < i1; i++) if (i != draft) rpart += (double)e_of(i) / sum;
        }
        const double rs = smp_block_sum(rpart, sh);
        const double u2 = smp_draw(P.seed, pos, 2);
        if (!(rs > 0.0)) tok = smp_walk_all(V, sum * u2, e_of, sh);
        else tok = smp_walk_all(V, rs * u2, r_of, sh);
      }
    }
  }
  if (tid == 0) {
    if (tok < 0 || tok >= V) { tok = top_i; atomicExch(err, 3u); }
    tok_out[t] = tok;
    val_out[t] = part_get(lg, l0 + tok);   // the raw logit of the emitted token (host/llb_host.c:1455-1456)
    if (acc_out) acc_out[t] = accepted;
  }
}

int op_smp_rows(cudaStream_t s, const SmpDev &P, PartIn lg, int V, float *adj, const SpecCtl *ctl, int rows, const int *t_draft, const long long *t_pos,
                const int *t_win, const int *t_nwin, int *tok_out, float *val_out, int *acc_out, unsigned int *err) {
  CU_OK(llb_launch(k_smp_rows, dim3(rows), dim3(SMP_THREADS), (size_t)0, s, P, lg, V, adj, ctl, ops_streams(), t_draft, t_pos, t_win, t_nwin, tok_out, val_out,
                   acc_out, err));
  return 0;
}

// host side: the parameters as the kernel takes them; -1 (and a message) for what has no device path
int smp_prepare(const llb_smp_params *p, SmpDev *d, bool *argmax_only) {
  memset(d, 0, sizeof *d);
  if (p->n_bias < 0 || p->n_bias > SMP_MAX_BIAS) return llb_fail("sampler: %d logit biases (at most %d)", p->n_bias, SMP_MAX_BIAS);
  const bool pen_on = !(p->repeat_last_n <= 0 || (p->repeat_penalty == 1.0f && p->frequency == 0.0f && p->presence == 0.0f));
  *argmax_only = p->temp <= 0.0f && p->n_bias == 0 && !pen_on;   // llb_smp_is_argmax (host/llb_sampler_impl.h:81-83)
  if (pen_on && p->repeat_last_n > SMP_MAX_WIN) return llb_fail("sampler: a penalty window of %d tokens (at most %d)", p->repeat_last_n, SMP_MAX_WIN);
  if (p->temp > 0.0f) {
    if (p->top_k > SMP_MAX_TOPK) return llb_fail("sampler: top_k %d (at most %d on the device)", p->top_k, SMP_MAX_TOPK);
    if (p->top_p < 1.0f && p->top_k <= 0) return llb_fail("sampler: top_p < 1 needs top_k in 1..%d (the reference's float sum over the whole vocabulary in id order has no device path)", SMP_MAX_TOPK);
  }
  d->temp = p->temp; d->top_p = p->top_p; d->min_p = p->min_p; d->top_k = p->top_k; d->repeat_penalty = p->repeat_penalty;
  d->repeat_last_n = p->repeat_last_n; d->presence = p->presence; d->frequency = p->frequency; d->seed = p->seed; d->min_keep = p->min_keep;
  d->pen_on = pen_on ? 1 : 0;
  d->log_min_p = p->min_p > 0.0f ? logf(p->min_p) : 0.0f;   // the host's logf, as the reference takes it
  d->n_bias = p->n_bias;
  for (int j = 0; j < p->n_bias; j++) { d->bias_ids[j] = p->bias_ids[j]; d->bias_vals[j] = p->bias_vals[j]; }
  return 0;
}
