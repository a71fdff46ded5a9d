/* oracle/ref_harness.c -- TEST INFRASTRUCTURE, not product code.
 *
 * Wraps the UNMODIFIED reference CPU engine (tools/qwen35_engine.c of
 * phenomenon0/eureka-engine) by including it where it lies, the way the
 * reference's own backends/windows/engine_cpu.c:41-44 does (#define main ... /
 * #include the engine).  No reference source is copied: the include path is
 * given on the compiler command line (-DREF_ENGINE_C=...), and everything this
 * file builds goes to oracle/_ref/.
 *
 * Two products from the same translation unit:
 *   oracle/_ref/qwen35_ref         the reference CLI (argv / stdout / stderr protocol
 *                                  of tools/qwen35_engine.c:15-17)
 *   oracle/_ref/libq35ref.so       the same code behind a few C entry points, so a test
 *                                  can step the reference token by token and read its
 *                                  logits, residual and layer state.
 *
 * Threads: the reference's sanctioned LLB_GEMV_ROWS hook (tools/qwen35_engine.c:481-486)
 * is filled with an OpenMP row split.  Every row is still one dot_fmt call over the same
 * bytes, so results are bit-identical to the serial loop (same argument as
 * backends/android/engine/patches/01-omp-rows.patch).
 */
#include <stdint.h>
#include <stddef.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int orh_gemv_rows(int fmt, const uint8_t *W, int rb, int rows, int cols, const float *x, float *y);
#define LLB_GEMV_ROWS orh_gemv_rows
#define main q35ref_cli_main
#include REF_ENGINE_C
#undef main

static int orh_threads = 0; /* 0: OpenMP default */

static int orh_gemv_rows(int fmt, const uint8_t *W, int rb, int rows, int cols, const float *x, float *y) {
  int r;
#ifdef _OPENMP
  int nt = orh_threads > 0 ? orh_threads : omp_get_max_threads();
  if (rows < 64) nt = 1;
#pragma omp parallel for schedule(static) num_threads(nt)
#endif
  for (r = 0; r < rows; r++) y[r] = dot_fmt(fmt, W + (size_t)r * rb, cols, x);
  return 1;
}

#ifdef Q35REF_CLI
int main(int argc, char **argv) {
  const char *t = getenv("Q35REF_THREADS");
  if (t) orh_threads = atoi(t);
  return q35ref_cli_main(argc, argv);
}
#else

#define API __attribute__((visibility("default")))

API void q35ref_threads(int n) { orh_threads = n; }

/* Load index.tsv + pack.bin of `dir` into RAM and allocate state for `cap` positions.
 * layers > 0 truncates the model like the CLI's --layers.  Returns 0 on success. */
API int q35ref_open(const char *dir, int layers, int cap) {
  char path[4096];
  FILE *f;
  long sz;
  uint8_t *buf;
  gNT = 0;
  load_index(dir);
  if (layers > 0 && layers < L) L = layers;
  snprintf(path, sizeof path, "%s/pack.bin", dir);
  f = fopen(path, "rb");
  if (!f) return 1;
  fseek(f, 0, SEEK_END);
  sz = ftell(f);
  fseek(f, 0, SEEK_SET);
  buf = (uint8_t *)malloc((size_t)sz);
  if (!buf || fread(buf, 1, (size_t)sz, f) != (size_t)sz) { fclose(f); return 2; }
  fclose(f);
  gPack = buf;
  gMapSz = 0;
  state_alloc(cap);
  buf_alloc();
  return 0;
}

/* The same with the pack bytes already in memory (borrowed): only index.tsv is read from `dir`. */
API int q35ref_open_mem(const char *dir, const uint8_t *pack, int layers, int cap) {
  gNT = 0;
  load_index(dir);
  if (layers > 0 && layers < L) L = layers;
  gPack = pack;
  gMapSz = 0;
  state_alloc(cap);
  buf_alloc();
  return 0;
}

/* cfg[0..18] = L D H KV HDIM dff V INTERVAL KC SZ GK TR VHD KDC VDC CONVD ROPEDIM, then
 * ROPE_BASE and EPS as float bits. */
API void q35ref_cfg(int *cfg) {
  int v[17] = {L, D, H, KV, HDIM, dff, V, INTERVAL, KC, SZ, GK, TR, VHD, KDC, VDC, CONVD, ROPEDIM};
  memcpy(cfg, v, sizeof v);
  memcpy(cfg + 17, &ROPE_BASE, 4);
  memcpy(cfg + 18, &EPS, 4);
}

API void q35ref_forward(int tok, int pos) { forward_token(tok, pos); }
/* runs output_norm + head on the current residual; returns the V logits */
API const float *q35ref_logits(void) { final_logits(); return LOGITS; }
API const float *q35ref_x(void) { return X; }            /* residual after the last layer   */
API const float *q35ref_hnorm(void) { return HH; }       /* output-normed hidden (after q35ref_logits) */
API void q35ref_top2(int *ids, float *vals) { top2(&ids[0], &vals[0], &ids[1], &vals[1]); }
API const float *q35ref_state_S(int il) { return gS + (size_t)il * TR * SZ * SZ; }
API const float *q35ref_state_conv(int il) { return gConv + (size_t)il * (KC - 1) * CONVD; }
API const float *q35ref_state_k(int il, int pos) { return gK + ((size_t)il * gCap + pos) * KV * HDIM; }
API const float *q35ref_state_v(int il, int pos) { return gV + ((size_t)il * gCap + pos) * KV * HDIM; }
API void q35ref_reset(void) {
  memset(gS, 0, (size_t)L * TR * SZ * SZ * 4);
  memset(gConv, 0, (size_t)L * (KC - 1) * CONVD * 4);
}

/* format leaves, for pinning a restatement or a device kernel against the reference */
API void q35ref_deq_row(int fmt, const uint8_t *row, int cols, float *out) { deq_row(fmt, row, cols, out); }
API float q35ref_dot(int fmt, const uint8_t *row, int cols, const float *x) { return dot_fmt(fmt, row, cols, x); }
API void q35ref_gemv(int fmt, const uint8_t *W, int rb, int rows, int cols, const float *x, float *y) {
  orh_gemv_rows(fmt, W, rb, rows, cols, x, y);
}
API float q35ref_half(uint16_t h) { return half_to_float(h); }
API float q35ref_silu(float x) { return hf_silu(x); }
API float q35ref_sigmoid(float x) { return hf_sigmoid(x); }
API float q35ref_softplus(float x) { return hf_softplus(x); }
#endif
