/* engine_main.c -- llb-engine-b200: the engine process the reference's CLI and server spawn, on libllb_b200.so.
 *
 * Speaks the protocol of the reference engines (tools/qwen35_engine.c:15-17 and :975-1013 for the CPU engine,
 * engine_qwen35_gpu.bend:13-24 for the GPU one; the command `llb run --spec` builds is
 * tools/llb/golden/dryrun-27b-fast-spec.txt):
 *
 *   llb-engine-b200 [--gpu SIZE] [--threads N] [--] PACKDIR id... [--steps N] [--layers L]
 *   env   LLB_SPEC=k     drafts per cycle, 0..7 (host/llb_host.c:1474; unset: plain greedy decoding)
 *         LLB_MTP=FILE   the MTP drafter as an AUX1 / MTP1 image (host/llb_host.c:1525-1603); with LLB_SPEC set and
 *                        LLB_MTP unset the cycle drafts by prompt lookup (host/llb_host.c:1936)
 *         LLB_GGUF=FILE  read the model from a GGUF instead of PACKDIR/pack.bin + index.tsv (host/llb_gguf.c:854-865)
 *         LLB_DEVICE=n   CUDA device ordinal (default 0)
 *         LLB_SAMPLE=SPEC  sampler parameters "key=val,key=val" (llb_smp_parse, host/llb_sampler_impl.h:26-75): temp top_p
 *                        top_k min_p repeat_penalty repeat_last_n presence frequency seed min_keep bias=ID:VAL;ID:VAL
 *                        preset=greedy|qwen_thinking|qwen_non_thinking; the verify step then follows llb_smp_verify on
 *                        the device (llb_spec_set_sampler).  --temp / --top-p / --seed set the same fields
 *   stdout  one generated id per line, then `wall_ms <ms>` and `tok_s <x>`
 *   stderr  `logits <pos> <id1> <bits1> <id2> <bits2>` for the row at <pos> (top-2 logits as raw f32 bits),
 *           `step <pos> <ms>` per generated token, and with LLB_SPEC the summary
 *           `spec: mtp|lookup k K cycles C rows R served S (x a cycle); accepted/drafted by position: a1/d1 ...`
 *           (host/llb_host.c:1513-1523)
 *
 * Every token goes through llb_spec_pass(pos, tok) -> [v1, id1, v2, id2], the reference's per-token operator
 * (spec_pass, host/llb_host.c:1902-1950): rows of a running cycle are served from its record, a new cycle starts where
 * the stream leaves the last one.  With sampling the row's id is the sampled token, which the caller feeds back.
 */
#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include "../../include/llb_b200.h"

static double now_ms(void) {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1000.0 + ts.tv_nsec / 1.0e6;
}

/* maps a whole file read-only; NULL (and a message) on failure */
static void *map_file(const char *path, size_t *size) {
  int fd = open(path, O_RDONLY);
  if (fd < 0) { perror(path); return NULL; }
  struct stat st;
  if (fstat(fd, &st) || st.st_size <= 0) { fprintf(stderr, "%s: cannot stat or empty\n", path); close(fd); return NULL; }
  void *p = mmap(NULL, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
  close(fd);
  if (p == MAP_FAILED) { perror("mmap"); return NULL; }
  *size = (size_t)st.st_size;
  return p;
}

static void usage(const char *p) {
  fprintf(stderr,
          "usage: %s [--gpu SIZE] [--threads N] [--] PACKDIR id... [--steps N] [--layers L]\n"
          "  env LLB_SPEC=k (0..7 drafts a cycle), LLB_MTP=FILE (AUX1 / MTP1 drafter image), LLB_GGUF=FILE, LLB_DEVICE=n,\n"
          "      LLB_SAMPLE=\"temp=0.7,top_k=20,top_p=0.8,seed=1\" (also --temp --top-p --top-k --seed)\n"
          "  stdout: ids, wall_ms, tok_s;  stderr: logits / step lines and the spec: summary\n", p);
}

static unsigned bits_of(float f) { unsigned u; memcpy(&u, &f, 4); return u; }

static void smp_defaults(llb_smp_params *p) {   /* llb_smp_defaults (host/llb_sampler_impl.h:15-18) */
  memset(p, 0, sizeof *p);
  p->top_p = 1.0f; p->repeat_penalty = 1.0f; p->repeat_last_n = 64;
}
/* "key=val,key=val" into p; 0, or -1 with a message on stderr */
static int smp_parse(llb_smp_params *p, const char *spec) {
  char buf[1024];
  if (!spec) return 0;
  if (strlen(spec) >= sizeof buf) { fprintf(stderr, "LLB_SAMPLE: too long\n"); return -1; }
  strcpy(buf, spec);
  for (char *tok = strtok(buf, ","); tok; tok = strtok(NULL, ",")) {
    char *eq = strchr(tok, '=');
    if (!eq) { fprintf(stderr, "LLB_SAMPLE: '%s' is not key=value\n", tok); return -1; }
    *eq = 0;
    const char *k = tok, *v = eq + 1;
    if (!strcmp(k, "temp")) p->temp = strtof(v, NULL);
    else if (!strcmp(k, "top_p")) p->top_p = strtof(v, NULL);
    else if (!strcmp(k, "top_k")) p->top_k = atoi(v);
    else if (!strcmp(k, "min_p")) p->min_p = strtof(v, NULL);
    else if (!strcmp(k, "repeat_penalty")) p->repeat_penalty = strtof(v, NULL);
    else if (!strcmp(k, "repeat_last_n")) p->repeat_last_n = atoi(v);
    else if (!strcmp(k, "presence")) p->presence = strtof(v, NULL);
    else if (!strcmp(k, "frequency")) p->frequency = strtof(v, NULL);
    else if (!strcmp(k, "seed")) p->seed = strtoull(v, NULL, 10);
    else if (!strcmp(k, "min_keep")) p->min_keep = atoi(v);
    else if (!strcmp(k, "max_tokens")) continue;             /* a policy field of the caller */
    else if (!strcmp(k, "preset")) {
      if (!strcmp(v, "greedy")) smp_defaults(p);
      else if (!strcmp(v, "qwen_thinking")) { p->temp = 1.0f; p->top_p = 0.95f; p->top_k = 20; p->presence = 1.5f; }
      else if (!strcmp(v, "qwen_non_thinking")) { p->temp = 0.7f; p->top_p = 0.8f; p->top_k = 20; p->presence = 1.5f; }
      else { fprintf(stderr, "LLB_SAMPLE: unknown preset '%s'\n", v); return -1; }
    } else if (!strcmp(k, "bias")) {
      for (const char *b = v; *b;) {
        char *end;
        const long id = strtol(b, &end, 10);
        if (*end != ':' || p->n_bias >= 64) { fprintf(stderr, "LLB_SAMPLE: bias wants ID:VAL;ID:VAL, at most 64\n"); return -1; }
        p->bias_ids[p->n_bias] = (int)id;
        p->bias_vals[p->n_bias++] = strtof(end + 1, &end);
        b = *end == ';' ? end + 1 : end;
        if (*end && *end != ';') { fprintf(stderr, "LLB_SAMPLE: bias wants ID:VAL;ID:VAL\n"); return -1; }
      }
    } else { fprintf(stderr, "LLB_SAMPLE: no key '%s' on this path\n", k); return -1; }
  }
  return 0;
}

int main(int argc, char **argv) {
  const char *dir = NULL;
  static int ids[1 << 20];
  int nids = 0, steps = 8, layers = 0;
  llb_smp_params smp;
  smp_defaults(&smp);
  if (smp_parse(&smp, getenv("LLB_SAMPLE"))) return 2;
  for (int a = 1; a < argc; a++) {
    if (!strcmp(argv[a], "--steps") && a + 1 < argc) steps = atoi(argv[++a]);
    else if (!strcmp(argv[a], "--layers") && a + 1 < argc) layers = atoi(argv[++a]);
    else if ((!strcmp(argv[a], "--gpu") || !strcmp(argv[a], "--threads")) && a + 1 < argc) a++;   /* the launcher's memory / thread hints */
    else if (!strcmp(argv[a], "--")) continue;
    else if (!strcmp(argv[a], "--ids") || !strcmp(argv[a], "--cpu") || !strcmp(argv[a], "--preload")) continue;
    else if (!strcmp(argv[a], "--temp") && a + 1 < argc) smp.temp = strtof(argv[++a], NULL);
    else if (!strcmp(argv[a], "--top-p") && a + 1 < argc) smp.top_p = strtof(argv[++a], NULL);
    else if (!strcmp(argv[a], "--top-k") && a + 1 < argc) smp.top_k = atoi(argv[++a]);
    else if (!strcmp(argv[a], "--seed") && a + 1 < argc) smp.seed = strtoull(argv[++a], NULL, 10);
    else if (argv[a][0] == '-' && argv[a][1] == '-') { fprintf(stderr, "unknown option %s\n", argv[a]); usage(argv[0]); return 2; }
    else if (!dir) dir = argv[a];
    else if (nids < (int)(sizeof ids / sizeof *ids)) ids[nids++] = atoi(argv[a]);
  }
  if (!dir || nids < 1 || steps < 1) { usage(argv[0]); return 2; }
  const char *e_spec = getenv("LLB_SPEC"), *e_mtp = getenv("LLB_MTP"), *e_gguf = getenv("LLB_GGUF"), *e_dev = getenv("LLB_DEVICE");
  const int k = e_spec ? atoi(e_spec) : 0;
  if (k < 0 || k > 7) { fprintf(stderr, "LLB_SPEC=%d: 0..7\n", k); return 2; }
  if (e_mtp && !e_spec) { fprintf(stderr, "LLB_MTP needs LLB_SPEC\n"); return 2; }

  if (llb_b200_init(e_dev ? atoi(e_dev) : 0)) { fprintf(stderr, "llb-engine-b200: %s\n", llb_b200_last_error()); return 1; }
  size_t n_mtp = 0;
  void *mtp = e_mtp && k > 0 ? map_file(e_mtp, &n_mtp) : NULL;
  if (e_mtp && k > 0 && !mtp) return 1;
  const int max_ctx = nids + steps + 16 + 2 * (k + 1);
  llb_spec *m = NULL;
  if (e_gguf) {
    m = llb_spec_open_gguf(e_gguf, mtp, n_mtp, 0, k, max_ctx, layers);
  } else {
    char path[4096];
    size_t n_idx = 0, n_pack = 0;
    snprintf(path, sizeof path, "%s/index.tsv", dir);
    char *idx_map = (char *)map_file(path, &n_idx);
    if (!idx_map) return 1;
    char *idx = (char *)malloc(n_idx + 1);
    memcpy(idx, idx_map, n_idx);
    idx[n_idx] = 0;
    snprintf(path, sizeof path, "%s/pack.bin", dir);
    void *pack = map_file(path, &n_pack);
    if (!pack) return 1;
    m = llb_spec_open(idx, pack, n_pack, 0, mtp, n_mtp, 0, k, max_ctx, layers);
    munmap(pack, n_pack);   /* every tensor now lives on the device */
    free(idx);
  }
  if (!m) { fprintf(stderr, "llb-engine-b200: %s\n", llb_b200_last_error()); return 1; }

  if (llb_spec_set_sampler(m, &smp)) { fprintf(stderr, "llb-engine-b200: %s\n", llb_b200_last_error()); return 1; }
  const double t0 = now_ms();
  float y[4];
  if (llb_spec_prefill(m, ids, nids) || llb_spec_pass(m, nids - 1, ids[nids - 1], y)) {
    fprintf(stderr, "llb-engine-b200: %s\n", llb_b200_last_error());
    return 1;
  }
  fprintf(stderr, "logits %d %d %u %d %u\n", nids - 1, (int)y[1], bits_of(y[0]), (int)y[3], bits_of(y[2]));
  int cur = (int)y[1], gen = 0;
  for (int s = 0; s < steps; s++) {
    printf("%d\n", cur);
    gen++;
    if (s + 1 >= steps) break;
    const double s0 = now_ms();
    if (llb_spec_pass(m, nids + s, cur, y)) { fprintf(stderr, "llb-engine-b200: %s\n", llb_b200_last_error()); return 1; }
    fprintf(stderr, "logits %d %d %u %d %u\n", nids + s, (int)y[1], bits_of(y[0]), (int)y[3], bits_of(y[2]));
    fprintf(stderr, "step %d %llu\n", nids + s, (unsigned long long)(now_ms() - s0));
    cur = (int)y[1];
  }
  const double t1 = now_ms();
  printf("wall_ms %llu\n", (unsigned long long)(t1 - t0));
  printf("tok_s %.4f\n", gen > 0 && t1 > t0 ? gen * 1000.0 / (t1 - t0) : 0.0);
  if (e_spec) {
    unsigned long long st[19];
    llb_spec_stats(m, st);
    fprintf(stderr, "spec: %s k %d cycles %llu rows %llu served %llu (%.3f a cycle); accepted/drafted by position:", mtp ? "mtp" : "lookup", k, st[0],
            st[1], st[2], st[0] ? (double)st[2] / (double)st[0] : 0.0);
    for (int j = 1; j <= k; j++) fprintf(stderr, " %llu/%llu", st[11 + j], st[3 + j]);
    fprintf(stderr, "\n");
  }
  llb_spec_close(m);
  return 0;
}
