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
 *   stdout  one generated id per line, then `wall_ms <ms>` and `tok_s <x>`
 *   stderr  `logits <pos> <id1> <bits1> <id2> <bits2>` for the row at <pos> (top-2 logits as raw f32 bits),
 *           `step <pos> <ms>` per generated token, and with LLB_SPEC the summary
 *           `spec: mtp|lookup k K cycles C rows R served S (x a cycle); accepted/drafted by position: a1/d1 ...`
 *           (host/llb_host.c:1513-1523)
 *
 * Every token goes through llb_spec_pass(pos, tok) -> [v1, id1, v2, id2], the reference's per-token operator
 * (spec_pass, host/llb_host.c:1902-1950): rows of a running cycle are served from its record, a new cycle starts where
 * the stream leaves the last one.  Sampling options of the reference CLI (--temp, --top-p) are refused: acceptance is
 * committed on the device under the greedy rule.
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
          "  env LLB_SPEC=k (0..7 drafts a cycle), LLB_MTP=FILE (AUX1 / MTP1 drafter image), LLB_GGUF=FILE, LLB_DEVICE=n\n"
          "  stdout: ids, wall_ms, tok_s;  stderr: logits / step lines and the spec: summary\n", p);
}

static unsigned bits_of(float f) { unsigned u; memcpy(&u, &f, 4); return u; }

int main(int argc, char **argv) {
  const char *dir = NULL;
  static int ids[1 << 20];
  int nids = 0, steps = 8, layers = 0;
  for (int a = 1; a < argc; a++) {
    if (!strcmp(argv[a], "--steps") && a + 1 < argc) steps = atoi(argv[++a]);
    else if (!strcmp(argv[a], "--layers") && a + 1 < argc) layers = atoi(argv[++a]);
    else if ((!strcmp(argv[a], "--gpu") || !strcmp(argv[a], "--threads")) && a + 1 < argc) a++;   /* the launcher's memory / thread hints */
    else if (!strcmp(argv[a], "--")) continue;
    else if (!strcmp(argv[a], "--ids") || !strcmp(argv[a], "--cpu") || !strcmp(argv[a], "--preload")) continue;
    else if (!strcmp(argv[a], "--temp") || !strcmp(argv[a], "--top-p") || !strcmp(argv[a], "--seed")) {
      fprintf(stderr, "%s: sampling is not available on this path (greedy acceptance is committed on the device)\n", argv[a]);
      return 2;
    }
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
