// api.cu -- the C ABI of include/llb_b200.h: backend primitives and operator entry points.
#include "../../include/llb_b200.h"
#include <stdlib.h>

#include "host.cuh"
#include "pf.cuh"
#include "tp.cuh"
#include "sampler.cuh"

LlbCtx g_llb;

struct llb_xp {
  XPlanes p;
  int T, planes;
  void *base;
};

// K-slice partial sums of the operator entry points (the engine owns its own scratch)
static float *g_parts = nullptr;
static size_t g_parts_floats = 0;

extern "C" {

int llb_b200_init(int device) {
  if (g_llb.stream) {
    // one device and one stream per process: the stream, the kernels' attributes and the library's own device words
    // belong to the first device; a second binding would leave them pointing into another GPU's memory
    if (g_llb.device == device) return 0;
    return llb_fail("llb_b200_init(%d): this process is already bound to device %d", device, g_llb.device);
  }
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess || n < 1) return llb_fail("no CUDA device: %s", cudaGetErrorString(e));
  if (device < 0 || device >= n) return llb_fail("device %d out of range (%d visible)", device, n);
  CU_OK(cudaSetDevice(device));
  cudaDeviceProp pr;
  CU_OK(cudaGetDeviceProperties(&pr, device));
  if (pr.major < 10) return llb_fail("device %d is sm_%d%d; this library is built for sm_100a only", device, pr.major, pr.minor);
  { const char *e = getenv("LLB_PDL"); g_llb.pdl = !(e && e[0] == '0'); }
  { const char *e = getenv("LLB_GEMM3"); g_llb.gemm3 = e && e[0] == '1'; }
  { const char *e = getenv("LLB_FFN_FUSED"); g_llb.ffn_fused = e && e[0] == '1'; }
  g_llb.sms = pr.multiProcessorCount;
  // a blocking stream: ordered after work a caller queued on the legacy default stream (torch's), so
  // device buffers produced there can be handed in without an explicit synchronisation
  cudaStream_t st = nullptr;
  CU_OK(cudaStreamCreate(&st));
  g_llb.device = device; g_llb.stream = st;
  if (gemm_setup()) { cudaStreamDestroy(st); g_llb.stream = nullptr; g_llb.device = -1; return -1; }
  return 0;
}
const char *llb_b200_last_error(void) { return g_llb.err; }
int llb_b200_sm_count(void) { return g_llb.sms; }

#define NEED_INIT(ret) \
  if (!g_llb.stream) { llb_fail("llb_b200_init has not been called"); return ret; }

llb_b200_dptr llb_b200_alloc_zero(size_t bytes) {
  NEED_INIT(0)
  if (backend_graph_bail()) return 0;
  void *p = nullptr;
  if (cudaMalloc(&p, bytes ? bytes : 4) != cudaSuccess) { llb_fail("cudaMalloc(%zu) failed", bytes); cudaGetLastError(); return 0; }
  if (cudaMemsetAsync(p, 0, bytes, g_llb.stream) != cudaSuccess) { cudaFree(p); llb_fail("memset failed"); return 0; }
  return (llb_b200_dptr)(uintptr_t)p;
}
int llb_b200_free(llb_b200_dptr p) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  CU_OK(cudaFree((void *)(uintptr_t)p));
  return 0;
}
int llb_b200_zero(llb_b200_dptr p, size_t bytes) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  CU_OK(cudaMemsetAsync((void *)(uintptr_t)p, 0, bytes, g_llb.stream));
  return 0;
}
int llb_b200_copy(llb_b200_dptr d, llb_b200_dptr s, size_t bytes) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  CU_OK(cudaMemcpyAsync((void *)(uintptr_t)d, (const void *)(uintptr_t)s, bytes, cudaMemcpyDeviceToDevice, g_llb.stream));
  return 0;
}
int llb_b200_write(llb_b200_dptr d, const void *h, size_t bytes) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  CU_OK(cudaMemcpyAsync((void *)(uintptr_t)d, h, bytes, cudaMemcpyHostToDevice, g_llb.stream));
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  return 0;
}
int llb_b200_read(void *h, llb_b200_dptr p, size_t bytes) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  CU_OK(cudaMemcpyAsync(h, (const void *)(uintptr_t)p, bytes, cudaMemcpyDeviceToHost, g_llb.stream));
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  return 0;
}
int llb_b200_sync(void) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  CU_OK(cudaGetLastError());
  return 0;
}
llb_b200_dptr llb_b200_stream(void) { return (llb_b200_dptr)(uintptr_t)g_llb.stream; }

size_t llb_b200_weight_bytes(int fmt, int rows, int cols) { return (size_t)rows * dev_row_bytes(fmt, cols); }

int llb_b200_weight_upload(int fmt, int rows, int cols, const void *src, int src_on_device, llb_b200_dptr dst) {
  NEED_INIT(-1)
  const size_t pb = (size_t)rows * pack_row_bytes(fmt, cols);
  if (!pack_row_bytes(fmt, cols)) return llb_fail("weight_upload: format %d / cols %d", fmt, cols);
  if (fmt != LLB_FM_Q6_K) {
    CU_OK(cudaMemcpyAsync((void *)(uintptr_t)dst, src, pb, src_on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice,
                          g_llb.stream));
    if (!src_on_device) CU_OK(cudaStreamSynchronize(g_llb.stream));
    return 0;
  }
  const uint8_t *s = (const uint8_t *)src;
  void *tmp = nullptr;
  if (!src_on_device) {
    CU_OK(cudaMalloc(&tmp, pb));
    const cudaError_t ce = cudaMemcpyAsync(tmp, src, pb, cudaMemcpyHostToDevice, g_llb.stream);
    if (ce != cudaSuccess) { cudaFree(tmp); return llb_fail("weight_upload: copy of %zu bytes: %s", pb, cudaGetErrorString(ce)); }
    s = (const uint8_t *)tmp;
  }
  int rc = ops_repack_q6k(g_llb.stream, s, (uint8_t *)(uintptr_t)dst, (size_t)rows * (cols / 256));
  if (tmp) {
    cudaStreamSynchronize(g_llb.stream);
    cudaFree(tmp);
  }
  return rc;
}

int llb_b200_dequant(int fmt, int rows, int cols, llb_b200_dptr w, llb_b200_dptr row_ids, int nrows, llb_b200_dptr out) {
  NEED_INIT(-1)
  return ops_dequant_rows(g_llb.stream, fmt, (const uint8_t *)(uintptr_t)w, rows, cols, (const int *)(uintptr_t)row_ids, nrows,
                          (float *)(uintptr_t)out);
}

llb_xp *llb_b200_xp_new(int K, int T, int planes) {
  NEED_INIT(nullptr)
  if (K % 256 || T < 1 || (planes != 1 && planes != 2) || T * planes > 32) { llb_fail("xp_new: K %d T %d planes %d", K, T, planes); return nullptr; }
  llb_xp *x = new llb_xp();
  x->T = T; x->planes = planes;
  const int NC = T * planes <= 8 ? 8 : T * planes <= 16 ? 16 : 32;
  if (cudaMalloc(&x->base, xp_bytes(K, NC)) != cudaSuccess) { llb_fail("xp_new: out of memory"); delete x; return nullptr; }
  cudaMemsetAsync(x->base, 0, xp_bytes(K, NC), g_llb.stream);
  x->p = xp_carve(x->base, K, NC);
  return x;
}
void llb_b200_xp_free(llb_xp *xp) {
  if (!xp) return;
  cudaStreamSynchronize(g_llb.stream);
  cudaFree(xp->base);
  delete xp;
}
int llb_b200_xp_set_f32(llb_xp *xp, llb_b200_dptr x) {
  NEED_INIT(-1)
  return ops_xp_from_f32(g_llb.stream, (const float *)(uintptr_t)x, xp->T, xp->planes, xp->p);
}
int llb_b200_xp_set_bf16(llb_xp *xp, llb_b200_dptr x) {
  NEED_INIT(-1)
  if (xp->planes != 1) return llb_fail("xp_set_bf16 needs planes == 1");
  return ops_xp_from_bf16(g_llb.stream, (const void *)(uintptr_t)x, xp->T, xp->p);
}

int llb_b200_gemm(int fmt, int nmat, const llb_b200_dptr *w, const int *rows, const llb_b200_dptr *out, int K, const llb_xp *xp, int ksplit) {
  NEED_INIT(-1)
  if (nmat < 1 || nmat > GEMM_MAXMAT) return llb_fail("gemm: nmat %d", nmat);
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.nmat = nmat; a.K = K; a.xp = xp->p; a.planes = xp->planes; a.T = xp->T;
  int ntiles = 0, total_rows = 0;
  for (int i = 0; i < nmat; i++) { ntiles += (rows[i] + 15) / 16; total_rows += rows[i]; }
  a.ksplit = gemm_fix_ksplit(fmt, xp->p.NC, K / 256, ksplit > 0 ? ksplit : gemm_pick_ksplit(fmt, xp->p.NC, ntiles, K / 256, g_llb.sms));
  const size_t per_split = (size_t)xp->T * total_rows;
  if (a.ksplit > 1 && per_split * a.ksplit > g_parts_floats) {
    if (g_parts) {
      float *old = g_parts;
      g_parts = nullptr; g_parts_floats = 0;   // nothing dangles if the calls below fail
      CU_OK(cudaStreamSynchronize(g_llb.stream)); CU_OK(cudaFree(old));
    }
    float *fresh = nullptr;
    CU_OK(cudaMalloc(&fresh, per_split * GEMM_MAXSPLIT * 4));
    g_parts = fresh; g_parts_floats = per_split * GEMM_MAXSPLIT;
  }
  size_t off = 0;
  for (int i = 0; i < nmat; i++) {
    a.m[i].W = (const uint8_t *)(uintptr_t)w[i];
    a.m[i].rows = rows[i];
    a.m[i].ostride = rows[i];
    a.m[i].tok_slot = nullptr;
    if (a.ksplit == 1) { a.m[i].out = (float *)(uintptr_t)out[i]; a.m[i].split_stride = 0; }
    else { a.m[i].out = g_parts + off; a.m[i].split_stride = (long long)per_split; off += (size_t)xp->T * rows[i]; }
  }
  if (gemm_launch(g_llb.stream, fmt, a)) return -1;
  if (a.ksplit > 1)
    for (int i = 0; i < nmat; i++)
      if (ops_sum_parts(g_llb.stream, a.m[i].out, a.ksplit, a.m[i].split_stride, xp->T * rows[i], (float *)(uintptr_t)out[i])) return -1;
  return 0;
}

int llb_b200_gemm_ksplit(int fmt, int nc, int ntiles, int nsb, int sms) { return gemm_pick_ksplit(fmt, nc, ntiles, nsb, sms); }
int llb_b200_ring_ksplit(int fmt, int nsb, int ntiles, int nc_spec, int nc_prefill, int sms) {
  return gemm_ring_ksplit(fmt, nsb, ntiles, nc_spec, nc_prefill, sms, 8);
}

int llb_b200_use_tcgen05(int on) {
  NEED_INIT(-1)
  const int was = g_llb.gemm3;
  g_llb.gemm3 = on != 0;
  return was;
}
int llb_b200_use_fused_ffn(int on) {
  NEED_INIT(-1)
  const int was = g_llb.ffn_fused;
  g_llb.ffn_fused = on != 0;
  return was;
}
int llb_b200_wait_errors(void) {
  NEED_INIT(-1)
  const int a = gemm_wait_errors(), b = pf_wait_errors(), c = tp_wait_errors();
  return a < 0 || b < 0 || c < 0 ? -1 : (a | b | c);
}
int llb_b200_wait_errors_clear(void) {
  NEED_INIT(-1)
  return gemm_wait_errors_clear() || pf_wait_errors_clear() || tp_wait_errors_clear() ? -1 : 0;
}
// the device sampler on T rows of given logits (test entry; the engine runs the same kernel from its control blocks)
int llb_b200_smp_rows(const llb_smp_params *p, llb_b200_dptr logits, int T, int V, const int *drafts, const long long *pos, const int *win,
                      const int *nwin, int *tok_out, int *acc_out, float *val_out) {
  NEED_INIT(-1)
  if (!p || T < 1 || T > 64 || V < 1) return llb_fail("smp_rows: T %d, V %d", T, V);
  SmpDev d;
  bool argmax_only = false;
  if (smp_prepare(p, &d, &argmax_only)) return -1;
  if (backend_graph_bail()) return -1;
  void *buf = nullptr;
  const size_t b_adj = (size_t)T * V * 4, b_win = (size_t)T * SMP_MAX_WIN * 4, b_i = (size_t)T * 4, b_l = (size_t)T * 8;
  CU_OK(cudaMalloc(&buf, b_adj + b_win + 5 * b_i + b_l + 16));
  char *c = (char *)buf;
  float *adj = (float *)c; c += b_adj;
  long long *d_pos = (long long *)c; c += b_l;
  int *d_win = (int *)c; c += b_win;
  int *d_draft = (int *)c; c += b_i;
  int *d_nwin = (int *)c; c += b_i;
  int *d_tok = (int *)c; c += b_i;
  int *d_acc = (int *)c; c += b_i;
  float *d_val = (float *)c; c += b_i;
  unsigned int *d_err = (unsigned int *)c;
  cudaStream_t s = g_llb.stream;
  int rc = 0;
  cudaError_t e = cudaMemsetAsync(buf, 0, b_adj + b_win + 5 * b_i + b_l + 16, s);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_pos, pos, b_l, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess) e = cudaMemcpyAsync(d_draft, drafts, b_i, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess && win) e = cudaMemcpyAsync(d_win, win, b_win, cudaMemcpyHostToDevice, s);
  if (e == cudaSuccess && nwin) e = cudaMemcpyAsync(d_nwin, nwin, b_i, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) rc = llb_fail("smp_rows: %s", cudaGetErrorString(e));
  if (!rc) rc = op_smp_rows(s, d, PartIn{(const float *)(uintptr_t)logits, 1, 0}, V, adj, nullptr, T, d_draft, d_pos, d_win, d_nwin, d_tok, d_val, d_acc, d_err);
  unsigned int err = 0;
  if (!rc) {
    e = cudaMemcpyAsync(tok_out, d_tok, b_i, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(acc_out, d_acc, b_i, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(val_out, d_val, b_i, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaMemcpyAsync(&err, d_err, 4, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) rc = llb_fail("smp_rows: %s", cudaGetErrorString(e));
  }
  cudaFree(buf);
  if (!rc && err) rc = llb_fail("smp_rows: the device sampler reported %u", err);
  return rc;
}
int llb_b200_wait_selftest(int which, int limit) {
  NEED_INIT(-1)
  if (backend_graph_bail()) return -1;
  return gemm_wait_selftest(g_llb.stream, which, limit);
}

int llb_b200_gemm_host(int fmt, llb_b200_dptr w, int rows, int K, const void *x_bf16, int T, float *y, llb_xp *xp, llb_b200_dptr x_dev,
                       llb_b200_dptr y_dev) {
  NEED_INIT(-1)
  CU_OK(cudaMemcpyAsync((void *)(uintptr_t)x_dev, x_bf16, (size_t)T * K * 2, cudaMemcpyHostToDevice, g_llb.stream));
  if (llb_b200_xp_set_bf16(xp, x_dev)) return -1;
  if (llb_b200_gemm(fmt, 1, &w, &rows, &y_dev, K, xp, 0)) return -1;
  CU_OK(cudaMemcpyAsync(y, (const void *)(uintptr_t)y_dev, (size_t)T * rows * 4, cudaMemcpyDeviceToHost, g_llb.stream));
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  return 0;
}

// ---- the GEMM for hosts that may not allocate -------------------------------------------------
// Some hosts give a library its memory once, at start-up, and refuse driver allocations afterwards:
// a serving process whose other streams must never stall on cudaMalloc's device-wide synchronisation,
// or a plugin sandbox that simply denies the call.  For them the scratch this GEMM needs -- the fp16
// activation planes and the K-slice partial sums -- lives in a fixed array inside the library image.
// Every GPU that loads the library carries these 8.5 MB until the process exits.
#define NOALLOC_MAX_K 8192
#define NOALLOC_MAX_T 4
#define NOALLOC_PART_FLOATS (2u << 20)                                   /* [K-slices][T][rows] f32 */
#define NOALLOC_XP_BYTES 172032                                          /* xp_bytes(8192, 8) = 163840, plus 8 KB of slack */
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_XP_BYTES + NOALLOC_PART_FLOATS * 4];
// In host code the array's name is only a handle for the runtime; the device address is looked up
// once per device, with that device current, and kept here.
static unsigned char *g_noalloc_ptr[64];

int llb_b200_gemm_noalloc(int fmt, llb_b200_dptr w, int rows, int K, llb_b200_dptr x_f32, int T, llb_b200_dptr out_f32) {
  NEED_INIT(-1)
  if (K < 256 || K % 256 || K > NOALLOC_MAX_K) return llb_fail("gemm_noalloc: K = %d; this entry point takes multiples of 256 up to %d", K, NOALLOC_MAX_K);
  if (T < 1 || T > NOALLOC_MAX_T) return llb_fail("gemm_noalloc: T = %d; this entry point takes 1..%d rows", T, NOALLOC_MAX_T);
  if (rows < 1) return llb_fail("gemm_noalloc: rows = %d", rows);
  if (!dev_row_bytes(fmt, K) || fmt == LLB_FM_F32) return llb_fail("gemm_noalloc: format %d has no kernel", fmt);
  const int NC = 8;
  const int ks = gemm_pick_ksplit(fmt, NC, (rows + 15) / 16, K / 256, g_llb.sms);
  if ((size_t)ks * T * rows > NOALLOC_PART_FLOATS)
    return llb_fail("gemm_noalloc: %d K-slices x %d rows x %d output rows need %zu floats of scratch, the built-in array holds %u",
                    ks, T, rows, (size_t)ks * T * rows, (unsigned)NOALLOC_PART_FLOATS);
  if (xp_bytes(K, NC) > NOALLOC_XP_BYTES) return llb_fail("gemm_noalloc: planes of %d columns do not fit", K);
  // the work is queued on the library's stream, so the array of the library's device is the one to use, whatever
  // device the calling thread has current
  const int dev = g_llb.device;
  if (dev < 0 || dev >= 64) return llb_fail("gemm_noalloc: device ordinal %d", dev);
  if (!g_noalloc_ptr[dev]) {
    int cur = -1;
    CU_OK(cudaGetDevice(&cur));
    if (cur != dev) CU_OK(cudaSetDevice(dev));
    void *p = nullptr;
    const cudaError_t ce = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (cur != dev && cur >= 0) cudaSetDevice(cur);
    if (ce != cudaSuccess) return llb_fail("gemm_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(ce));
    g_noalloc_ptr[dev] = (unsigned char *)p;
  }
  unsigned char *scratch = g_noalloc_ptr[dev];
  // the array keeps the previous call's contents: the planes start from zero every time (unused
  // columns would otherwise carry stale values into the tensor-core tiles); the partial sums are
  // fully rewritten before they are read
  CU_OK(cudaMemsetAsync(scratch, 0, xp_bytes(K, NC), g_llb.stream));
  XPlanes xp = xp_carve(scratch, K, NC);
  if (ops_xp_from_f32(g_llb.stream, (const float *)(uintptr_t)x_f32, T, 2, xp)) return -1;
  float *parts = (float *)(scratch + NOALLOC_XP_BYTES);
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.nmat = 1; a.K = K; a.xp = xp; a.planes = 2; a.T = T; a.ksplit = ks;
  a.m[0].W = (const uint8_t *)(uintptr_t)w; a.m[0].rows = rows; a.m[0].ostride = rows;
  a.m[0].out = ks == 1 ? (float *)(uintptr_t)out_f32 : parts;
  a.m[0].split_stride = ks == 1 ? 0 : (long long)T * rows;
  if (gemm_launch(g_llb.stream, fmt, a)) return -1;
  if (ks > 1 && ops_sum_parts(g_llb.stream, parts, ks, (long long)T * rows, T * rows, (float *)(uintptr_t)out_f32)) return -1;
  return 0;
}

}  // extern "C"
