// ops.cu -- format and activation-plane utility kernels.
#include <vector>

#include "host.cuh"

// ---- activations -> fp16 planes ----------------------------------------------------------------
__global__ void k_xp_from_f32(const float *__restrict__ x, int K, int planes, XPlanes xp) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  if (c0 >= K) return;
  xp_store32(xp, t, planes, c0, x[(size_t)t * K + c0 + lane], lane);
}
__global__ void k_xp_from_bf16(const unsigned short *__restrict__ x, int K, XPlanes xp) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.y, lane = threadIdx.x & 31;
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) & ~31;
  if (c0 >= K) return;
  float v = __uint_as_float((uint32_t)x[(size_t)t * K + c0 + lane] << 16);
  xp_store32(xp, t, 1, c0, v, lane);
}
int ops_xp_from_f32(cudaStream_t s, const float *x, int T, int planes, XPlanes xp) {
  if (xp.K % 32) return llb_fail("xp: K %d", xp.K);
  if (T * planes > xp.NC) return llb_fail("xp: %d rows x %d planes do not fit %d columns", T, planes, xp.NC);
  CU_OK(llb_launch(k_xp_from_f32, dim3((xp.K + 255) / 256, T), dim3(256), (size_t)(0), s, x, xp.K, planes, xp));
  CU_OK(cudaGetLastError());
  return 0;
}
int ops_xp_from_bf16(cudaStream_t s, const void *x, int T, XPlanes xp) {
  if (xp.K % 32) return llb_fail("xp: K %d", xp.K);
  if (T > xp.NC) return llb_fail("xp: %d rows do not fit %d columns", T, xp.NC);
  CU_OK(llb_launch(k_xp_from_bf16, dim3((xp.K + 255) / 256, T), dim3(256), (size_t)(0), s, (const unsigned short *)x, xp.K, xp));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- bit-exact row dequantisation (embedding rows; the dequant parity check) -------------------
__global__ void k_dequant_rows(int fmt, const uint8_t *__restrict__ W, int cols, const int *__restrict__ row_ids,
                               float *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  const int r = blockIdx.y;
  const int row = row_ids ? row_ids[r] : r;
  const uint8_t *src = W + (size_t)row * dev_row_bytes(fmt, cols);
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x)
    out[(size_t)r * cols + c] = deq_elem(fmt, src, cols, c);
}
int ops_dequant_rows(cudaStream_t s, int fmt, const uint8_t *W, int rows, int cols, const int *row_ids, int nrows,
                     float *out) {
  (void)rows;
  if (nrows < 1) return 0;
  int gx = (cols + 255) / 256;
  if (gx > 64) gx = 64;
  // gridDim.y is limited to 65535 rows per launch
  for (int r0 = 0; r0 < nrows; r0 += 65535) {
    int n = nrows - r0 < 65535 ? nrows - r0 : 65535;
    CU_OK(llb_launch(k_dequant_rows, dim3(gx, n), dim3(256), (size_t)(0), s, fmt, row_ids ? W : W + (size_t)r0 * dev_row_bytes(fmt, cols), cols,
                                              row_ids ? row_ids + r0 : nullptr, out + (size_t)r0 * cols));
    CU_OK(cudaGetLastError());
  }
  return 0;
}

// ---- Q6_K: 210-byte stored super-blocks -> 224-byte device super-blocks ------------------------
__global__ void k_repack_q6k(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t nblocks) {
  pdl_trigger();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  size_t n = nblocks * 224;
  for (; i < n; i += (size_t)gridDim.x * blockDim.x) {
    size_t b = i / 224;
    int o = (int)(i - b * 224);
    dst[i] = o < 210 ? src[b * 210 + o] : 0;
  }
}
int ops_repack_q6k(cudaStream_t s, const uint8_t *src210, uint8_t *dst224, size_t nblocks) {
  if (!nblocks) return 0;
  size_t n = nblocks * 224;
  int grid = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  CU_OK(llb_launch(k_repack_q6k, dim3(grid), dim3(256), (size_t)(0), s, src210, dst224, nblocks));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- fixed-order sum of K-slice partials --------------------------------------------------------
__global__ void k_sum_parts(const float *__restrict__ parts, int nsplit, long long stride, int n, float *__restrict__ out) {
  pdl_trigger();
  pdl_wait();
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float v = parts[i];
  for (int k = 1; k < nsplit; k++) v += parts[(size_t)k * stride + i];
  out[i] = v;
}
int ops_sum_parts(cudaStream_t s, const float *parts, int nsplit, long long split_stride, int n, float *out) {
  CU_OK(llb_launch(k_sum_parts, dim3((n + 255) / 256), dim3(256), (size_t)(0), s, parts, nsplit, split_stride, n, out));
  CU_OK(cudaGetLastError());
  return 0;
}

// ---- the launch half of the backend contract ----------------------------------------------------
// host/llb_backend.h:9-24 asks a backend for LLB_LAUNCH(k, gx, gy, bx, &a0, ...) / LLB_LAUNCH_SM: kernels are fetched
// by name (cuModuleGetFunction in the reference, tools/payload-spec.patch:9-23), every argument is the address of a
// host variable copied at the call, launches run in call order on one stream.  host/llb_backend_cuda.h:125-184 adds a
// recorder: between llb_graph_begin and llb_graph_end the launches are kept and then run as one CUDA graph, a repeated
// kernel sequence re-uses its graph, and any other device call ends the recording first ("bail").
//
// The kernels reachable by name are the library's own leaves with plain argument lists; the reference's kernel names
// (llb_spec_gu3, ...) are not among them: their argument lists carry its two-plane int8 activation format, so an
// unknown name returns NULL and the caller fails cleanly.
struct llb_b200_kernel { const char *name; const void *fn; int nparams; };
static const llb_b200_kernel g_kernels[] = {
    {"llb_b200_k_dequant_rows", (const void *)k_dequant_rows, 5},   // (int fmt, const u8 *W, int cols, const int *row_ids, float *out), grid (x, rows)
    {"llb_b200_k_sum_parts", (const void *)k_sum_parts, 5},         // (const float *parts, int nsplit, long long stride, int n, float *out)
    {"llb_b200_k_repack_q6k", (const void *)k_repack_q6k, 3},       // (const u8 *src210, u8 *dst224, size_t nblocks)
    {"llb_b200_k_xp_from_f32", (const void *)k_xp_from_f32, 4},     // (const float *x, int K, int planes, XPlanes xp), grid (K / 256, T)
};

#define GRAPH_SLOTS 16      // cached kernel sequences (LLB_GSLOT of the reference)
#define GRAPH_MAXNODES 2048 // launches per recorded step (LLB_GMAX)
struct GraphSig { const void *fn; unsigned gx, gy, bx, sm; };
static bool g_rec = false;
static std::vector<GraphSig> g_rec_sig;
static struct { std::vector<const void *> fns; cudaGraphExec_t exec = nullptr; } g_slot[GRAPH_SLOTS];
static int g_victim = 0;
static unsigned long long g_gstat[4];   // graphs built, steps replayed, steps that re-used a cached graph, bails

// ends a recording by running what was recorded once, outside any cache
static int graph_flush(bool count_bail) {
  if (!g_rec) return 0;
  g_rec = false;
  cudaGraph_t g = nullptr;
  CU_OK(cudaStreamEndCapture(g_llb.stream, &g));
  if (count_bail) g_gstat[3] += 1;
  if (!g) return 0;
  cudaGraphExec_t ex = nullptr;
  cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
  if (e == cudaSuccess) e = cudaGraphLaunch(ex, g_llb.stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(g_llb.stream);
  if (ex) cudaGraphExecDestroy(ex);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return llb_fail("graph recorder: %s", cudaGetErrorString(e));
  return 0;
}
int backend_graph_bail(void) { return graph_flush(true); }

extern "C" {
__attribute__((visibility("default"))) const llb_b200_kernel *llb_b200_kernel_by_name(const char *name) {
  if (name)
    for (const llb_b200_kernel &k : g_kernels)
      if (!strcmp(k.name, name)) return &k;
  llb_fail("kernel_by_name: the library has no kernel called %s", name ? name : "(null)");
  return nullptr;
}

__attribute__((visibility("default"))) int llb_b200_launch(const llb_b200_kernel *k, unsigned gx, unsigned gy, unsigned bx, unsigned sm, void **args, unsigned na) {
  if (!g_llb.stream) return llb_fail("llb_b200_init has not been called");
  if (!k) return llb_fail("launch: no kernel (an unknown name?)");
  if ((int)na != k->nparams) return llb_fail("launch: %s takes %d arguments, %u given", k->name, k->nparams, na);
  if (!gx || !gy || !bx || bx > 1024) return llb_fail("launch: %s with grid %u x %u, block %u", k->name, gx, gy, bx);
  if (g_rec) {
    if (g_rec_sig.size() >= GRAPH_MAXNODES) return llb_fail("graph recorder: more than %d launches in one step", GRAPH_MAXNODES);
    g_rec_sig.push_back({k->fn, gx, gy, bx, sm});
  }
  const cudaError_t e = cudaLaunchKernel(k->fn, dim3(gx, gy, 1), dim3(bx, 1, 1), args, sm, g_llb.stream);
  if (e != cudaSuccess) return llb_fail("launch of %s: %s", k->name, cudaGetErrorString(e));
  return 0;
}

__attribute__((visibility("default"))) int llb_b200_graph_begin(void) {
  if (!g_llb.stream) return llb_fail("llb_b200_init has not been called");
  if (g_rec) return 0;
  CU_OK(cudaStreamBeginCapture(g_llb.stream, cudaStreamCaptureModeThreadLocal));
  g_rec = true;
  g_rec_sig.clear();
  return 0;
}

__attribute__((visibility("default"))) int llb_b200_graph_end(void) {
  if (!g_rec) return 0;
  g_rec = false;
  cudaGraph_t g = nullptr;
  CU_OK(cudaStreamEndCapture(g_llb.stream, &g));
  if (!g || g_rec_sig.empty()) { if (g) cudaGraphDestroy(g); return 0; }
  // a step with the kernel sequence of a cached graph only updates that graph's nodes
  int sl = -1;
  for (int i = 0; i < GRAPH_SLOTS && sl < 0; i++) {
    if (!g_slot[i].exec || g_slot[i].fns.size() != g_rec_sig.size()) continue;
    bool same = true;
    for (size_t j = 0; same && j < g_rec_sig.size(); j++) same = g_slot[i].fns[j] == g_rec_sig[j].fn;
    if (same) sl = i;
  }
  cudaError_t e = cudaSuccess;
  if (sl >= 0) {
    cudaGraphExecUpdateResultInfo info;
    if (cudaGraphExecUpdate(g_slot[sl].exec, g, &info) == cudaSuccess) g_gstat[2] += 1;
    else { cudaGetLastError(); cudaGraphExecDestroy(g_slot[sl].exec); g_slot[sl].exec = nullptr; sl = -1; }
  }
  if (sl < 0) {
    sl = g_victim; g_victim = (g_victim + 1) % GRAPH_SLOTS;
    if (g_slot[sl].exec) cudaGraphExecDestroy(g_slot[sl].exec);
    g_slot[sl].exec = nullptr;
    e = cudaGraphInstantiate(&g_slot[sl].exec, g, 0);
    g_slot[sl].fns.clear();
    for (const GraphSig &q : g_rec_sig) g_slot[sl].fns.push_back(q.fn);
    g_gstat[0] += 1;
  }
  cudaGraphDestroy(g);
  if (e == cudaSuccess) e = cudaGraphLaunch(g_slot[sl].exec, g_llb.stream);
  if (e != cudaSuccess) return llb_fail("graph recorder: %s", cudaGetErrorString(e));
  g_gstat[1] += 1;
  return 0;
}

__attribute__((visibility("default"))) int llb_b200_graph_bail(void) { return backend_graph_bail(); }
__attribute__((visibility("default"))) void llb_b200_graph_stats(unsigned long long out[4]) { for (int i = 0; i < 4; i++) out[i] = g_gstat[i]; }
}  // extern "C"
