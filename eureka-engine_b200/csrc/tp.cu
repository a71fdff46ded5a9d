// tp.cu -- tensor parallelism across the GPUs of one box: the collective of the sharded engine (engine.cu splits the
// projections by columns and by rows; what is left to exchange is ONE all-reduce(sum) of a [T, d_model] tile after each
// row-split projection: attn_output / ssm_out and ffn_down, two per layer).  The reference has no multi-GPU code at all
// ("One GPU only", docs/limits.md:96); this is the split its benchmark configuration asks for.
//
// NCCL is loaded at run time from the library the process already has (torch's bundled libnccl.so.2, or the system one):
// no link-time dependency, and a process that never asks for tensor parallelism never touches it.  The communicator is
// created from a unique id that rank 0 makes and the host program hands to the other ranks (torch.distributed, a file, a
// socket: this library does not care).  All-reduces are enqueued on the library's stream, so they are captured into the
// cycle's CUDA graph like every kernel.
#include <dlfcn.h>
#include <nccl.h>

#include "host.cuh"
#include "tp.cuh"

static struct {
  void *lib = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, size = 1;
  ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  const char *(*GetErrorString)(ncclResult_t) = nullptr;
} g_tp;

static int tp_load(const char *path) {
  if (g_tp.lib) return 0;
  const char *cands[] = {path, "libnccl.so.2", "libnccl.so"};
  for (const char *c : cands) {
    if (!c || !*c) continue;
    g_tp.lib = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
    if (g_tp.lib) break;
  }
  if (!g_tp.lib) return llb_fail("tensor parallel: cannot load NCCL (%s)", dlerror());
#define TP_SYM(field, name) \
  *(void **)&g_tp.field = dlsym(g_tp.lib, name); \
  if (!g_tp.field) return llb_fail("tensor parallel: NCCL has no %s", name)
  TP_SYM(GetUniqueId, "ncclGetUniqueId");
  TP_SYM(CommInitRank, "ncclCommInitRank");
  TP_SYM(AllReduce, "ncclAllReduce");
  TP_SYM(CommDestroy, "ncclCommDestroy");
  TP_SYM(GetErrorString, "ncclGetErrorString");
#undef TP_SYM
  return 0;
}

int tp_plan(int rank, int size, int H, int KV, int f, int GK, int TR, TpPlan *p) {
  if (size < 1 || rank < 0 || rank >= size) return llb_fail("tensor parallel: rank %d of %d", rank, size);
  if (H % size || GK % size || TR % GK || (KV >= size ? KV % size : size % KV) || f % 256 || f / 256 < size)
    return llb_fail("tensor parallel: %d heads / %d kv heads / %d q-k groups / %d value heads / FFN %d do not split %d ways", H, KV, GK, TR, f, size);
  p->rank = rank; p->size = size;
  p->H_l = H / size; p->h0 = rank * p->H_l;
  if (KV >= size) { p->KV_l = KV / size; p->kv0 = rank * p->KV_l; }
  else { p->KV_l = 1; p->kv0 = p->h0 / (H / KV); }             // fewer kv heads than ranks: the one head this rank's queries read
  if ((p->h0 + p->H_l - 1) / (H / KV) >= p->kv0 + p->KV_l) return llb_fail("tensor parallel: the query heads of rank %d span kv heads it does not hold", rank);
  const int nsb = f / 256, base = nsb / size, extra = nsb % size;
  p->f_l = 256 * (base + (rank < extra)); p->f0 = 256 * (rank * base + (rank < extra ? rank : extra));
  p->GK_l = GK / size; p->g0 = rank * p->GK_l; p->reps = TR / GK; p->TR_l = p->reps * p->GK_l;
  return 0;
}

// ---- the one-shot all-reduce over peer memory ---------------------------------------------------------------------------
// What NCCL costs here is latency: 128 all-reduces of an 80 KB tile per pass, about 21 us each.  The tile is small enough
// for the simplest scheme there is: every rank STORES its tile into a slot of every peer's buffer (plain stores through a
// peer mapping, NVLink) and adds the N slots of its own buffer in rank order (so every rank gets the same bits).  One
// kernel per all-reduce, captured into the cycle graph like the NCCL call it replaces; the K-slice sum of the projection's
// partial results is folded into the same kernel.
//   Data and flag travel together (the scheme of NCCL's low-latency protocol): a 16-byte line is {value, call number,
//   value, call number}, stored with one 16-byte store whose 8-byte halves arrive whole, so the reader needs no fence and
//   no separate flag: it polls the line itself until both numbers are this call's.  A float4 of the tile is two lines.
//   A first version with bulk stores, __threadfence_system and a release flag per chunk took 23 us per all-reduce --
//   slower than NCCL's 21: the fence waits for every store's round trip over NVLink, then the flag makes another.
//   buffer of a rank: lines[2][PEER_MAXR][2 * PEER_CAP / 4] (double-buffered by the parity of the call's number: a rank
//   that runs ahead writes the other half; it cannot run two calls ahead, since its next call needs the slow rank's
//   data of that call), then local words: the call counter, the CTAs that have finished, the error flag.
//   No multicast, no multimem: plain peer stores and volatile local loads.  Every poll is bounded: a peer whose lines
//   never arrive makes the wait run out, the error word is set (llb_b200_wait_errors reports it) and the kernel goes on.
#define PEER_MAXR 8
#define PEER_CAP (8 * 8192)        // floats of a tile: 8 rows of d_model <= 8192
#define PEER_WAIT_LIMIT (1u << 22)   // polls of one line (a few seconds)
struct PeerBuf {
  uint4 lines[2][PEER_MAXR][PEER_CAP / 2];
  unsigned int call, done, err, pad;
};
struct PeerPtrs { PeerBuf *p[PEER_MAXR]; };
static struct {
  PeerBuf *mine = nullptr;
  PeerPtrs ptrs = {};
  bool open = false;
  bool opened[PEER_MAXR] = {false};
} g_peer;

__device__ __forceinline__ void peer_store_line(uint4 *dst, float a, float b, unsigned int call) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(__float_as_uint(a)), "r"(call), "r"(__float_as_uint(b)), "r"(call) : "memory");
}
// polls a line of this rank's own buffer until both halves carry this call's number; false when the limit ran out
__device__ __forceinline__ bool peer_wait_line(const uint4 *src, unsigned int call, unsigned int limit, float &a, float &b) {
  for (unsigned int it = 0; it < limit; it++) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
    if (v.y == call && v.w == call) { a = __uint_as_float(v.x); b = __uint_as_float(v.z); return true; }
  }
  a = b = 0.0f;
  return false;
}

__global__ void __launch_bounds__(256) k_ar_peer(PeerPtrs pp, int rank, int size, const float *__restrict__ part, int ns, long long stride, int n4,
                                                  float *__restrict__ whole, unsigned int limit) {
  pdl_trigger();
  PeerBuf *me = pp.p[rank];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  pdl_wait();
  // this call's number: the last CTA of the previous call stored its own (read after the wait: that kernel has completed)
  const unsigned int call = *(volatile unsigned int *)&me->call + 1u;
  const int par = call & 1u;
  if (i < n4) {
    // this rank's values: the K-slices of the projection added in slice order; out to every peer at once
    float4 v = __ldcg((const float4 *)part + i);
    for (int k = 1; k < ns; k++) { const float4 w = __ldcg((const float4 *)(part + (size_t)k * stride) + i); v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w; }
    for (int r = 0; r < size; r++) {
      if (r == rank) continue;
      uint4 *dst = &pp.p[r]->lines[par][rank][2 * i];
      peer_store_line(dst, v.x, v.y, call);
      peer_store_line(dst + 1, v.z, v.w, call);
    }
    // the sum in rank order, this rank's own values taken from registers
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    bool ok = true;
    for (int r = 0; r < size; r++) {
      float4 w = v;
      if (r != rank) {
        const uint4 *src = &me->lines[par][r][2 * i];
        ok = peer_wait_line(src, call, limit, w.x, w.y) && ok;
        ok = peer_wait_line(src + 1, call, limit, w.z, w.w) && ok;
      }
      if (r == 0) acc = w;
      else { acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w; }
    }
    if (!ok) atomicExch(&me->err, 1u);
    ((float4 *)whole)[i] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(&me->done, 1u) == gridDim.x - 1) { me->done = 0; *(volatile unsigned int *)&me->call = call; __threadfence(); }
  }
}

bool tp_peer_ready(void) { return g_peer.open && g_tp.size > 1; }
int tp_wait_errors(void) {
  if (!g_peer.mine) return 0;
  unsigned int v = 0;
  if (cudaMemcpy(&v, &g_peer.mine->err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)v;
}
int tp_wait_errors_clear(void) {
  if (g_peer.mine) CU_OK(cudaMemset(&g_peer.mine->err, 0, 4));
  return 0;
}
// Ranks drive their own host loops; before a stretch of passes every rank meets the others on the host (a four-byte NCCL
// all-reduce and a stream synchronisation), so that the device-side waits above only ever bridge the skew of ranks that
// run in step, never the seconds one rank's host may spend elsewhere.
int tp_host_barrier(void) {
  if (g_tp.size <= 1 || !g_tp.comm) return 0;
  static float *word = nullptr;
  if (!word) { CU_OK(cudaMalloc(&word, 4)); CU_OK(cudaMemset(word, 0, 4)); }
  const ncclResult_t r = g_tp.AllReduce(word, word, 1, ncclFloat32, ncclSum, g_tp.comm, g_llb.stream);
  if (r != ncclSuccess) return llb_fail("ncclAllReduce: %s", g_tp.GetErrorString(r));
  CU_OK(cudaStreamSynchronize(g_llb.stream));
  return 0;
}
// whole[n] = sum over ranks of (sum over K-slices of part): one kernel on the library's stream
int tp_allreduce_parts(const float *part, int ns, long long stride, size_t n, float *whole) {
  if (!tp_peer_ready()) return llb_fail("tensor parallel: the peer buffers are not open");
  if (n % 4 || n > PEER_CAP) return llb_fail("tensor parallel: a tile of %zu floats (multiples of 4 up to %d)", n, PEER_CAP);
  const int ctas = (int)((n / 4 + 255) / 256);
  CU_OK(llb_launch(k_ar_peer, dim3(ctas), dim3(256), (size_t)0, g_llb.stream, g_peer.ptrs, g_tp.rank, g_tp.size, part, ns, stride, (int)(n / 4), whole,
                   (unsigned int)PEER_WAIT_LIMIT));
  return 0;
}

int tp_rank(void) { return g_tp.rank; }
int tp_size(void) { return g_tp.size; }

// sum over all ranks, in place, n floats, on the library's stream
int tp_allreduce(float *buf, size_t n) {
  if (g_tp.size == 1) return 0;
  if (!g_tp.comm) return llb_fail("tensor parallel: llb_b200_tp_init has not been called");
  const ncclResult_t r = g_tp.AllReduce(buf, buf, n, ncclFloat32, ncclSum, g_tp.comm, g_llb.stream);
  if (r != ncclSuccess) return llb_fail("ncclAllReduce: %s", g_tp.GetErrorString(r));
  return 0;
}

extern "C" {
// 128 bytes that rank 0 makes and every rank passes to llb_b200_tp_init; nccl_path may be NULL
__attribute__((visibility("default"))) int llb_b200_tp_unique_id(const char *nccl_path, void *id128) {
  if (tp_load(nccl_path)) return -1;
  static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
  const ncclResult_t r = g_tp.GetUniqueId((ncclUniqueId *)id128);
  if (r != ncclSuccess) return llb_fail("ncclGetUniqueId: %s", g_tp.GetErrorString(r));
  return 0;
}
// joins the communicator of `size` ranks (after llb_b200_init has bound this process to its GPU); engines opened with
// llb_spec_open_tp afterwards use it
__attribute__((visibility("default"))) int llb_b200_tp_init(const char *nccl_path, int rank, int size, const void *id128) {
  if (!g_llb.stream) return llb_fail("llb_b200_init has not been called");
  if (size < 1 || size > 8 || rank < 0 || rank >= size) return llb_fail("tp_init: rank %d of %d", rank, size);
  if (g_tp.comm) return g_tp.rank == rank && g_tp.size == size ? 0 : llb_fail("tp_init: this process already is rank %d of %d", g_tp.rank, g_tp.size);
  if (size == 1) { g_tp.rank = 0; g_tp.size = 1; return 0; }
  if (tp_load(nccl_path)) return -1;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof id);
  const ncclResult_t r = g_tp.CommInitRank(&g_tp.comm, size, id, rank);
  if (r != ncclSuccess) { g_tp.comm = nullptr; return llb_fail("ncclCommInitRank: %s", g_tp.GetErrorString(r)); }
  g_tp.rank = rank; g_tp.size = size;
  return 0;
}
__attribute__((visibility("default"))) int llb_b200_tp_plan(int rank, int size, int H, int KV, int f, int GK, int TR, int *out10) {
  TpPlan p;
  if (tp_plan(rank, size, H, KV, f, GK, TR, &p)) return -1;
  const int v[10] = {p.H_l, p.h0, p.KV_l, p.kv0, p.f_l, p.f0, p.GK_l, p.g0, p.TR_l, p.reps};
  memcpy(out10, v, sizeof v);
  return 0;
}
// The peer buffers of the one-shot all-reduce.  Every rank allocates its buffer and gets a 64-byte handle for it
// (llb_b200_tp_peer_alloc); the host program gathers the handles of all ranks, in rank order, and every rank opens the
// others' (llb_b200_tp_peer_open).  Engines opened afterwards exchange their tiles through these buffers instead of NCCL.
__attribute__((visibility("default"))) int llb_b200_tp_peer_alloc(void *handle64) {
  if (!g_llb.stream) return llb_fail("llb_b200_init has not been called");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "an IPC handle is 64 bytes");
  if (!g_peer.mine) {
    CU_OK(cudaMalloc(&g_peer.mine, sizeof(PeerBuf)));
    CU_OK(cudaMemset(g_peer.mine, 0, sizeof(PeerBuf)));
  }
  cudaIpcMemHandle_t h;
  CU_OK(cudaIpcGetMemHandle(&h, g_peer.mine));
  memcpy(handle64, &h, 64);
  return 0;
}
__attribute__((visibility("default"))) int llb_b200_tp_peer_open(const void *handles, int n) {
  if (!g_peer.mine) return llb_fail("tp_peer_open: llb_b200_tp_peer_alloc first");
  if (n != g_tp.size || n < 2 || n > PEER_MAXR) return llb_fail("tp_peer_open: %d handles, the communicator has %d ranks", n, g_tp.size);
  if (g_peer.open) return 0;
  for (int r = 0; r < n; r++) {
    if (r == g_tp.rank) { g_peer.ptrs.p[r] = g_peer.mine; continue; }
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char *)handles + 64 * (size_t)r, 64);
    void *p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { cudaGetLastError(); return llb_fail("tp_peer_open: rank %d's buffer: %s", r, cudaGetErrorString(e)); }
    g_peer.ptrs.p[r] = (PeerBuf *)p; g_peer.opened[r] = true;
  }
  g_peer.open = true;
  return 0;
}
// 1 when the engines of this process exchange through the peer buffers, 0 when through NCCL
__attribute__((visibility("default"))) int llb_b200_tp_peer_active(void) { return tp_peer_ready() ? 1 : 0; }
__attribute__((visibility("default"))) void llb_b200_tp_finalize(void) {
  if (g_peer.mine) {
    cudaStreamSynchronize(g_llb.stream);
    for (int r = 0; r < PEER_MAXR; r++) if (g_peer.opened[r]) { cudaIpcCloseMemHandle(g_peer.ptrs.p[r]); g_peer.opened[r] = false; }
    cudaFree(g_peer.mine);
    g_peer.mine = nullptr; g_peer.open = false; g_peer.ptrs = PeerPtrs{};
  }
  if (g_tp.comm) { cudaStreamSynchronize(g_llb.stream); g_tp.CommDestroy(g_tp.comm); g_tp.comm = nullptr; }
  g_tp.rank = 0; g_tp.size = 1;
}
}  // extern "C"
