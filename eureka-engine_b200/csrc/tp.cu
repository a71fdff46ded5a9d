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
__attribute__((visibility("default"))) void llb_b200_tp_finalize(void) {
  if (g_tp.comm) { cudaStreamSynchronize(g_llb.stream); g_tp.CommDestroy(g_tp.comm); g_tp.comm = nullptr; }
  g_tp.rank = 0; g_tp.size = 1;
}
}  // extern "C"
