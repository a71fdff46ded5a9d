// host.cuh -- host-side state shared by the translation units of libllb_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"
#include "gemm.cuh"

struct LlbCtx {
  int device = -1;
  int sms = 0;
  int ffn_fused = 0;   // the FFN as one launch with a grid barrier (LLB_FFN_FUSED=1)
  int gemm3 = 0;   // Q4_K, T <= 4 on the tcgen05 kernel (LLB_GEMM3=1)
  int pdl = 1;     // programmatic dependent launch on every kernel of a pass (LLB_PDL=0 turns it off)
  cudaStream_t stream = nullptr;
  char err[512] = {0};
};
extern LlbCtx g_llb;

inline int llb_fail(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_llb.err, sizeof g_llb.err, fmt, ap);
  va_end(ap);
  return -1;
}
#define CU_OK(call)                                                                              \
  do {                                                                                           \
    cudaError_t e_ = (call);                                                                     \
    if (e_ != cudaSuccess) return llb_fail("%s: %s (%s:%d)", #call, cudaGetErrorString(e_), __FILE__, __LINE__); \
  } while (0)

// Launch with (optionally) the programmatic-serialization attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t llb_launch(void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at; cfg.numAttrs = g_llb.pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, k, KArgs(args)...);
}

// gemm.cu
int gemm_pick_ksplit(int fmt, int NC, int ntiles, int nsb, int sms, bool sel = false);   // sel: for a routed-expert launch
int gemm_fix_ksplit(int fmt, int NC, int nsb, int ks, bool sel = false);   // clamps a requested K-split to what the format's kernel can take
int gemm_ring_ksplit(int fmt, int nsb, int ntiles, int nc_spec, int nc_pf, int sms, int cap);
int gemm_launch(cudaStream_t s, int fmt, GemmArgs &a);   // fills tile0 / nsb, picks NT from xp.NC
int gemm_setup(void);
int gemm_wait_errors(void);
int gemm_wait_errors_clear(void);
int gemm_wait_selftest(cudaStream_t s, int which, int limit);
bool gemm_ffn_fusable(int fmt_gu, int fmt_dn, int NC, int d);
int gemm_launch_ffn(cudaStream_t s, GemmArgs &a1, int fmt2, GemmArgs &a2);   // gate|up (Q4_K, one K-slice), silu, down in one launch
int gemm_launch_moe(cudaStream_t s, int fmt, bool down, const XPlanes &xp, MoeArgs &m, int *ksplit, const float *wt_silu);   // moe.cuh

// ops.cu
int backend_graph_bail(void);   // ends a launch recording in progress by running it (the memory primitives call it first)
int ops_xp_from_f32(cudaStream_t s, const float *x, int T, int planes, XPlanes xp);
int ops_xp_from_bf16(cudaStream_t s, const void *x, int T, XPlanes xp);
int ops_dequant_rows(cudaStream_t s, int fmt, const uint8_t *W, int rows, int cols, const int *row_ids, int nrows, float *out);
int ops_repack_q6k(cudaStream_t s, const uint8_t *src210, uint8_t *dst224, size_t nblocks);
int ops_sum_parts(cudaStream_t s, const float *parts, int nsplit, long long split_stride, int n, float *out);
