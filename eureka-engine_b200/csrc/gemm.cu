// gemm.cu -- host side of the dequant-fused skinny GEMM (kernel in gemm.cuh).
#include "host.cuh"

template <int FMT, int NT> static int launch_one(cudaStream_t s, const GemmArgs &a, int grid) {
  k_gemm<FMT, NT><<<grid, GEMM_WARPS * 32, gemm_smem_bytes<FMT>(), s>>>(a);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return llb_fail("k_gemm launch: %s", cudaGetErrorString(e));
  return 0;
}

template <int FMT> static int setup_fmt() {
  CU_OK(cudaFuncSetAttribute(k_gemm<FMT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_smem_bytes<FMT>()));
  CU_OK(cudaFuncSetAttribute(k_gemm<FMT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, gemm_smem_bytes<FMT>()));
  return 0;
}

int gemm_setup(void) {
  if (setup_fmt<LLB_FM_Q4_K>() || setup_fmt<LLB_FM_Q5_K>() || setup_fmt<LLB_FM_Q6_K>() || setup_fmt<LLB_FM_Q8_0>()) return -1;
  return 0;
}

// K-slices per row tile: balance (tiles * slices) over the resident warps against the length of the
// longest slice, with a small charge per slice for the partial sums the consumer has to add.
int gemm_pick_ksplit(int ntiles, int nsb, int sms) {
  const long long nw = (long long)sms * GEMM_WARPS;
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= GEMM_MAXSPLIT && ks <= nsb; ks++) {
    long long rounds = ((long long)ntiles * ks + nw - 1) / nw;
    int slice = (nsb + ks - 1) / ks;
    double cost = (double)rounds * slice * (1.0 + 0.02 * (ks - 1));
    if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
  }
  return best;
}

int gemm_launch(cudaStream_t s, int fmt, GemmArgs &a) {
  if (a.nmat < 1 || a.nmat > GEMM_MAXMAT) return llb_fail("gemm: nmat %d", a.nmat);
  if (a.K % 256) return llb_fail("gemm: K %d is not a multiple of 256", a.K);
  if (a.xp.NC != 8 && a.xp.NC != 16) return llb_fail("gemm: NC %d", a.xp.NC);
  if (a.xp.K != a.K) return llb_fail("gemm: planes hold %d columns, K is %d", a.xp.K, a.K);
  a.nsb = a.K / 256;
  a.tile0[0] = 0;
  for (int i = 0; i < a.nmat; i++) a.tile0[i + 1] = a.tile0[i] + (a.m[i].rows + 15) / 16;
  for (int i = a.nmat; i < GEMM_MAXMAT; i++) a.tile0[i + 1] = a.tile0[a.nmat];
  if (a.ksplit < 1 || a.ksplit > GEMM_MAXSPLIT || a.ksplit > a.nsb) return llb_fail("gemm: ksplit %d", a.ksplit);
  const int nunits = a.tile0[a.nmat] * a.ksplit;
  int grid = (nunits + GEMM_WARPS - 1) / GEMM_WARPS;
  if (grid > g_llb.sms) grid = g_llb.sms;
  if (grid < 1) return 0;
  const int NT = a.xp.NC / 8;
#define GO(F)                                                                     \
  case F: return NT == 1 ? launch_one<F, 1>(s, a, grid) : launch_one<F, 2>(s, a, grid);
  switch (fmt) {
    GO(LLB_FM_Q4_K)
    GO(LLB_FM_Q5_K)
    GO(LLB_FM_Q6_K)
    GO(LLB_FM_Q8_0)
  }
#undef GO
  return llb_fail("gemm: format %d has no kernel", fmt);
}
