// gemm.cu -- host side of the dequant-fused skinny GEMMs (kernel in gemm2.cuh, its arithmetic in gemm.cuh).
#include "gemm2.cuh"
#include "gemm3.cuh"
#include "ffn_fused.cuh"
#include "moe.cuh"
#include "host.cuh"

static int g2_max_sb(int fmt, int NC, bool sel = false) {
  return fmt == LLB_FM_Q4_K ? g2_max_slice_sb<LLB_FM_Q4_K>(NC, sel) : fmt == LLB_FM_Q5_K ? g2_max_slice_sb<LLB_FM_Q5_K>(NC, sel)
       : fmt == LLB_FM_Q8_0 ? g2_max_slice_sb<LLB_FM_Q8_0>(NC, sel) : g2_max_slice_sb<LLB_FM_Q6_K>(NC, sel);
}
// the tcgen05 kernel takes Q4_K with T <= 4 (8 plane columns)
static bool is_g3(int fmt, int NC) { return g_llb.gemm3 && fmt == LLB_FM_Q4_K && NC == 8; }
static unsigned int *g_ffn_sync = nullptr;   // the fused FFN's grid barrier: two counters
static unsigned int *g_g3_err = nullptr;   // device word: set when a bounded wait of k_gemm3 ran out
static int g2_warps_of(int fmt, int NC, bool sel = false) {
  return fmt == LLB_FM_Q6_K ? g2_warps<LLB_FM_Q6_K>(NC, sel) : fmt == LLB_FM_Q8_0 ? g2_warps<LLB_FM_Q8_0>(NC, sel)
       : fmt == LLB_FM_Q5_K ? g2_warps<LLB_FM_Q5_K>(NC, sel) : g2_warps<LLB_FM_Q4_K>(NC, sel);
}

template <int FMT, int NT> static int launch_two(cudaStream_t s, const GemmArgs &a) {
  const int NC = 8 * NT, nsl = (a.nsb + a.ksplit - 1) / a.ksplit;
  int cps = g_llb.sms * G2_CPSM / a.ksplit;
  if (cps < 1) cps = 1;
  // every SM takes part as long as there is a tile for it: the tiles are dealt out one per CTA in turn
  constexpr int G2_WARPS = g2_warps<FMT>(8 * NT);
  if (cps > a.tile0[a.nmat]) cps = a.tile0[a.nmat];
  const size_t smem = (size_t)g2_xp_bytes<FMT>(nsl, NC) + g2_ring_bytes<FMT>(NC);
  if (smem > G2_SMEM_MAX) return llb_fail("k_gemm2: a K-slice of %d super-blocks needs %zu bytes of shared memory", nsl, smem);
  cudaError_t e = llb_launch(k_gemm2<FMT, NT>, dim3(cps * a.ksplit), dim3(G2_WARPS * 32), smem, s, a, cps);
  if (e != cudaSuccess) return llb_fail("k_gemm2 launch: %s", cudaGetErrorString(e));
  return 0;
}

static int launch_three(cudaStream_t s, const GemmArgs &a) {
  const int nsl = (a.nsb + a.ksplit - 1) / a.ksplit;
  int ntiles = 0;
  for (int i = 0; i < a.nmat; i++) ntiles += (a.m[i].rows + 127) / 128;
  int cps = g_llb.sms / a.ksplit;
  if (cps < 1) cps = 1;
  if (cps > ntiles) cps = ntiles;
  const size_t smem = (size_t)g3_smem_bytes(nsl);
  if (smem > G3_SMEM_MAX) return llb_fail("k_gemm3: a K-slice of %d super-blocks needs %zu bytes of shared memory", nsl, smem);
  cudaError_t e = llb_launch(k_gemm3, dim3(cps * a.ksplit), dim3(G3_BLOCK), smem, s, a, cps, g_g3_err);
  if (e != cudaSuccess) return llb_fail("k_gemm3 launch: %s", cudaGetErrorString(e));
  return 0;
}
// 1 when a bounded wait of the tcgen05 kernel or of the fused FFN's barrier has run out since the library was
// initialised (or since the word was last cleared)
int gemm_wait_errors(void) {
  unsigned int v = 0;
  if (g_g3_err && cudaMemcpy(&v, g_g3_err, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -1;
  return (int)v;
}
int gemm_wait_errors_clear(void) {
  if (g_g3_err) CU_OK(cudaMemset(g_g3_err, 0, 4));
  return 0;
}

// The two device-side waits of this file, each made to run out on purpose with a small limit: an mbarrier nobody
// arrives on (the wait of k_gemm3 and k_pfmm, tc5.cuh) and the fused FFN's grid barrier told to expect one block more
// than the launch has.  One block, one waiting thread; the wait gives up after `limit` tries, sets the error word
// exactly as in the real kernels and the kernel returns.
__global__ void k_wait_selftest(int which, unsigned int limit, unsigned int *sync, unsigned int *err) {
  __shared__ __align__(8) uint64_t bar;
  if (which == 0) {
    const uint32_t bar_s = smem_u32(&bar);
    if (threadIdx.x == 0) {
      mbar_init(bar_s, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0 && !mbar_wait(bar_s, 0, limit)) atomicExch(err, 1u);
  } else {
    ffn_grid_sync(sync, 2u, err, limit);
    if (threadIdx.x == 0) { sync[0] = 0; sync[1] = 0; }   // the block that never came would have reset them
  }
}
int gemm_wait_selftest(cudaStream_t s, int which, int limit) {
  if (which < 0 || which > 1 || limit < 1 || limit > 100000) return llb_fail("wait selftest: which 0..1, limit 1..100000");
  unsigned int *sync = nullptr;
  CU_OK(cudaMalloc(&sync, 8));           // a private pair of counters: the barrier of real launches is not touched
  CU_OK(cudaMemsetAsync(sync, 0, 8, s));
  k_wait_selftest<<<1, 32, 0, s>>>(which, (unsigned int)limit, sync, g_g3_err);
  CU_OK(cudaGetLastError());
  CU_OK(cudaStreamSynchronize(s));
  CU_OK(cudaFree(sync));
  return 0;
}

template <int FMT> static int setup_fmt2() {
  CU_OK(cudaFuncSetAttribute(k_gemm2<FMT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_gemm2<FMT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_gemm2<FMT, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  return 0;
}

template <int FMT> static int setup_moe() {
  CU_OK(cudaFuncSetAttribute(k_moe_gu<FMT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_moe_gu<FMT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_moe_dn<FMT, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_moe_dn<FMT, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_moe_gu<FMT, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_moe_dn<FMT, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_moe_dn_silu<FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  return 0;
}

int gemm_setup(void) {
  if (setup_fmt2<LLB_FM_Q4_K>() || setup_fmt2<LLB_FM_Q5_K>() || setup_fmt2<LLB_FM_Q6_K>() || setup_fmt2<LLB_FM_Q8_0>()) return -1;
  CU_OK(cudaFuncSetAttribute(k_gemm3, cudaFuncAttributeMaxDynamicSharedMemorySize, G3_SMEM_MAX));
  if (setup_moe<LLB_FM_Q4_K>() || setup_moe<LLB_FM_Q5_K>() || setup_moe<LLB_FM_Q6_K>()) return -1;
  CU_OK(cudaFuncSetAttribute(k_ffn<LLB_FM_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_ffn<LLB_FM_Q5_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  CU_OK(cudaFuncSetAttribute(k_ffn<LLB_FM_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, G2_SMEM_MAX));
  if (!g_ffn_sync) {
    CU_OK(cudaMalloc(&g_ffn_sync, 8));
    CU_OK(cudaMemset(g_ffn_sync, 0, 8));
  }
  if (!g_g3_err) {
    CU_OK(cudaMalloc(&g_g3_err, 4));
    CU_OK(cudaMemset(g_g3_err, 0, 4));
  }
  return 0;
}

// sel: a routed-expert launch (its own warp count and ring depth at 32 plane columns)
int gemm_fix_ksplit(int fmt, int NC, int nsb, int ks, bool sel) {
  if (ks < 1) ks = 1;
  if (!sel && is_g3(fmt, NC)) {
    const int mx = g3_max_slice_sb();
    const int lo = (nsb + mx - 1) / mx;
    if (ks < lo) ks = lo;
  } else {
    const int mx = g2_max_sb(fmt, NC, sel);
    const int lo = (nsb + mx - 1) / mx;       // the activation slice of a CTA has to fit in shared memory
    if (ks < lo) ks = lo;
  }
  if (ks > GEMM_MAXSPLIT) ks = GEMM_MAXSPLIT;
  if (ks > nsb) ks = nsb;
  return ks;
}

// K-slices per row tile: the longest chain of work of any warp (tiles per warp x super-blocks per
// slice), with a small charge per slice for the partial sums the consumer has to add.
int gemm_pick_ksplit(int fmt, int NC, int ntiles, int nsb, int sms, bool sel) {
  int best = 1;
  double best_cost = 1e30;
  for (int ks = 1; ks <= GEMM_MAXSPLIT && ks <= nsb; ks++) {
    if (gemm_fix_ksplit(fmt, NC, nsb, ks, sel) != ks) continue;
    long long rounds;
    if (!sel && is_g3(fmt, NC)) {
      // 128-row tiles, one CTA per (tile, slice) at a time; 1.5 super-blocks of pipeline fill per tile
      const int cps = sms / ks > 0 ? sms / ks : 1, nt128 = (ntiles + 7) / 8;
      rounds = (nt128 + cps - 1) / cps;
      const int slice = (nsb + ks - 1) / ks;
      const double cost = (double)rounds * (slice + 1.5) * (1.0 + 0.02 * (ks - 1));
      if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
      continue;
    } else {
      const int cps = sms * G2_CPSM / ks > 0 ? sms * G2_CPSM / ks : 1;
      rounds = (ntiles + (long long)cps * g2_warps_of(fmt, NC, sel) - 1) / ((long long)cps * g2_warps_of(fmt, NC, sel));
    }
    const int slice = (nsb + ks - 1) / ks;
    const double cost = (double)rounds * slice * (1.0 + 0.02 * (ks - 1));
    if (cost < best_cost - 1e-9) { best_cost = cost; best = ks; }
  }
  return gemm_fix_ksplit(fmt, NC, nsb, best, sel);
}

// One K-split for a launch whose partial sums outlive the pass (attn_qkv into the conv ring): valid at both
// plane widths in use, the cost model's choice at the speculative width where that fits, at most `cap`.
// Returns 0 when no split up to `cap` fits both widths.
int gemm_ring_ksplit(int fmt, int nsb, int ntiles, int nc_spec, int nc_pf, int sms, int cap) {
  const int lo_a = gemm_fix_ksplit(fmt, nc_spec, nsb, 1), lo_b = gemm_fix_ksplit(fmt, nc_pf, nsb, 1);
  const int lo = lo_a > lo_b ? lo_a : lo_b;
  if (cap > nsb) cap = nsb;
  if (lo > cap) return 0;
  int ks = gemm_pick_ksplit(fmt, nc_spec, ntiles, nsb, sms);
  if (ks < lo) ks = lo;
  if (ks > cap) ks = cap;
  return ks;
}

// fills nsb and the tile table of a launch and checks its shape
static int gemm_prepare(int fmt, GemmArgs &a) {
  if (a.nmat < 1 || a.nmat > GEMM_MAXMAT) return llb_fail("gemm: nmat %d", a.nmat);
  if (a.K % 256) return llb_fail("gemm: K %d is not a multiple of 256", a.K);
  if (a.xp.NC != 8 && a.xp.NC != 16 && a.xp.NC != 32) return llb_fail("gemm: NC %d", a.xp.NC);
  if (a.xp.K != a.K) return llb_fail("gemm: planes hold %d columns, K is %d", a.xp.K, a.K);
  a.nsb = a.K / 256;
  a.tile0[0] = 0;
  for (int i = 0; i < a.nmat; i++) a.tile0[i + 1] = a.tile0[i] + (a.m[i].rows + 15) / 16;
  for (int i = a.nmat; i < GEMM_MAXMAT; i++) a.tile0[i + 1] = a.tile0[a.nmat];
  if (a.ksplit != gemm_fix_ksplit(fmt, a.xp.NC, a.nsb, a.ksplit)) return llb_fail("gemm: ksplit %d is not valid for this shape", a.ksplit);
  return 0;
}

// ---- the fused FFN launch (ffn_fused.cuh) ------------------------------------------------------
template <int FMT2> static int launch_ffn(cudaStream_t s, const GemmArgs &a1, const GemmArgs &a2) {
  int cps1 = g_llb.sms, cps2 = g_llb.sms / a2.ksplit;
  if (cps1 > a1.tile0[a1.nmat]) cps1 = a1.tile0[a1.nmat];
  if (cps2 < 1) cps2 = 1;
  if (cps2 > a2.tile0[a2.nmat]) cps2 = a2.tile0[a2.nmat];
  const int grid = cps1 > cps2 * a2.ksplit ? cps1 : cps2 * a2.ksplit;
  if (grid > g_llb.sms) return llb_fail("k_ffn: %d CTAs do not fit %d SMs", grid, g_llb.sms);   // the barrier needs them all resident
  const size_t s1 = (size_t)g2_xp_bytes<LLB_FM_Q4_K>(a1.nsb, 8) + 16 * G2_STAGES * 16 * G2Traits<LLB_FM_Q4_K>::RS;
  const int nsl2 = (a2.nsb + a2.ksplit - 1) / a2.ksplit;
  const size_t s2 = (size_t)g2_xp_bytes<FMT2>(nsl2, 8) + 16 * G2_STAGES * 16 * G2Traits<FMT2>::RS;
  const size_t smem = s1 > s2 ? s1 : s2;
  if (smem > G2_SMEM_MAX) return llb_fail("k_ffn: %zu bytes of shared memory", smem);
  cudaError_t e = llb_launch(k_ffn<FMT2>, dim3(grid), dim3(512), smem, s, a1, a2, cps1, cps2, g_ffn_sync, g_g3_err);
  if (e != cudaSuccess) return llb_fail("k_ffn launch: %s", cudaGetErrorString(e));
  return 0;
}
// can the FFN of these formats and widths run as one launch?  (gate|up in one K-slice, T <= 4)
bool gemm_ffn_fusable(int fmt_gu, int fmt_dn, int NC, int d) {
  return g_llb.ffn_fused && g_ffn_sync && NC == 8 && fmt_gu == LLB_FM_Q4_K &&
         (fmt_dn == LLB_FM_Q4_K || fmt_dn == LLB_FM_Q5_K || fmt_dn == LLB_FM_Q6_K) && d % 256 == 0 &&
         d / 256 <= g2_max_slice_sb<LLB_FM_Q4_K>(8);
}
// a1: gate and up (two matrices, Q4_K, ksplit 1, outputs complete); a2: down in format fmt2 with its own K-split
int gemm_launch_ffn(cudaStream_t s, GemmArgs &a1, int fmt2, GemmArgs &a2) {
  if (a1.nmat != 2 || a1.ksplit != 1 || a2.nmat != 1 || a1.xp.NC != 8 || a2.xp.NC != 8) return llb_fail("k_ffn: unsupported launch shape");
  if (gemm_prepare(LLB_FM_Q4_K, a1) || gemm_prepare(fmt2, a2)) return -1;
  if (a2.K != a1.m[0].rows || a1.m[1].rows != a1.m[0].rows) return llb_fail("k_ffn: down takes %d columns, gate/up have %d/%d rows", a2.K, a1.m[0].rows, a1.m[1].rows);
  if (fmt2 == LLB_FM_Q4_K) return launch_ffn<LLB_FM_Q4_K>(s, a1, a2);
  if (fmt2 == LLB_FM_Q5_K) return launch_ffn<LLB_FM_Q5_K>(s, a1, a2);
  if (fmt2 == LLB_FM_Q6_K) return launch_ffn<LLB_FM_Q6_K>(s, a1, a2);
  return llb_fail("k_ffn: down format %d", fmt2);
}

// ---- the routed experts' GEMMs (moe.cuh) ---------------------------------------------------------
template <int FMT, int NT> static int launch_moe(cudaStream_t s, bool down, const GemmArgs &a, const MoeArgs &m, int ntiles, const float *wt_silu) {
  const int NC = 8 * NT, nsl = (a.nsb + a.ksplit - 1) / a.ksplit;
  int cps = g_llb.sms * G2_CPSM / a.ksplit;
  if (cps < 1) cps = 1;
  if (cps > ntiles) cps = ntiles;
  constexpr bool sel = moe_ntc<NT>() != NT;
  const size_t smem = (size_t)g2_xp_bytes<FMT>(nsl, NC) + g2_ring_bytes<FMT>(NC, sel);
  if (smem > G2_SMEM_MAX) return llb_fail("moe gemm: a K-slice of %d super-blocks needs %zu bytes of shared memory", nsl, smem);
  cudaError_t e;
  if (down && wt_silu) {
    if constexpr (NT == 1) e = llb_launch(k_moe_dn_silu<FMT>, dim3(cps * a.ksplit), dim3(G2Traits<FMT>::WARPS * 32), smem, s, a, m, wt_silu, cps);
    else return llb_fail("moe gemm: the down launch builds its own activations for T <= 4 only");
  } else {
    e = down ? llb_launch(k_moe_dn<FMT, NT>, dim3(cps * a.ksplit), dim3(g2_warps<FMT>(NC, sel) * 32), smem, s, a, m, cps)
             : llb_launch(k_moe_gu<FMT, NT>, dim3(cps * a.ksplit), dim3(g2_warps<FMT>(NC, sel) * 32), smem, s, a, m, cps);
  }
  if (e != cudaSuccess) return llb_fail("moe gemm launch: %s", cudaGetErrorString(e));
  return 0;
}
// down == false: gate|up of every (token, slot) on planes of K = d columns, one K-slice (the epilogue needs whole sums);
// down == true: the per-token virtual matrices of K = nslot * ef columns, *ksplit slices (0: chosen here) into m.out
// wt_silu (down only, T <= 4): the launch builds wt * silu(m.g) * m.u in shared memory itself; xp then only gives K and NC
int gemm_launch_moe(cudaStream_t s, int fmt, bool down, const XPlanes &xp, MoeArgs &m, int *ksplit, const float *wt_silu) {
  if (fmt != LLB_FM_Q4_K && fmt != LLB_FM_Q5_K && fmt != LLB_FM_Q6_K) return llb_fail("moe gemm: expert stacks of format %d have no kernel", fmt);
  if (m.ef % 256 || m.d % 256) return llb_fail("moe gemm: widths %d, %d are not multiples of 256", m.ef, m.d);
  GemmArgs a;
  memset(&a, 0, sizeof a);
  a.K = down ? m.nslot * m.ef : m.d;
  if (xp.K != a.K || (xp.NC != 8 && xp.NC != 16 && xp.NC != 32)) return llb_fail("moe gemm: planes of %d x %d columns, K is %d", xp.K, xp.NC, a.K);
  a.nsb = a.K / 256; a.xp = xp; a.planes = 2; a.T = m.T; a.nmat = 0;
  const int ntiles = down ? m.T * (m.d / 16) : m.T * m.nslot * (m.ef / 8);
  int ks = 1;
  const bool sel = xp.NC >= 32;
  if (down) ks = *ksplit > 0 ? *ksplit : gemm_pick_ksplit(fmt, xp.NC, ntiles, a.nsb, g_llb.sms, sel);
  ks = gemm_fix_ksplit(fmt, xp.NC, a.nsb, ks, sel);
  if (!down && ks != 1) return llb_fail("moe gemm: %d columns do not fit one K-slice", a.K);
  a.ksplit = ks;
  if (ksplit) *ksplit = ks;
  const int NT = xp.NC / 8;
#define MOE_GO(F) return NT == 1 ? launch_moe<F, 1>(s, down, a, m, ntiles, wt_silu) : NT == 2 ? launch_moe<F, 2>(s, down, a, m, ntiles, wt_silu) : launch_moe<F, 4>(s, down, a, m, ntiles, wt_silu)
  if (fmt == LLB_FM_Q4_K) MOE_GO(LLB_FM_Q4_K);
  if (fmt == LLB_FM_Q5_K) MOE_GO(LLB_FM_Q5_K);
  MOE_GO(LLB_FM_Q6_K);
#undef MOE_GO
}

int gemm_launch(cudaStream_t s, int fmt, GemmArgs &a) {
  if (gemm_prepare(fmt, a)) return -1;
  if (a.tile0[a.nmat] < 1) return 0;
  const int NT = a.xp.NC / 8;
  if (is_g3(fmt, a.xp.NC)) return launch_three(s, a);
  if (fmt == LLB_FM_Q4_K) return NT == 1 ? launch_two<LLB_FM_Q4_K, 1>(s, a) : NT == 2 ? launch_two<LLB_FM_Q4_K, 2>(s, a) : launch_two<LLB_FM_Q4_K, 4>(s, a);
  if (fmt == LLB_FM_Q5_K) return NT == 1 ? launch_two<LLB_FM_Q5_K, 1>(s, a) : NT == 2 ? launch_two<LLB_FM_Q5_K, 2>(s, a) : launch_two<LLB_FM_Q5_K, 4>(s, a);
  if (fmt == LLB_FM_Q6_K) return NT == 1 ? launch_two<LLB_FM_Q6_K, 1>(s, a) : NT == 2 ? launch_two<LLB_FM_Q6_K, 2>(s, a) : launch_two<LLB_FM_Q6_K, 4>(s, a);
  if (fmt == LLB_FM_Q8_0) return NT == 1 ? launch_two<LLB_FM_Q8_0, 1>(s, a) : NT == 2 ? launch_two<LLB_FM_Q8_0, 2>(s, a) : launch_two<LLB_FM_Q8_0, 4>(s, a);
  return llb_fail("gemm: format %d has no kernel", fmt);
}
