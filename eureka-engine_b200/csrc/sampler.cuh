// sampler.cuh -- the device sampler's parameters and launcher (sampler.cu).
#pragma once
#include "../../include/llb_b200.h"
#include "model.cuh"

#define SMP_MAX_BIAS 64     // LLB_SMP_MAX_BIAS (host/llb_sampler.h:35)
#define SMP_MAX_TOPK 256    // the reference's own partial-selection bound (LLB_SMP_SEL, host/llb_sampler_impl.h:168)
#define SMP_MAX_WIN 256     // longest penalty window on the device

struct SmpDev {
  float temp, top_p, min_p, log_min_p;
  int top_k;
  float repeat_penalty;
  int repeat_last_n;
  float presence, frequency;
  unsigned long long seed;
  int min_keep, pen_on, n_bias;
  int bias_ids[SMP_MAX_BIAS];
  float bias_vals[SMP_MAX_BIAS];
};

int smp_prepare(const llb_smp_params *p, SmpDev *d, bool *argmax_only);
// rows blocks: engine mode takes draft / position / window of every row from the control blocks at ctl (stream geometry
// as set by ops_set_streams); test mode (ctl == null) from t_draft[rows], t_pos[rows], t_win[rows][SMP_MAX_WIN], t_nwin[rows]
int op_smp_rows(cudaStream_t s, const SmpDev &P, PartIn lg, int V, float *adj, const SpecCtl *ctl, int rows, const int *t_draft, const long long *t_pos,
                const int *t_win, const int *t_nwin, int *tok_out, float *val_out, int *acc_out, unsigned int *err);
