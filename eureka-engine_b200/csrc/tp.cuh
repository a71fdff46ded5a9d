// tp.cuh -- the tensor-parallel collective (tp.cu) and the partition of one model over the ranks.
#pragma once
#include <stddef.h>

int tp_rank(void);
int tp_size(void);
int tp_allreduce(float *buf, size_t n);   // sum over the ranks, in place, on the library's stream (NCCL)
// the one-shot all-reduce over peer memory (when the peer buffers are open): whole[n] = sum over ranks of the sum over the
// ns K-slices of part, one kernel on the library's stream
bool tp_peer_ready(void);
int tp_allreduce_parts(const float *part, int ns, long long stride, size_t n, float *whole);
int tp_host_barrier(void);   // all ranks meet on the host (no-op on one rank)
int tp_wait_errors(void);
int tp_wait_errors_clear(void);

// A set of half-open ranges [start, start + count) of rows or columns, in order.
struct TpSel {
  int n = 0;
  int start[8] = {0}, count[8] = {0};
  int total() const { int t = 0; for (int i = 0; i < n; i++) t += count[i]; return t; }
  void add(int s, int c) { start[n] = s; count[n] = c; n++; }
};
// What rank r of n owns of a model (tools/qwen35_engine.c:581-726 for the shapes):
//   query heads [h0, h0 + H_l); kv heads [kv0, kv0 + KV_l) (replicated when n > KV: the one head its queries read);
//   FFN columns [f0, f0 + f_l), whole super-blocks, the first f_sb % n ranks one super-block more;
//   DeltaNet q/k groups [g0, g0 + GK_l) and the value heads that read them: value head hh reads group hh % GK
//   (:621-626), so the rank owns heads rep * GK + g for its groups g and every repeat rep.
struct TpPlan {
  int rank, size;
  int H_l, h0, KV_l, kv0, f_l, f0, GK_l, g0, TR_l, reps;
};
int tp_plan(int rank, int size, int H, int KV, int f, int GK, int TR, TpPlan *p);   // -1 (and a message) if the model does not split that way
