/* oracle/q35_oracle.h -- TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the reference algorithm for the speculative-decoding path of the Qwen3.5
 * hybrid model.  Only tests, the package smoke check and the benchmark's CPU-baseline leg may
 * load this library; the product path never does.
 *
 * What it follows (paths inside phenomenon0/eureka-engine):
 *   format leaves, trunk forward   tools/qwen35_engine.c:45-778
 *   MTP drafter (NextN block)      host/llb_host.c:1771-1829, tools/mtp27/mtp_pack.py:14-30
 *   cycle / accept / rollback      host/llb_host.c:1902-1950, tools/payload-spec2.patch:375-410
 *   greedy accept rule             host/llb_sampler_impl.h:400-405
 *   routed-expert FFN              host/llb_host.c:622-724, tools/payload-moeany.patch
 *
 * Parity pin: the trunk forward, logits and top-2 of this restatement are bit-identical to the
 * reference engine compiled from its own sources (oracle/_ref, see oracle/Makefile) on the same
 * packs; tests/golden holds vectors produced by that reference build.  The MTP drafter and the
 * cycle have no CPU code in the reference ("parity unpinned" for draft ids): they are pinned only
 * through the lossless property (spec ids == plain greedy ids).  The routed-expert FFN has no CPU code in
 * the reference either; it is pinned against the reference's float64 checker
 * (reports/metal-catchup/tools/mx_ref.py) run on this restatement's outputs (tests/golden/moe_ffn.npz).
 */
#ifndef Q35_ORACLE_H
#define Q35_ORACLE_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct Q35 Q35;

typedef struct {
  int n_layers, d_model, n_heads, n_kv_heads, head_dim, d_ff, vocab, interval, conv_kernel, ssm_state,
      ssm_groups, ssm_heads, vhd, kdc, vdc, convd, rope_dim;
  float rope_base, eps;
  int n_experts, n_used, d_expert, d_shared; /* routed-expert FFN (0 experts: dense) */
} Q35Cfg;

typedef struct {
  uint64_t cycles, rows, served;
  uint64_t drafted[8], accepted[8]; /* by draft position 1..k, as the reference's "spec:" line */
} Q35SpecStats;

void q35_threads(int n);

/* leaves */
float q35_half(uint16_t h);
void q35_deq_row(int fmt, const uint8_t *row, int cols, float *out);
float q35_dot(int fmt, const uint8_t *row, int cols, const float *x);
void q35_gemv(int fmt, const uint8_t *W, int row_bytes, int rows, int cols, const float *x, float *y);
float q35_silu(float x);
float q35_sigmoid(float x);
float q35_softplus(float x);
float q35_exp(float x);
void q35_rope(float *x, int pos, int rope_dim, float base);

/* model */
Q35 *q35_open_dir(const char *dir, int layers, int cap);
Q35 *q35_open_mem(const char *index_text, const uint8_t *pack, size_t pack_bytes, int layers, int cap);
void q35_close(Q35 *m);
void q35_cfg(const Q35 *m, Q35Cfg *out);
void q35_reset(Q35 *m);

/* trunk, one token at a time (tools/qwen35_engine.c:726-778) */
void q35_forward(Q35 *m, int tok, int pos);
const float *q35_logits(Q35 *m);            /* output_norm + head on the current residual */
const float *q35_residual(const Q35 *m);
const float *q35_hnorm(const Q35 *m);       /* output-normed hidden, valid after q35_logits */
void q35_top2(const float *z, int n, int *ids, float *vals);
const float *q35_state_S(const Q35 *m, int il);
const float *q35_state_conv(const Q35 *m, int il);
const float *q35_state_k(const Q35 *m, int il, int pos);
const float *q35_state_v(const Q35 *m, int il, int pos);

/* the routed-expert FFN of layer il on one normed row h2[d] (no residual): out[d], ids[k], wts[k + 1]
 * (host/llb_host.c:622-724, tools/payload-moeany.patch) */
int q35_moe_ffn(Q35 *m, int il, const float *h2, float *out, int *ids, float *wts);

/* plain greedy: ids[steps]; top2[steps][4] = id1, bits1, id2, bits2 (may be NULL) */
int q35_greedy(Q35 *m, const int *prompt, int np, int steps, int *ids, uint32_t *top2);

/* MTP drafter from an AUX1 or MTP1 image; speculative greedy loop with k drafts per cycle */
int q35_mtp_load(Q35 *m, const uint8_t *img, size_t bytes);
int q35_spec_greedy(Q35 *m, const int *prompt, int np, int steps, int k, int *ids, uint32_t *top2,
                    Q35SpecStats *st);
/* prompt-lookup drafter (host/llb_host.c:1655-1676) and the greedy loop that uses it in place of the MTP head */
int q35_lookup_draft(const int *hist, int pos, int k, int *out);
int q35_spec_lookup(Q35 *m, const int *prompt, int np, int steps, int k, int *ids, uint32_t *top2, Q35SpecStats *st);
/* one drafter call for tests: n rows at positions pa.., tokens tk, hidden rows hs[n][d];
 * returns the draft id; hn_out[n][d] gets the drafter's own normed hidden */
int q35_mtp_rows(Q35 *m, int n, int pa, const int *tk, const float *hs, float *hn_out);

#ifdef __cplusplus
}
#endif
#endif
