/* llb_b200.h -- C ABI of libllb_b200.so, a B200 (sm_100a) implementation of the
 * speculative-decoding path of phenomenon0/eureka-engine.
 *
 * Plain C: integers, sizes, device addresses as 64-bit integers (the reference's llb_b200_dptr,
 * host/llb_backend.h:7-9) and host pointers.  Every call returns 0 / a handle on success and
 * -1 / 0 on failure with llb_b200_last_error() holding the reason; nothing falls back to the CPU.
 * All work is queued on one in-order stream per process (the reference's null-stream contract,
 * host/llb_backend.h:14-18): each call sees the effects of every earlier one.
 *
 * Three layers, bottom up:
 *   1. backend primitives      -- what host/llb_backend.h:7-34 asks of a backend
 *   2. operator entry points   -- the T-row leaves of tools/payload-spec*.patch, one call each
 *   3. llb_spec_*              -- the whole draft -> verify -> accept -> commit cycle of
 *                                 host/llb_host.c:1902-1950 on the device
 */
#ifndef LLB_B200_H
#define LLB_B200_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef unsigned long long llb_b200_dptr; /* a device address; the type host/llb_backend_cuda.h:5 gives llb_dptr */

#if defined(__GNUC__)
#define LLB_API __attribute__((visibility("default")))
#else
#define LLB_API
#endif

/* weight formats: the reference registry, host/llb_formats.h:4-15 */
enum { LLB_F32 = 0, LLB_Q8_0 = 1, LLB_Q4_K = 3, LLB_Q6_K = 4, LLB_Q5_K = 9 };

/* ---- 1. backend primitives ------------------------------------------------------------------ */
/* Binds the process to a GPU and creates the library's stream.  One device per process: a second call with the
 * same ordinal is a no-op, with another ordinal it fails ("already bound"). */
LLB_API int llb_b200_init(int device);
LLB_API const char *llb_b200_last_error(void);
LLB_API int llb_b200_sm_count(void);
LLB_API llb_b200_dptr llb_b200_alloc_zero(size_t bytes);      /* host/llb_backend.h:25-26, host/llb_backend_cuda.h:186-191 (0 on failure) */
LLB_API int llb_b200_free(llb_b200_dptr p);
LLB_API int llb_b200_zero(llb_b200_dptr p, size_t bytes);     /* host/llb_backend.h:27, host/llb_backend_cuda.h:193-196 */
LLB_API int llb_b200_copy(llb_b200_dptr d, llb_b200_dptr s, size_t bytes);        /* host/llb_backend.h:28, host/llb_backend_cuda.h:204-207 (device to device, in order) */
LLB_API int llb_b200_write(llb_b200_dptr d, const void *h, size_t bytes);    /* host/llb_backend.h:29, host/llb_backend_cuda.h:210-213 */
LLB_API int llb_b200_read(void *h, llb_b200_dptr p, size_t bytes);           /* host/llb_backend.h:30-31, host/llb_backend_cuda.h:198-201 (synchronises) */
LLB_API int llb_b200_sync(void);                                        /* host/llb_backend_cuda.h:216-219 */
LLB_API llb_b200_dptr llb_b200_stream(void);                  /* the cudaStream_t all calls queue on, for event timing */

/* The launch half of the contract.  A kernel is fetched by name (the reference: cuModuleGetFunction(&h, gpu_lib,
 * "llb_spec_gu3"), tools/payload-spec.patch:9-23) and launched with gx * gy blocks of bx threads, sm bytes of
 * dynamic shared memory and `na` arguments, each the address of a host variable copied at the call
 * (LLB_LAUNCH / LLB_LAUNCH_SM, host/llb_backend.h:9-24; llb_launch, host/llb_backend_cuda.h:86-106).  Reachable by
 * name are the library's leaves with plain argument lists:
 *   llb_b200_k_dequant_rows (int fmt, W, int cols, const int *row_ids or 0, float *out)     grid (<= 64, rows), block 256
 *   llb_b200_k_sum_parts    (const float *parts, int nsplit, long long stride, int n, float *out)   grid ((n + 255) / 256, 1), block 256
 *   llb_b200_k_repack_q6k   (src 210-byte blocks, dst 224-byte blocks, size_t nblocks)
 *   llb_b200_k_xp_from_f32  (const float *x, int K, int planes, planes descriptor by value)
 * Any other name -- the reference's kernel names included, whose argument lists carry its two-plane int8
 * activations -- returns NULL; a launch with a NULL kernel or a wrong argument count returns -1 and queues nothing. */
typedef struct llb_b200_kernel llb_b200_kernel;
LLB_API const llb_b200_kernel *llb_b200_kernel_by_name(const char *name);
LLB_API int llb_b200_launch(const llb_b200_kernel *k, unsigned gx, unsigned gy, unsigned bx, unsigned sm, void **args, unsigned na);
/* The recorder of host/llb_backend_cuda.h:125-184 (llb_graph_begin / llb_graph_end / llb_graph_bail): launches made
 * between begin and end are recorded, then run as ONE CUDA graph; a step with the kernel sequence of one of the 16 cached
 * graphs updates that graph's nodes instead of building a new one; at most 2048 launches a step.  A memory primitive
 * called while recording first runs what was recorded ("bail"), as in the reference.  Only llb_b200_launch records:
 * do not call operator or llb_spec_* entry points between begin and end.  stats: graphs built, steps replayed,
 * steps that re-used a cached graph, bails. */
LLB_API int llb_b200_graph_begin(void);
LLB_API int llb_b200_graph_end(void);
LLB_API int llb_b200_graph_bail(void);
LLB_API void llb_b200_graph_stats(unsigned long long out[4]);

/* ---- 2. operator entry points --------------------------------------------------------------- */
/* Bytes of a [rows x cols] matrix in the device layout (Q6_K super-blocks are padded from 210 to
 * 224 bytes at upload; every other format is stored as in a pack). */
LLB_API size_t llb_b200_weight_bytes(int fmt, int rows, int cols);
/* Pack bytes (host pointer, or device address when src_on_device) -> device layout at dst. */
LLB_API int llb_b200_weight_upload(int fmt, int rows, int cols, const void *src, int src_on_device, llb_b200_dptr dst);
/* Bit-exact dequantisation of `nrows` rows (row_ids on the device, or 0 for rows 0..nrows-1) into
 * f32 [nrows][cols].  Replaces llb_embedk / deq_row (tools/payload-kpair.patch:526,
 * tools/qwen35_engine.c:233-327). */
LLB_API int llb_b200_dequant(int fmt, int rows, int cols, llb_b200_dptr w, llb_b200_dptr row_ids, int nrows, llb_b200_dptr out_f32);

/* Activation planes of a T-row GEMM input (replaces the two-plane int8 quantiser llb_t_q8x2,
 * tools/payload-spec2.patch:126-145).  `planes` = 2 keeps about 22 bits of each f32 value in two
 * fp16 columns (T <= 8); `planes` = 1 takes up to 16 bf16 rows as they are. */
typedef struct llb_xp llb_xp;
LLB_API llb_xp *llb_b200_xp_new(int K, int T, int planes);
LLB_API void llb_b200_xp_free(llb_xp *xp);
LLB_API int llb_b200_xp_set_f32(llb_xp *xp, llb_b200_dptr x_f32 /* [T][K] */);
LLB_API int llb_b200_xp_set_bf16(llb_xp *xp, llb_b200_dptr x_bf16 /* [T][K] */);

/* Y_i[t][r] = sum_c W_i[r][c] x[t][c] for up to four matrices of one format sharing x
 * (replaces llb_spec_gu / _re / _q8 / _q6, tools/payload-spec.patch:226-236).
 * out_i: f32 [T][rows_i].  ksplit = 0 picks the K-split; scratch for the partial sums is internal. */
LLB_API int llb_b200_gemm(int fmt, int nmat, const llb_b200_dptr *w, const int *rows, const llb_b200_dptr *out, int K, const llb_xp *xp,
                  int ksplit);
/* Q4_K GEMMs with T <= 4 on the tcgen05 kernel (weights unpacked into tensor memory, tcgen05.mma) instead
 * of the mma.sync one; returns the previous setting.  Also set by LLB_GEMM3=1 at llb_b200_init.  Off by
 * default: at the 27B shapes the mma.sync kernel is the faster of the two.  A speculative engine keeps the
 * kernels it was opened with. */
LLB_API int llb_b200_use_tcgen05(int on);
/* The SwiGLU FFN of engines opened from now on as ONE launch (gate|up GEMM, grid-wide barrier, silu(gate) * up built in
 * shared memory, down GEMM) instead of three; returns the previous setting.  Also LLB_FFN_FUSED=1 at llb_b200_init.  Off by
 * default: measured no faster at the 27B shape.  Applies where gate and up are Q4_K and T <= 4. */
LLB_API int llb_b200_use_fused_ffn(int on);
/* 1 when a bounded wait inside a kernel (an mbarrier of the tcgen05 GEMM, the fused FFN's grid barrier) has run out since
 * llb_b200_init: the results of that launch are not valid.  0 otherwise; -1 on a CUDA error. */
LLB_API int llb_b200_wait_errors(void);
/* Puts that status back to 0. */
LLB_API int llb_b200_wait_errors_clear(void);
/* Failure-detection check: one small launch whose only wait can never be satisfied -- which 0: an mbarrier nobody arrives
 * on, waited for with the tcgen05 kernels' own bounded wait; which 1: the fused FFN's grid barrier told to expect a block
 * that does not exist -- with a limit of `limit` tries (1..100000) instead of the kernels' 2^22.  The wait runs out, the
 * kernel sets the status word and returns: afterwards llb_b200_wait_errors() is 1 and the device keeps working.  Returns 0
 * when the launch completed. */
LLB_API int llb_b200_wait_selftest(int which, int limit);
/* The same through HOST buffers: bf16 x [T][K] in, f32 y [T][rows] out, copies included. */
LLB_API int llb_b200_gemm_host(int fmt, llb_b200_dptr w, int rows, int K, const void *x_bf16, int T, float *y, llb_xp *xp,
                       llb_b200_dptr x_dev, llb_b200_dptr y_dev);

/* The prompt path's dense GEMM alone (replaces the reference's chunked tensor-core prefill GEMM, tools/pf27/pfmm.cuh:311-384):
 * Y[r][n] = sum_c W[n][c] x[r][c] for R <= 256 rows (two units of 128 against every dequantised weight stage) of f32 activations x [R][K] against a weight matrix in the device
 * layout, out f32 [R][rows]; tcgen05.mma with both operands as two fp16 planes (about 22 bits) and fp32 sums in tensor memory.  ksplit = 0
 * picks the K-split (at most K / 256 slices of whole super-blocks).  Synchronises; scratch is allocated and freed inside the call. */
LLB_API int llb_b200_pf_gemm(int fmt, llb_b200_dptr w, int rows, int K, llb_b200_dptr x_f32, int R, llb_b200_dptr out_f32, int ksplit);

/* Y[t][r] = sum_c W[r][c] x[t][c] for callers that are not allowed to allocate.  No counterpart in the
 * reference.  Meant for hosts that fix a library's memory at start-up and forbid driver allocations
 * afterwards (a serving process that cannot afford cudaMalloc's device-wide synchronisation, a plugin
 * sandbox that denies it).  x: f32 [T][K], out: f32 [T][rows], w: device layout, all caller-owned.
 * Planes and K-slice partial sums live in a fixed 8.5 MB array inside the library (held on every GPU that
 * loads it until exit); the call itself makes no cudaMalloc / cudaFree / allocating library call.
 * Limits: K a multiple of 256 up to 8192, T <= 4, (K-slices x T x rows) <= 2 Mi floats; anything larger
 * returns -1 with the reason.  The first call on a device looks up the array's device address
 * (cudaGetSymbolAddress): make that call before any stream capture begins.  All calls share the one array,
 * so two calls whose GPU work overlaps (different streams, different threads) race. */
LLB_API int llb_b200_gemm_noalloc(int fmt, llb_b200_dptr w, int rows, int K, llb_b200_dptr x_f32, int T, llb_b200_dptr out_f32);

/* ---- 3. the speculative cycle ----------------------------------------------------------------- */
/* Replaces host/llb_host.c:1474-1950 for greedy decoding with either of the reference's drafters.
 * index_text: the pack's index.tsv (tools/qwen35_engine.c:379-433); pack: pack.bin bytes (host, or a
 * device address when pack_on_device); mtp: the MTP drafter as an AUX1 or MTP1 image
 * (host/llb_host.c:1525-1603), or NULL: with k > 0 the cycle then drafts by prompt lookup over the token
 * history (spec_draft, host/llb_host.c:1655-1676; 1 + found rows per cycle); k: drafts per cycle (0..7, LLB_SPEC);
 * max_ctx: positions of KV kept per full-attention layer; layers: > 0 truncates the model like the
 * reference engine's --layers. */
typedef struct llb_spec llb_spec;
LLB_API llb_spec *llb_spec_open(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp,
                                size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers);
/* Tensor parallelism over the GPUs of one box (the reference is single-GPU, docs/limits.md:96; this is the split its
 * benchmark configuration asks for).  One process per GPU.  Rank 0 makes a 128-byte id with llb_b200_tp_unique_id and the
 * host program hands it to the other ranks; every rank then calls llb_b200_tp_init (after llb_b200_init) and opens the
 * engine with llb_spec_open_tp(..., tp_size).  nccl_path: the NCCL library to load at run time (NULL: libnccl.so.2 as the
 * process finds it).  A rank keeps its share of the column-split projections (attn_q by query head, attn_k / attn_v by kv
 * head, attn_qkv / attn_gate / ssm_beta / ssm_alpha by DeltaNet group, ffn_gate / ffn_up by FFN column) and of the
 * row-split ones (attn_output, ssm_out, ffn_down), whose [T, d_model] results are summed by an NCCL all-reduce on the
 * library's stream, two per layer, inside the cycle's CUDA graph.  Embedding, head and norms are replicated, so every rank
 * emits the same tokens.  All ranks must make the same calls in the same order.  Heads, kv heads (or ranks per kv head),
 * DeltaNet groups and FFN super-blocks must split tp_size ways; routed-expert models and the dense prompt path are not split. */
LLB_API int llb_b200_tp_unique_id(const char *nccl_path, void *id128);
LLB_API int llb_b200_tp_init(const char *nccl_path, int rank, int size, const void *id128);
LLB_API void llb_b200_tp_finalize(void);
/* The library's own all-reduce instead of NCCL's: ONE kernel per all-reduce that adds the projection's K-slices, stores the
 * rank's [T, d_model] tile into a slot of every peer's buffer (plain stores through a peer mapping over NVLink; no multicast,
 * no multimem), raises a flag beside it, waits -- bounded, llb_b200_wait_errors reports a wait that ran out -- for the peers'
 * flags and adds the slots in rank order.  Every rank allocates its buffer and gets a 64-byte inter-process handle for it
 * (llb_b200_tp_peer_alloc, after llb_b200_tp_init); the host program gathers the handles of all ranks in rank order and
 * every rank opens them (llb_b200_tp_peer_open).  Engines opened afterwards use the peer buffers; the ranks meet on the host
 * (a four-byte NCCL all-reduce) at the start of every call that enqueues passes, so the device-side waits only bridge the
 * skew of ranks running in step. */
LLB_API int llb_b200_tp_peer_alloc(void *handle64);
LLB_API int llb_b200_tp_peer_open(const void *handles, int n);
LLB_API int llb_b200_tp_peer_active(void);
LLB_API llb_spec *llb_spec_open_tp(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp,
                                   size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers, int tp_size);
/* Sampling-mode verify (the llb_sampler contract beyond greedy, host/llb_sampler.h).  The fields are LlbSmpParams' (:38-52;
 * n_logprobs and max_tokens, which the path does not use, left out): temp <= 0 greedy; top_p >= 1, top_k <= 0, min_p <= 0,
 * repeat_last_n <= 0 switch their stage off.  With parameters that leave the argmax untouched (llb_smp_is_argmax) the cycle is
 * the greedy one.  Otherwise every row of a verify pass gets, on the device and inside the cycle's graph, the token
 * llb_smp_verify (a row with a draft; both drafters are deterministic, so q is one-hot) or llb_smp_sample (the row without)
 * would return for its logits, with the reference's counter RNG (seed, position, draw), and the accept step takes those
 * tokens in place of the argmax: the emitted stream is distributed as plain sampling's, whatever the drafter proposes.
 * Limits, refused by name: top_k <= 256; top_p < 1 needs top_k; penalty window <= 256; min_keep above what min_p keeps.
 * Must be set before llb_spec_prefill; the result record's top-2 words then carry (emitted id, its raw logit, argmax's
 * runner-up id and value). */
typedef struct {
  float temp, top_p, min_p;
  int top_k;
  float repeat_penalty;
  int repeat_last_n;
  float presence, frequency;
  unsigned long long seed;
  int min_keep;
  int n_bias;
  int bias_ids[64];
  float bias_vals[64];
} llb_smp_params;
LLB_API int llb_spec_set_sampler(llb_spec *m, const llb_smp_params *p);
/* 0, or the device sampler's error word since the engine was opened (2: min_keep above what min_p kept; 3: a token out of range). */
LLB_API int llb_spec_sampler_errors(llb_spec *m);
/* Test entry: the device sampler on T rows of logits given on the device (f32 [T][V]): drafts[T] (-1: a plain draw),
 * pos[T] (the position each token will occupy), the penalty windows win[T][256] with their lengths nwin[T] (host arrays);
 * tok_out / acc_out / val_out[T] on the host. */
LLB_API int llb_b200_smp_rows(const llb_smp_params *p, llb_b200_dptr logits, int T, int V, const int *drafts, const long long *pos,
                              const int *win, const int *nwin, int *tok_out, int *acc_out, float *val_out);

/* Several streams per engine (multi-stream batching inside one GPU; the reference's analogue is its prefill-only
 * LLB_BATCH, host/llb_host.c:2151-2793).  `streams` independent sequences share every weight read: a pass carries the k + 1
 * rows of each stream through every GEMM together (streams x (k + 1) <= 16 rows), while attention,
 * the DeltaNet scan, the drafter and the accept step run per stream inside the same launches, each stream on its own KV
 * cache, conv ring, state ring, control block and result ring.  A stream's tokens do not depend on what the other
 * streams do (a row's GEMM result does not depend on its neighbours).  Prompts go in per stream, at any time; a cycle
 * advances every stream that has a prompt.  The one-stream calls (llb_spec_cycle, _generate, _pass, _run_cycles) are
 * refused by an engine of several streams; _prefill, _stats, _position and _read_state mean stream 0. */
LLB_API llb_spec *llb_spec_open_streams(const char *index_text, const void *pack, size_t pack_bytes, int pack_on_device, const void *mtp,
                                        size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers, int streams);
LLB_API int llb_spec_streams(const llb_spec *m);
/* Another engine on the weights `first` has on the device: its own k, context, streams, sequence state and graphs, no
 * second copy of the model.  Streams beyond the 16 rows of one pass go into siblings, whose passes run one after the other
 * (each streams the weights once).  Its tokens are those of an engine opened the usual way with the same k and streams, bit
 * for bit.  `first` may be closed before its siblings: the weights are freed with the last engine that uses them.
 * Refused: a tensor-parallel `first`; k > 0 where `first` was opened without the drafter the sibling would load. */
LLB_API llb_spec *llb_spec_open_sibling(llb_spec *first, int k, int max_ctx, int streams);
/* Bytes of weights the engine allocated itself (0 for a sibling). */
LLB_API size_t llb_spec_weight_bytes(const llb_spec *m);
LLB_API int llb_spec_prefill_stream(llb_spec *m, int stream, const int *ids, int n);
/* The prompts of several streams at once: streams[i] gets ids[i][0 .. n[i]-1].  The prompts' rows share the prompt passes
 * (every stream feeds its own k + 1 rows of a pass), so n_prompts prompts take about the passes of the longest one; each
 * stream ends in the state llb_spec_prefill_stream would have left it in.  A stream named twice is refused. */
LLB_API int llb_spec_prefill_streams(llb_spec *m, int n_prompts, const int *streams, const int *const *ids, const int *n);
/* One cycle of every stream that has a prompt, as one graph launch: ids_out[stream * 8 + i], i < n_out[stream], are that
 * stream's emitted tokens (n_out = 0 for a stream without a prompt); top2_out (may be NULL) [stream][8][4] words. */
LLB_API int llb_spec_cycle_streams(llb_spec *m, int *ids_out, int *n_out, uint32_t *top2_out);
/* n cycles back to back without a host round trip; tokens[stream] = tokens that stream emitted. */
LLB_API int llb_spec_run_cycles_streams(llb_spec *m, int n, int *tokens);
LLB_API int llb_spec_position_stream(const llb_spec *m, int stream);
/* The result record of a stream's last cycle: out[0..2] = p0, rows T, rows served; out[3..10] the verify inputs (the
 * committed token, then the drafts); out[11..18] every row's emitted id; out[19 + 4 r ..] = [id1, bits1, id2, bits2] of row r. */
LLB_API int llb_spec_last_record(const llb_spec *m, int stream, unsigned int *out51);
LLB_API int llb_spec_stats_stream(const llb_spec *m, int stream, unsigned long long *out19);
LLB_API int llb_spec_read_state_stream(llb_spec *m, int stream, int what, int il, int pos, float *out, size_t n);

/* Test entry (no GPU needed): rank `rank` of `size`'s share of a model with H query heads, KV kv heads, FFN width f, GK
 * DeltaNet groups and TR value heads: out[10] = H_l, h0, KV_l, kv0, f_l, f0, GK_l, g0, TR_l, reps; -1 if it does not split. */
LLB_API int llb_b200_tp_plan(int rank, int size, int H, int KV, int f, int GK, int TR, int *out10);

/* What llb_spec_open checks before it touches the GPU, callable without one: the index parses, its #cfg values are
 * complete and consistent (no zero divisor, widths that agree), and every tensor's [offset, offset + bytes) lies inside
 * a pack of pack_bytes bytes -- a truncated pack.bin or a stale index.tsv is an error naming the tensor. */
LLB_API int llb_spec_check_index(const char *index_text, size_t pack_bytes);
/* Test entry (no GPU needed): the K-split a GEMM launch of `ntiles` 16-row tiles over nsb super-blocks gets at nc plane
 * columns on `sms` SMs, and the one split fixed for a DeltaNet layer's attn_qkv launch, whose partial sums live on in
 * the conv ring across passes of both widths (0: none fits). */
LLB_API int llb_b200_gemm_ksplit(int fmt, int nc, int ntiles, int nsb, int sms);
LLB_API int llb_b200_ring_ksplit(int fmt, int nsb, int ntiles, int nc_spec, int nc_prefill, int sms);
LLB_API void llb_spec_close(llb_spec *m);
LLB_API int llb_spec_reset(llb_spec *m);                       /* host/llb_host.c:1915-1928 */
LLB_API int llb_spec_prefill(llb_spec *m, const int *ids, int n);
/* one cycle: ids_out[0 .. *n_out-1] emitted; top2_out[i] = id1, bits(v1), id2, bits(v2) of row i
 * (the reference's "logits" line, tools/qwen35_engine.c:985) */
LLB_API int llb_spec_cycle(llb_spec *m, int *ids_out, int *n_out, uint32_t *top2_out);
LLB_API int llb_spec_generate(llb_spec *m, int steps, int *ids, uint32_t *top2);
/* the reference's per-token operator (spec_pass, host/llb_host.c:1902-1950): y = [v1, id1, v2, id2] */
LLB_API int llb_spec_pass(llb_spec *m, int pos, int tok, float *y);
LLB_API int llb_spec_position(const llb_spec *m);
/* How llb_spec_prefill feeds a prompt.  mode 0 (default): every row through the T-row verify pass, eight rows a pass, at
 * the verify path's precision.  mode 1 (also LLB_PREFILL=fast in the environment at open, the reference's switch,
 * host/llb_host.c:206): all but the last k + 1 rows in chunks of 128 rows through dense tcgen05 GEMMs (operands as two fp16 planes)
 * (replaces pf_take / spec_pf / spec_take, host/llb_pf.h:551, host/llb_host.c:1831-1899): trunk K/V, conv history and
 * DeltaNet state, and the drafter's K/V rows, are left as the T-row pass would have left them, within the path's
 * tolerance.  Models with routed experts always take mode 0.  Returns the previous mode.
 * llb_spec_fast_rows: prompt rows that went through the dense path since the engine was opened. */
LLB_API int llb_spec_set_prefill(llb_spec *m, int mode);
LLB_API double llb_spec_fast_rows(const llb_spec *m);
/* n cycles enqueued back to back, no host round trip between them; returns the tokens emitted */
LLB_API int llb_spec_run_cycles(llb_spec *m, int n, int *ids, int cap);
/* measurement helpers: device time (CUDA events on the library's stream) of the verify pass alone and
 * of the largest GEMM launch; kernels per graph replay (which: 0 cycle, 2 verify pass) */
LLB_API int llb_spec_time_verify(llb_spec *m, int iters, float *ms_per_pass);
/* the verify pass timed with `rows` rows whatever the drafter found (missing rows repeat the first token); overwrites
 * those rows' cache slots: a measurement entry, to be called after the generation that matters */
LLB_API int llb_spec_time_verify_rows(llb_spec *m, int iters, int rows, float *ms_per_pass);
LLB_API int llb_spec_time_gemm(llb_spec *m, int iters, float *us_per_launch, double *bytes_per_launch);
LLB_API int llb_spec_graph_nodes(const llb_spec *m, int which);
/* one eager verify pass with an event after every op: "name\tcount\ttotal_us" lines */
LLB_API int llb_spec_profile_verify(llb_spec *m, char *buf, int cap);
/* out[19] = cycles, rows, served, drafted[8], accepted[8] by draft position (host/llb_host.c:1513-1523) */
LLB_API int llb_spec_stats(const llb_spec *m, unsigned long long *out);
LLB_API int llb_spec_read_state(llb_spec *m, int what, int il, int pos, float *out, size_t n);
/* The engine straight from a GGUF file of architecture qwen35 or qwen35moe (replaces the reference's GGUF ->
 * pack step, tools/gguf2pack.c, and its in-place reader host/llb_gguf.c:854-865): configuration from the
 * metadata keys of tools/gguf2pack.c:541-600, tensors uploaded from the mapped file (F32, Q4_K, Q5_K, Q6_K
 * verbatim; Q8_0 re-sliced from GGUF blocks to the pack's row-split layout), tied head when the file has no
 * output.weight, nextn blocks left out of the trunk.  mtp: an optional AUX1 / MTP1 drafter image as for
 * llb_spec_open; without one, a dense model's own nextn block (blk.<trunk length>.nextn.* and its attention / FFN
 * tensors) is the drafter, with the file's head over the whole vocabulary; without either, prompt lookup.
 * NULL on failure (llb_last_error). */
LLB_API llb_spec *llb_spec_open_gguf(const char *path, const void *mtp, size_t mtp_bytes, int mtp_on_device, int k, int max_ctx, int layers);
/* the index text derived from a GGUF header ("#cfg" lines, then name, file offset, bytes, rows, cols, type per
 * tensor); returns its length or -1; needs no GPU */
LLB_API int llb_b200_gguf_index(const char *path, char *buf, int cap);
LLB_API int llb_spec_read_logits(llb_spec *m, int r, float *out);
/* Test entry for models with a routed-expert FFN (host/llb_host.c:622-724 llb_moe_run; kernels llb_moe_topk,
 * llb_moe_gu, llb_moe_dn of tools/payload-moeany.patch): layer il's expert FFN alone on T normed rows h2[T][d] in
 * host memory.  out[T][d]: sum_j wt_j down_j(silu(gate_j h2) * up_j h2) + sigmoid(shared gate) * shared(h2), no
 * residual; ids, wt [T][k + 1]: the chosen experts in rank order and their weights, slot k = the shared expert (id =
 * expert count) and its gate.  Resets the sequence state. */
LLB_API int llb_spec_moe_ffn(llb_spec *m, int il, int T, const float *h2, float *out, int *ids, float *wt);

#ifdef __cplusplus
}
#endif
#endif
