/*
 * llamd_cuda.h -- C ABI of libllamd_cuda.so, the B200 (sm_100a) backend for
 * llamd's quantized decode/prefill hot path.
 *
 * The entry points mirror, one for one, the `extern "C"` surface that the
 * reference's device backend crate binds (crates/llamd-rocm/src/lib.rs:73-136
 * and crates/llamd-rocm/src/forward.rs:269-618), so a `llamd-cuda` crate can
 * declare them with the same shapes. Each declaration cites the reference
 * interface it replaces.
 *
 * Conventions (same as the reference's):
 *   - `llamd_cuda_*` host-facing calls take HOST pointers unless a parameter
 *     is named d_*, synchronise before returning, and return 0 / -1.
 *   - `llamd_fwd_*` calls take DEVICE pointers, enqueue on the one stream the
 *     library owns, never synchronise, and return void. A failure is sticky
 *     and surfaces from llamd_fwd_sync() / llamd_fwd_last_error().
 *   - The caller owns every buffer; the library owns the stream, the captured
 *     graph and its grow-only scratch.
 *   - Not re-entrant: one stream, one thread at a time.
 *
 * Q6_K weights live on the device in a tiled layout (see "weights" below); the
 * bytes a caller uploads are always the reference's own 210-byte blocks.
 */
#ifndef LLAMD_CUDA_H
#define LLAMD_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLAMD_QK_K 256
#define LLAMD_Q6K_BLOCK_BYTES 210
#define LLAMD_Q8_0_BLOCK_BYTES 34
#define LLAMD_MAX_SEQ 8 /* crates/llamd-rocm/kernels/llamd_batch.hip:41 MAX_SEQ: sequences per launch of the nseq kernels */
#define LLAMD_MAX_BATCH 256 /* sequences a model can hold; a pass of more than LLAMD_MAX_SEQ takes several launches for its large matrices, or the prefill GEMM kernels */

/* ---- device discovery: crates/llamd-rocm/src/lib.rs:74-85 ------------- */
int llamd_cuda_device_count(void);
int llamd_cuda_device_info(int dev, char *name, int name_len, char *arch, int arch_len,
                           size_t *total_mem, int *sm_count, int *warp_size);
size_t llamd_cuda_free_mem(void);
/* One process drives one GPU: pick it before anything else is called. */
int llamd_cuda_set_device(int dev);
/* Message for the last failure on this thread's library state ("" if none). */
const char *llamd_cuda_last_error_string(void);

/* ---- raw device memory: crates/llamd-rocm/src/lib.rs:86-90,
 *      crates/llamd-rocm/src/forward.rs:270-277 --------------------------- */
void *llamd_cuda_upload(const void *host, size_t bytes); /* NULL on failure */
void llamd_cuda_release(void *dev);
void *llamd_fwd_alloc(size_t bytes);
void llamd_fwd_free(void *p);
int llamd_fwd_upload(void *dst, const void *src, size_t bytes);
int llamd_fwd_download(void *dst, const void *src, size_t bytes);
int llamd_fwd_memset(void *p, int value, size_t bytes);
int llamd_fwd_sync(void);
size_t llamd_fwd_free_mem(void);
int llamd_fwd_last_error(void);
int llamd_fwd_stream_init(void); /* forward.rs:552 */
/* Kernel launches issued through the library since load (graph nodes count once, at capture). */
unsigned long long llamd_fwd_launch_count(void);
/* Programmatic dependent launch of the decode-path kernels: 1 (default) lets a
 * kernel's weight prefetch overlap the previous kernel's tail; 0 serialises. */
void llamd_fwd_set_pdl(int on);
/* Batched decode (nseq > 1) of matrices too small to fill the GPU with one CTA per 256 (row, block) units: the
 * sequences are cut into groups of g per CTA (default 2; 0 = one CTA takes all nseq). Results do not depend on g. */
void llamd_fwd_set_batch_group(int g);
/* The library's stream as a cudaStream_t, for callers that time with events. */
void *llamd_fwd_stream(void);

/* Device-time stopwatch: CUDA events on the library stream (the discipline of
 * crates/llamd-rocm/kernels/llamd.hip:1120-1141). stop synchronises. */
int llamd_fwd_timer_start(void);
int llamd_fwd_timer_stop(float *ms_out);

/* ---- graph capture: crates/llamd-rocm/src/forward.rs:613-617 ----------- */
int llamd_fwd_begin_capture(void);
int llamd_fwd_end_capture(void);
int llamd_fwd_graph_launch(void);
int llamd_fwd_has_graph(void);
void llamd_fwd_graph_destroy(void);

/* ---- weights ----------------------------------------------------------
 * Device layout "T32": blocks are taken in the reference's own order
 * (row-major, `blocks` per row, experts on the slowest axis) and cut into
 * tiles of 32 blocks; a tile is 6720 bytes (= 32 x 210, so the repack is a
 * bit permutation): 12 x 32 x 16 B of 6-bit codes, 32 x 16 B of scales and
 * 32 x 2 B of f16 d. It plays the role of the reference's planar repack
 * (crates/llamd-quant/src/dot.rs:379-423, crates/llamd-rocm/src/lib.rs:685-695).
 */
size_t llamd_cuda_q6k_tiled_bytes(size_t n_blocks);
/* d_src: n_blocks x 210 B in the reference layout, on the device. */
void llamd_fwd_repack_q6k(const void *d_src, void *d_dst, size_t n_blocks);
/* The same into blocks [dst_first, dst_first+n_blocks) of a larger tiled buffer that was zero-filled. */
void llamd_fwd_repack_q6k_at(const void *d_src, void *d_dst, size_t n_blocks, size_t dst_first);
/* Host blocks in, tiled device buffer out (upload + repack + sync). NULL on failure. */
void *llamd_cuda_upload_q6k(const void *host_blocks, size_t n_blocks);
/* Inverse of the repack, for checking that no bit moved wrongly. */
void llamd_fwd_unpack_q6k(const void *d_tiled, void *d_dst, size_t n_blocks);
/* Dequantize blocks [first, first+n) of a tiled buffer to f32, with the
 * reference's arithmetic d * sc * q (crates/llamd-quant/src/lib.rs:181-226). */
void llamd_fwd_dequantize_q6k(const void *d_tiled, size_t first_block, size_t n_blocks, float *d_out);
/* Q8_0: same idea, tiles of 32 rows x 1 block. rows must be what matvec gets. */
size_t llamd_cuda_q8_0_tiled_bytes(size_t rows, size_t blocks_per_row);
void llamd_fwd_repack_q8_0(const void *d_src, void *d_dst, size_t rows, size_t blocks_per_row);
void *llamd_cuda_upload_q8_0(const void *host_blocks, size_t rows, size_t blocks_per_row);
/* crates/llamd-quant/src/lib.rs:154-162, from the tiled buffer. */
void llamd_fwd_dequantize_q8_0(const void *d_tiled, size_t rows, size_t blocks_per_row, float *d_out);

/* ---- host-facing compute: crates/llamd-rocm/src/lib.rs:91-135 ---------- */
/* d_w: tiled Q6_K, rows x blocks. aq/ad: one Q8_K activation (qs and d planes). */
int llamd_cuda_matvec_q6k_resident(const void *d_w, const int8_t *aq, const float *ad, float *out,
                                   int blocks, int rows);
/* d_w holds n_expert matrices of `rows` rows; out is [n_used][rows]. */
int llamd_cuda_matvec_grouped(const void *d_w, const int32_t *eid, const int8_t *aq, const float *ad,
                              float *out, int blocks, int rows, int n_used);
int llamd_cuda_matvec_bench(const void *d_w, const int8_t *aq, const float *ad, int blocks, int rows,
                            int iters, float *ms_out);
int llamd_cuda_matvec_grouped_bench(const void *d_w, const int32_t *eid, const int8_t *aq,
                                    const float *ad, int blocks, int rows, int n_used, int iters,
                                    float *ms_out);
int llamd_cuda_quantize_q8k(const float *x, int nblocks, int8_t *qs, float *d, int16_t *bsums);
/* f32 activations in, f32 out: quantize + matvec for `nseq` activations at
 * once (Model::matvec_quant, crates/llamd-models/src/model.rs:241-276). The
 * whole call is what a host caller pays: H2D, kernels, D2H. */
int llamd_cuda_matvec_q6k_f32(const void *d_w, const float *x, float *out, int blocks, int rows, int nseq);
/* Q8_0 weights: dequantize-then-f32-dot in the reference's order (model.rs:253-263). */
int llamd_cuda_matvec_q8_0_f32(const void *d_w, const float *x, float *out, int blocks32, int rows, int nseq);

/* ---- device-pointer ops: crates/llamd-rocm/src/forward.rs:279-612 ------ */
void llamd_fwd_quantize(const float *x, int8_t *qs, float *d, int nblocks);              /* :375 */
void llamd_fwd_quantize_bsums(const float *x, int8_t *qs, float *d, int16_t *bsums, int nblocks);
void llamd_fwd_matvec(const void *w, const int8_t *aq, const float *ad, float *out, int blocks, int rows); /* :347 */
/* nseq activations [nseq][blocks*256] / [nseq][blocks] -> out [nseq][rows]
 * (crates/llamd-rocm/src/batch.rs bop::matvec). */
void llamd_fwd_matvec_batch(const void *w, const int8_t *aq, const float *ad, float *out, int blocks,
                            int rows, int nseq);
void llamd_fwd_matvec_x3(const void *w0, const void *w1, const void *w2, const int8_t *aq,
                         const float *ad, float *o0, float *o1, float *o2, int blocks, int rows0,
                         int rows1, int rows2); /* :524 */
void llamd_fwd_matvec_x3_batch(const void *w0, const void *w1, const void *w2, const int8_t *aq,
                               const float *ad, float *o0, float *o1, float *o2, int blocks, int rows0,
                               int rows1, int rows2, int nseq);
void llamd_fwd_matvec_grouped(const void *w, const int32_t *ids, const int8_t *aq, const float *ad,
                              float *out, int blocks, int rows, int n_used); /* :355 */
void llamd_fwd_matvec_grouped_x2(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq,
                                 const float *ad, float *oa, float *ob, int blocks, int rows,
                                 int n_used); /* :539 */
/* per-expert activation aq[e], ad[e] (:365) */
void llamd_fwd_matvec_grouped_pa(const void *w, const int32_t *ids, const int8_t *aq, const float *ad,
                                 float *out, int blocks, int rows, int n_used);
/* Batched grouped forms: ids [nseq][n_used]; activations [nseq][blocks*256]
 * (x2) or [nseq][n_used][blocks*256] (pa); outputs [nseq][n_used][rows]. */
void llamd_fwd_matvec_grouped_x2_batch(const void *wa, const void *wb, const int32_t *ids,
                                       const int8_t *aq, const float *ad, float *oa, float *ob,
                                       int blocks, int rows, int n_used, int nseq);
void llamd_fwd_matvec_grouped_pa_batch(const void *w, const int32_t *ids, const int8_t *aq,
                                       const float *ad, float *out, int blocks, int rows, int n_used,
                                       int nseq);
/* Fused forms: the activation's Q8_K quantization (:375), and for the down
 * projection also silu(gate)*up (:316), happen inside the matvec. x is f32
 * [nseq][blocks*256]; gate/up are f32 [nseq*n_used][blocks*256]. Same results
 * as the separate launches. */
void llamd_fwd_matvec_f32act(const void *w, const float *x, float *out, int blocks, int rows, int nseq);
void llamd_fwd_matvec_grouped_pa_silu(const void *w, const int32_t *ids, const float *gate, const float *up,
                                      float *out, int blocks, int rows, int n_used, int nseq);
/* f32 weights [rows][k] (the router): sequential f32 dot per row (:340). */
void llamd_fwd_matvec_f32(const float *w, const float *x, float *out, int k, int rows);
void llamd_fwd_matvec_f32_batch(const float *w, const float *x, float *out, int k, int rows, int nseq);
void llamd_fwd_transpose_f32(const float *w, float *wt, int rows, int k);
void llamd_fwd_matvec_q8_0(const void *w, const float *x, float *out, int blocks32, int rows, int nseq);
/* Small and medium matrices run with their weights brought into shared memory by bulk copies whose waits are
 * bounded: 0 while every copy has arrived within its limit, else 1 + the first CTA whose wait ran out (its 32 rows
 * were not written). Synchronises the stream. No counterpart in the reference. */
int llamd_fwd_matvec_q8_0_status(void);

void llamd_fwd_embed(const void *table, int token, float *out, int blocks);              /* :279 */
void llamd_fwd_embed_meta(const void *table, const int32_t *meta, float *out, int blocks, int nseq); /* :594 */
void llamd_fwd_rms_norm_mul(const float *x, const float *w, float *out, int n, float eps, int nseq); /* :280 */
void llamd_fwd_head_rms_norm_mul(const float *x, const float *w, float *out, int n_head, int hd, float eps); /* :287 */
/* norm*w, then Q8_K of the result, one pass (:576). */
void llamd_fwd_rms_norm_quant(const float *x, const float *w, float *out, int8_t *qs, float *d, int n,
                              float eps, int nseq);
/* x + residual -> sum_out, then norm*w (f32 to out, may be NULL) and its Q8_K
 * form: the residual add of crates/llamd-runtime/src/layer.rs:170 fused into
 * the norm of :173-174. */
void llamd_fwd_add_rms_norm_quant(const float *x, const float *residual, float *sum_out, const float *w,
                                  float *out, int8_t *qs, float *d, int n, float eps, int nseq);
/* x + sum_e weights[e]*down[e] -> sum_out (the MoE combine and residual, :586,
 * e in routing order), then norm*w and its Q8_K form: a layer's tail fused
 * with the next layer's attention norm (or the output norm). */
void llamd_fwd_combine_rms_norm_quant(const float *x, const float *down, const float *weights, int n_used,
                                      float *sum_out, const float *w, float *out, int8_t *qs, float *d, int n,
                                      float eps, int nseq);
/* rope_tab: [max_pos][hd/2][2] (sin, cos) built by llamd_cuda_rope_table. */
int llamd_cuda_rope_table(float *host_out, int max_pos, int hd, float freq_base);
void llamd_fwd_rope(float *x, int pos, int n_head, int hd, const float *rope_tab);       /* :295 */
void llamd_fwd_norm_rope(float *x, const float *w, int n_head, int hd, const int32_t *meta,
                         const float *rope_tab, float eps, int nseq);                   /* :553 */
void llamd_fwd_k_norm_rope_store(float *k, const float *w, const float *v, float *kc, float *vc,
                                 int n_head_kv, int hd, int kv_dim, const int32_t *meta,
                                 const float *rope_tab, float eps, int nseq, int max_kv); /* :563 */
/* :553 and :563 in one launch: query heads and key heads together. */
void llamd_fwd_qk_norm_rope_store(float *q, const float *wq, float *k, const float *wk, const float *v, float *kc,
                                  float *vc, int n_head, int n_head_kv, int hd, const int32_t *meta,
                                  const float *rope_tab, float eps, int nseq, int max_kv);
void llamd_fwd_kv_store(float *kc, float *vc, const float *k, const float *v, int pos, int kv_dim); /* :296 */
void llamd_fwd_attention(const float *q, const float *kc, const float *vc, float *out, float *scores,
                         int n_head, int n_head_kv, int hd, int n_kv);                  /* :304 */
void llamd_fwd_attention_meta(const float *q, const float *kc, const float *vc, float *out,
                              float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta,
                              int max_kv, int nseq);                                    /* :601 */
/* No counterpart in the reference. llamd_fwd_attention for hosts that cannot
 * allocate device memory when they call (a server whose own pool owns the whole
 * GPU, a loop that must not hit the allocator's device synchronisation): the
 * score scratch is a 1 MiB array built into the library, so this call and
 * everything under it allocate nothing. q, kc, vc, out are device pointers as
 * in llamd_fwd_attention; enqueues on the library stream, does not synchronise.
 * Limits: n_head * n_kv <= 262144 (64 heads x 4096 positions), and one head's
 * score row must fit shared memory beside the K/V tiles: (hd + n_kv +
 * 128 (hd + 1)) * 4 bytes <= 200 KiB, i.e. n_kv <= 34560 at head_dim 128 (the
 * first limit is the tighter one from 8 heads up). Shapes beyond either are
 * refused with -1 and a message in llamd_cuda_last_error_string(). The call
 * also returns -1, launching nothing, while an earlier error of the library is
 * still unread (llamd_fwd_last_error / llamd_fwd_sync read and clear it): a
 * return of 0 therefore means THIS call's launches were accepted.
 * "Allocates nothing" holds from the second call on: the first call on a
 * device creates the library stream if llamd_fwd_stream_init has not, looks up
 * the array's device address (that device must be current; the lookup may
 * load the module, which is when the 1 MiB is taken) and loads the kernels.
 * Make llamd_fwd_stream_init and one warm-up call at start-up, outside the
 * host's no-allocation window and before any stream capture begins. The
 * library drives one device per process (the one its stream was made on).
 * All calls share the one array: two calls whose kernels overlap on the GPU
 * (different streams or processes' threads) race on it. Returns 0 / -1. */
int llamd_fwd_attention_noalloc(const float *q, const float *kc, const float *vc, float *out, int n_head,
                                int n_head_kv, int hd, int n_kv);
void llamd_fwd_add(const float *a, const float *b, float *out, int n);                   /* :315 */
void llamd_fwd_silu_mul(const float *gate, const float *up, float *out, int n);          /* :316 */
/* silu(gate)*up, then Q8_K of the result (fuses :316 and :375). */
void llamd_fwd_silu_mul_quant(const float *gate, const float *up, float *out, int8_t *qs, float *d, int n);
void llamd_fwd_router(const float *logits, int n_expert, int n_used, int32_t *ids, float *weights,
                      float *probs, int nseq);                                          /* :317 */
/* The router's f32 matvec (:340) and the routing (:317) in one launch. w is
 * [n_expert][k]; logits [nseq][n_expert] is required (the CTAs meet there);
 * probs may be NULL; counter is nseq zeroed words, left zeroed. */
void llamd_fwd_router_matvec(const float *w, const float *x, int k, int n_expert, int n_used, float *logits,
                             int32_t *ids, float *weights, float *probs, unsigned int *counter, int nseq);
/* The FFN norm fused in front of it (no counterpart in the reference, which launches them apart:
 * crates/llamd-rocm/src/forward.rs op::rms_norm_quant then op::router): x_out = x + residual; xn = rms_norm(x_out) *
 * w_norm; qs / d = Q8_K of xn (for the experts); logits / ids / weights = the router over xn. x_out must be a buffer
 * other than x and residual (every CTA of the launch reads them); xn_out and probs may be NULL. Same bits as
 * llamd_fwd_add_rms_norm_quant followed by llamd_fwd_router_matvec. */
void llamd_fwd_norm_router(const float *w, const float *x, const float *residual, float *x_out, const float *w_norm,
                           float *xn_out, int8_t *qs, float *d, int k, float eps, int n_expert, int n_used, float *logits,
                           int32_t *ids, float *weights, float *probs, unsigned int *counter, int nseq);
void llamd_fwd_moe_combine(const float *down, const float *weights, float *out, int n_used, int n_embd); /* :325 */
void llamd_fwd_moe_combine_add(const float *down, const float *weights, const float *residual,
                               float *out, int n_used, int n_embd, int nseq);           /* :586 */
void llamd_fwd_argmax(const float *x, int n, float *scratch_v, int32_t *scratch_i, int32_t *out,
                      int nblocks, int nseq);                                           /* :332 */

/* Expert scatter plan (crates/llamd-vulkan/shaders/moe_group.comp:40-82):
 * counting sort of the nseq*n_used (token, slot) pairs by expert. Within an
 * expert, pairs are in ascending pair order. */
void llamd_fwd_moe_group(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart,
                         int32_t *gcount, int32_t *ptoken, int32_t *pslot);
/* The same plus a work list for the expert-major matvec: entries
 * (expert, first pair, count <= 8), 3 ints each, and their number. */
void llamd_fwd_moe_group_work(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart,
                              int32_t *gcount, int32_t *ptoken, int32_t *pslot, int32_t *work,
                              int32_t *n_work);

/* ---- many tokens at once: the prefill path of VulkanModel::run
 *      (crates/llamd-runtime/src/vulkan_model.rs:378-853) ------------------- */
/* Up to three matrices (w1/w2 may be NULL) against ntok activations
 * [ntok][blocks*256]; outputs [ntok][rows_i]. Weights are reused for 8 tokens
 * per CTA. */
void llamd_fwd_matvec_tokens(const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad,
                             float *o0, float *o1, float *o2, int blocks, int rows0, int rows1, int rows2, int ntok);
/* Expert-major grouped matvec over the plan of llamd_fwd_moe_group_work
 * (q6k_expert_major.comp / q6k_expert_major_pa.comp): pair p reads activation
 * aq[act_map[p]] (ptoken for gate/up, pslot for down) and writes
 * out[pslot[p]][rows]. wb/ob may be NULL; max_items >= npair/8 + n_expert. */
void llamd_fwd_expert_major(const void *wa, const void *wb, const int32_t *work, const int32_t *n_work, int max_items,
                            const int32_t *act_map, const int32_t *pslot, const int8_t *aq, const float *ad,
                            float *oa, float *ob, int blocks, int rows, int n_expert);
/* The same two on the integer tensor path (mma.sync s8 x s8 -> s32 per
 * (block, residue) slice, f32 scaling per slice as crates/llamd-vulkan/shaders/
 * q6k_expert_cm.comp:18-31 does per 16-K group); results identical to the two
 * above. Activations are the residue-major words llamd_fwd_q8k_residue_major
 * makes from Q8_K quants; the expert form takes gstart/gcount of the plan. */
void llamd_fwd_q8k_residue_major(const int8_t *aq, void *aq_rm, size_t nblocks);
void llamd_fwd_gemm_tokens(const void *w0, const void *w1, const void *w2, const void *aq_rm, const float *ad, float *o0,
                           float *o1, float *o2, int blocks, int rows0, int rows1, int rows2, int ntok);
void llamd_fwd_expert_gemm(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount,
                           const int32_t *act_map, const int32_t *pslot, const void *aq_rm, const float *ad, float *oa,
                           float *ob, int blocks, int rows, int n_expert);
/* QK-norm/RoPE/KV-store and attention for the ntok tokens of one tile: every
 * row is a position (meta[2i+1]) of ONE sequence whose cache is kc/vc.
 * scores: [ntok][n_head][max_kv] floats. */
void llamd_fwd_qk_norm_rope_store_tile(float *q, const float *wq, float *k, const float *wk, const float *v, float *kc,
                                       float *vc, int n_head, int n_head_kv, int hd, const int32_t *meta,
                                       const float *rope_tab, float eps, int ntok);
void llamd_fwd_attention_tile(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head,
                              int n_head_kv, int hd, const int32_t *meta, int max_kv, int ntok);
/* ---- a binary16 K/V cache (no counterpart in the reference, whose caches are f32, crates/llamd-runtime/src/kv.rs:27-170;
 * the benchmark configuration names an f16 cache). kc / vc hold IEEE binary16 elements, same shapes as above. A value is
 * rounded to nearest-even ONCE, by the store; every load widens it exactly, and all arithmetic stays f32 in the
 * reference's order, so results are those of the f32 path over a cache of f16-representable values.
 * llamd_fwd_kv16_expand widens rows [0, n_pos) of both caches into f32 buffers: what the tiled prefill attention
 * (llamd_fwd_attention_prefill / _tile) reads in place of an f32 cache. */
void llamd_fwd_qk_norm_rope_store_kv16(float *q, const float *wq, float *k, const float *wk, const float *v, void *kc,
                                       void *vc, int n_head, int n_head_kv, int hd, const int32_t *meta,
                                       const float *rope_tab, float eps, int nseq, int max_kv);
void llamd_fwd_qk_norm_rope_store_tile_kv16(float *q, const float *wq, float *k, const float *wk, const float *v, void *kc,
                                            void *vc, int n_head, int n_head_kv, int hd, const int32_t *meta,
                                            const float *rope_tab, float eps, int ntok);
void llamd_fwd_attention_meta_kv16(const float *q, const void *kc, const void *vc, float *out, float *scores, int n_head,
                                   int n_head_kv, int hd, const int32_t *meta, int max_kv, int nseq);
void llamd_fwd_kv16_expand(const void *kc16, const void *vc16, float *kc32, float *vc32, int n_pos, int kv_dim);
/* ---- one decode launch fewer per layer: QK-norm, RoPE and the K/V store inside the attention-scores launch ----
 * (no counterpart in the reference, which launches op::norm_rope, op::k_norm_rope_store and op::attention_meta apart,
 * crates/llamd-rocm/src/forward.rs). q, k, v are the projections as the matvec left them (not modified); the K and V rows
 * of each sequence's position meta[2s+1] are stored; out gets the attention output. Same bits as
 * llamd_fwd_qk_norm_rope_store followed by llamd_fwd_attention_meta (_kv16: over binary16 caches). */
void llamd_fwd_attention_rope_meta(const float *q, const float *wq, const float *k, const float *wk, const float *v, float *kc,
                                   float *vc, float *out, float *scores, int n_head, int n_head_kv, int hd,
                                   const int32_t *meta, const float *rope_tab, float eps, int max_kv, int nseq);
void llamd_fwd_attention_rope_meta_kv16(const float *q, const float *wq, const float *k, const float *wk, const float *v,
                                        void *kc, void *vc, float *out, float *scores, int n_head, int n_head_kv, int hd,
                                        const int32_t *meta, const float *rope_tab, float eps, int max_kv, int nseq);
/* ---- two decode launches fewer per layer: the producer's last CTA does the small follow-up op itself ----
 * llamd_fwd_matvec_grouped_x2_silu_quant = llamd_fwd_matvec_grouped_x2 (crates/llamd-rocm/src/forward.rs: planar_grouped_x2)
 * followed by llamd_fwd_silu_mul_quant of oa, ob: qs [slots][rows], d [slots][rows/256]; rows % 256 == 0.
 * llamd_fwd_attention_meta_quant = llamd_fwd_attention_meta followed by llamd_fwd_quantize of out:
 * qs [nseq][n_head*hd], d [nseq][n_head*hd/256]; needs the scores buffer.
 * counter: one zero-initialised word per slot / per sequence; a launch leaves them at zero again. Same bits as the
 * separate launches. */
void llamd_fwd_matvec_grouped_x2_silu_quant(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq,
                                            const float *ad, float *oa, float *ob, unsigned int *counter, int8_t *qs,
                                            float *d, int blocks, int rows, int n_used, int nseq);
void llamd_fwd_attention_meta_quant(const float *q, const float *kc, const float *vc, float *out, float *scores,
                                    int n_head, int n_head_kv, int hd, const int32_t *meta, int max_kv, int nseq,
                                    unsigned int *counter, int8_t *qs, float *d);

/* ---- the same matmuls at TOLERANCE level on tcgen05 (f16 tiles dequantized in shared memory, f32
 * accumulators in TMEM, one accumulation over all of K). Outputs agree with llamd_fwd_gemm_tokens /
 * llamd_fwd_expert_gemm within QUANTIZED_MATMUL = 1e-3 (crates/llamd-core/src/tolerance.rs:41-66), not bit for bit.
 * act16: the activations as two f16 terms each, from llamd_fwd_act_f16_rm: blocks*256*4 bytes per index. max_count bounds the tokens of any one
 * expert (the number of pairs always does). llamd_fwd_gemm_tc_status synchronises and returns 0 unless a wait
 * inside a kernel ran out (outputs then incomplete). */
void llamd_fwd_act_f16_rm(const int8_t *aq, const float *ad, void *act16, size_t nblocks);
void llamd_fwd_gemm_tokens_tc(const void *w0, const void *w1, const void *w2, const void *act16, float *o0, float *o1,
                              float *o2, int blocks, int rows0, int rows1, int rows2, int ntok);
void llamd_fwd_expert_gemm_tc(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount,
                              const int32_t *act_map, const int32_t *pslot, const void *act16, float *oa, float *ob,
                              int blocks, int rows, int n_expert, int max_count);
int llamd_fwd_gemm_tc_status(void);

/* ---- expert parallelism (no counterpart in the reference, which has no multi-GPU path) ----
 * After llamd_cuda_ep_init (llamd_cuda_model.h) this rank holds experts [own_lo, own_hi) of every expert tensor,
 * stored from local index 0. The owned-range matvecs are llamd_fwd_matvec_grouped_x2 / _pa over n_slots flat
 * slots (ids[n_slots], slot s reading activation s / n_used or its own): a slot whose expert is not owned is
 * skipped and its output rows are left untouched.
 * dispatch: all-gather of every rank's (ids[n_used], ad[blocks], aq[blocks*256]) into [world][...] buffers.
 * combine: block t of send ([world][n_used][n_embd]) goes to rank t, block r of recv comes from rank r; then
 * down[slot] = recv[owner(ids[slot])][slot]: the eight expert outputs in routing order, as on one GPU.
 * Both enqueue NCCL calls on the library stream and may be captured into the graph. */
void llamd_fwd_matvec_grouped_x2_owned(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                                       float *oa, float *ob, int blocks, int rows, int n_used, int n_slots, int own_lo,
                                       int own_hi);
void llamd_fwd_matvec_grouped_pa_owned(const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out,
                                       int blocks, int rows, int n_slots, int own_lo, int own_hi);
void llamd_fwd_ep_dispatch(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *ids_all, float *ad_all,
                           int8_t *aq_all, int n_used, int blocks);
void llamd_fwd_ep_combine(const float *send, float *recv, const int32_t *ids, float *down, int n_used, int n_embd,
                          int n_expert);

/* ---- the operations of `llamd_tensor::Backend` (crates/llamd-tensor/src/lib.rs:148-174) in their general row-wise
 * form, with CpuBackend's arithmetic (crates/llamd-cpu/src/lib.rs:55-225): every sum one in-order f32 chain from +0.0.
 * Device pointers; `add` is llamd_fwd_add above. ---- */
void llamd_fwd_rms_norm_rows(const float *x, float *out, int n, int rows, float eps); /* cpu/lib.rs:55-75: no weight */
void llamd_fwd_softmax_rows(const float *x, float *out, int n, int rows);            /* :81-101 */
void llamd_fwd_silu(const float *x, float *out, size_t n);                            /* :103-106 */
/* f32::exp as the reference's CPU path evaluates it (the host libm's expf), elementwise. The library's exponential
 * is the correctly rounded one corrected, input by input, to the host's expf: when the stream is made, every float
 * for which exp is not 1, 0 or infinite is evaluated on the device and compared with expf on the host, and the
 * inputs that differ (llamd_cuda_exp_exceptions of them) are kept in a table the kernels consult. Softmax, SiLU,
 * the router and attention are therefore bit-identical to the CPU path, not merely within an ulp of it.
 * LLAMD_EXP_TABLE=0 in the environment switches the table off (correctly rounded exp, ~1 s less start-up). */
void llamd_fwd_expf(const float *x, float *out, size_t n);
long long llamd_cuda_exp_exceptions(void);
int llamd_cuda_exp_window_on(void); /* > 0: only results this close (in 2^-29 ulp) to a rounding midpoint are looked up; measured at start-up */
void llamd_fwd_mul(const float *a, const float *b, float *out, size_t n);             /* :112-114 */
void llamd_fwd_scale(const float *x, float by, float *out, size_t n);                 /* :116-118 */
/* w [m rows][k], x [n rows][k] -> out [n][m], out[j*m+i] (:126-149); any k. */
void llamd_fwd_matmul_f32(const float *w, const float *x, float *out, int k, int m, int n);
/* NeoX pairing (i, i + head_dim/2) per head (:158-209). sincos [rows][head_dim/2][2] = (sin, cos) of
 * theta = pos*freq_scale / freq_base^(2i/head_dim), tabulated by the caller with the host libm the reference calls. */
void llamd_fwd_rope_rows(const float *x, float *out, int row_len, int rows, int head_dim, const float *sincos);
/* out[i] = table[ids[i]] (:211-224); the caller has refused ids outside the table. */
void llamd_fwd_get_rows_f32(const float *table, const uint32_t *ids, float *out, int row_len, int n_ids);

/* llamd_fwd_matvec_f32 for the ntok tokens of a tile: out[t][row] = fold(-0.0, +) of w[row][i]*x[t][i], i
 * ascending (crates/llamd-models/src/model.rs:253-263). w [rows][k] f32, x [ntok][k], out [ntok][rows]; k % 4 == 0. */
void llamd_fwd_matmul_f32_tokens(const float *w, const float *x, float *out, int k, int rows, int ntok);
/* The same result from register-tiled kernels (scores, softmax rows, weighted
 * sum of V: each output element still one in-order chain of unfused multiply
 * and add, as `attend` in crates/llamd-cpu/src/lib.rs computes it).
 * n_kv_max bounds pos+1 over the tile's tokens. Shapes the tiled kernels do
 * not cover fall through to llamd_fwd_attention_tile. */
void llamd_fwd_attention_prefill(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head,
                                 int n_head_kv, int hd, const int32_t *meta, int max_kv, int ntok, int n_kv_max);

#ifdef __cplusplus
}
#endif
#endif /* LLAMD_CUDA_H */
