/*
 * llamd_cuda_model.h -- C ABI of the resident decode model in libllamd_cuda.so.
 *
 * The counterpart of `DeviceModel` (crates/llamd-runtime/src/device.rs:94-144):
 * load once, then `forward(token, pos) -> token` with one synchronise per
 * token. The reference loads from a GGUF-backed `Model`
 * (device.rs:262-471); here tensors are handed over one at a time in the
 * reference's own byte layouts, which also serves random-init weights that
 * have no file.
 */
#ifndef LLAMD_CUDA_MODEL_H
#define LLAMD_CUDA_MODEL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* crates/llamd-models/src/hparams.rs:54-75 (the fields the decode loop reads) */
typedef struct {
    int32_t n_layer, n_embd, n_head, n_head_kv, head_dim;
    int32_t n_expert, n_expert_used, n_ff_expert, n_vocab;
    float rope_freq_base, rms_eps;
} llamd_hparams;

typedef struct llamd_model llamd_model;

/* Tensor ids for llamd_model_set_tensor. Names follow
 * crates/llamd-models/src/model.rs LayerNames. */
enum {
    LLAMD_T_TOK_EMBD = 0,   /* Q6_K [n_vocab x n_embd]                      */
    LLAMD_T_OUTPUT_NORM,    /* f32  [n_embd]                                */
    LLAMD_T_OUTPUT,         /* Q6_K [n_vocab x n_embd]; absent = tied       */
    LLAMD_T_ATTN_NORM,      /* f32  [n_embd]                                */
    LLAMD_T_ATTN_Q,         /* Q6_K [n_head*head_dim x n_embd]              */
    LLAMD_T_ATTN_K,         /* Q6_K [n_head_kv*head_dim x n_embd]           */
    LLAMD_T_ATTN_V,
    LLAMD_T_ATTN_Q_NORM,    /* f32  [head_dim], optional                    */
    LLAMD_T_ATTN_K_NORM,
    LLAMD_T_ATTN_OUT,       /* Q6_K [n_embd x n_head*head_dim]              */
    LLAMD_T_FFN_NORM,       /* f32  [n_embd]                                */
    LLAMD_T_FFN_GATE_INP,   /* f32  [n_expert x n_embd]                     */
    LLAMD_T_FFN_GATE_EXPS,  /* Q6_K [n_expert][n_ff_expert x n_embd]        */
    LLAMD_T_FFN_UP_EXPS,
    LLAMD_T_FFN_DOWN_EXPS   /* Q6_K [n_expert][n_embd x n_ff_expert]        */
};

/* Expert parallelism (no counterpart in the reference, which is single-GPU):
 * one process per GPU. Rank 0 makes 128 bytes with llamd_cuda_ep_unique_id and
 * shares them with the other ranks by any host channel; every rank then calls
 * llamd_cuda_ep_init(rank, world, id) after llamd_cuda_set_device and BEFORE
 * llamd_model_create. A model created afterwards keeps only experts
 * [rank*n_expert/world, (rank+1)*n_expert/world) of what set_tensor is given,
 * decodes its own sequence(s), and per MoE layer all-gathers the routed
 * requests (ids + Q8_K activation) and returns expert outputs to their home rank
 * over NCCL. Every rank must make the same sequence of forward calls.
 * With max_seq > 1 (peer-memory form only, below): llamd_model_forward_batch of 2..max_seq sequences runs as one tile
 * of the peer-memory exchange -- one rendezvous each way per layer for ALL of a rank's sequences, the expert matmuls
 * as grouped GEMMs over every rank's sequences -- and gives each sequence the single-sequence pass's bits. A batch may
 * not exceed llamd_model_ep_tile_cap; the ranks' batch sizes need not agree, their sequence of calls must. */
int llamd_cuda_ep_unique_id(void *out128);
int llamd_cuda_ep_init(int rank, int world, const void *id128);
void llamd_cuda_ep_finalize(void);
int llamd_cuda_ep_rank(void);
/* Expert parallelism over peer memory: both collectives of a MoE layer replaced by stores over NVLink into the
 * other ranks' buffers plus arrival counters (one process per GPU, buffers shared through CUDA IPC). Every rank pushes
 * its request record (expert ids, Q8_K activation) into every rank's gathered buffers; an owned expert's rows go
 * straight into the home rank's expert-output buffer.
 * llamd_model_ep_p2p_export writes LLAMD_EP_P2P_RECORD bytes (ten IPC handles); every rank collects all ranks'
 * records in rank order and calls llamd_model_ep_p2p_attach(m, all, world) -- a synchronisation point: no rank may
 * run a pass before every rank has attached. The waits are bounded: if a peer does not deliver, the pass fails with a
 * message in llamd_model_error instead of hanging. Same tokens as one GPU, bit for bit. */
#define LLAMD_EP_P2P_RECORD 640
int llamd_model_ep_p2p_export(llamd_model *m, void *out_record);
int llamd_model_ep_p2p_attach(llamd_model *m, const void *all, int world);
int llamd_cuda_ep_ipc_export(const void *dev, void *handle64);
void *llamd_cuda_ep_ipc_open(const void *handle64);
void llamd_cuda_ep_ipc_close(void *mapped);
int llamd_cuda_ep_world(void);
/* Failure detection (no counterpart in the reference). Nothing here hangs on a rank that is missing:
 *  - llamd_cuda_ep_init waits at most the time-out below for the communicator (a rank that never joins) and then
 *    fails with a message; a pass with NCCL collectives in it is waited for on the host with the same limit, after which
 *    the communicator is aborted (ncclCommAbort) and the call fails;
 *  - in the peer-memory form every device-side wait gives up after "ep_poll_limit" polls (llamd_model_set_option;
 *    default 2^24, seconds), records which wait it was in a status word (llamd_model_ep_status: 1 expert rows,
 *    2 requests), and the pass fails with a message. The later waits of that model then return at once. A model whose
 *    wait ran out, or whose communicator was aborted, must be freed and recreated on every rank. */
void llamd_cuda_ep_set_timeout_ms(int ms); /* default 60000 */
int llamd_model_ep_status(llamd_model *m);
/* Expert parallelism over peer memory without a communicator: sets rank and world only. The model must then be
 * attached (llamd_model_ep_p2p_attach or _attach_ptrs) before its first pass. */
int llamd_cuda_ep_init_local(int rank, int world);
/* Attach with device pointers the caller already holds (ranks inside one process, or memory the caller mapped):
 * llamd_model_ep_p2p_buffers gives this rank's LLAMD_EP_P2P_RECORD / 64 shared buffers (expert outputs, arrival
 * counter, gathered ids / scales / quants, dispatch counter of the decode pass; expert outputs and gathered
 * quants / scales / ids of a prefill tile); ptrs is [world][that many] in the same order (row `rank` ignored). */
int llamd_model_ep_p2p_buffers(llamd_model *m, void **out);
/* Expert-parallel prefill (peer-memory form): llamd_model_prefill cuts the prompt into tiles of at most this many
 * tokens, min("prefill_tile" at the time the buffers were shared, 40960 / (world * n_expert_used), max_kv). Per MoE
 * layer every rank stores its tile (Q8_K activations, routed ids) into every rank's gathered buffers, runs the pairs
 * whose expert it owns over ALL ranks' tokens on the grouped integer GEMM, and the down projection stores each
 * pair's rows into the buffer of the rank the token lives on; the ordered combine there is the single-GPU one, so
 * tokens and logits equal one GPU's bit for bit. Every rank must call llamd_model_prefill with prompts that give
 * the same NUMBER of tiles (their lengths may differ). With the NCCL exchanges instead of peer memory, prefill
 * feeds the prompt through the decode pass token by token. */
int llamd_model_ep_tile_cap(llamd_model *m);
int llamd_model_ep_p2p_attach_ptrs(llamd_model *m, void *const *ptrs, int world);

/* DeviceModel::load_batched (device.rs:270): room for max_seq sequences of
 * max_kv positions. NULL on failure (llamd_cuda_last_error_string says why). */
llamd_model *llamd_model_create(const llamd_hparams *hp, int max_kv, int max_seq);
void llamd_model_free(llamd_model *m);
const char *llamd_model_error(llamd_model *m);

/* Upload (part of) one tensor from host memory. For Q6_K tensors `host` holds
 * `count` 210-byte blocks that land at blocks [first_block, first_block+count)
 * of the tensor (so the 128 experts of a layer can be sent one by one); for
 * f32 tensors `count` is the element count and first_block must be 0.
 * layer is ignored for the three model-level tensors. 0 / -1. */
int llamd_model_set_tensor(llamd_model *m, int layer, int which, size_t first_block, const void *host, size_t count);
size_t llamd_model_weight_bytes(llamd_model *m); /* device.rs:473 */

/* Public knobs of DeviceModel (device.rs:126-143): "use_graph" (default 1),
 * "trace" (record per-layer hidden state and expert ids; disables the graph),
 * "ep_poll_limit" (polls before a device-side wait on another rank gives up).
 * Launch structure of the decode pass, none of which changes a bit of the result: "fuse_norm_router" (for passes of fewer
 * than "fuse_norm_router_max" sequences, default 2: single sequences), "fuse_rope_attn"
 * (default 1), "fuse_attn_quant", "fuse_norm_qkv", "fuse_silu_down", "fuse_tails" (default 0: measured no faster):
 * neighbouring launches as one ("fuse_attn_quant": the attention-output launch writes the Q8_K form of its result itself,
 * as thread-block clusters of the eight CTAs of a 256-element block; heads of 128, the separate quantize launch
 * otherwise); "attn_gqa" (default 1): a batch of four or more sequences runs attention with one CTA per kv head for all
 * the query heads that share it (eight heads of 128 per kv head; the per-head kernels otherwise); "sort_slots" = n
 * (default 8): from n sequences per pass the expert launches take their (sequence, expert) slots in expert order, so that
 * sequences that chose the same expert read it side by side; "head_gemm" = n (default 4): from n sequences per pass the
 * output projection runs on the integer GEMM over a folded copy of its matrix (made at the first such pass, +2 bytes per
 * weight; the matvec when the memory is not there); "dense_gemm" = n (default 8): the same for the four attention
 * projections of every layer; "early_loads"
 * (default 1): the down projection reads its expert ids, and attention its positions and the cached rows of earlier
 * positions, before the launch's dependency wait, so their bytes travel while the launch in front still runs.
 * Prefill: "prefill_tile" (tokens per tile, 1..4096, default 512), "prefill_gemm" (1: the exact integer tensor path,
 * default; 0: dp4a, 8 tokens per weight pass, exact; 2: tcgen05 on f16 pairs, tolerance level), "prefill_attn" (1: the
 * register-tiled attention kernels, default; 0: the per-token decode kernels), "prefill_prefold" (1: keep the expert
 * matrices a second time, folded for the integer GEMM, +2 bytes per weight; same bits).
 * Experiments kept for A/B runs, results unchanged: "pdl" (mask of launch classes that use programmatic dependent
 * launch), "prefetch" (1: matvec launches ask L2 for the next matvec's weights), "batch_group" (sequences per CTA for
 * small matrices at batch > 1, default 2), "ep_rank_arrive" (expert parallelism: 1 = one arrival per rank and launch on
 * the return path instead of one per CTA; the same on every rank). An unknown name or a value out of range: -1, message. */
int llamd_model_set_option(llamd_model *m, const char *name, int value);

/* The resident decode kernel (no counterpart in the reference): option "resident" = 1 runs a single-sequence pass as
 * ONE cooperative launch per token (every layer inside it, grid barriers between a layer's phases) instead of a dozen
 * launches per layer; the same arithmetic in the same order, so the same bits. Falls back to the per-op pass when the
 * dimensions do not fit (shared memory, heads x 4 > SMs) or with max_seq > 1 / expert parallelism. Option
 * "resident_profile" = 1 makes its CTA 0 accumulate nanoseconds per phase, read by llamd_model_resident_profile
 * (32 values in the kernel's phase order; [30] SM cycles and [31] nanoseconds of the whole kernel).
 *
 * Option "kv_f16" = 1 (the benchmark configuration's "KV cache is f16"; the reference's caches are f32): the K/V caches
 * hold binary16 values, rounded to nearest-even once at the store and widened exactly at every load; nothing else changes,
 * so a pass is bit-identical to the f32 arithmetic over a cache of f16-representable values (which is what the oracle's
 * f16-store mode computes). The caches are re-allocated and EMPTY after the option changes: set it before the first pass
 * (and before a peer-memory attach). Every path honours it: per-op decode, batches, the tiled prefill (through an f32 view
 * of the rows it attends), the resident kernel, llamd_model_read_kv (returns the widened values).
 *
 * Option "arith" = 1, or a mask of 2 (norms) | 4 (router) | 8 (attention) (no counterpart in the reference's CPU path; its
 * device backends reduce in parallel too): a decode pass sums the 2048-term sums of the two norms and of the router's
 * dots, the softmax sum and the weighted values of attention as reduction trees instead of walking them in the reference's
 * order. Integers, indices, `exp` and every other float operation are unchanged, so results agree with arith = 0 to the
 * last bits of those sums, NOT bit for bit, and a near-tie in a router can then choose another expert. Deterministic (fixed
 * tree shapes). Honoured by the graph of separate launches (any batch that takes the matvec pass; needs "fuse_norm_router", the default) and by
 * the resident kernel; refused (-1, message) with expert parallelism. Prefill tiles and wide batches always use the exact
 * arithmetic. */
int llamd_model_resident_profile(llamd_model *m, unsigned long long *out32);

/* DeviceModel::forward (device.rs:689-722): one token, greedy next token. */
int llamd_model_forward(llamd_model *m, int32_t token, int32_t pos, int32_t *out_token);
/* DeviceModel::forward_batch (device.rs:741-962): nseq independent sequences. Up to LLAMD_MAX_SEQ (8) they share
 * each weight read inside the nseq kernels; up to option "matvec_batch_max" (default 56) the same pass runs with one
 * launch per 8 sequences for its large matrices; beyond that, up to max_seq (at most LLAMD_MAX_BATCH), the pass runs as
 * a prefill tile whose tokens belong to different sequences, on the integer GEMM (with sharded experts: from 2 on,
 * through the tile exchange over peer memory). Either way sequence s gets exactly the single-sequence pass's bits. */
int llamd_model_forward_batch(llamd_model *m, const int32_t *tokens, const int32_t *positions, int nseq,
                              int32_t *out_tokens);
/* VulkanModel::prefill (crates/llamd-runtime/src/vulkan_model.rs:877-907):
 * consume n_tokens prompt ids at positions base_pos.., return the greedy token
 * after the last one. */
int llamd_model_prefill(llamd_model *m, const int32_t *tokens, int n_tokens, int base_pos, int32_t *out_token);
/* Verification for speculative decoding (the reference plans it "verified only": docs/porting-matrix.md row 20). Consumes
 * n_tokens at base_pos.. like llamd_model_prefill, but out_tokens[i] = the greedy token after tokens[0..=i], for every
 * i. A drafter keeps the longest prefix with tokens[i + 1] == out_tokens[i]; output with drafting equals output
 * without it, because the tiled pass equals token-by-token decode bit for bit. */
int llamd_model_verify(llamd_model *m, const int32_t *tokens, int n_tokens, int base_pos, int32_t *out_tokens);
/* Resident greedy decode: n passes back to back, each pass's token fed to the
 * next on the device, one synchronise at the end; the same tokens as n calls
 * of llamd_model_forward. ms_out (may be NULL) gets the device time of the n
 * passes. The kernel-only counterpart of the reference's tg64 loop
 * (crates/llamd-testing/tests/device_forward.rs:136-279). */
int llamd_model_decode(llamd_model *m, int32_t first_token, int32_t start_pos, int n, int32_t *out_tokens, float *ms_out);
/* Device time of `iters` repetitions of only the Q6_K matvec launches of one
 * pass (the kernel-only discipline of DeviceWeights::bench_kernel_only,
 * crates/llamd-rocm/src/lib.rs:378-423, over a whole token's weights). */
int llamd_model_bench_matvecs(llamd_model *m, int iters, int nseq, float *ms_out, int *launches_out);
/* Kernel launches one pass queues (the nodes of its graph). */
unsigned long long llamd_model_launches_per_pass(llamd_model *m);
/* Phase profile of one pass (the counterpart of DeviceModel::profile,
 * device.rs:136-199): an un-graphed pass with an event after every launch
 * group; ms_out[LLAMD_PH_COUNT] gets each phase's time summed over the layers.
 * A diagnostic: the events serialise the pass, the total is not a throughput. */
enum {
    LLAMD_PH_EMBED = 0, LLAMD_PH_ATTN_NORM, LLAMD_PH_QKV, LLAMD_PH_ROPE, LLAMD_PH_ATTENTION, LLAMD_PH_QUANT, LLAMD_PH_ATTN_OUT,
    LLAMD_PH_FFN_NORM, LLAMD_PH_ROUTER, LLAMD_PH_GATE_UP, LLAMD_PH_SILU, LLAMD_PH_DOWN, LLAMD_PH_LM_HEAD, LLAMD_PH_ARGMAX,
    LLAMD_PH_COUNT
};
int llamd_model_profile_pass(llamd_model *m, int32_t token, int32_t pos, float *ms_out);
/* Logits of the last pass, [nseq][n_vocab], to host memory (device.rs:966). */
int llamd_model_logits(llamd_model *m, float *host_out, int nseq);
/* With "trace" on: x after every layer [n_layer][max_seq][n_embd] and the
 * routed expert ids [n_layer][max_seq][n_expert_used] of the last pass. */
int llamd_model_read_trace(llamd_model *m, float *x_out, int32_t *ids_out);
/* K and V of positions [0, n_pos) of one layer and sequence, to host memory. */
int llamd_model_read_kv(llamd_model *m, int layer, int seq, int n_pos, float *k_out, float *v_out);

#ifdef __cplusplus
}
#endif
#endif /* LLAMD_CUDA_MODEL_H */
