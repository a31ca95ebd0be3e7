// CudaModel: the resident decode model, the counterpart of DeviceModel
// (crates/llamd-runtime/src/device.rs:94-144, 262-471, 486-722, 741-962).
//
// Weights are uploaded once (tensor by tensor, from the reference's byte
// layouts) and stay on the device; a token is one queue of launches on the
// library stream reading (token, pos) from a device-resident meta buffer, so
// the captured CUDA graph is valid for every later token; the host pays 8 bytes
// up and 4 bytes down per token and one synchronise.
#include <string.h>

#include <string>
#include <vector>

#include "common.cuh"
#include "mega.cuh"
#include "../../include/llamd_cuda_model.h"

extern "C" {
void llamd_fwd_repack_q6k_at(const void *d_src, void *d_dst, size_t n_blocks, size_t dst_first);
void llamd_fwd_add_rms_norm_quant(const float *x, const float *residual, float *sum_out, const float *w, float *out, int8_t *qs,
                                  float *d, int n, float eps, int nseq);
void llamd_fwd_combine_rms_norm_quant(const float *x, const float *down, const float *weights, int n_used, float *sum_out,
                                      const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq);
void llamd_fwd_qk_norm_rope_store(float *q, const float *wq, float *k, const float *wk, const float *v, float *kc, float *vc, int n_head,
                                  int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int nseq, int max_kv);
void llamd_fwd_matvec_tokens(const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad, float *o0, float *o1,
                             float *o2, int blocks, int rows0, int rows1, int rows2, int ntok);
void llamd_fwd_expert_major(const void *wa, const void *wb, const int32_t *work, const int32_t *n_work, int max_items,
                            const int32_t *act_map, const int32_t *pslot, const int8_t *aq, const float *ad, float *oa, float *ob,
                            int blocks, int rows, int n_expert);
void llamd_fwd_qk_norm_rope_store_tile(float *q, const float *wq, float *k, const float *wk, const float *v, float *kc, float *vc,
                                       int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int ntok);
void llamd_fwd_attention_tile(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                              int hd, const int32_t *meta, int max_kv, int ntok);
void llamd_fwd_attention_prefill(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                                 int hd, const int32_t *meta, int max_kv, int ntok, int n_kv_max);
void llamd_fwd_matmul_f32_tokens(const float *w, const float *x, float *out, int k, int rows, int ntok);
void llamd_fwd_norm_router(const float *w, const float *x, const float *residual, float *x_out, const float *w_norm, float *xn_out,
                           int8_t *qs, float *d, int k, float eps, int n_expert, int n_used, float *logits, int32_t *ids, float *weights,
                           float *probs, unsigned int *counter, int nseq);
void llamd_fwd_attention_rope_meta(const float *q, const float *wq, const float *k, const float *wk, const float *v, float *kc, float *vc,
                                   float *out, float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab,
                                   float eps, int max_kv, int nseq);
void llamd_fwd_attention_rope_meta_kv16(const float *q, const float *wq, const float *k, const float *wk, const float *v, void *kc, void *vc,
                                        float *out, float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta,
                                        const float *rope_tab, float eps, int max_kv, int nseq);
void llamd_fwd_qk_norm_rope_store_kv16(float *q, const float *wq, float *k, const float *wk, const float *v, void *kc, void *vc, int n_head,
                                       int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int nseq, int max_kv);
void llamd_fwd_qk_norm_rope_store_tile_kv16(float *q, const float *wq, float *k, const float *wk, const float *v, void *kc, void *vc,
                                            int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int ntok);
void llamd_fwd_attention_meta_kv16(const float *q, const void *kc, const void *vc, float *out, float *scores, int n_head, int n_head_kv,
                                   int hd, const int32_t *meta, int max_kv, int nseq);
void llamd_fwd_kv16_expand(const void *kc16, const void *vc16, float *kc32, float *vc32, int n_pos, int kv_dim);
void llamd_fwd_matvec_grouped_x2_silu_quant(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                                            float *oa, float *ob, unsigned int *counter, int8_t *qs, float *d, int blocks, int rows,
                                            int n_used, int nseq);
void llamd_fwd_attention_meta_quant(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                                    int hd, const int32_t *meta, int max_kv, int nseq, unsigned int *counter, int8_t *qs, float *d);
void llamd_fwd_matvec_f32act(const void *w, const float *x, float *out, int blocks, int rows, int nseq);
void llamd_fwd_matvec_grouped_pa_silu(const void *w, const int32_t *ids, const float *gate, const float *up, float *out, int blocks,
                                      int rows, int n_used, int nseq);
void llamd_fwd_matvec_grouped_x2_owned(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad, float *oa,
                                       float *ob, int blocks, int rows, int n_used, int n_slots, int own_lo, int own_hi);
void llamd_fwd_matvec_grouped_pa_owned(const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out, int blocks,
                                       int rows, int n_slots, int own_lo, int own_hi);
void llamd_fwd_ep_dispatch(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *ids_all, float *ad_all, int8_t *aq_all,
                           int n_used, int blocks);
void llamd_fwd_ep_combine(const float *send, float *recv, const int32_t *ids, float *down, int n_used, int n_embd, int n_expert);
int llamd_cuda_ep_rank(void);
int llamd_cuda_ep_world(void);
int llamd_cuda_ep_ipc_export(const void *dev, void *handle64);
void *llamd_cuda_ep_ipc_open(const void *handle64);
void llamd_cuda_ep_ipc_close(void *mapped);
void llamd_fwd_ep_push(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *const *ids_tab, float *const *ad_tab,
                       int8_t *const *aq_tab, unsigned int *const *disp_tab, unsigned int *epoch, int n_used, int blocks);
void llamd_fwd_q8k_residue_major(const int8_t *aq, void *aq_rm, size_t nblocks);
void llamd_fwd_act_f16_rm(const int8_t *aq, const float *ad, void *act16, size_t nblocks);
void llamd_fwd_gemm_tokens_tc(const void *w0, const void *w1, const void *w2, const void *act16, float *o0, float *o1, float *o2,
                              int blocks, int rows0, int rows1, int rows2, int ntok);
void llamd_fwd_expert_gemm_tc(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount, const int32_t *act_map,
                              const int32_t *pslot, const void *act16, float *oa, float *ob, int blocks, int rows, int n_expert,
                              int max_count);
int llamd_fwd_gemm_tc_status(void);
void llamd_fwd_gemm_tokens(const void *w0, const void *w1, const void *w2, const void *aq_rm, const float *ad, float *o0, float *o1,
                           float *o2, int blocks, int rows0, int rows1, int rows2, int ntok);
void llamd_fwd_expert_gemm(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount, const int32_t *act_map,
                           const int32_t *pslot, const void *aq_rm, const float *ad, float *oa, float *ob, int blocks, int rows,
                           int n_expert);
void llamd_fwd_router_matvec(const float *w, const float *x, int k, int n_expert, int n_used, float *logits, int32_t *ids,
                             float *weights, float *probs, unsigned int *counter, int nseq);
void llamd_fwd_moe_group_work(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart, int32_t *gcount,
                              int32_t *ptoken, int32_t *pslot, int32_t *work, int32_t *n_work);
}

using namespace llamd;

namespace llamd {
int ep_bounded_sync();  // ep.cu: the stream synchronise of a pass that has NCCL collectives in it, with a host time-out
}

namespace {

constexpr int kArgmaxBlocks = 512;  // crates/llamd-runtime/src/device.rs ARGMAX_BLOCKS

struct Buf {
    void *p = nullptr;
    size_t bytes = 0;
    bool alloc(size_t n) {
        bytes = n ? n : 1;
        if (cudaMalloc(&p, bytes) != cudaSuccess) {
            set_error(cudaGetLastError(), "model cudaMalloc");
            p = nullptr;
            return false;
        }
        cudaMemsetAsync(p, 0, bytes, stream());
        return true;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
    }
    template <typename T>
    T *as() const {
        return (T *)p;
    }
};

struct Layer {
    Buf attn_norm, attn_q, attn_k, attn_v, attn_q_norm, attn_k_norm, attn_out, ffn_norm, ffn_gate_inp;
    Buf gate_exps, up_exps, down_exps;
    Buf gate_fold, up_fold, down_fold;  // option "prefill_prefold": the expert matrices folded once for the prefill GEMM
    Buf q_fold, k_fold, v_fold, o_fold;  // option "dense_gemm": the attention projections folded for batched decode
    bool has_q_norm = false, has_k_norm = false;
    Buf kc, vc;
};

struct Model {
    llamd_hparams hp;
    int max_kv, max_seq;
    std::vector<Layer> layers;
    Buf tok_embd, output_norm, output, rope_tab;
    // scratch (crates/llamd-runtime/src/device.rs:407-434)
    Buf x, xb, xb2, q, k, v, attn, aq, ad, aq2, ad2, router_logits, router_probs, expert_ids, expert_w;
    Buf head_fold, head_rm;  // the output matrix folded for the integer GEMM (option "head_gemm"), and a batch's activations in its operand order
    bool head_fold_ready = false, head_fold_failed = false;
    Buf slot_order;          // [max_seq * n_expert_used] a batch's (sequence, slot) pairs sorted by expert (decode pass, 8 sequences and more)
    Buf e_gate, e_up, e_down, logits, amax_v, amax_i, out_token, meta;
    Buf trace_x, trace_ids;  // [n_layer][max_seq][n_embd], [n_layer][max_seq][n_used]
    Buf scores;              // [max_seq][n_head][max_kv] scaled attention logits
    Buf router_counter;      // the router kernel's arrival counters, one per sequence
    Buf tail_counter;        // arrival counters of the fused tails: [max_seq * n_expert_used] (also covers [max_seq])
    Buf tok_log, tok_count;  // device-side record of emitted tokens, for the resident decode loop
    unsigned long long launches_per_pass = 0;
    // prefill tile buffers (allocated on first use), token dimension = prefill_tile
    struct Prefill {
        int tile = 0;
        Buf x, xb, xb2, q, k, v, attn, aq, ad, aq2, ad2, ids, w, logits, counter, gate, up, down, scores, meta;
        Buf gstart, gcount, ptoken, pslot, work, n_work;
        Buf logits_all, amax_v, amax_i, out_tokens;  // every token's logits and greedy pick (verification, wide batches)
        int32_t *h_out_tokens = nullptr;             // pinned [tile]
        Buf aq_rm, aq2_rm;  // the GEMMs' view of aq / aq2: residue-major bytes (integer path) or two f16 terms per element (tcgen05 path)
        int32_t *h_meta = nullptr;
        // Expert parallelism over peer memory: every rank's tile (activations, scales, routed ids) gathered here by the
        // ranks' own stores, [world][ep_cap] token rows; then this rank's share of the expert work over all of them.
        int ep_cap = 0;  // tokens per rank the shared buffers hold; fixed once they have been exported to the peers
        Buf aq_all, ad_all, ids_all, aq_all_rm, gate_all, up_all, aq2_all, ad2_all, aq2_all_rm, push_done;
        Buf down_tab, aq_tab, ad_tab, ids_tab;  // device arrays [world]: every rank's down / aq_all / ad_all / ids_all
    } pf;
    // expert parallelism (ep_world > 1): this rank holds experts [own_lo, own_hi)
    int ep_rank = 0, ep_world = 1, own_lo = 0, own_hi = 0;
    Buf ids_all, ad_all, aq_all, gate_all, up_all, aq2_all, ad2_all, down_all, recv_all;
    // peer-written expert outputs (llamd_model_ep_p2p_attach): every rank's e_down and arrival counter, mapped here
    int ep_p2p = 0;
    unsigned int ep_poll_limit = 1u << 24;  // polls (with back-off: seconds) before a wait on another rank gives up; option "ep_poll_limit"
    Buf ep_arrive, ep_status, ep_out_tab, ep_arrive_tab;  // counter word, status word, device pointer tables [world]
    Buf ep_local_done;       // this rank's CTA count of a down projection with peer outputs
    int ep_rank_arrive = 0;  // option "ep_rank_arrive": one arrival per rank and launch (1) or one per CTA (0, measured 0.8 % faster at 4
                             // GPUs: 847 against 840 tok/s); the same on every rank
    Buf ep_disp, ep_epoch, ep_ids_tab, ep_ad_tab, ep_aq_tab, ep_disp_tab;  // dispatch counter, this rank's epoch, tables [world]
    std::vector<void *> ep_mapped;                         // what cudaIpcOpenMemHandle returned, to close
    // Opt-in phase profile (the counterpart of DeviceModel::profile, crates/llamd-runtime/src/device.rs:136-199):
    // events between the launches of an un-graphed pass; totals are never a throughput figure.
    bool profiling = false;
    std::vector<cudaEvent_t> prof_events;
    std::vector<int> prof_phase;
    // The resident decode kernel (mega.cu): one cooperative launch per token instead of a dozen launches per layer.
    int resident = 0;        // option "resident": 1 = use it for single-sequence passes when the dimensions allow
    Buf mega_layers, mega_bar, mega_status, mega_prof;
    int arith_fast = 0;      // option "arith": non-zero = tree reductions for the long ordered sums of a decode token
    int resident_profile = 0;  // option "resident_profile": CTA 0 of the resident kernel accumulates nanoseconds per phase
    bool mega_ready = false;
    int fuse_tails = 0;      // 1: the attention output's and the gate/up outputs' follow-up ops run in the producer's last CTA
                             // (measured slower: fence + arrival + reload cost more than a graph's kernel boundary)
    int prefetch = 0;        // 1: every matvec launch asks L2 for the weights of the matvec after it (measured: no gain)
    int prefill_attn = 1;    // 1: register-tiled attention kernels for a tile; 0: the per-token decode kernels
    int early_loads = 1;     // option "early_loads": the down projection reads its expert ids, and attention its positions and the cached rows
                             // of earlier positions, before the dependency wait (what they read was complete before the launch in front began)
    int matvec_batch_max = 56;  // option "matvec_batch_max": batches up to this many sequences run the decode pass of matvec launches (beyond
                                // LLAMD_MAX_SEQ its large matrices take one launch per LLAMD_MAX_SEQ sequences), larger ones the tile pass.
                                // Measured at position ~500, tok/s aggregate, matvec / tile: 9 sequences 1109 / 529, 16: 1547 / 776,
                                // 32: 1810 / 1247, 40: 1797 / 1446, 48: 1882 / 1649, 64: 1968 / 2048, 80: 1972 / 2330
    int dense_gemm = 8;      // option "dense_gemm" = n: from n sequences per pass the attention projections run on the integer GEMM over folded
                             // copies of their matrices (as "head_gemm"; +2 bytes per weight of the four matrices of every layer); 0: never
    bool dense_fold_ready = false, dense_fold_failed = false;
    int head_gemm = 4;       // option "head_gemm" = n: from n sequences per pass the output projection runs on the integer GEMM over a folded
                             // copy of the matrix (2 bytes per weight once per pass, where the matvec repeats its integer work per sequence;
                             // +0.6 GB for a 151936 x 2048 matrix, made at the first such pass); 0: never
    int fuse_norm_router_max = 2;  // option "fuse_norm_router_max": the fused norm + router launch serves passes of fewer sequences than this.
                                   // Measured, tok/s aggregate, fused / separate: 1 sequence 281.3 / 275.7 (when it was built), 2: 460.5 / 485.0,
                                   // 4: 727.1 / 736.8, 8: 1112.5 / 1149.2, 24: 1644.5 / 1718.7, 48: 1876.2 / 1941.4
    int sort_slots = 8;      // option "sort_slots" = n: from n sequences per pass the expert launches take their slots in expert order (0: never)
    int attn_gqa = 1;        // option "attn_gqa": batches of sequences run attention with one CTA per kv head for all its query heads (the same bits)
    int fuse_attn_quant = 0; // option "fuse_attn_quant": the attention-output launch leaves its result quantized (clusters of the CTAs of a
                             // 256-element block exchange their maxima through distributed shared memory); needs fuse_rope_attn. The same
                             // bits, one launch fewer, and measured 7 % SLOWER (270.4 against 291.2 tok/s): a launch of 16 clusters of
                             // eight co-scheduled CTAs starts later behind a running kernel than 128 free CTAs do, so off
    int fuse_silu_down = 0;  // option "fuse_silu_down": silu(gate) * up and its Q8_K form inside the down projection's launch (decode pass);
                             // the same bits and the same speed (290.3 against 290.5 tok/s: 200 CTAs each redo their slot's 768 exps), so off
    int fuse_norm_qkv = 0;   // option "fuse_norm_qkv": the attention norm (and the combine before it) inside the QKV matvec (one sequence);
                             // the same bits, measured 0.8 % slower (288.1 against 290.5 tok/s: 160 CTAs each repeat the combine), so off
    int fuse_rope_attn = 1;  // option "fuse_rope_attn": QK-norm, RoPE and the KV store inside the attention-scores launch (decode pass)
    int fuse_norm_router = 1;  // option "fuse_norm_router": the FFN norm and the router as one launch (decode pass)
    int kv16 = 0;            // option "kv_f16": the caches hold binary16 values (rounded at the store)
    Buf kc32, vc32;          // a prefill tile's view of one layer's binary16 cache, widened to f32 ([max_kv][kv_dim] each)
    int prefold = 0;         // option "prefill_prefold"; prefold_ready once the folded copies exist
    bool prefold_ready = false;
    int prefill_gemm = 1;    // 1: integer tensor path (mma.sync), exact; 0: dp4a, 8 tokens per weight pass, exact;
                             // 2: tcgen05 on f16 pairs, tolerance level (gemm_tc.cu)
    int prefill_tile = 512;  // VulkanModel::prefill_tile default max_seq.min(512), vulkan_model.rs:343
    int32_t *h_meta = nullptr;  // pinned
    int32_t *h_out = nullptr;   // pinned
    size_t weight_bytes = 0;
    int use_graph = 1, trace = 0;
    int graph_nseq = 0;         // nseq the captured graph was recorded for
    unsigned long long id = 0;
    std::string err;
};

unsigned long long g_next_id = 1, g_graph_owner = 0;

// After the argmax: record the emitted tokens and make them the next pass's
// input at pos+1, so passes can be queued back to back without the host.
// forward() overwrites meta before every pass, so this only matters to the
// resident decode loop.
__global__ void advance_meta_kernel(int32_t *__restrict__ meta, const int32_t *__restrict__ out_token, int32_t *__restrict__ tok_log,
                                    int32_t *__restrict__ tok_count, int nseq, int log_cap) {
    pdl_trigger();
    pdl_wait();
    const int s = threadIdx.x;
    const int c = *tok_count;
    __syncthreads();
    if (s < nseq) {
        const int t = out_token[s];
        if ((c + 1) * nseq <= log_cap) tok_log[c * nseq + s] = t;
        meta[2 * s] = t;
        meta[2 * s + 1] += 1;
    }
    if (s == 0) *tok_count = c + 1;
}

size_t q6k_blocks_for(size_t rows, size_t k) { return rows * (k / LLAMD_QK_K); }

bool upload_q6k_slice(Buf &dst, size_t total_blocks, size_t first, const void *host, size_t n_blocks) {
    if (!dst.p && !dst.alloc(llamd_cuda_q6k_tiled_bytes(total_blocks))) return false;
    if (first + n_blocks > total_blocks) {
        set_error_msg("set_tensor: slice outside the tensor");
        return false;
    }
    const size_t bytes = n_blocks * LLAMD_Q6K_BLOCK_BYTES;
    void *raw = scratch(6, bytes);
    if (!raw) return false;
    if (cudaMemcpyAsync(raw, host, bytes, cudaMemcpyHostToDevice, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "set_tensor H2D");
        return false;
    }
    llamd_fwd_repack_q6k_at(raw, dst.p, n_blocks, first);
    // the staging buffer is reused by the next call and the host array may go away
    return llamd_fwd_sync() == 0;
}

bool upload_f32(Buf &dst, const void *host, size_t n) {
    if (!dst.p && !dst.alloc(n * sizeof(float))) return false;
    if (cudaMemcpyAsync(dst.p, host, n * sizeof(float), cudaMemcpyHostToDevice, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "set_tensor H2D");
        return false;
    }
    return llamd_fwd_sync() == 0;
}

// ---- L2 prefetch plans (common.cuh: PrefetchPlan): set just before a matvec launch, naming what follows it ----
static MatvecPlans plan_static(const Model &m, const Buf *a, const Buf *b = nullptr, const Buf *c = nullptr, size_t cap = 0) {
    MatvecPlans pl = {};
    if (!m.prefetch) return pl;
    PrefetchPlan pf = {};
    const Buf *r[3] = {a, b, c};
    for (int i = 0; i < 3; i++) {
        if (!r[i] || !r[i]->p) continue;
        size_t n = r[i]->bytes & ~(size_t)15;
        if (cap && n > cap) n = cap;
        pf.base[i] = (const uint8_t *)r[i]->p;
        pf.bytes[i] = n;
    }
    pl.pf = pf;
    return pl;
}
static MatvecPlans plan_experts(const Model &m, const Buf &w, const int32_t *ids, int n_ids) {
    MatvecPlans pl = {};
    if (!m.prefetch || !w.p) return pl;
    const int lo = m.ep_world > 1 ? m.own_lo : 0, hi = m.ep_world > 1 ? m.own_hi : m.hp.n_expert;
    if (hi <= lo || n_ids > 256) return pl;
    PrefetchPlan pf = {};
    pf.base[0] = (const uint8_t *)w.p;
    pf.bytes[0] = (w.bytes / (size_t)(hi - lo)) & ~(size_t)15;
    pf.ids = ids;
    pf.n_ids = n_ids;
    pf.own_lo = lo;
    pf.own_hi = hi;
    pl.pf = pf;
    return pl;
}
constexpr size_t kHeadPrefetchBytes = (size_t)48 << 20;  // of the 256 MB lm_head: what comfortably stays in L2

// The resident kernel reads the layers' pointers from a device table, made once all tensors are there.
bool mega_prepare(Model &m) {
    if (m.mega_ready) return true;
    if (!mega_supported(m.hp, m.max_kv)) return false;
    std::vector<MegaLayer> tab(m.layers.size());
    for (size_t i = 0; i < m.layers.size(); i++) {
        Layer &l = m.layers[i];
        tab[i] = MegaLayer{l.attn_q.as<uint8_t>(), l.attn_k.as<uint8_t>(), l.attn_v.as<uint8_t>(), l.attn_out.as<uint8_t>(),
                           l.gate_exps.as<uint8_t>(), l.up_exps.as<uint8_t>(), l.down_exps.as<uint8_t>(), l.attn_norm.as<float>(),
                           l.has_q_norm ? l.attn_q_norm.as<float>() : nullptr, l.has_k_norm ? l.attn_k_norm.as<float>() : nullptr,
                           l.ffn_norm.as<float>(), l.ffn_gate_inp.as<float>(), l.kc.as<float>(), l.vc.as<float>()};
    }
    for (Buf *b : {&m.mega_layers, &m.mega_bar, &m.mega_status, &m.mega_prof}) b->release();  // (made again after the caches moved)
    if (!m.mega_layers.alloc(tab.size() * sizeof(MegaLayer)) || !m.mega_bar.alloc(256) || !m.mega_status.alloc(256) || !m.mega_prof.alloc(32 * 8))
        return false;
    if (cudaMemcpyAsync(m.mega_layers.p, tab.data(), tab.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice, stream()) != cudaSuccess ||
        llamd_fwd_sync() != 0)
        return false;
    m.mega_ready = true;
    return true;
}

// One token through the resident kernel, then the head as in the per-op pass.
void queue_token_resident(Model &m) {
    const llamd_hparams &hp = m.hp;
    const int eb = hp.n_embd / 256;
    MegaParams p = {};
    p.n_layer = hp.n_layer; p.E = hp.n_embd; p.H = hp.n_head; p.HKV = hp.n_head_kv; p.hd = hp.head_dim;
    p.n_expert = hp.n_expert; p.nu = hp.n_expert_used; p.ffe = hp.n_ff_expert; p.max_kv = m.max_kv;
    p.eps = hp.rms_eps;
    p.layers = m.mega_layers.as<MegaLayer>();
    p.tok_embd = m.tok_embd.as<uint8_t>();
    p.output_norm = m.output_norm.as<float>();
    p.rope_tab = m.rope_tab.as<float>();
    p.meta = m.meta.as<int32_t>();
    p.q = m.q.as<float>(); p.k = m.k.as<float>(); p.v = m.v.as<float>(); p.attn = m.attn.as<float>(); p.xb2 = m.xb2.as<float>();
    p.scores = m.scores.as<float>();
    p.logits = m.router_logits.as<float>(); p.e_gate = m.e_gate.as<float>(); p.e_up = m.e_up.as<float>(); p.e_down = m.e_down.as<float>();
    p.x_out = m.x.as<float>(); p.expert_w = m.expert_w.as<float>(); p.expert_ids = m.expert_ids.as<int32_t>();
    p.aq_out = m.aq.as<int8_t>(); p.ad_out = m.ad.as<float>();
    p.trace_x = m.trace ? m.trace_x.as<float>() : nullptr;
    p.trace_ids = m.trace ? m.trace_ids.as<int32_t>() : nullptr;
    p.bar = m.mega_bar.as<unsigned int>();
    p.status = m.mega_status.as<int>();
    p.spin_limit = 1u << 22;
    p.prof = m.resident_profile ? m.mega_prof.as<unsigned long long>() : nullptr;
    p.fast = m.arith_fast;
    p.kv16 = m.kv16;
    launch_decode_mega(p, hp);
    matvec_batch(MatvecPlans{}, m.output.p ? m.output.p : m.tok_embd.p, m.aq.as<int8_t>(), m.ad.as<float>(), m.logits.as<float>(), eb,
                 hp.n_vocab, 1);
    llamd_fwd_argmax(m.logits.as<float>(), hp.n_vocab, m.amax_v.as<float>(), m.amax_i.as<int32_t>(), m.out_token.as<int32_t>(),
                     kArgmaxBlocks, 1);
    launch_k("advance_meta", advance_meta_kernel, dim3(1), dim3(32), 0, m.meta.as<int32_t>(), (const int32_t *)m.out_token.as<int32_t>(),
             m.tok_log.as<int32_t>(), m.tok_count.as<int32_t>(), 1, m.max_kv * m.max_seq);
}

// Queue one pass for `nseq` sequences. Does not synchronise.
// The order is crates/llamd-runtime/src/device.rs:486-655 (itself the CPU
// order of crates/llamd-runtime/src/layer.rs:85-203, 230-304).
void queue_token(Model &m, int nseq) {
    const llamd_hparams &hp = m.hp;
    const int E = hp.n_embd, H = hp.n_head, HKV = hp.n_head_kv, hd = hp.head_dim;
    const int kvd = HKV * hd, qd = H * hd, nu = hp.n_expert_used, ffe = hp.n_ff_expert;
    const int eb = E / 256;
    const int32_t *meta = m.meta.as<int32_t>();
    float *x = m.x.as<float>();

    if (m.resident && nseq == 1 && m.max_seq == 1 && m.ep_world == 1 && !m.profiling && mega_prepare(m)) {
        queue_token_resident(m);
        return;
    }
    // what this pass asks of the norm, router and attention launches (an argument of theirs): the `fast` arithmetic's mask
    // (option arith; the fused norm + router launch carries the router's tree, so the mask needs it on), the loads before
    // the dependency wait, the batch form of attention
    const int pf = (m.arith_fast && m.fuse_norm_router && !m.fuse_tails ? m.arith_fast : 0) | (m.early_loads ? kPassEarlyLoads : 0) |
                   (m.attn_gqa ? kPassAttnGqa : 0);
    const bool dense_gemm = m.dense_gemm && nseq >= m.dense_gemm && m.dense_fold_ready && !m.fuse_norm_qkv;
    size_t n_marks = 0;
    auto mark = [&](int phase) {
        if (!m.profiling) return;
        if (n_marks == m.prof_events.size()) {
            cudaEvent_t e;
            cudaEventCreate(&e);
            m.prof_events.push_back(e);
            m.prof_phase.push_back(0);
        }
        m.prof_phase[n_marks] = phase;
        cudaEventRecord(m.prof_events[n_marks++], stream());
    };
    mark(-1);
    llamd_fwd_embed_meta(m.tok_embd.p, meta, x, eb, nseq);
    mark(LLAMD_PH_EMBED);
    auto trace_x = [&](int il) {
        if (m.trace)
            cudaMemcpyAsync(m.trace_x.as<float>() + (size_t)il * m.max_seq * E, x, (size_t)nseq * E * sizeof(float), cudaMemcpyDeviceToDevice,
                            stream());
    };
    // peer-written expert outputs: the norm that combines them waits for n_used x (CTAs per slot of the down projection) arrivals
    bool ep_wait_pending = false;
    auto plan_ep_wait = [&]() -> WaitPlan {
        if (!ep_wait_pending) return WaitPlan{};
        // every rank arrives once, when all CTAs of its down projection are done (owners after their stores, the others
        // after reading the request)
        const int rows_per_cta = 256 / (ffe / 256);
        const unsigned target = m.ep_rank_arrive ? (unsigned)m.ep_world
                                                 : (unsigned)m.ep_world * (unsigned)nu * (unsigned)((E + rows_per_cta - 1) / rows_per_cta);
        ep_wait_pending = false;
        return WaitPlan{m.ep_arrive.as<unsigned int>(), target, m.ep_status.as<int>(), m.ep_poll_limit};
    };
    // what the down projection of layer il is followed by: the next layer's Q, K, V, or the head's first megabytes
    auto plan_after_down = [&](int il) -> MatvecPlans {
        if (il + 1 < hp.n_layer) return plan_static(m, &m.layers[il + 1].attn_q, &m.layers[il + 1].attn_k, &m.layers[il + 1].attn_v);
        return plan_static(m, m.output.p ? &m.output : &m.tok_embd, nullptr, nullptr, kHeadPrefetchBytes);
    };
    // where the residual stream lives: m.x, or m.xb after a fused norm + router launch (which may not write in place: its
    // other CTAs still read the old stream); the combine that opens the next layer moves it back to m.x
    const float *x_res = x;
    // (the fused launch repeats the norm in each of its n_expert / 4 CTAs per sequence; it wins for a single sequence, where a
    // launch boundary is what it saves, and loses from two sequences on -- m.fuse_norm_router_max -- where the norm as a
    // launch of its own and the router rows behind it cost less; the `fast` arithmetic's router tree lives in the fused kernel)
    const bool fuse_nr = m.fuse_norm_router && (size_t)6 * E * sizeof(float) <= 200 * 1024 && E % 256 == 0 && hp.n_expert <= 4 * E &&
                         (nseq < m.fuse_norm_router_max || m.arith_fast);
    for (int il = 0; il < hp.n_layer; il++) {
        Layer &l = m.layers[il];
        // Attention norm, f32 and Q8_K in one pass (Q, K and V read the same
        // activation). From the second layer on the same launch first finishes
        // the previous layer: x += sum_e w_e * down_e.
        // (with one sequence on one GPU both fold into the QKV matvec, whose every CTA then makes its own activation: one
        // launch fewer; it may not update the stream in place, so it needs the stream in m.xb, where a fused norm + router
        // launch leaves it)
        const bool fuse_nq = m.fuse_norm_qkv && nseq == 1 && m.ep_world == 1 && (il == 0 || x_res != x);
        if (fuse_nq) {
            MatvecPlans pl = plan_static(m, &l.attn_out);
            pl.norm = NormPlan{x_res, il ? m.e_down.as<float>() : nullptr, m.expert_w.as<float>(), nu, il ? x : nullptr, l.attn_norm.as<float>(),
                               hp.rms_eps};
            matvec_x3_norm(pl, l.attn_q.p, l.attn_k.p, l.attn_v.p, m.q.as<float>(), m.k.as<float>(), m.v.as<float>(), eb, qd, kvd, kvd);
            if (il) {
                x_res = x;
                trace_x(il - 1);
            }
            mark(LLAMD_PH_ATTN_NORM);
        } else {
            if (il == 0) {
                rms_norm_quant_flags(x, l.attn_norm.as<float>(), nullptr, m.aq.as<int8_t>(), m.ad.as<float>(), E, hp.rms_eps, nseq, pf);
            } else {
                combine_rms_norm_quant_wait(plan_ep_wait(), x_res, m.e_down.as<float>(), m.expert_w.as<float>(), nu, x, l.attn_norm.as<float>(),
                                            nullptr, m.aq.as<int8_t>(), m.ad.as<float>(), E, hp.rms_eps, nseq, pf);
                x_res = x;
                trace_x(il - 1);
            }
            mark(LLAMD_PH_ATTN_NORM);
            if (dense_gemm) {
                // a batch: the folded matrices once for all the sequences, on the integer tensor path (the same bits)
                llamd_fwd_q8k_residue_major(m.aq.as<int8_t>(), m.head_rm.p, (size_t)nseq * eb);
                gemm_tokens_folded3(l.q_fold.p, l.k_fold.p, l.v_fold.p, m.head_rm.p, m.ad.as<float>(), m.q.as<float>(), m.k.as<float>(),
                                    m.v.as<float>(), eb, qd, kvd, kvd, nseq);
            } else {
                matvec_x3_batch(plan_static(m, &l.attn_out), l.attn_q.p, l.attn_k.p, l.attn_v.p, m.aq.as<int8_t>(), m.ad.as<float>(),
                                m.q.as<float>(), m.k.as<float>(), m.v.as<float>(), eb, qd, kvd, kvd, nseq);
            }
        }
        mark(LLAMD_PH_QKV);
        // QK-norm per head BEFORE RoPE; K and V go into the cache at pos
        const bool fuse = m.fuse_tails && !m.kv16 && qd % 256 == 0 && hd % 16 == 0 && ffe % 256 == 0;
        const bool fuse_ra = m.fuse_rope_attn && !fuse && hd % 16 == 0 && hd <= 256;
        const float *wqn = l.has_q_norm ? l.attn_q_norm.as<float>() : nullptr, *wkn = l.has_k_norm ? l.attn_k_norm.as<float>() : nullptr;
        if (fuse_ra) {
            // ... inside the attention-scores launch: one launch fewer, the same bits; with fuse_attn_quant the Q8_K form of the
            // result is made by the output launch itself (a cluster per 256-element block) where the shape allows
            const bool quant_in_launch = m.fuse_attn_quant != 0;
            attention_rope_quant(m.q.as<float>(), wqn, m.k.as<float>(), wkn, m.v.as<float>(), l.kc.p, l.vc.p, m.attn.as<float>(),
                                 m.scores.as<float>(), H, HKV, hd, meta, m.rope_tab.as<float>(), hp.rms_eps, m.max_kv, nseq, m.kv16,
                                 quant_in_launch ? m.aq.as<int8_t>() : nullptr, quant_in_launch ? m.ad.as<float>() : nullptr, pf);
            mark(LLAMD_PH_ROPE);
            mark(LLAMD_PH_ATTENTION);
            if (!quant_in_launch) llamd_fwd_quantize(m.attn.as<float>(), m.aq.as<int8_t>(), m.ad.as<float>(), nseq * (qd / 256));
        } else {
            if (m.kv16)
                llamd_fwd_qk_norm_rope_store_kv16(m.q.as<float>(), wqn, m.k.as<float>(), wkn, m.v.as<float>(), l.kc.p, l.vc.p, H, HKV, hd, meta,
                                                  m.rope_tab.as<float>(), hp.rms_eps, nseq, m.max_kv);
            else
                llamd_fwd_qk_norm_rope_store(m.q.as<float>(), wqn, m.k.as<float>(), wkn, m.v.as<float>(), l.kc.as<float>(), l.vc.as<float>(), H,
                                             HKV, hd, meta, m.rope_tab.as<float>(), hp.rms_eps, nseq, m.max_kv);
            mark(LLAMD_PH_ROPE);
            if (fuse) {
                // the CTA that finishes a sequence's attention last also writes its Q8_K form
                llamd_fwd_attention_meta_quant(m.q.as<float>(), l.kc.as<float>(), l.vc.as<float>(), m.attn.as<float>(), m.scores.as<float>(), H,
                                               HKV, hd, meta, m.max_kv, nseq, m.tail_counter.as<unsigned int>(), m.aq.as<int8_t>(),
                                               m.ad.as<float>());
                mark(LLAMD_PH_ATTENTION);
            } else {
                attention_meta_flags(m.q.as<float>(), l.kc.p, l.vc.p, m.attn.as<float>(), m.scores.as<float>(), H, HKV, hd, meta, m.max_kv, nseq,
                                     m.kv16, pf);
                mark(LLAMD_PH_ATTENTION);
                // (llamd_fwd_matvec_f32act fuses these two; measured 2 % slower per token: every CTA repeats the quantization)
                llamd_fwd_quantize(m.attn.as<float>(), m.aq.as<int8_t>(), m.ad.as<float>(), nseq * (qd / 256));
            }
        }
        mark(LLAMD_PH_QUANT);
        if (dense_gemm) {
            llamd_fwd_q8k_residue_major(m.aq.as<int8_t>(), m.head_rm.p, (size_t)nseq * (qd / 256));
            gemm_tokens_folded(l.o_fold.p, m.head_rm.p, m.ad.as<float>(), m.xb2.as<float>(), qd / 256, E, nseq);
        } else {
            matvec_batch(plan_static(m, &l.ffn_gate_inp), l.attn_out.p, m.aq.as<int8_t>(), m.ad.as<float>(), m.xb2.as<float>(), qd / 256, E,
                         nseq);
        }
        mark(LLAMD_PH_ATTN_OUT);
        // residual, then the FFN norm (f32 for the router, Q8_K for the experts)
        if (fuse_nr) {
            norm_router_flags(l.ffn_gate_inp.as<float>(), x, m.xb2.as<float>(), m.xb.as<float>(), l.ffn_norm.as<float>(), nullptr,
                              m.aq.as<int8_t>(), m.ad.as<float>(), E, hp.rms_eps, hp.n_expert, nu, m.router_logits.as<float>(),
                              m.expert_ids.as<int32_t>(), m.expert_w.as<float>(), nullptr, m.router_counter.as<unsigned int>(), nseq, pf);
            x_res = m.xb.as<float>();
            mark(LLAMD_PH_FFN_NORM);
        } else {
            add_rms_norm_quant_flags(x, m.xb2.as<float>(), x, l.ffn_norm.as<float>(), m.xb.as<float>(), m.aq.as<int8_t>(), m.ad.as<float>(), E,
                                     hp.rms_eps, nseq, pf);
            mark(LLAMD_PH_FFN_NORM);
            llamd_fwd_router_matvec(l.ffn_gate_inp.as<float>(), m.xb.as<float>(), E, hp.n_expert, nu, m.router_logits.as<float>(),
                                    m.expert_ids.as<int32_t>(), m.expert_w.as<float>(), nullptr, m.router_counter.as<unsigned int>(), nseq);
        }
        mark(LLAMD_PH_ROUTER);
        if (m.ep_world > 1) {
            // Expert parallelism: gather every rank's routed request, run the experts this
            // rank owns for all of them, return each token's rows to its home rank.
            const int W = m.ep_world;
            MatvecPlans gu = plan_experts(m, l.down_exps, m.ids_all.as<int32_t>(), W * nu);
            if (m.ep_p2p) {
                // every rank pushes its request record into every rank's gathered buffers; the gate/up launch waits for
                // all of them (no collective)
                llamd_fwd_ep_push(m.expert_ids.as<int32_t>(), m.ad.as<float>(), m.aq.as<int8_t>(), m.ep_ids_tab.as<int32_t *>(),
                                  m.ep_ad_tab.as<float *>(), m.ep_aq_tab.as<int8_t *>(), m.ep_disp_tab.as<unsigned int *>(),
                                  m.ep_epoch.as<unsigned int>(), nu, eb);
                gu.dwait = DispatchWait{m.ep_disp.as<unsigned int>(), m.ep_epoch.as<unsigned int>(), (unsigned)W, m.ep_status.as<int>(), m.ep_poll_limit};
            } else {
                llamd_fwd_ep_dispatch(m.expert_ids.as<int32_t>(), m.ad.as<float>(), m.aq.as<int8_t>(), m.ids_all.as<int32_t>(),
                                      m.ad_all.as<float>(), m.aq_all.as<int8_t>(), nu, eb);
            }
            matvec_grouped_x2_owned(gu, l.gate_exps.p, l.up_exps.p, m.ids_all.as<int32_t>(), m.aq_all.as<int8_t>(), m.ad_all.as<float>(),
                                    m.gate_all.as<float>(), m.up_all.as<float>(), eb, ffe, nu, W * nu, m.own_lo, m.own_hi);
            llamd_fwd_silu_mul_quant(m.gate_all.as<float>(), m.up_all.as<float>(), nullptr, m.aq2_all.as<int8_t>(), m.ad2_all.as<float>(),
                                     W * nu * ffe);
            MatvecPlans dn = plan_after_down(il);
            dn.ids_early = m.early_loads;  // (the gathered ids were complete before the gate+up launch let anything start behind it)
            if (m.ep_p2p) {
                // no return collective: an owned slot's rows go straight into its home rank's e_down (routing-order slot),
                // each CTA bumps that rank's counter, and the home rank's next norm waits for all of them
                dn.peer = PeerOutPlan{m.ep_out_tab.as<float *>(), m.ep_arrive_tab.as<unsigned int *>(), nu, m.ep_world, m.ep_rank_arrive ? m.ep_local_done.as<unsigned int>() : nullptr};
                matvec_grouped_pa_owned(dn, l.down_exps.p, m.ids_all.as<int32_t>(), m.aq2_all.as<int8_t>(), m.ad2_all.as<float>(),
                                        m.down_all.as<float>(), ffe / 256, E, W * nu, m.own_lo, m.own_hi);
                ep_wait_pending = true;
            } else {
                matvec_grouped_pa_owned(dn, l.down_exps.p, m.ids_all.as<int32_t>(), m.aq2_all.as<int8_t>(), m.ad2_all.as<float>(),
                                        m.down_all.as<float>(), ffe / 256, E, W * nu, m.own_lo, m.own_hi);
                llamd_fwd_ep_combine(m.down_all.as<float>(), m.recv_all.as<float>(), m.expert_ids.as<int32_t>(), m.e_down.as<float>(), nu,
                                     E, hp.n_expert);
            }
            if (m.trace)
                cudaMemcpyAsync(m.trace_ids.as<int32_t>() + (size_t)il * m.max_seq * nu, m.expert_ids.p, (size_t)nseq * nu * sizeof(int32_t),
                                cudaMemcpyDeviceToDevice, stream());
            continue;
        }
        MatvecPlans gu = plan_experts(m, l.down_exps, m.expert_ids.as<int32_t>(), nseq * nu);
        // a batch's slots in expert order, so that the sequences that chose the same expert read it side by side (one small
        // launch; measured worth it from 8 sequences on)
        const int32_t *order = nullptr;
        if (m.sort_slots && nseq >= m.sort_slots) {
            slot_order_launch(m.expert_ids.as<int32_t>(), nseq * nu, m.slot_order.as<int32_t>());
            order = m.slot_order.as<int32_t>();
        }
        gu.slot_order = order;
        // SiLU on the gate only, times up, quantized per expert; each expert's down projection reads its OWN activation
        if (fuse) {
            gu.tail = TailPlan{m.tail_counter.as<unsigned int>(), m.aq2.as<int8_t>(), m.ad2.as<float>()};
            matvec_grouped_x2_batch(gu, l.gate_exps.p, l.up_exps.p, m.expert_ids.as<int32_t>(), m.aq.as<int8_t>(), m.ad.as<float>(),
                                    m.e_gate.as<float>(), m.e_up.as<float>(), eb, ffe, nu, nseq);
            mark(LLAMD_PH_GATE_UP);
        } else {
            matvec_grouped_x2_batch(gu, l.gate_exps.p, l.up_exps.p, m.expert_ids.as<int32_t>(), m.aq.as<int8_t>(), m.ad.as<float>(),
                                    m.e_gate.as<float>(), m.e_up.as<float>(), eb, ffe, nu, nseq);
            mark(LLAMD_PH_GATE_UP);
            if (!m.fuse_silu_down)
                llamd_fwd_silu_mul_quant(m.e_gate.as<float>(), m.e_up.as<float>(), nullptr, m.aq2.as<int8_t>(), m.ad2.as<float>(),
                                         nseq * nu * ffe);
        }
        mark(LLAMD_PH_SILU);
        // (the ids were complete before the gate+up launch let anything start behind it: the down projection's weights
        // travel while the SiLU launch runs)
        MatvecPlans dn_plan = plan_after_down(il);
        dn_plan.ids_early = m.early_loads;
        dn_plan.slot_order = order;
        if (!fuse && m.fuse_silu_down)  // every CTA of a slot makes the slot's activation itself: one launch fewer, the same bits
            matvec_grouped_pa_silu(dn_plan, l.down_exps.p, m.expert_ids.as<int32_t>(), m.e_gate.as<float>(), m.e_up.as<float>(),
                                   m.e_down.as<float>(), ffe / 256, E, nu, nseq);
        else
            matvec_grouped_pa_batch(dn_plan, l.down_exps.p, m.expert_ids.as<int32_t>(), m.aq2.as<int8_t>(), m.ad2.as<float>(),
                                    m.e_down.as<float>(), ffe / 256, E, nu, nseq);
        mark(LLAMD_PH_DOWN);
        if (m.trace)
            cudaMemcpyAsync(m.trace_ids.as<int32_t>() + (size_t)il * m.max_seq * nu, m.expert_ids.p, (size_t)nseq * nu * sizeof(int32_t),
                            cudaMemcpyDeviceToDevice, stream());
    }
    // the last layer's combine, fused with the output norm
    combine_rms_norm_quant_wait(plan_ep_wait(), x_res, m.e_down.as<float>(), m.expert_w.as<float>(), nu, x, m.output_norm.as<float>(), nullptr,
                                m.aq.as<int8_t>(), m.ad.as<float>(), E, hp.rms_eps, nseq, pf);
    trace_x(hp.n_layer - 1);
    mark(LLAMD_PH_ATTN_NORM);
    if (m.head_gemm && nseq >= m.head_gemm && m.head_fold_ready) {
        // a batch: the folded matrix once for all the sequences, on the integer tensor path (the same bits)
        llamd_fwd_q8k_residue_major(m.aq.as<int8_t>(), m.head_rm.p, (size_t)nseq * eb);
        gemm_tokens_folded(m.head_fold.p, m.head_rm.p, m.ad.as<float>(), m.logits.as<float>(), eb, hp.n_vocab, nseq);
    } else {
        // (the prefetch plan names where the next token starts)
        matvec_batch(plan_static(m, &m.layers[0].attn_q, &m.layers[0].attn_k, &m.layers[0].attn_v), m.output.p ? m.output.p : m.tok_embd.p,
                     m.aq.as<int8_t>(), m.ad.as<float>(), m.logits.as<float>(), eb, hp.n_vocab, nseq);
    }
    mark(LLAMD_PH_LM_HEAD);
    llamd_fwd_argmax(m.logits.as<float>(), hp.n_vocab, m.amax_v.as<float>(), m.amax_i.as<int32_t>(), m.out_token.as<int32_t>(),
                     kArgmaxBlocks, nseq);
    mark(LLAMD_PH_ARGMAX);
    launch_k("advance_meta", advance_meta_kernel, dim3(1), dim3(32), 0, m.meta.as<int32_t>(), (const int32_t *)m.out_token.as<int32_t>(),
             m.tok_log.as<int32_t>(), m.tok_count.as<int32_t>(), nseq, m.max_kv * m.max_seq);
}

// Only the Q6_K matvec launches of one pass, with whatever activations and
// expert ids the last pass left in the scratch buffers: what the dominant
// kernel costs per token, for the roofline figure.
void queue_matvecs_only(Model &m, int nseq) {
    const llamd_hparams &hp = m.hp;
    const int E = hp.n_embd, kvd = hp.n_head_kv * hp.head_dim, qd = hp.n_head * hp.head_dim, nu = hp.n_expert_used, ffe = hp.n_ff_expert;
    const int eb = E / 256;
    // the same prefetch plans as the full pass sets
    for (int il = 0; il < hp.n_layer; il++) {
        Layer &l = m.layers[il];
        matvec_x3_batch(plan_static(m, &l.attn_out), l.attn_q.p, l.attn_k.p, l.attn_v.p, m.aq.as<int8_t>(), m.ad.as<float>(), m.q.as<float>(),
                        m.k.as<float>(), m.v.as<float>(), eb, qd, kvd, kvd, nseq);
        matvec_batch(plan_static(m, &l.ffn_gate_inp), l.attn_out.p, m.aq.as<int8_t>(), m.ad.as<float>(), m.xb2.as<float>(), qd / 256, E, nseq);
        matvec_grouped_x2_batch(plan_experts(m, l.down_exps, m.expert_ids.as<int32_t>(), nseq * nu), l.gate_exps.p, l.up_exps.p,
                                m.expert_ids.as<int32_t>(), m.aq.as<int8_t>(), m.ad.as<float>(), m.e_gate.as<float>(), m.e_up.as<float>(), eb,
                                ffe, nu, nseq);
        MatvecPlans dn = il + 1 < hp.n_layer
                             ? plan_static(m, &m.layers[il + 1].attn_q, &m.layers[il + 1].attn_k, &m.layers[il + 1].attn_v)
                             : plan_static(m, m.output.p ? &m.output : &m.tok_embd, nullptr, nullptr, kHeadPrefetchBytes);
        dn.ids_early = m.early_loads;
        matvec_grouped_pa_batch(dn, l.down_exps.p, m.expert_ids.as<int32_t>(), m.aq2.as<int8_t>(), m.ad2.as<float>(), m.e_down.as<float>(),
                                ffe / 256, E, nu, nseq);
    }
    matvec_batch(plan_static(m, &m.layers[0].attn_q, &m.layers[0].attn_k, &m.layers[0].attn_v), m.output.p ? m.output.p : m.tok_embd.p,
                 m.aq.as<int8_t>(), m.ad.as<float>(), m.logits.as<float>(), eb, hp.n_vocab, nseq);
}

// The device-side waits of the peer-memory form are bounded; what the status word they leave behind means.
std::string ep_wait_message(int status) {
    return std::string("expert parallelism: a wait for the other ranks' ") + (status == 2 ? "requests" : "expert rows") +
           " ran out (status " + std::to_string(status) + "); the pass is incomplete and the model must be recreated";
}

bool check_ready(Model &m) {
    if (!m.tok_embd.p || !m.output_norm.p) {
        m.err = "model: token_embd / output_norm not set";
        return false;
    }
    for (size_t i = 0; i < m.layers.size(); i++) {
        Layer &l = m.layers[i];
        if (!l.attn_norm.p || !l.attn_q.p || !l.attn_k.p || !l.attn_v.p || !l.attn_out.p || !l.ffn_norm.p || !l.ffn_gate_inp.p ||
            !l.gate_exps.p || !l.up_exps.p || !l.down_exps.p) {
            m.err = "model: layer " + std::to_string(i) + " has tensors missing";
            return false;
        }
    }
    return true;
}

int run(Model &m, const int32_t *tokens, const int32_t *positions, int nseq, int32_t *out_tokens) {
    const llamd_hparams &hp = m.hp;
    if (nseq < 1 || nseq > m.max_seq) {
        m.err = "forward: nseq outside 1..max_seq";
        return -1;
    }
    for (int s = 0; s < nseq; s++) {
        if (positions[s] < 0 || positions[s] >= m.max_kv) {
            m.err = "forward: position " + std::to_string(positions[s]) + " beyond the " + std::to_string(m.max_kv) + " allocated";
            return -1;
        }
        if (tokens[s] < 0 || tokens[s] >= hp.n_vocab) {
            m.err = "forward: token id outside the vocabulary";
            return -1;
        }
        m.h_meta[2 * s] = tokens[s];
        m.h_meta[2 * s + 1] = positions[s];
    }
    if (!check_ready(m)) return -1;
    if (m.resident) mega_prepare(m);  // (uploads a pointer table: not inside a capture)
    if (m.dense_gemm && nseq >= m.dense_gemm && !m.dense_fold_ready && !m.dense_fold_failed) {
        // the attention projections folded once for batched passes (not inside a capture); the matvec without the memory
        const int eb = hp.n_embd / 256, qd = hp.n_head * hp.head_dim, kvd = hp.n_head_kv * hp.head_dim;
        const size_t need = (size_t)hp.n_layer * (expert_fold_bytes(eb, qd, 1) + 2 * expert_fold_bytes(eb, kvd, 1) + expert_fold_bytes(qd / 256, hp.n_embd, 1));
        bool ok = qd % 256 == 0 && need + ((size_t)1 << 30) <= llamd_cuda_free_mem();
        for (size_t i = 0; ok && i < m.layers.size(); i++) {
            Layer &l = m.layers[i];
            ok = l.q_fold.alloc(expert_fold_bytes(eb, qd, 1)) && l.k_fold.alloc(expert_fold_bytes(eb, kvd, 1)) &&
                 l.v_fold.alloc(expert_fold_bytes(eb, kvd, 1)) && l.o_fold.alloc(expert_fold_bytes(qd / 256, hp.n_embd, 1));
            if (!ok) break;
            expert_prefold(l.attn_q.p, l.q_fold.p, eb, qd, 1);
            expert_prefold(l.attn_k.p, l.k_fold.p, eb, kvd, 1);
            expert_prefold(l.attn_v.p, l.v_fold.p, eb, kvd, 1);
            expert_prefold(l.attn_out.p, l.o_fold.p, qd / 256, hp.n_embd, 1);
        }
        const size_t rm_bytes = (size_t)m.max_seq * (size_t)(qd / 256 > eb ? qd / 256 : eb) * 256;
        if (ok && m.head_rm.bytes < rm_bytes) {
            m.head_rm.release();
            ok = m.head_rm.alloc(rm_bytes);
        }
        m.dense_fold_ready = ok && llamd_fwd_sync() == 0;
        if (!m.dense_fold_ready) {
            for (auto &l : m.layers)
                for (Buf *b : {&l.q_fold, &l.k_fold, &l.v_fold, &l.o_fold}) b->release();
            m.dense_fold_failed = true;
            if (error_code() != 0) return -1;
        }
    }
    if (m.head_gemm && nseq >= m.head_gemm && !m.head_fold_ready && !m.head_fold_failed) {
        // the output matrix folded once for the batched output projection (not inside a capture); without the memory for
        // it the matvec serves batches as it serves one sequence
        const int eb = hp.n_embd / 256;
        const size_t need = expert_fold_bytes(eb, hp.n_vocab, 1);
        if (need + ((size_t)1 << 30) <= llamd_cuda_free_mem() && m.head_fold.alloc(need) && (m.head_rm.p || m.head_rm.alloc((size_t)m.max_seq * eb * 256))) {
            expert_prefold(m.output.p ? m.output.p : m.tok_embd.p, m.head_fold.p, eb, hp.n_vocab, 1);
            m.head_fold_ready = llamd_fwd_sync() == 0;
        }
        if (!m.head_fold_ready) {
            m.head_fold.release();
            m.head_fold_failed = true;
            if (error_code() != 0) return -1;
        }
    }
    // the only per-token host->device traffic: 8 bytes per sequence
    if (cudaMemcpyAsync(m.meta.p, m.h_meta, (size_t)nseq * 8, cudaMemcpyHostToDevice, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "meta H2D");
        return -1;
    }
    if (m.use_graph && !m.trace) {
        // a graph recorded for another model, or another nseq, points at the wrong buffers
        if (!llamd_fwd_has_graph() || g_graph_owner != m.id || m.graph_nseq != nseq) {
            llamd_fwd_graph_destroy();
            if (llamd_fwd_begin_capture() != 0) return -1;
            const unsigned long long before = g_launches;
            queue_token(m, nseq);
            m.launches_per_pass = g_launches - before;
            if (llamd_fwd_end_capture() != 0 || error_code() != 0) {
                llamd_fwd_graph_destroy();
                return -1;
            }
            g_graph_owner = m.id;
            m.graph_nseq = nseq;
        }
        if (llamd_fwd_graph_launch() != 0) return -1;
    } else {
        const unsigned long long before = g_launches;
        queue_token(m, nseq);
        m.launches_per_pass = g_launches - before;
    }
    if (cudaMemcpyAsync(m.h_out, m.out_token.p, (size_t)nseq * 4, cudaMemcpyDeviceToHost, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "token D2H");
        return -1;
    }
    m.h_out[m.max_seq] = 0;
    if (m.ep_p2p) cudaMemcpyAsync(m.h_out + m.max_seq, m.ep_status.p, 4, cudaMemcpyDeviceToHost, stream());
    if (m.mega_ready && m.resident) cudaMemcpyAsync(m.h_out + m.max_seq, m.mega_status.p, 4, cudaMemcpyDeviceToHost, stream());
    // THE ONE SYNCHRONISE (with NCCL collectives in the pass: bounded on the host, see ep_bounded_sync)
    if ((m.ep_world > 1 && !m.ep_p2p ? ep_bounded_sync() : llamd_fwd_sync()) != 0) return -1;
    if (m.h_out[m.max_seq] != 0) {
        m.err = m.ep_p2p ? ep_wait_message(m.h_out[m.max_seq])
                         : std::string("resident decode kernel: a grid barrier was not completed within its limit; the pass is incomplete");
        return -1;
    }
    for (int s = 0; s < nseq; s++) {
        if (m.h_out[s] < 0 || m.h_out[s] >= hp.n_vocab) {
            m.err = "argmax returned " + std::to_string(m.h_out[s]);
            return -1;
        }
        out_tokens[s] = m.h_out[s];
    }
    return 0;
}

}  // namespace

extern "C" {

llamd_model *llamd_model_create(const llamd_hparams *hp, int max_kv, int max_seq) {
    if (!hp || max_kv <= 0 || max_seq < 1 || max_seq > LLAMD_MAX_BATCH) {
        set_error_msg("model: max_kv of 0 or max_seq outside 1..256");
        return nullptr;
    }
    if (hp->n_layer <= 0 || hp->n_embd % 256 || (hp->n_head * hp->head_dim) % 256 || hp->n_ff_expert % 256 || hp->head_dim % 4 ||
        hp->n_head_kv <= 0 || hp->n_head % hp->n_head_kv || hp->n_expert <= 0 || hp->n_expert > 1024 || hp->n_expert_used <= 0 ||
        hp->n_expert_used > hp->n_expert || hp->n_expert_used > 64 || hp->head_dim / 2 > 1024) {
        set_error_msg("model: unsupported hyperparameters (widths must be multiples of 256, MoE only)");
        return nullptr;
    }
    if (!stream()) return nullptr;
    Model *m = new Model();
    m->hp = *hp;
    m->max_kv = max_kv;
    m->max_seq = max_seq;
    m->id = g_next_id++;
    m->layers.resize(hp->n_layer);
    m->ep_rank = llamd_cuda_ep_rank();
    m->ep_world = llamd_cuda_ep_world();
    if (m->ep_world > 1 && hp->n_expert % m->ep_world != 0) {
        set_error_msg("model: expert parallelism needs n_expert divisible by the world size");
        delete m;
        return nullptr;
    }
    m->own_lo = m->ep_rank * (hp->n_expert / m->ep_world);
    m->own_hi = m->own_lo + hp->n_expert / m->ep_world;
    const size_t E = hp->n_embd, qd = (size_t)hp->n_head * hp->head_dim, kvd = (size_t)hp->n_head_kv * hp->head_dim;
    const size_t nu = hp->n_expert_used, ffe = hp->n_ff_expert, S = max_seq;
    const size_t max_act = E > qd ? E : qd;
    bool ok = true;
    auto f = [&](Buf &b, size_t n) { ok = ok && b.alloc(n * S * sizeof(float)); };
    f(m->x, E); f(m->xb, E); f(m->xb2, E); f(m->q, qd); f(m->k, kvd); f(m->v, kvd); f(m->attn, qd);
    ok = ok && m->aq.alloc(max_act * S);
    f(m->ad, max_act / 256);
    ok = ok && m->aq2.alloc(nu * ffe * S);
    f(m->ad2, nu * ffe / 256);
    f(m->router_logits, hp->n_expert); f(m->router_probs, hp->n_expert);
    ok = ok && m->expert_ids.alloc(nu * 4 * S) && m->slot_order.alloc(nu * 4 * S);
    f(m->expert_w, nu); f(m->e_gate, nu * ffe); f(m->e_up, nu * ffe); f(m->e_down, nu * E);
    f(m->logits, hp->n_vocab); f(m->amax_v, kArgmaxBlocks);
    ok = ok && m->amax_i.alloc(kArgmaxBlocks * 4 * S) && m->out_token.alloc(4 * S) && m->meta.alloc(8 * S);
    ok = ok && m->tok_log.alloc((size_t)max_kv * 4 * S) && m->tok_count.alloc(4) && m->router_counter.alloc(4 * S) && m->tail_counter.alloc(4 * (size_t)S * hp->n_expert_used) &&
         m->scores.alloc((size_t)S * hp->n_head * max_kv * sizeof(float));
    if (m->ep_world > 1) {
        const size_t W = m->ep_world;
        ok = ok && m->ids_all.alloc(W * nu * 4) && m->ad_all.alloc(W * (E / 256) * 4) && m->aq_all.alloc(W * E) &&
             m->gate_all.alloc(W * nu * ffe * 4) && m->up_all.alloc(W * nu * ffe * 4) && m->aq2_all.alloc(W * nu * ffe) &&
             m->ad2_all.alloc(W * nu * (ffe / 256) * 4) && m->down_all.alloc(W * nu * E * 4) && m->recv_all.alloc(W * nu * E * 4) &&
             m->ep_arrive.alloc(256) && m->ep_status.alloc(256) && m->ep_out_tab.alloc(W * sizeof(void *)) &&
             m->ep_arrive_tab.alloc(W * sizeof(void *)) && m->ep_local_done.alloc(256) && m->ep_disp.alloc(256) && m->ep_epoch.alloc(256) &&
             m->ep_ids_tab.alloc(W * sizeof(void *)) && m->ep_ad_tab.alloc(W * sizeof(void *)) && m->ep_aq_tab.alloc(W * sizeof(void *)) &&
             m->ep_disp_tab.alloc(W * sizeof(void *));
    }
    for (auto &l : m->layers) {
        ok = ok && l.kc.alloc((size_t)max_kv * kvd * 4 * S) && l.vc.alloc((size_t)max_kv * kvd * 4 * S);
    }
    // RoPE angles from the host libm
    if (ok) {
        std::vector<float> tab((size_t)max_kv * hp->head_dim);
        llamd_cuda_rope_table(tab.data(), max_kv, hp->head_dim, hp->rope_freq_base);
        ok = m->rope_tab.alloc(tab.size() * sizeof(float)) &&
             cudaMemcpyAsync(m->rope_tab.p, tab.data(), tab.size() * sizeof(float), cudaMemcpyHostToDevice, stream()) == cudaSuccess &&
             llamd_fwd_sync() == 0;
    }
    ok = ok && cudaMallocHost((void **)&m->h_meta, 8 * S) == cudaSuccess && cudaMallocHost((void **)&m->h_out, 4 * (S + 1)) == cudaSuccess;  // + the peer-wait status word
    if (!ok) {
        llamd_model_free((llamd_model *)m);
        return nullptr;
    }
    return (llamd_model *)m;
}

void llamd_model_free(llamd_model *h) {
    if (!h) return;
    Model *m = (Model *)h;
    cudaStreamSynchronize(stream());
    if (g_graph_owner == m->id) {
        // a captured graph must not outlive the buffers it points at
        llamd_fwd_graph_destroy();
        g_graph_owner = 0;
    }
    for (auto &l : m->layers)
        for (Buf *b : {&l.attn_norm, &l.attn_q, &l.attn_k, &l.attn_v, &l.attn_q_norm, &l.attn_k_norm, &l.attn_out, &l.ffn_norm,
                       &l.ffn_gate_inp, &l.gate_exps, &l.up_exps, &l.down_exps, &l.gate_fold, &l.up_fold, &l.down_fold, &l.q_fold, &l.k_fold,
                       &l.v_fold, &l.o_fold, &l.kc, &l.vc})
            b->release();
    for (Buf *b : {&m->tok_embd, &m->output_norm, &m->output, &m->rope_tab, &m->x, &m->xb, &m->xb2, &m->q, &m->k, &m->v, &m->attn,
                   &m->aq, &m->ad, &m->aq2, &m->ad2, &m->router_logits, &m->router_probs, &m->expert_ids, &m->slot_order, &m->head_fold, &m->head_rm, &m->expert_w, &m->e_gate,
                   &m->e_up, &m->e_down, &m->logits, &m->amax_v, &m->amax_i, &m->out_token, &m->meta, &m->trace_x, &m->trace_ids,
                   &m->tok_log, &m->tok_count, &m->router_counter, &m->tail_counter, &m->scores, &m->ids_all, &m->ad_all, &m->aq_all, &m->gate_all,
                   &m->up_all, &m->aq2_all, &m->ad2_all, &m->down_all, &m->recv_all, &m->ep_arrive, &m->ep_status, &m->ep_out_tab,
                   &m->ep_arrive_tab, &m->ep_disp, &m->ep_epoch, &m->ep_ids_tab, &m->ep_ad_tab, &m->ep_aq_tab, &m->ep_disp_tab, &m->mega_layers, &m->mega_bar, &m->mega_status, &m->mega_prof,
                   &m->kc32, &m->vc32, &m->ep_local_done})
        b->release();
    for (void *p : m->ep_mapped) llamd_cuda_ep_ipc_close(p);
    for (Buf *b : {&m->pf.x, &m->pf.xb, &m->pf.xb2, &m->pf.q, &m->pf.k, &m->pf.v, &m->pf.attn, &m->pf.aq, &m->pf.ad, &m->pf.aq2, &m->pf.ad2,
                   &m->pf.ids, &m->pf.w, &m->pf.logits, &m->pf.counter, &m->pf.gate, &m->pf.up, &m->pf.down, &m->pf.scores, &m->pf.meta,
                   &m->pf.gstart, &m->pf.gcount, &m->pf.ptoken, &m->pf.pslot, &m->pf.work, &m->pf.n_work, &m->pf.aq_rm, &m->pf.aq2_rm,
                   &m->pf.aq_all, &m->pf.ad_all, &m->pf.ids_all, &m->pf.aq_all_rm, &m->pf.gate_all, &m->pf.up_all, &m->pf.aq2_all,
                   &m->pf.ad2_all, &m->pf.aq2_all_rm, &m->pf.push_done, &m->pf.down_tab, &m->pf.aq_tab, &m->pf.ad_tab, &m->pf.ids_tab})
        b->release();
    if (m->pf.h_meta) cudaFreeHost(m->pf.h_meta);
    for (Buf *b : {&m->pf.logits_all, &m->pf.amax_v, &m->pf.amax_i, &m->pf.out_tokens}) b->release();
    if (m->pf.h_out_tokens) cudaFreeHost(m->pf.h_out_tokens);
    for (cudaEvent_t e : m->prof_events) cudaEventDestroy(e);
    if (m->h_meta) cudaFreeHost(m->h_meta);
    if (m->h_out) cudaFreeHost(m->h_out);
    delete m;
}

const char *llamd_model_error(llamd_model *h) {
    Model *m = (Model *)h;
    if (!m) return llamd_cuda_last_error_string();
    if (m->err.empty()) return llamd_cuda_last_error_string();
    return m->err.c_str();
}

int llamd_model_set_tensor(llamd_model *h, int layer, int which, size_t first_block, const void *host, size_t count) {
    Model *m = (Model *)h;
    if (!m || !host) return -1;
    const llamd_hparams &hp = m->hp;
    const size_t E = hp.n_embd, qd = (size_t)hp.n_head * hp.head_dim, kvd = (size_t)hp.n_head_kv * hp.head_dim;
    const size_t ffe = hp.n_ff_expert, ne = hp.n_expert;
    bool ok = false;
    size_t total = 0;
    if (which == LLAMD_T_TOK_EMBD || which == LLAMD_T_OUTPUT) {
        total = q6k_blocks_for(hp.n_vocab, E);
        ok = upload_q6k_slice(which == LLAMD_T_TOK_EMBD ? m->tok_embd : m->output, total, first_block, host, count);
        if (m->head_fold_ready || m->head_fold_failed) {  // the folded copy of the output matrix is of the old bytes
            if (g_graph_owner == m->id) llamd_fwd_graph_destroy();
            m->head_fold.release();
            m->head_fold_ready = m->head_fold_failed = false;
        }
    } else if (which == LLAMD_T_OUTPUT_NORM) {
        ok = count == E && upload_f32(m->output_norm, host, E);
    } else {
        if (layer < 0 || layer >= hp.n_layer) {
            m->err = "set_tensor: layer out of range";
            return -1;
        }
        Layer &l = m->layers[layer];
        if ((which == LLAMD_T_ATTN_Q || which == LLAMD_T_ATTN_K || which == LLAMD_T_ATTN_V || which == LLAMD_T_ATTN_OUT) &&
            (m->dense_fold_ready || m->dense_fold_failed)) {  // the folded copies are of the old bytes
            if (g_graph_owner == m->id) llamd_fwd_graph_destroy();
            for (auto &ll : m->layers)
                for (Buf *b : {&ll.q_fold, &ll.k_fold, &ll.v_fold, &ll.o_fold}) b->release();
            m->dense_fold_ready = m->dense_fold_failed = false;
        }
        switch (which) {
        case LLAMD_T_ATTN_NORM: ok = count == E && upload_f32(l.attn_norm, host, E); break;
        case LLAMD_T_FFN_NORM: ok = count == E && upload_f32(l.ffn_norm, host, E); break;
        case LLAMD_T_ATTN_Q_NORM: ok = count == (size_t)hp.head_dim && upload_f32(l.attn_q_norm, host, count); l.has_q_norm = ok; break;
        case LLAMD_T_ATTN_K_NORM: ok = count == (size_t)hp.head_dim && upload_f32(l.attn_k_norm, host, count); l.has_k_norm = ok; break;
        case LLAMD_T_ATTN_Q: total = q6k_blocks_for(qd, E); ok = upload_q6k_slice(l.attn_q, total, first_block, host, count); break;
        case LLAMD_T_ATTN_K: total = q6k_blocks_for(kvd, E); ok = upload_q6k_slice(l.attn_k, total, first_block, host, count); break;
        case LLAMD_T_ATTN_V: total = q6k_blocks_for(kvd, E); ok = upload_q6k_slice(l.attn_v, total, first_block, host, count); break;
        case LLAMD_T_ATTN_OUT: total = q6k_blocks_for(E, qd); ok = upload_q6k_slice(l.attn_out, total, first_block, host, count); break;
        case LLAMD_T_FFN_GATE_EXPS:
        case LLAMD_T_FFN_UP_EXPS:
        case LLAMD_T_FFN_DOWN_EXPS: {
            // Only the experts this rank owns are kept (all of them without expert
            // parallelism): the caller's block range is cut to [own_lo, own_hi).
            const size_t per = q6k_blocks_for(ffe, E);
            total = (size_t)(m->own_hi - m->own_lo) * per;
            Buf &dst = which == LLAMD_T_FFN_GATE_EXPS ? l.gate_exps : (which == LLAMD_T_FFN_UP_EXPS ? l.up_exps : l.down_exps);
            if (first_block + count > ne * per) {
                m->err = "set_tensor: slice outside the tensor";
                return -1;
            }
            size_t lo = first_block, hi = first_block + count;
            const size_t own0 = (size_t)m->own_lo * per, own1 = (size_t)m->own_hi * per;
            if (lo < own0) lo = own0;
            if (hi > own1) hi = own1;
            if (!dst.p && !dst.alloc(llamd_cuda_q6k_tiled_bytes(total))) break;
            if (lo >= hi) {
                ok = true;  // nothing of this slice lives here
                count = 0;
            } else {
                ok = upload_q6k_slice(dst, total, lo - own0, (const uint8_t *)host + (lo - first_block) * LLAMD_Q6K_BLOCK_BYTES, hi - lo);
                count = hi - lo;
            }
        } break;
        case LLAMD_T_FFN_GATE_INP: ok = count == ne * E && upload_f32(l.ffn_gate_inp, host, ne * E); break;
        default: m->err = "set_tensor: unknown tensor id"; return -1;
        }
    }
    if (!ok) {
        if (m->err.empty()) m->err = std::string("set_tensor failed: ") + llamd_cuda_last_error_string();
        return -1;
    }
    if (total) m->weight_bytes += count * LLAMD_Q6K_BLOCK_BYTES;
    else m->weight_bytes += count * sizeof(float);
    return 0;
}

size_t llamd_model_weight_bytes(llamd_model *h) { return h ? ((Model *)h)->weight_bytes : 0; }

int llamd_model_set_option(llamd_model *h, const char *name, int value) {
    Model *m = (Model *)h;
    if (!m || !name) return -1;
    if (!strcmp(name, "use_graph")) {
        m->use_graph = value;
        return 0;
    }
    if (!strcmp(name, "resident")) {
        if (m->resident != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other pass
        m->resident = value;
        return 0;
    }
    if (!strcmp(name, "arith")) {
        // 0: every f32 sum in the reference's order (bit-exact against the CPU path). 1: the 2048-term sums of the two norms
        // and the router, the softmax sum and the weighted-value sum of attention as reduction trees; integers, indices and
        // every other float operation unchanged. Decode passes on one GPU: the graph of separate launches (any number of
        // sequences up to 8) and the resident kernel; prefill tiles and wide batches keep the exact arithmetic.
        if (value && m->ep_world != 1) {
            m->err = "option arith: the fast arithmetic is a single-GPU decode mode";
            return -1;
        }
        if (value < 0 || value > 14 || (value > 1 && (value & 1))) {
            m->err = "option arith: 0 (exact), 1 (fast: all three sums) or a mask of 2 (norms) | 4 (router) | 8 (attention)";
            return -1;
        }
        value = value == 1 ? 7 : value >> 1;  // (the kernel's mask: 1 norms, 2 router, 4 attention)
        if (m->arith_fast != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();
        m->arith_fast = value;
        return 0;
    }
    if (!strcmp(name, "resident_profile")) {
        if (m->resident_profile != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();
        m->resident_profile = value;
        if (m->mega_prof.p) cudaMemsetAsync(m->mega_prof.p, 0, 32 * 8, stream());
        return 0;
    }
    if (!strcmp(name, "fuse_tails")) {
        if (m->fuse_tails != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_tails = value;
        return 0;
    }
    if (!strcmp(name, "prefetch")) {
        if (m->prefetch != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->prefetch = value;
        return 0;
    }
    if (!strcmp(name, "prefill_attn")) {
        m->prefill_attn = value;
        return 0;
    }
    if (!strcmp(name, "ep_rank_arrive")) {
        if (m->ep_rank_arrive != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();
        m->ep_rank_arrive = value != 0;
        return 0;
    }
    if (!strcmp(name, "matvec_batch_max")) {
        if (value < LLAMD_MAX_SEQ || value > LLAMD_MAX_BATCH) {
            m->err = "option matvec_batch_max: 8..256";
            return -1;
        }
        m->matvec_batch_max = value;
        return 0;
    }
    if (!strcmp(name, "dense_gemm")) {
        if (value < 0 || value > LLAMD_MAX_BATCH) {
            m->err = "option dense_gemm: 0 (never) or the number of sequences from which on, up to 256";
            return -1;
        }
        if (m->dense_gemm != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->dense_gemm = value;
        return 0;
    }
    if (!strcmp(name, "head_gemm")) {
        if (value < 0 || value > LLAMD_MAX_BATCH) {
            m->err = "option head_gemm: 0 (never) or the number of sequences from which on, up to 256";
            return -1;
        }
        if (m->head_gemm != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->head_gemm = value;
        return 0;
    }
    if (!strcmp(name, "fuse_norm_router_max")) {
        if (value < 1 || value > LLAMD_MAX_BATCH + 1) {
            m->err = "option fuse_norm_router_max: 1..257";
            return -1;
        }
        if (m->fuse_norm_router_max != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_norm_router_max = value;
        return 0;
    }
    if (!strcmp(name, "sort_slots")) {
        if (value < 0 || value > LLAMD_MAX_BATCH) {
            m->err = "option sort_slots: 0 (never) or the number of sequences from which on, up to 256";
            return -1;
        }
        if (m->sort_slots != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->sort_slots = value;
        return 0;
    }
    if (!strcmp(name, "attn_gqa")) {
        if (m->attn_gqa != (value != 0) && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->attn_gqa = value != 0;
        return 0;
    }
    if (!strcmp(name, "fuse_attn_quant")) {
        if (m->fuse_attn_quant != (value != 0) && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_attn_quant = value != 0;
        return 0;
    }
    if (!strcmp(name, "early_loads")) {
        if (m->early_loads != (value != 0) && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->early_loads = value != 0;
        return 0;
    }
    if (!strcmp(name, "fuse_silu_down")) {
        if (m->fuse_silu_down != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_silu_down = value;
        return 0;
    }
    if (!strcmp(name, "fuse_norm_qkv")) {
        if (m->fuse_norm_qkv != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_norm_qkv = value;
        return 0;
    }
    if (!strcmp(name, "fuse_rope_attn")) {
        if (m->fuse_rope_attn != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_rope_attn = value;
        return 0;
    }
    if (!strcmp(name, "fuse_norm_router")) {
        if (m->fuse_norm_router != value && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other setting
        m->fuse_norm_router = value;
        return 0;
    }
    if (!strcmp(name, "kv_f16")) {
        // 1: the K/V caches hold binary16 values (the benchmark configuration's "KV cache is f16"; the reference's caches are
        // f32): a value is rounded to nearest-even once, at the store, and widened exactly at every load, nothing else
        // changes. The caches are re-allocated and EMPTY afterwards: set it before the first pass.
        if ((value != 0) == (m->kv16 != 0)) return 0;
        if (m->ep_world > 1 && m->ep_p2p) {
            m->err = "option kv_f16: set it before the peer-memory attach";
            return -1;
        }
        cudaStreamSynchronize(stream());
        if (g_graph_owner == m->id) llamd_fwd_graph_destroy();
        const size_t kvd = (size_t)m->hp.n_head_kv * m->hp.head_dim, elem = value ? 2 : 4;
        bool ok = true;
        for (auto &l : m->layers) {
            l.kc.release();
            l.vc.release();
            ok = ok && l.kc.alloc((size_t)m->max_kv * kvd * elem * m->max_seq) && l.vc.alloc((size_t)m->max_kv * kvd * elem * m->max_seq);
        }
        m->kc32.release();
        m->vc32.release();
        if (value) ok = ok && m->kc32.alloc((size_t)m->max_kv * kvd * 4) && m->vc32.alloc((size_t)m->max_kv * kvd * 4);
        if (!ok) {
            m->err = std::string("option kv_f16: ") + llamd_cuda_last_error_string();
            return -1;
        }
        m->kv16 = value != 0;
        m->mega_ready = false;  // (the resident kernel's layer table names the caches)
        return 0;
    }
    if (!strcmp(name, "prefill_prefold")) {
        // 1: keep every expert matrix a second time, folded into the integer MMA's operand order (2 bytes per weight:
        // +58 GB for the 48-layer model), so that a prefill tile's grouped GEMMs copy operands instead of folding them.
        // Built at the next prefill; 0 releases the copies. Same bits either way.
        if (!value && m->prefold_ready) {
            cudaStreamSynchronize(stream());
            for (auto &l : m->layers)
                for (Buf *b : {&l.gate_fold, &l.up_fold, &l.down_fold}) b->release();
            m->prefold_ready = false;
        }
        m->prefold = value != 0;
        return 0;
    }
    if (!strcmp(name, "prefill_gemm")) {
        m->prefill_gemm = value;
        return 0;
    }
    if (!strcmp(name, "prefill_tile")) {
        if (value < 1 || value > 4096) return -1;
        m->prefill_tile = value;
        return 0;
    }
    if (!strcmp(name, "batch_group")) {
        llamd_fwd_set_batch_group(value);
        if (g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other grouping
        return 0;
    }
    if (!strcmp(name, "pdl")) {
        llamd_fwd_set_pdl(value);
        if (g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded in the other mode
        return 0;
    }
    if (!strcmp(name, "ep_poll_limit")) {
        // polls (128 ns back-off each after the first 32) before a wait on another rank gives up: the default, 2^24, is seconds
        if (value < 1) return -1;
        if ((unsigned)value != m->ep_poll_limit && g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the other limit
        m->ep_poll_limit = (unsigned)value;
        return 0;
    }
    if (!strcmp(name, "trace")) {
        if (value && !m->trace_x.p) {
            if (!m->trace_x.alloc((size_t)m->hp.n_layer * m->max_seq * m->hp.n_embd * sizeof(float)) ||
                !m->trace_ids.alloc((size_t)m->hp.n_layer * m->max_seq * m->hp.n_expert_used * sizeof(int32_t)))
                return -1;
        }
        m->trace = value;
        return 0;
    }
    m->err = "set_option: unknown option";
    return -1;
}

static int run_wide_batch(Model &m, const int32_t *tokens, const int32_t *positions, int nseq, int32_t *out_tokens);

int llamd_model_forward(llamd_model *h, int32_t token, int32_t pos, int32_t *out_token) {
    Model *m = (Model *)h;
    if (!m || !out_token) return -1;
    m->err.clear();
    return run(*m, &token, &pos, 1, out_token);
}

int llamd_model_forward_batch(llamd_model *h, const int32_t *tokens, const int32_t *positions, int nseq, int32_t *out_tokens) {
    Model *m = (Model *)h;
    if (!m || !tokens || !positions || !out_tokens) return -1;
    m->err.clear();
    if (nseq > m->matvec_batch_max && nseq > LLAMD_MAX_SEQ && nseq <= m->max_seq) return run_wide_batch(*m, tokens, positions, nseq, out_tokens);
    // sharded experts: the per-op pass exchanges one sequence per rank; several go through the tile exchange
    if (m->ep_world > 1 && nseq > 1 && nseq <= m->max_seq) return run_wide_batch(*m, tokens, positions, nseq, out_tokens);
    return run(*m, tokens, positions, nseq, out_tokens);
}

// ---- prefill ------------------------------------------------------------------
// VulkanModel::prefill / run (crates/llamd-runtime/src/vulkan_model.rs:378-907):
// the prompt is cut into tiles of at most `prefill_tile` tokens; a tile runs the
// layer graph once with a token dimension: weights are streamed once per 8
// tokens, the routed experts go expert-major through the counting-sort plan
// (moe_group), and attention needs no mask because every token of the tile has
// stored its K and V before any query of the tile runs. Per token the
// arithmetic is the decode pass's, so prefill == sequential decode exactly.
constexpr int kGroupMaxPairs = 40960;  // what one scatter plan takes (ops.cu: moe_group_kernel)

// The folded copies of the expert matrices (option "prefill_prefold"), made once all tensors are there.
static bool ensure_prefold(Model &m) {
    if (!m.prefold || m.prefold_ready) return true;
    const llamd_hparams &hp = m.hp;
    const int eb = hp.n_embd / 256, fb = hp.n_ff_expert / 256, n_local = m.own_hi - m.own_lo;
    const size_t gu = expert_fold_bytes(eb, hp.n_ff_expert, n_local), dn = expert_fold_bytes(fb, hp.n_embd, n_local);
    const size_t need = (size_t)hp.n_layer * (2 * gu + dn);
    if (need + ((size_t)2 << 30) > llamd_cuda_free_mem()) {
        m.err = "prefill_prefold: the folded expert matrices need " + std::to_string(need >> 20) + " MiB of device memory";
        return false;
    }
    for (auto &l : m.layers) {
        if (!l.gate_fold.alloc(gu) || !l.up_fold.alloc(gu) || !l.down_fold.alloc(dn)) {
            m.err = std::string("prefill_prefold: ") + llamd_cuda_last_error_string();
            return false;
        }
        expert_prefold(l.gate_exps.p, l.gate_fold.p, eb, hp.n_ff_expert, n_local);
        expert_prefold(l.up_exps.p, l.up_fold.p, eb, hp.n_ff_expert, n_local);
        expert_prefold(l.down_exps.p, l.down_fold.p, fb, hp.n_embd, n_local);
    }
    if (llamd_fwd_sync() != 0) {
        m.err = std::string("prefill_prefold: ") + llamd_cuda_last_error_string();
        return false;
    }
    m.prefold_ready = true;
    return true;
}

static bool prefill_alloc(Model &m, int tile) {
    if (!ensure_prefold(m)) return false;
    Model::Prefill &p = m.pf;
    if (p.tile >= tile) return true;
    if (p.ep_cap) {
        m.err = "prefill: the tile buffers have been shared with the other ranks and cannot grow (set prefill_tile before the attach)";
        return false;
    }
    for (Buf *b : {&p.x, &p.xb, &p.xb2, &p.q, &p.k, &p.v, &p.attn, &p.aq, &p.ad, &p.aq2, &p.ad2, &p.ids, &p.w, &p.logits, &p.counter,
                   &p.gate, &p.up, &p.down, &p.scores, &p.meta, &p.gstart, &p.gcount, &p.ptoken, &p.pslot, &p.work, &p.n_work, &p.aq_rm,
                   &p.aq2_rm})
        b->release();
    if (p.h_meta) cudaFreeHost(p.h_meta);
    p.h_meta = nullptr;
    for (Buf *b : {&p.logits_all, &p.amax_v, &p.amax_i, &p.out_tokens}) b->release();
    if (p.h_out_tokens) cudaFreeHost(p.h_out_tokens);
    p.h_out_tokens = nullptr;
    const llamd_hparams &hp = m.hp;
    const size_t T = tile, E = hp.n_embd, qd = (size_t)hp.n_head * hp.head_dim, kvd = (size_t)hp.n_head_kv * hp.head_dim;
    const size_t nu = hp.n_expert_used, ffe = hp.n_ff_expert, ne = hp.n_expert, max_act = E > qd ? E : qd;
    bool ok = p.x.alloc(T * E * 4) && p.xb.alloc(T * E * 4) && p.xb2.alloc(T * E * 4) && p.q.alloc(T * qd * 4) && p.k.alloc(T * kvd * 4) &&
              p.v.alloc(T * kvd * 4) && p.attn.alloc(T * qd * 4) && p.aq.alloc(T * max_act) && p.ad.alloc(T * (max_act / 256) * 4) &&
              p.aq2.alloc(T * nu * ffe) && p.ad2.alloc(T * nu * (ffe / 256) * 4) && p.ids.alloc(T * nu * 4) && p.w.alloc(T * nu * 4) &&
              p.logits.alloc(T * ne * 4) && p.counter.alloc(T * 4) && p.gate.alloc(T * nu * ffe * 4) && p.up.alloc(T * nu * ffe * 4) &&
              p.down.alloc(T * nu * E * 4) && p.scores.alloc(T * hp.n_head * (size_t)((m.max_kv + 3) & ~3) * 4) && p.meta.alloc(T * 8) &&
              p.gstart.alloc(ne * 4) && p.gcount.alloc(ne * 4) && p.ptoken.alloc(T * nu * 4 * (size_t)m.ep_world) &&
              p.pslot.alloc(T * nu * 4 * (size_t)m.ep_world) &&
              p.work.alloc((T * nu / 8 + ne + 1) * 12) && p.n_work.alloc(4) && p.aq_rm.alloc(T * max_act * 4) && p.aq2_rm.alloc(T * nu * ffe * 4) &&
              cudaMallocHost((void **)&p.h_meta, T * 8) == cudaSuccess;
    if (ok && m.ep_world > 1) {
        for (Buf *b : {&p.aq_all, &p.ad_all, &p.ids_all, &p.aq_all_rm, &p.gate_all, &p.up_all, &p.aq2_all, &p.ad2_all, &p.aq2_all_rm, &p.push_done,
                       &p.down_tab, &p.aq_tab, &p.ad_tab, &p.ids_tab})
            b->release();
        const size_t W = m.ep_world, G = W * T;  // gathered token rows
        ok = p.aq_all.alloc(G * E) && p.ad_all.alloc(G * (E / 256) * 4) && p.ids_all.alloc(G * nu * 4) && p.aq_all_rm.alloc(G * E) &&
             p.gate_all.alloc(G * nu * ffe * 4) && p.up_all.alloc(G * nu * ffe * 4) && p.aq2_all.alloc(G * nu * ffe) &&
             p.ad2_all.alloc(G * nu * (ffe / 256) * 4) && p.aq2_all_rm.alloc(G * nu * ffe) && p.push_done.alloc(W * 4) &&
             p.down_tab.alloc(W * sizeof(void *)) && p.aq_tab.alloc(W * sizeof(void *)) && p.ad_tab.alloc(W * sizeof(void *)) &&
             p.ids_tab.alloc(W * sizeof(void *)) && p.gstart.p && llamd_fwd_sync() == 0;
    }
    if (!ok) {
        m.err = std::string("prefill buffers: ") + llamd_cuda_last_error_string();
        return false;
    }
    p.tile = tile;
    return true;
}

static bool prefill_alloc_all_logits(Model &m, bool own_logits) {
    Model::Prefill &p = m.pf;
    const size_t T = p.tile;
    if (p.out_tokens.p && p.out_tokens.bytes >= T * 4 && (!own_logits || (p.logits_all.p && p.logits_all.bytes >= T * (size_t)m.hp.n_vocab * 4))) return true;
    for (Buf *b : {&p.amax_v, &p.amax_i, &p.out_tokens}) b->release();
    if (own_logits) p.logits_all.release();
    if (p.h_out_tokens) cudaFreeHost(p.h_out_tokens);
    p.h_out_tokens = nullptr;
    const bool ok = p.amax_v.alloc(T * kArgmaxBlocks * 4) && p.amax_i.alloc(T * kArgmaxBlocks * 4) && p.out_tokens.alloc(T * 4) &&
                    (!own_logits || p.logits_all.alloc(T * (size_t)m.hp.n_vocab * 4)) &&
                    cudaMallocHost((void **)&p.h_out_tokens, T * 4) == cudaSuccess;
    if (!ok) m.err = std::string("verification buffers: ") + llamd_cuda_last_error_string();
    return ok;
}

// The largest tile expert-parallel prefill can take: the scatter plan covers the pairs of ALL ranks' tiles.
static int ep_tile_cap(const Model &m) {
    int cap = kGroupMaxPairs / (m.ep_world * m.hp.n_expert_used);
    if (cap > m.prefill_tile) cap = m.prefill_tile;
    if (cap > m.max_kv) cap = m.max_kv;
    return cap < 1 ? 1 : cap;
}

// multi_seq: the T tokens belong to T different sequences, token i with its own cache (sequence i) and position:
// K/V go to the per-sequence caches and attention runs the per-sequence decode kernels. all_logits: the head runs for
// every token of the tile (logits into `logits_out`, greedy picks into pf.out_tokens), not only for the last one.
static void queue_prefill_tile(Model &m, int T, int n_kv_max, bool last, bool multi_seq = false, bool all_logits = false,
                               float *logits_out = nullptr) {
    const llamd_hparams &hp = m.hp;
    Model::Prefill &p = m.pf;
    const int E = hp.n_embd, H = hp.n_head, HKV = hp.n_head_kv, hd = hp.head_dim;
    const int kvd = HKV * hd, qd = H * hd, nu = hp.n_expert_used, ffe = hp.n_ff_expert, ne = hp.n_expert, eb = E / 256;
    const int32_t *meta = p.meta.as<int32_t>();
    float *x = p.x.as<float>();
    const int max_items = T * nu / 8 + ne;
    llamd_fwd_embed_meta(m.tok_embd.p, meta, x, eb, T);
    for (int il = 0; il < hp.n_layer; il++) {
        Layer &l = m.layers[il];
        if (il == 0)
            llamd_fwd_rms_norm_quant(x, l.attn_norm.as<float>(), nullptr, p.aq.as<int8_t>(), p.ad.as<float>(), E, hp.rms_eps, T);
        else
            llamd_fwd_combine_rms_norm_quant(x, p.down.as<float>(), p.w.as<float>(), nu, x, l.attn_norm.as<float>(), nullptr,
                                             p.aq.as<int8_t>(), p.ad.as<float>(), E, hp.rms_eps, T);
        const bool ep = m.ep_world > 1;  // sharded experts run on the integer GEMM; so then do the dense matmuls
        const bool gemm = m.prefill_gemm != 0 || ep, tc = m.prefill_gemm == 2 && !ep;
        if (tc) {
            llamd_fwd_act_f16_rm(p.aq.as<int8_t>(), p.ad.as<float>(), p.aq_rm.p, (size_t)T * eb);
            llamd_fwd_gemm_tokens_tc(l.attn_q.p, l.attn_k.p, l.attn_v.p, p.aq_rm.p, p.q.as<float>(), p.k.as<float>(), p.v.as<float>(), eb, qd,
                                     kvd, kvd, T);
        } else if (gemm) {
            llamd_fwd_q8k_residue_major(p.aq.as<int8_t>(), p.aq_rm.p, (size_t)T * eb);
            llamd_fwd_gemm_tokens(l.attn_q.p, l.attn_k.p, l.attn_v.p, p.aq_rm.p, p.ad.as<float>(), p.q.as<float>(), p.k.as<float>(),
                                  p.v.as<float>(), eb, qd, kvd, kvd, T);
        } else {
            llamd_fwd_matvec_tokens(l.attn_q.p, l.attn_k.p, l.attn_v.p, p.aq.as<int8_t>(), p.ad.as<float>(), p.q.as<float>(),
                                    p.k.as<float>(), p.v.as<float>(), eb, qd, kvd, kvd, T);
        }
        const float *kc_view = l.kc.as<float>(), *vc_view = l.vc.as<float>();  // what the tile's attention reads
        const float *wqn = l.has_q_norm ? l.attn_q_norm.as<float>() : nullptr, *wkn = l.has_k_norm ? l.attn_k_norm.as<float>() : nullptr;
        if (multi_seq && m.fuse_rope_attn && hd % 16 == 0 && hd <= 256) {
            // every token is another sequence at its own position, as in a decode pass: the decode pass's attention launches
            // (QK-norm, RoPE and the K/V store inside the scores launch; one CTA per kv head for all its query heads where
            // the shape allows; the rows of earlier positions read before the dependency wait -- earlier passes wrote them)
            attention_rope_quant(p.q.as<float>(), wqn, p.k.as<float>(), wkn, p.v.as<float>(), l.kc.p, l.vc.p, p.attn.as<float>(),
                                 p.scores.as<float>(), H, HKV, hd, meta, m.rope_tab.as<float>(), hp.rms_eps, m.max_kv, T, m.kv16, nullptr, nullptr,
                                 (m.early_loads ? kPassEarlyLoads : 0) | (m.attn_gqa ? kPassAttnGqa : 0));
        } else if (multi_seq && m.kv16) {
            llamd_fwd_qk_norm_rope_store_kv16(p.q.as<float>(), wqn, p.k.as<float>(), wkn, p.v.as<float>(), l.kc.p, l.vc.p, H, HKV, hd, meta,
                                              m.rope_tab.as<float>(), hp.rms_eps, T, m.max_kv);
            llamd_fwd_attention_meta_kv16(p.q.as<float>(), l.kc.p, l.vc.p, p.attn.as<float>(), p.scores.as<float>(), H, HKV, hd, meta, m.max_kv, T);
        } else if (multi_seq) {
            llamd_fwd_qk_norm_rope_store(p.q.as<float>(), wqn, p.k.as<float>(), wkn, p.v.as<float>(), l.kc.as<float>(), l.vc.as<float>(), H, HKV,
                                         hd, meta, m.rope_tab.as<float>(), hp.rms_eps, T, m.max_kv);
            llamd_fwd_attention_meta(p.q.as<float>(), l.kc.as<float>(), l.vc.as<float>(), p.attn.as<float>(), p.scores.as<float>(), H, HKV,
                                     hd, meta, m.max_kv, T);
        } else if (m.kv16) {
            // one sequence's tile over a binary16 cache: store rounded, then widen the rows the tile attends (exactly) into an
            // f32 view that the tiled kernels read as they read an f32 cache
            llamd_fwd_qk_norm_rope_store_tile_kv16(p.q.as<float>(), wqn, p.k.as<float>(), wkn, p.v.as<float>(), l.kc.p, l.vc.p, H, HKV, hd, meta,
                                                   m.rope_tab.as<float>(), hp.rms_eps, T);
            llamd_fwd_kv16_expand(l.kc.p, l.vc.p, m.kc32.as<float>(), m.vc32.as<float>(), n_kv_max, kvd);
            kc_view = m.kc32.as<float>();
            vc_view = m.vc32.as<float>();
        } else {
            llamd_fwd_qk_norm_rope_store_tile(p.q.as<float>(), wqn, p.k.as<float>(), wkn, p.v.as<float>(), l.kc.as<float>(), l.vc.as<float>(), H,
                                              HKV, hd, meta, m.rope_tab.as<float>(), hp.rms_eps, T);
        }
        if (!multi_seq) {  // (a batch of sequences attended above)
            if (m.prefill_attn)
                llamd_fwd_attention_prefill(p.q.as<float>(), kc_view, vc_view, p.attn.as<float>(), p.scores.as<float>(), H, HKV, hd, meta,
                                            (m.max_kv + 3) & ~3, T, n_kv_max);  // score rows padded to 16 bytes
            else
                llamd_fwd_attention_tile(p.q.as<float>(), kc_view, vc_view, p.attn.as<float>(), p.scores.as<float>(), H, HKV, hd, meta,
                                         m.max_kv, T);
        }
        llamd_fwd_quantize(p.attn.as<float>(), p.aq.as<int8_t>(), p.ad.as<float>(), T * (qd / 256));
        if (tc) {
            llamd_fwd_act_f16_rm(p.aq.as<int8_t>(), p.ad.as<float>(), p.aq_rm.p, (size_t)T * (qd / 256));
            llamd_fwd_gemm_tokens_tc(l.attn_out.p, nullptr, nullptr, p.aq_rm.p, p.xb2.as<float>(), nullptr, nullptr, qd / 256, E, 0, 0, T);
        } else if (gemm) {
            llamd_fwd_q8k_residue_major(p.aq.as<int8_t>(), p.aq_rm.p, (size_t)T * (qd / 256));
            llamd_fwd_gemm_tokens(l.attn_out.p, nullptr, nullptr, p.aq_rm.p, p.ad.as<float>(), p.xb2.as<float>(), nullptr, nullptr, qd / 256,
                                  E, 0, 0, T);
        } else {
            llamd_fwd_matvec_tokens(l.attn_out.p, nullptr, nullptr, p.aq.as<int8_t>(), p.ad.as<float>(), p.xb2.as<float>(), nullptr, nullptr,
                                    qd / 256, E, 0, 0, T);
        }
        llamd_fwd_add_rms_norm_quant(x, p.xb2.as<float>(), x, l.ffn_norm.as<float>(), p.xb.as<float>(), p.aq.as<int8_t>(), p.ad.as<float>(),
                                     E, hp.rms_eps, T);
        if (m.prefill_attn && T > 1) {
            llamd_fwd_matmul_f32_tokens(l.ffn_gate_inp.as<float>(), p.xb.as<float>(), p.logits.as<float>(), E, ne, T);
            llamd_fwd_router(p.logits.as<float>(), ne, nu, p.ids.as<int32_t>(), p.w.as<float>(), nullptr, T);
        } else {
            llamd_fwd_router_matvec(l.ffn_gate_inp.as<float>(), p.xb.as<float>(), E, ne, nu, p.logits.as<float>(), p.ids.as<int32_t>(),
                                    p.w.as<float>(), nullptr, p.counter.as<unsigned int>(), T);
        }
        if (m.ep_world > 1) {
            // Expert parallelism (peer-memory form). Every rank stores its tile's Q8_K activations and routed ids into every
            // rank's gathered buffers; each rank then plans and runs the pairs whose expert it owns, over all ranks'
            // tokens, with the integer GEMM, and the down projection stores each pair's rows straight into the buffer of
            // the rank the token lives on, at the pair's own (token, slot) place: the combine that follows adds them in
            // routing order exactly as one GPU does. Gathered pair id = (rank * cap + token) * n_used + slot.
            const int W = m.ep_world, cap = p.ep_cap, G = W * cap, n_local = m.own_hi - m.own_lo;
            ep_push_tile(p.ids.as<int32_t>(), p.ad.as<float>(), p.aq.as<int8_t>(), p.ids_tab.as<int32_t *>(), p.ad_tab.as<float *>(),
                         p.aq_tab.as<int8_t *>(), m.ep_disp_tab.as<unsigned int *>(), m.ep_epoch.as<unsigned int>(),
                         p.push_done.as<unsigned int>(), T, cap, nu, eb);
            ep_wait_requests(m.ep_disp.as<unsigned int>(), m.ep_epoch.as<unsigned int>(), m.ep_status.as<int>(), m.ep_poll_limit);
            moe_group_owned(p.ids_all.as<int32_t>(), ne, nu, G, p.gstart.as<int32_t>(), p.gcount.as<int32_t>(), p.ptoken.as<int32_t>(),
                            p.pslot.as<int32_t>(), nullptr, nullptr, m.own_lo, m.own_hi);
            llamd_fwd_q8k_residue_major(p.aq_all.as<int8_t>(), p.aq_all_rm.p, (size_t)G * eb);
            const bool pre = m.prefold_ready;
            expert_gemm_scatter(l.gate_exps.p, l.up_exps.p, p.gstart.as<int32_t>() + m.own_lo, p.gcount.as<int32_t>() + m.own_lo,
                                p.ptoken.as<int32_t>(), p.pslot.as<int32_t>(), p.aq_all_rm.p, p.ad_all.as<float>(), p.gate_all.as<float>(),
                                p.up_all.as<float>(), eb, ffe, n_local, nullptr, 1, pre ? l.gate_fold.p : nullptr, pre ? l.up_fold.p : nullptr);
            // (every gathered pair, owned or not: the others' rows are never read)
            llamd_fwd_silu_mul_quant(p.gate_all.as<float>(), p.up_all.as<float>(), nullptr, p.aq2_all.as<int8_t>(), p.ad2_all.as<float>(),
                                     G * nu * ffe);
            llamd_fwd_q8k_residue_major(p.aq2_all.as<int8_t>(), p.aq2_all_rm.p, (size_t)G * nu * (ffe / 256));
            expert_gemm_scatter(l.down_exps.p, nullptr, p.gstart.as<int32_t>() + m.own_lo, p.gcount.as<int32_t>() + m.own_lo,
                                p.pslot.as<int32_t>(), p.pslot.as<int32_t>(), p.aq2_all_rm.p, p.ad2_all.as<float>(), p.down.as<float>(), nullptr,
                                ffe / 256, E, n_local, p.down_tab.as<float *>(), cap * nu);
            ep_signal_rows(m.ep_arrive_tab.as<unsigned int *>());
            ep_wait_rows(m.ep_arrive.as<unsigned int>(), (unsigned)W, m.ep_status.as<int>(), m.ep_poll_limit);
            continue;
        }
        // the expert scatter plan: (token, slot) pairs sorted by expert
        llamd_fwd_moe_group_work(p.ids.as<int32_t>(), ne, nu, T, p.gstart.as<int32_t>(), p.gcount.as<int32_t>(), p.ptoken.as<int32_t>(),
                                 p.pslot.as<int32_t>(), p.work.as<int32_t>(), p.n_work.as<int32_t>());
        if (tc) {
            llamd_fwd_act_f16_rm(p.aq.as<int8_t>(), p.ad.as<float>(), p.aq_rm.p, (size_t)T * eb);
            llamd_fwd_expert_gemm_tc(l.gate_exps.p, l.up_exps.p, p.gstart.as<int32_t>(), p.gcount.as<int32_t>(), p.ptoken.as<int32_t>(),
                                     p.pslot.as<int32_t>(), p.aq_rm.p, p.gate.as<float>(), p.up.as<float>(), eb, ffe, ne, T);
            llamd_fwd_silu_mul_quant(p.gate.as<float>(), p.up.as<float>(), nullptr, p.aq2.as<int8_t>(), p.ad2.as<float>(), T * nu * ffe);
            llamd_fwd_act_f16_rm(p.aq2.as<int8_t>(), p.ad2.as<float>(), p.aq2_rm.p, (size_t)T * nu * (ffe / 256));
            llamd_fwd_expert_gemm_tc(l.down_exps.p, nullptr, p.gstart.as<int32_t>(), p.gcount.as<int32_t>(), p.pslot.as<int32_t>(),
                                     p.pslot.as<int32_t>(), p.aq2_rm.p, p.down.as<float>(), nullptr, ffe / 256, E, ne, T);
        } else if (gemm) {
            llamd_fwd_q8k_residue_major(p.aq.as<int8_t>(), p.aq_rm.p, (size_t)T * eb);
            const bool pre = m.prefold_ready;
            expert_gemm_scatter(l.gate_exps.p, l.up_exps.p, p.gstart.as<int32_t>(), p.gcount.as<int32_t>(), p.ptoken.as<int32_t>(),
                                p.pslot.as<int32_t>(), p.aq_rm.p, p.ad.as<float>(), p.gate.as<float>(), p.up.as<float>(), eb, ffe, ne, nullptr, 1,
                                pre ? l.gate_fold.p : nullptr, pre ? l.up_fold.p : nullptr);
            llamd_fwd_silu_mul_quant(p.gate.as<float>(), p.up.as<float>(), nullptr, p.aq2.as<int8_t>(), p.ad2.as<float>(), T * nu * ffe);
            llamd_fwd_q8k_residue_major(p.aq2.as<int8_t>(), p.aq2_rm.p, (size_t)T * nu * (ffe / 256));
            expert_gemm_scatter(l.down_exps.p, nullptr, p.gstart.as<int32_t>(), p.gcount.as<int32_t>(), p.pslot.as<int32_t>(),
                                p.pslot.as<int32_t>(), p.aq2_rm.p, p.ad2.as<float>(), p.down.as<float>(), nullptr, ffe / 256, E, ne, nullptr, 1,
                                pre ? l.down_fold.p : nullptr, nullptr);
        } else {
            llamd_fwd_expert_major(l.gate_exps.p, l.up_exps.p, p.work.as<int32_t>(), p.n_work.as<int32_t>(), max_items,
                                   p.ptoken.as<int32_t>(), p.pslot.as<int32_t>(), p.aq.as<int8_t>(), p.ad.as<float>(), p.gate.as<float>(),
                                   p.up.as<float>(), eb, ffe, ne);
            llamd_fwd_silu_mul_quant(p.gate.as<float>(), p.up.as<float>(), nullptr, p.aq2.as<int8_t>(), p.ad2.as<float>(), T * nu * ffe);
            llamd_fwd_expert_major(l.down_exps.p, nullptr, p.work.as<int32_t>(), p.n_work.as<int32_t>(), max_items, p.pslot.as<int32_t>(),
                                   p.pslot.as<int32_t>(), p.aq2.as<int8_t>(), p.ad2.as<float>(), p.down.as<float>(), nullptr, ffe / 256, E,
                                   ne);
        }
    }
    if (all_logits) {
        // the head for every token of the tile: combine + output norm + Q8_K per row, lm_head as a GEMM, greedy pick per row
        llamd_fwd_combine_rms_norm_quant(x, p.down.as<float>(), p.w.as<float>(), nu, x, m.output_norm.as<float>(), nullptr,
                                         p.aq.as<int8_t>(), p.ad.as<float>(), E, hp.rms_eps, T);
        llamd_fwd_q8k_residue_major(p.aq.as<int8_t>(), p.aq_rm.p, (size_t)T * eb);
        llamd_fwd_gemm_tokens(m.output.p ? m.output.p : m.tok_embd.p, nullptr, nullptr, p.aq_rm.p, p.ad.as<float>(), logits_out, nullptr,
                              nullptr, eb, hp.n_vocab, 0, 0, T);
        llamd_fwd_argmax(logits_out, hp.n_vocab, p.amax_v.as<float>(), p.amax_i.as<int32_t>(), p.out_tokens.as<int32_t>(), kArgmaxBlocks, T);
        return;
    }
    if (!last) return;
    // logits for the tile's last token only (vulkan_model.rs:793-818)
    const size_t r = (size_t)(T - 1);
    llamd_fwd_combine_rms_norm_quant(x + r * E, p.down.as<float>() + r * nu * E, p.w.as<float>() + r * nu, nu, m.x.as<float>(),
                                     m.output_norm.as<float>(), nullptr, m.aq.as<int8_t>(), m.ad.as<float>(), E, hp.rms_eps, 1);
    llamd_fwd_matvec_batch(m.output.p ? m.output.p : m.tok_embd.p, m.aq.as<int8_t>(), m.ad.as<float>(), m.logits.as<float>(), eb, hp.n_vocab,
                           1);
    llamd_fwd_argmax(m.logits.as<float>(), hp.n_vocab, m.amax_v.as<float>(), m.amax_i.as<int32_t>(), m.out_token.as<int32_t>(), kArgmaxBlocks,
                     1);
}

int llamd_model_prefill(llamd_model *h, const int32_t *tokens, int n_tokens, int base_pos, int32_t *out_token) {
    Model *m = (Model *)h;
    if (!m || !tokens || n_tokens <= 0 || !out_token) return -1;
    m->err.clear();
    if (base_pos < 0 || base_pos + n_tokens > m->max_kv) {
        m->err = "prefill: positions beyond the " + std::to_string(m->max_kv) + " allocated";
        return -1;
    }
    for (int i = 0; i < n_tokens; i++)
        if (tokens[i] < 0 || tokens[i] >= m->hp.n_vocab) {
            m->err = "prefill: token id outside the vocabulary";
            return -1;
        }
    if (!check_ready(*m)) return -1;
    if (m->ep_world > 1 && !(m->ep_p2p && m->pf.ep_cap)) {
        // With sharded experts and the NCCL exchanges the prompt goes through the decode pass position by position
        // (every rank makes the same number of passes, so the collectives stay in step).
        int32_t out = -1;
        for (int i = 0; i < n_tokens; i++) {
            const int32_t pos = base_pos + i;
            if (run(*m, &tokens[i], &pos, 1, &out) != 0) return -1;
        }
        *out_token = out;
        return 0;
    }
    // (expert parallelism over peer memory: tiles of at most the shared capacity; every rank must bring the same number
    // of tiles, of any length, or the others' bounded waits run out)
    int tile = m->prefill_tile < 1 ? 1 : m->prefill_tile;
    if (m->ep_world > 1 && tile > m->pf.ep_cap) tile = m->pf.ep_cap;
    if (tile > n_tokens) tile = n_tokens;
    if (!prefill_alloc(*m, tile)) return -1;
    for (int t0 = 0; t0 < n_tokens; t0 += tile) {
        const int T = n_tokens - t0 < tile ? n_tokens - t0 : tile;
        if (llamd_fwd_sync() != 0) return -1;  // the pinned meta staging is reused per tile
        for (int i = 0; i < T; i++) {
            m->pf.h_meta[2 * i] = tokens[t0 + i];
            m->pf.h_meta[2 * i + 1] = base_pos + t0 + i;
        }
        if (cudaMemcpyAsync(m->pf.meta.p, m->pf.h_meta, (size_t)T * 8, cudaMemcpyHostToDevice, stream()) != cudaSuccess) {
            set_error(cudaGetLastError(), "prefill meta H2D");
            return -1;
        }
        queue_prefill_tile(*m, T, base_pos + t0 + T, t0 + T >= n_tokens);
    }
    if (cudaMemcpyAsync(m->h_out, m->out_token.p, 4, cudaMemcpyDeviceToHost, stream()) != cudaSuccess) return -1;
    m->h_out[m->max_seq] = 0;
    if (m->ep_p2p) cudaMemcpyAsync(m->h_out + m->max_seq, m->ep_status.p, 4, cudaMemcpyDeviceToHost, stream());
    if (llamd_fwd_sync() != 0) return -1;
    if (m->h_out[m->max_seq] != 0) {
        m->err = ep_wait_message(m->h_out[m->max_seq]);
        return -1;
    }
    if (m->prefill_gemm == 2 && llamd_fwd_gemm_tc_status() != 0) {
        m->err = "prefill: a wait inside the tcgen05 GEMM ran out; the pass is incomplete";
        return -1;
    }
    if (m->h_out[0] < 0 || m->h_out[0] >= m->hp.n_vocab) {
        m->err = "argmax returned " + std::to_string(m->h_out[0]);
        return -1;
    }
    *out_token = m->h_out[0];
    return 0;
}

// Verification of drafted tokens (speculative decoding, "verified only": the target model always decides). The n
// tokens are consumed at positions base_pos.. exactly as llamd_model_prefill consumes them -- the same tiles, the same
// arithmetic as token-by-token decode -- but the head runs for EVERY token: out_tokens[i] is the greedy token after
// tokens[0..=i]. A caller that drafted tokens[1..] keeps the longest prefix with tokens[i + 1] == out_tokens[i] and
// continues from there: K/V rows written beyond the accepted position are simply overwritten later. Because the
// tiled pass equals sequential decode bit for bit, output with drafting equals output without it.
int llamd_model_verify(llamd_model *h, const int32_t *tokens, int n_tokens, int base_pos, int32_t *out_tokens) {
    Model *m = (Model *)h;
    if (!m || !tokens || n_tokens <= 0 || !out_tokens) return -1;
    m->err.clear();
    if (m->ep_world > 1) {
        m->err = "verify: not available with sharded experts";
        return -1;
    }
    if (base_pos < 0 || base_pos + n_tokens > m->max_kv) {
        m->err = "verify: positions beyond the " + std::to_string(m->max_kv) + " allocated";
        return -1;
    }
    for (int i = 0; i < n_tokens; i++)
        if (tokens[i] < 0 || tokens[i] >= m->hp.n_vocab) {
            m->err = "verify: token id outside the vocabulary";
            return -1;
        }
    if (!check_ready(*m)) return -1;
    int tile = m->prefill_tile < 1 ? 1 : m->prefill_tile;
    if (tile > 64) tile = 64;  // every token's logits are kept: 0.6 MB each
    if (tile > n_tokens) tile = n_tokens;
    if (!prefill_alloc(*m, tile) || !prefill_alloc_all_logits(*m, true)) return -1;
    for (int t0 = 0; t0 < n_tokens; t0 += tile) {
        const int T = n_tokens - t0 < tile ? n_tokens - t0 : tile;
        if (llamd_fwd_sync() != 0) return -1;  // the pinned staging is reused per tile
        for (int i = 0; i < T; i++) {
            m->pf.h_meta[2 * i] = tokens[t0 + i];
            m->pf.h_meta[2 * i + 1] = base_pos + t0 + i;
        }
        if (cudaMemcpyAsync(m->pf.meta.p, m->pf.h_meta, (size_t)T * 8, cudaMemcpyHostToDevice, stream()) != cudaSuccess) {
            set_error(cudaGetLastError(), "verify meta H2D");
            return -1;
        }
        queue_prefill_tile(*m, T, base_pos + t0 + T, true, false, true, m->pf.logits_all.as<float>());
        if (cudaMemcpyAsync(m->pf.h_out_tokens, m->pf.out_tokens.p, (size_t)T * 4, cudaMemcpyDeviceToHost, stream()) != cudaSuccess) return -1;
        if (llamd_fwd_sync() != 0) return -1;
        for (int i = 0; i < T; i++) {
            if (m->pf.h_out_tokens[i] < 0 || m->pf.h_out_tokens[i] >= m->hp.n_vocab) {
                m->err = "argmax returned " + std::to_string(m->pf.h_out_tokens[i]);
                return -1;
            }
            out_tokens[t0 + i] = m->pf.h_out_tokens[i];
        }
    }
    return 0;
}

// forward_batch beyond LLAMD_MAX_SEQ sequences: the pass of a prefill tile whose tokens belong to nseq different
// sequences (own cache, own position), so that the matmuls run on the integer GEMM with every weight read once for all
// sequences. Per sequence the arithmetic is the single-sequence pass's.
static int run_wide_batch(Model &m, const int32_t *tokens, const int32_t *positions, int nseq, int32_t *out_tokens) {
    if (m.ep_world > 1 && (!m.ep_p2p || nseq > m.pf.ep_cap)) {
        // sharded experts: the batch runs as one tile of the peer-memory exchange (one rendezvous each way per layer for
        // all of a rank's sequences); every rank must make the same sequence of calls, with any batch size of its own
        m.err = "forward_batch: with sharded experts a batch needs the peer-memory attach, and at most as many sequences as its tile capacity";
        return -1;
    }
    for (int s = 0; s < nseq; s++) {
        if (positions[s] < 0 || positions[s] >= m.max_kv || tokens[s] < 0 || tokens[s] >= m.hp.n_vocab) {
            m.err = "forward_batch: a position beyond the allocated cache or a token outside the vocabulary";
            return -1;
        }
    }
    if (!check_ready(m)) return -1;
    if (m.hp.n_expert_used * nseq > kGroupMaxPairs) {
        m.err = "forward_batch: too many (sequence, expert) pairs for one scatter plan";
        return -1;
    }
    if (!prefill_alloc(m, nseq) || !prefill_alloc_all_logits(m, false)) return -1;
    if (llamd_fwd_sync() != 0) return -1;
    int n_kv_max = 0;
    for (int s = 0; s < nseq; s++) {
        m.pf.h_meta[2 * s] = tokens[s];
        m.pf.h_meta[2 * s + 1] = positions[s];
        if (positions[s] + 1 > n_kv_max) n_kv_max = positions[s] + 1;
    }
    if (cudaMemcpyAsync(m.pf.meta.p, m.pf.h_meta, (size_t)nseq * 8, cudaMemcpyHostToDevice, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "batch meta H2D");
        return -1;
    }
    queue_prefill_tile(m, nseq, n_kv_max, true, true, true, m.logits.as<float>());
    if (cudaMemcpyAsync(m.pf.h_out_tokens, m.pf.out_tokens.p, (size_t)nseq * 4, cudaMemcpyDeviceToHost, stream()) != cudaSuccess) return -1;
    m.h_out[m.max_seq] = 0;
    if (m.ep_p2p) cudaMemcpyAsync(m.h_out + m.max_seq, m.ep_status.p, 4, cudaMemcpyDeviceToHost, stream());
    if (llamd_fwd_sync() != 0) return -1;
    if (m.h_out[m.max_seq] != 0) {
        m.err = ep_wait_message(m.h_out[m.max_seq]);
        return -1;
    }
    for (int s = 0; s < nseq; s++) {
        if (m.pf.h_out_tokens[s] < 0 || m.pf.h_out_tokens[s] >= m.hp.n_vocab) {
            m.err = "argmax returned " + std::to_string(m.pf.h_out_tokens[s]);
            return -1;
        }
        out_tokens[s] = m.pf.h_out_tokens[s];
    }
    return 0;
}

// Resident greedy decode: n passes queued back to back, each feeding its
// token to the next on the device; one synchronise at the end. Equivalent to
// n calls of llamd_model_forward with the returned token fed back.
// ms_out (optional): device time of the n passes, from events on the library stream.
int llamd_model_decode(llamd_model *h, int32_t first_token, int32_t start_pos, int n, int32_t *out_tokens, float *ms_out) {
    Model *m = (Model *)h;
    if (!m || n <= 0 || !out_tokens) return -1;
    m->err.clear();
    if (start_pos < 0 || start_pos + n > m->max_kv || first_token < 0 || first_token >= m->hp.n_vocab) {
        m->err = "decode: positions beyond the allocated KV cache, or a bad token";
        return -1;
    }
    if (!check_ready(*m)) return -1;
    if (m->resident) mega_prepare(*m);
    m->h_meta[0] = first_token;
    m->h_meta[1] = start_pos;
    LLAMD_TRY(cudaMemcpyAsync(m->meta.p, m->h_meta, 8, cudaMemcpyHostToDevice, stream()), "decode meta H2D");
    LLAMD_TRY(cudaMemsetAsync(m->tok_count.p, 0, 4, stream()), "decode counter reset");
    if (m->use_graph && (!llamd_fwd_has_graph() || g_graph_owner != m->id || m->graph_nseq != 1)) {
        llamd_fwd_graph_destroy();
        if (llamd_fwd_begin_capture() != 0) return -1;
        const unsigned long long before = g_launches;
        queue_token(*m, 1);
        m->launches_per_pass = g_launches - before;
        if (llamd_fwd_end_capture() != 0 || error_code() != 0) {
            llamd_fwd_graph_destroy();
            return -1;
        }
        g_graph_owner = m->id;
        m->graph_nseq = 1;
    }
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    int rc = 0;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess || cudaEventRecord(e0, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "decode events");
        rc = -1;
    }
    for (int i = 0; rc == 0 && i < n; i++) {
        if (m->use_graph) {
            if (llamd_fwd_graph_launch() != 0) rc = -1;
        } else {
            queue_token(*m, 1);
        }
    }
    if (rc == 0 && cudaEventRecord(e1, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "decode events");
        rc = -1;
    }
    if (rc == 0 && cudaMemcpyAsync(out_tokens, m->tok_log.p, (size_t)n * 4, cudaMemcpyDeviceToHost, stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "decode D2H");
        rc = -1;
    }
    m->h_out[m->max_seq] = 0;
    if (rc == 0 && m->ep_p2p) cudaMemcpyAsync(m->h_out + m->max_seq, m->ep_status.p, 4, cudaMemcpyDeviceToHost, stream());
    if (rc == 0 && m->mega_ready && m->resident) cudaMemcpyAsync(m->h_out + m->max_seq, m->mega_status.p, 4, cudaMemcpyDeviceToHost, stream());
    // whatever was queued is drained before the events go away, also after a failure
    const int sync_rc = (m->ep_world > 1 && !m->ep_p2p) ? ep_bounded_sync() : llamd_fwd_sync();
    if (sync_rc != 0) rc = -1;
    if (rc == 0 && ms_out) cudaEventElapsedTime(ms_out, e0, e1);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (rc == 0 && m->h_out[m->max_seq] != 0) {
        m->err = m->ep_p2p ? ep_wait_message(m->h_out[m->max_seq])
                           : std::string("resident decode kernel: a grid barrier was not completed within its limit; the tokens are not valid");
        rc = -1;
    }
    return rc;
}

// Device time of `iters` repetitions of one pass's Q6_K matvec launches only.
int llamd_model_bench_matvecs(llamd_model *h, int iters, int nseq, float *ms_out, int *launches_out) {
    Model *m = (Model *)h;
    if (!m || iters <= 0 || !ms_out || nseq < 1 || nseq > m->max_seq || !check_ready(*m)) return -1;
    if (m->ep_world > 1) {
        m->err = "bench_matvecs: not available with sharded experts";
        return -1;
    }
    const unsigned long long before = g_launches;
    queue_matvecs_only(*m, nseq);  // warm
    if (launches_out) *launches_out = (int)(g_launches - before);
    if (llamd_fwd_sync() != 0) return -1;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    cudaEventRecord(e0, stream());
    for (int i = 0; i < iters; i++) queue_matvecs_only(*m, nseq);
    cudaEventRecord(e1, stream());
    const int rc = llamd_fwd_sync();
    cudaEventElapsedTime(ms_out, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return rc;
}

unsigned long long llamd_model_launches_per_pass(llamd_model *h) { return h ? ((Model *)h)->launches_per_pass : 0; }

// One un-graphed pass with an event after every launch group; ms_out[LLAMD_PH_COUNT] receives the time
// from the previous mark to each phase's mark, summed over the layers (so it includes the launch gap).
int llamd_model_profile_pass(llamd_model *h, int32_t token, int32_t pos, float *ms_out) {
    Model *m = (Model *)h;
    if (!m || !ms_out || m->ep_world > 1) return -1;
    m->err.clear();
    const int saved_graph = m->use_graph;
    m->use_graph = 0;
    m->profiling = true;
    int32_t out = 0;
    const int rc = run(*m, &token, &pos, 1, &out);
    m->profiling = false;
    m->use_graph = saved_graph;
    if (rc != 0) return -1;
    for (int i = 0; i < LLAMD_PH_COUNT; i++) ms_out[i] = 0.0f;
    for (size_t i = 1; i < m->prof_events.size(); i++) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, m->prof_events[i - 1], m->prof_events[i]) != cudaSuccess) {
            cudaGetLastError();
            break;
        }
        const int ph = m->prof_phase[i];
        if (ph >= 0 && ph < LLAMD_PH_COUNT) ms_out[ph] += ms;
    }
    return 0;
}

// ---- expert parallelism over peer memory (no collective in the pass) ----
// export: LLAMD_EP_P2P_RECORD bytes = the IPC handles of this rank's expert-output buffer, arrival counter, gathered
// ids / scales / quants buffers and dispatch counter.
// attach: the records of ALL ranks in rank order; maps the peers' buffers and switches the decode pass to the form in
// which requests are pushed to the peers and an owned expert's rows are stored straight into the home rank's buffer.
// Every rank must attach.
constexpr int kEpShared = LLAMD_EP_P2P_RECORD / 64;  // buffers every rank shares with the others
static Buf *ep_shared_buf(Model &m, int i) {
    Buf *b[kEpShared] = {&m.e_down, &m.ep_arrive, &m.ids_all, &m.ad_all, &m.aq_all, &m.ep_disp,
                         &m.pf.down, &m.pf.aq_all, &m.pf.ad_all, &m.pf.ids_all};  // the last four: a prefill tile's
    return b[i];
}
static Buf *ep_table_buf(Model &m, int i) {
    Buf *b[kEpShared] = {&m.ep_out_tab, &m.ep_arrive_tab, &m.ep_ids_tab, &m.ep_ad_tab, &m.ep_aq_tab, &m.ep_disp_tab,
                         &m.pf.down_tab, &m.pf.aq_tab, &m.pf.ad_tab, &m.pf.ids_tab};
    return b[i];
}
// The tile buffers must exist before they can be shared: made here for the current prefill_tile (capped by what one
// scatter plan over all ranks' tiles can take), and fixed from then on.
static bool ep_prepare_shared(Model &m) {
    if (m.pf.ep_cap) return true;
    const int cap = ep_tile_cap(m);
    if (!prefill_alloc(m, cap)) return false;
    m.pf.ep_cap = m.pf.tile;
    return true;
}
int llamd_model_ep_p2p_export(llamd_model *h, void *out) {
    Model *m = (Model *)h;
    if (!m || !out || m->ep_world < 2 || !ep_prepare_shared(*m)) return -1;
    for (int i = 0; i < kEpShared; i++)
        if (llamd_cuda_ep_ipc_export(ep_shared_buf(*m, i)->p, (char *)out + 64 * i) != 0) return -1;
    return 0;
}
int llamd_model_ep_p2p_attach(llamd_model *h, const void *all, int world) {
    Model *m = (Model *)h;
    if (!m || !all || world != m->ep_world || world < 2 || !ep_prepare_shared(*m)) return -1;
    std::vector<void *> tab[kEpShared];
    for (int i = 0; i < kEpShared; i++) tab[i].resize(world);
    for (int r = 0; r < world; r++) {
        for (int i = 0; i < kEpShared; i++) {
            if (r == m->ep_rank) {
                tab[i][r] = ep_shared_buf(*m, i)->p;
                continue;
            }
            void *p = llamd_cuda_ep_ipc_open((const char *)all + (size_t)r * LLAMD_EP_P2P_RECORD + 64 * i);
            if (!p) {
                m->err = "ep_p2p_attach: a peer's buffer could not be mapped";
                return -1;
            }
            m->ep_mapped.push_back(p);
            tab[i][r] = p;
        }
    }
    for (int i = 0; i < kEpShared; i++)
        if (cudaMemcpyAsync(ep_table_buf(*m, i)->p, tab[i].data(), world * sizeof(void *), cudaMemcpyHostToDevice, stream()) != cudaSuccess) return -1;
    // (the counters are zero since the model was created and only this protocol touches them: clearing them here
    // could erase the arrival of a peer that attached first)
    if (llamd_fwd_sync() != 0) return -1;
    if (g_graph_owner == m->id) llamd_fwd_graph_destroy();  // recorded with the collectives
    m->ep_p2p = 1;
    return 0;
}

// The same switch for ranks that can hand each other device pointers directly (several models in one process, or
// memory mapped by the caller): ptrs is [world][6] in the order of llamd_model_ep_p2p_buffers; row `rank` is ignored.
int llamd_model_ep_p2p_buffers(llamd_model *h, void **out6) {
    Model *m = (Model *)h;
    if (!m || !out6 || m->ep_world < 2 || !ep_prepare_shared(*m)) return -1;
    for (int i = 0; i < kEpShared; i++) out6[i] = ep_shared_buf(*m, i)->p;
    return 0;
}
int llamd_model_ep_p2p_attach_ptrs(llamd_model *h, void *const *ptrs, int world) {
    Model *m = (Model *)h;
    if (!m || !ptrs || world != m->ep_world || world < 2 || !ep_prepare_shared(*m)) return -1;
    std::vector<void *> tab[kEpShared];
    for (int i = 0; i < kEpShared; i++) {
        tab[i].resize(world);
        for (int r = 0; r < world; r++) {
            tab[i][r] = r == m->ep_rank ? ep_shared_buf(*m, i)->p : ptrs[(size_t)r * kEpShared + i];
            if (!tab[i][r]) {
                m->err = "ep_p2p_attach_ptrs: a null buffer";
                return -1;
            }
        }
    }
    for (int i = 0; i < kEpShared; i++)
        if (cudaMemcpyAsync(ep_table_buf(*m, i)->p, tab[i].data(), world * sizeof(void *), cudaMemcpyHostToDevice, stream()) != cudaSuccess) return -1;
    if (llamd_fwd_sync() != 0) return -1;
    if (g_graph_owner == m->id) llamd_fwd_graph_destroy();
    m->ep_p2p = 1;
    return 0;
}
// Nanoseconds per phase of the resident decode kernel, accumulated by its CTA 0 since "resident_profile" was set:
// 14 slots in the kernel's order (phases A, B1, B2, C, D, E, F, each followed by its barrier); out32 gets 32 values.
int llamd_model_resident_profile(llamd_model *h, unsigned long long *out32) {
    Model *m = (Model *)h;
    if (!m || !out32 || !m->mega_prof.p) return -1;
    return llamd_fwd_download(out32, m->mega_prof.p, 32 * 8);
}
// Tokens per rank and tile that expert-parallel prefill takes (fixed when the buffers are shared); 0 before that.
int llamd_model_ep_tile_cap(llamd_model *h) { return h ? ((Model *)h)->pf.ep_cap : 0; }
// The status word of the bounded device-side waits: 0, or what the first wait that ran out left (1: expert rows, 2: requests).
int llamd_model_ep_status(llamd_model *h) {
    Model *m = (Model *)h;
    if (!m || !m->ep_status.p) return 0;
    int st = 0;
    if (llamd_fwd_download(&st, m->ep_status.p, 4) != 0) return -1;
    return st;
}

int llamd_model_logits(llamd_model *h, float *host_out, int nseq) {
    Model *m = (Model *)h;
    if (!m || !host_out || nseq < 1 || nseq > m->max_seq) return -1;
    return llamd_fwd_download(host_out, m->logits.p, (size_t)nseq * m->hp.n_vocab * sizeof(float));
}

int llamd_model_read_trace(llamd_model *h, float *x_out, int32_t *ids_out) {
    Model *m = (Model *)h;
    if (!m || !m->trace_x.p) return -1;
    if (x_out && llamd_fwd_download(x_out, m->trace_x.p, m->trace_x.bytes) != 0) return -1;
    if (ids_out && llamd_fwd_download(ids_out, m->trace_ids.p, m->trace_ids.bytes) != 0) return -1;
    return 0;
}

int llamd_model_read_kv(llamd_model *h, int layer, int seq, int n_pos, float *k_out, float *v_out) {
    Model *m = (Model *)h;
    if (!m || layer < 0 || layer >= m->hp.n_layer || seq < 0 || seq >= m->max_seq || n_pos < 0 || n_pos > m->max_kv) return -1;
    const size_t kvd = (size_t)m->hp.n_head_kv * m->hp.head_dim;
    const size_t off = (size_t)seq * m->max_kv * kvd;
    if (m->kv16) {
        // (one sequence's rows widened on the device into the f32 view, then read: the values are the cache's, exactly)
        const uint8_t *k16 = (const uint8_t *)m->layers[layer].kc.p + off * 2, *v16 = (const uint8_t *)m->layers[layer].vc.p + off * 2;
        llamd_fwd_kv16_expand(k16, v16, m->kc32.as<float>(), m->vc32.as<float>(), n_pos, (int)kvd);
        if (k_out && llamd_fwd_download(k_out, m->kc32.p, n_pos * kvd * sizeof(float)) != 0) return -1;
        if (v_out && llamd_fwd_download(v_out, m->vc32.p, n_pos * kvd * sizeof(float)) != 0) return -1;
        return 0;
    }
    if (k_out && llamd_fwd_download(k_out, m->layers[layer].kc.as<float>() + off, n_pos * kvd * sizeof(float)) != 0) return -1;
    if (v_out && llamd_fwd_download(v_out, m->layers[layer].vc.as<float>() + off, n_pos * kvd * sizeof(float)) != 0) return -1;
    return 0;
}

}  // extern "C"
