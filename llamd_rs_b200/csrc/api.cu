// extern "C" entry points of the Q6_K matvec family, and the host-facing
// (host pointers in, host pointers out, synchronising) calls that mirror
// crates/llamd-rocm/src/lib.rs:91-135 / crates/llamd-rocm/kernels/llamd.hip:1053-1292.
#include <string.h>

#include "common.cuh"

using namespace llamd;

// The grouped device-pointer forms do not know how many experts the tensor
// holds (the reference's do not either: its Rust wrappers check the ids,
// crates/llamd-rocm/src/lib.rs:461-470). The in-kernel guard therefore accepts
// any non-negative id.
static const int kAnyExpert = 0x7fffffff;

namespace llamd {
void matvec_batch(const MatvecPlans &pl, const void *w, const int8_t *aq, const float *ad, float *out, int blocks, int rows, int nseq) {
    const void *ws[1] = {w};
    float *os[1] = {out};
    launch_matvec(1, ws, os, &rows, blocks, aq, ad, nseq, nullptr, 1, 0, 1, 0, nullptr, nullptr, 0, 0x7fffffff, pl);
}
void matvec_x3_batch(const MatvecPlans &pl, const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad, float *o0,
                     float *o1, float *o2, int blocks, int rows0, int rows1, int rows2, int nseq) {
    const void *ws[3] = {w0, w1, w2};
    float *os[3] = {o0, o1, o2};
    const int rows[3] = {rows0, rows1, rows2};
    launch_matvec(3, ws, os, rows, blocks, aq, ad, nseq, nullptr, 1, 0, 1, 0, nullptr, nullptr, 0, 0x7fffffff, pl);
}
void matvec_grouped_pa_silu(const MatvecPlans &pl, const void *w, const int32_t *ids, const float *gate, const float *up, float *out, int blocks,
                            int rows, int n_used, int nseq) {
    const void *ws[1] = {w};
    float *os[1] = {out};
    launch_matvec(1, ws, os, &rows, blocks, nullptr, nullptr, 1, ids, n_used * nseq, kAnyExpert, 1, 2, gate, up, 0, 0x7fffffff, pl);
}
// Q, K, V of one sequence with the attention norm (and the MoE combine before it) folded in: pl.norm says from what.
void matvec_x3_norm(const MatvecPlans &pl, const void *w0, const void *w1, const void *w2, float *o0, float *o1, float *o2, int blocks,
                    int rows0, int rows1, int rows2) {
    const void *ws[3] = {w0, w1, w2};
    float *os[3] = {o0, o1, o2};
    const int rows[3] = {rows0, rows1, rows2};
    launch_matvec(3, ws, os, rows, blocks, nullptr, nullptr, 1, nullptr, 1, 0, 1, /*ACT_NORM*/ 3, nullptr, nullptr, 0, 0x7fffffff, pl);
}
void matvec_grouped_x2_batch(const MatvecPlans &pl, const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                             float *oa, float *ob, int blocks, int rows, int n_used, int nseq) {
    const void *ws[2] = {wa, wb};
    float *os[2] = {oa, ob};
    const int r2[2] = {rows, rows};
    launch_matvec(2, ws, os, r2, blocks, aq, ad, 1, ids, n_used * nseq, kAnyExpert, n_used, 0, nullptr, nullptr, 0, 0x7fffffff, pl);
}
void matvec_grouped_pa_batch(const MatvecPlans &pl, const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out,
                             int blocks, int rows, int n_used, int nseq) {
    const void *ws[1] = {w};
    float *os[1] = {out};
    launch_matvec(1, ws, os, &rows, blocks, aq, ad, 1, ids, n_used * nseq, kAnyExpert, 1, 0, nullptr, nullptr, 0, 0x7fffffff, pl);
}
void matvec_grouped_x2_owned(const MatvecPlans &pl, const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                             float *oa, float *ob, int blocks, int rows, int n_used, int n_slots, int own_lo, int own_hi) {
    const void *ws[2] = {wa, wb};
    float *os[2] = {oa, ob};
    const int r2[2] = {rows, rows};
    launch_matvec(2, ws, os, r2, blocks, aq, ad, 1, ids, n_slots, kAnyExpert, n_used, 0, nullptr, nullptr, own_lo, own_hi, pl);
}
void matvec_grouped_pa_owned(const MatvecPlans &pl, const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out,
                             int blocks, int rows, int n_slots, int own_lo, int own_hi) {
    const void *ws[1] = {w};
    float *os[1] = {out};
    launch_matvec(1, ws, os, &rows, blocks, aq, ad, 1, ids, n_slots, kAnyExpert, 1, 0, nullptr, nullptr, own_lo, own_hi, pl);
}
}  // namespace llamd

extern "C" {

void llamd_fwd_matvec_batch(const void *w, const int8_t *aq, const float *ad, float *out, int blocks, int rows, int nseq) {
    matvec_batch(MatvecPlans{}, w, aq, ad, out, blocks, rows, nseq);
}
void llamd_fwd_matvec(const void *w, const int8_t *aq, const float *ad, float *out, int blocks, int rows) {
    llamd_fwd_matvec_batch(w, aq, ad, out, blocks, rows, 1);
}
void llamd_fwd_matvec_x3_batch(const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad, float *o0, float *o1,
                               float *o2, int blocks, int rows0, int rows1, int rows2, int nseq) {
    matvec_x3_batch(MatvecPlans{}, w0, w1, w2, aq, ad, o0, o1, o2, blocks, rows0, rows1, rows2, nseq);
}
void llamd_fwd_matvec_x3(const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad, float *o0, float *o1,
                         float *o2, int blocks, int rows0, int rows1, int rows2) {
    llamd_fwd_matvec_x3_batch(w0, w1, w2, aq, ad, o0, o1, o2, blocks, rows0, rows1, rows2, 1);
}
void llamd_fwd_matvec_grouped(const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out, int blocks, int rows,
                              int n_used) {
    const void *ws[1] = {w};
    float *os[1] = {out};
    launch_matvec(1, ws, os, &rows, blocks, aq, ad, 1, ids, n_used, kAnyExpert, n_used);
}
void llamd_fwd_matvec_grouped_x2_batch(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad, float *oa,
                                       float *ob, int blocks, int rows, int n_used, int nseq) {
    matvec_grouped_x2_batch(MatvecPlans{}, wa, wb, ids, aq, ad, oa, ob, blocks, rows, n_used, nseq);
}
// llamd_fwd_matvec_grouped_x2_batch followed by llamd_fwd_silu_mul_quant of its outputs, in one launch: the CTA
// that completes a slot last writes act = silu(gate) * up as Q8_K into qs [slots][rows], d [slots][rows/256].
// counter: n_used*nseq zero-initialised words the launch leaves at zero again. rows must be a multiple of 256.
void llamd_fwd_matvec_grouped_x2_silu_quant(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                                            float *oa, float *ob, unsigned int *counter, int8_t *qs, float *d, int blocks, int rows,
                                            int n_used, int nseq) {
    if (!counter || !qs || !d || rows % 256) {
        set_error_msg("matvec_grouped_x2_silu_quant: counter, qs, d must be given and rows a multiple of 256");
        return;
    }
    MatvecPlans pl = {};
    pl.tail = TailPlan{counter, qs, d};
    matvec_grouped_x2_batch(pl, wa, wb, ids, aq, ad, oa, ob, blocks, rows, n_used, nseq);
}
void llamd_fwd_matvec_grouped_x2(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad, float *oa,
                                 float *ob, int blocks, int rows, int n_used) {
    llamd_fwd_matvec_grouped_x2_batch(wa, wb, ids, aq, ad, oa, ob, blocks, rows, n_used, 1);
}
void llamd_fwd_matvec_grouped_pa_batch(const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out, int blocks,
                                       int rows, int n_used, int nseq) {
    matvec_grouped_pa_batch(MatvecPlans{}, w, ids, aq, ad, out, blocks, rows, n_used, nseq);
}
void llamd_fwd_matvec_grouped_pa(const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out, int blocks, int rows,
                                 int n_used) {
    llamd_fwd_matvec_grouped_pa_batch(w, ids, aq, ad, out, blocks, rows, n_used, 1);
}

// f32 activations quantized inside the matvec (fuses the separate `quantize`
// launch of crates/llamd-runtime/src/device.rs:580 into the attn_out projection).
void llamd_fwd_matvec_f32act(const void *w, const float *x, float *out, int blocks, int rows, int nseq) {
    const void *ws[1] = {w};
    float *os[1] = {out};
    launch_matvec(1, ws, os, &rows, blocks, nullptr, nullptr, nseq, nullptr, 1, 0, 1, 1, x, nullptr);
}
// The down projection with silu(gate)*up and its quantization inside
// (fuses device.rs:615-618 into :622): gate/up are [nseq*n_used][blocks*256].
void llamd_fwd_matvec_grouped_pa_silu(const void *w, const int32_t *ids, const float *gate, const float *up, float *out, int blocks,
                                      int rows, int n_used, int nseq) {
    matvec_grouped_pa_silu(MatvecPlans{}, w, ids, gate, up, out, blocks, rows, n_used, nseq);
}

// Expert-parallel forms: `ids` are GLOBAL expert ids for n_slots slots; this GPU holds experts
// [own_lo, own_hi) in `w*` from local index 0 and computes only the slots it owns.
// x2: slot s reads activation aq[s / n_used]; pa: slot s reads aq[s].
void llamd_fwd_matvec_grouped_x2_owned(const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad, float *oa,
                                       float *ob, int blocks, int rows, int n_used, int n_slots, int own_lo, int own_hi) {
    matvec_grouped_x2_owned(MatvecPlans{}, wa, wb, ids, aq, ad, oa, ob, blocks, rows, n_used, n_slots, own_lo, own_hi);
}
void llamd_fwd_matvec_grouped_pa_owned(const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out, int blocks,
                                       int rows, int n_slots, int own_lo, int own_hi) {
    matvec_grouped_pa_owned(MatvecPlans{}, w, ids, aq, ad, out, blocks, rows, n_slots, own_lo, own_hi);
}

// ---- many tokens at once (prefill) -------------------------------------------
// Up to three matrices that share ntok activations [ntok][blocks*256]; outputs [ntok][rows_i].
void llamd_fwd_matvec_tokens(const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad, float *o0, float *o1,
                             float *o2, int blocks, int rows0, int rows1, int rows2, int ntok) {
    const void *ws[3] = {w0, w1, w2};
    float *os[3] = {o0, o1, o2};
    const int rows[3] = {rows0, rows1, rows2};
    const int njobs = w2 ? 3 : (w1 ? 2 : 1);
    launch_matvec_multi(njobs, ws, os, rows, blocks, aq, ad, ntok, nullptr, nullptr, 0, nullptr, nullptr, 0);
}
// Expert-major grouped matvec over the scatter plan of llamd_fwd_moe_group_work
// (crates/llamd-vulkan/shaders/q6k_expert_major.comp, q6k_expert_major_pa.comp):
// for every work item (expert, first, count) the expert's rows are streamed once
// for `count` pairs. Pair p reads activation aq[act_map[p]] (act_map = ptoken
// for gate/up, pslot for down) and writes out[pslot[p]][rows]. wb/ob may be NULL.
// max_items bounds the list length: npair/8 + n_expert always suffices.
void llamd_fwd_expert_major(const void *wa, const void *wb, const int32_t *work, const int32_t *n_work, int max_items,
                            const int32_t *act_map, const int32_t *pslot, const int8_t *aq, const float *ad, float *oa, float *ob,
                            int blocks, int rows, int n_expert) {
    const void *ws[2] = {wa, wb};
    float *os[2] = {oa, ob};
    const int r2[2] = {rows, rows};
    launch_matvec_multi(wb ? 2 : 1, ws, os, r2, blocks, aq, ad, 0, work, n_work, max_items, act_map, pslot, n_expert);
}

// ---- host-facing -----------------------------------------------------------
// scratch slots: 0 aq, 1 ad, 2 out, 3 ids, 4 x(f32), 5 bsums

static int stage_act(const int8_t *aq, const float *ad, int blocks, int nact, int8_t **d_aq, float **d_ad) {
    *d_aq = (int8_t *)scratch(0, (size_t)nact * blocks * 256);
    *d_ad = (float *)scratch(1, (size_t)nact * blocks * sizeof(float));
    if (!*d_aq || !*d_ad) return -1;
    LLAMD_TRY(cudaMemcpyAsync(*d_aq, aq, (size_t)nact * blocks * 256, cudaMemcpyHostToDevice, stream()), "aq H2D");
    LLAMD_TRY(cudaMemcpyAsync(*d_ad, ad, (size_t)nact * blocks * sizeof(float), cudaMemcpyHostToDevice, stream()), "ad H2D");
    return 0;
}

int llamd_cuda_matvec_q6k_resident(const void *d_w, const int8_t *aq, const float *ad, float *out, int blocks, int rows) {
    if (!d_w || !aq || !ad || !out || blocks <= 0 || rows <= 0) return -1;
    int8_t *d_aq;
    float *d_ad;
    if (stage_act(aq, ad, blocks, 1, &d_aq, &d_ad)) return -1;
    float *d_out = (float *)scratch(2, (size_t)rows * sizeof(float));
    if (!d_out) return -1;
    llamd_fwd_matvec(d_w, d_aq, d_ad, d_out, blocks, rows);
    LLAMD_TRY(cudaMemcpyAsync(out, d_out, (size_t)rows * sizeof(float), cudaMemcpyDeviceToHost, stream()), "out D2H");
    return llamd_fwd_sync();
}

int llamd_cuda_matvec_grouped(const void *d_w, const int32_t *eid, const int8_t *aq, const float *ad, float *out, int blocks, int rows,
                              int n_used) {
    if (!d_w || !eid || !aq || !ad || !out || blocks <= 0 || rows <= 0 || n_used <= 0) return -1;
    for (int i = 0; i < n_used; i++)
        if (eid[i] < 0) return -1;
    int8_t *d_aq;
    float *d_ad;
    if (stage_act(aq, ad, blocks, 1, &d_aq, &d_ad)) return -1;
    float *d_out = (float *)scratch(2, (size_t)rows * n_used * sizeof(float));
    int32_t *d_ids = (int32_t *)scratch(3, (size_t)n_used * sizeof(int32_t));
    if (!d_out || !d_ids) return -1;
    LLAMD_TRY(cudaMemcpyAsync(d_ids, eid, (size_t)n_used * sizeof(int32_t), cudaMemcpyHostToDevice, stream()), "ids H2D");
    llamd_fwd_matvec_grouped(d_w, d_ids, d_aq, d_ad, d_out, blocks, rows, n_used);
    LLAMD_TRY(cudaMemcpyAsync(out, d_out, (size_t)rows * n_used * sizeof(float), cudaMemcpyDeviceToHost, stream()), "out D2H");
    return llamd_fwd_sync();
}

// Kernel-only time: one warm launch, then `iters` back-to-back launches
// between two events (the discipline of llamd.hip:1101-1148).
static int bench_loop(int iters, float *ms_out, void (*launch)(void *), void *ctx) {
    if (iters <= 0 || !ms_out) return -1;
    cudaEvent_t e0, e1;
    LLAMD_TRY(cudaEventCreate(&e0), "event");
    LLAMD_TRY(cudaEventCreate(&e1), "event");
    launch(ctx);
    LLAMD_TRY(cudaStreamSynchronize(stream()), "bench warm sync");
    cudaEventRecord(e0, stream());
    for (int i = 0; i < iters; i++) launch(ctx);
    cudaEventRecord(e1, stream());
    LLAMD_TRY(cudaEventSynchronize(e1), "bench sync");
    cudaEventElapsedTime(ms_out, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    return error_code() == 0 ? 0 : -1;
}

struct BenchCtx {
    const void *w;
    const int32_t *ids;
    const int8_t *aq;
    const float *ad;
    float *out;
    int blocks, rows, n_used;
};

int llamd_cuda_matvec_bench(const void *d_w, const int8_t *aq, const float *ad, int blocks, int rows, int iters, float *ms_out) {
    if (!d_w || !aq || !ad || blocks <= 0 || rows <= 0) return -1;
    int8_t *d_aq;
    float *d_ad;
    if (stage_act(aq, ad, blocks, 1, &d_aq, &d_ad)) return -1;
    float *d_out = (float *)scratch(2, (size_t)rows * sizeof(float));
    if (!d_out) return -1;
    BenchCtx c = {d_w, nullptr, d_aq, d_ad, d_out, blocks, rows, 0};
    return bench_loop(iters, ms_out, [](void *p) {
        BenchCtx *c = (BenchCtx *)p;
        llamd_fwd_matvec(c->w, c->aq, c->ad, c->out, c->blocks, c->rows);
    }, &c);
}

int llamd_cuda_matvec_grouped_bench(const void *d_w, const int32_t *eid, const int8_t *aq, const float *ad, int blocks, int rows,
                                    int n_used, int iters, float *ms_out) {
    if (!d_w || !eid || !aq || !ad || blocks <= 0 || rows <= 0 || n_used <= 0) return -1;
    int8_t *d_aq;
    float *d_ad;
    if (stage_act(aq, ad, blocks, 1, &d_aq, &d_ad)) return -1;
    float *d_out = (float *)scratch(2, (size_t)rows * n_used * sizeof(float));
    int32_t *d_ids = (int32_t *)scratch(3, (size_t)n_used * sizeof(int32_t));
    if (!d_out || !d_ids) return -1;
    LLAMD_TRY(cudaMemcpyAsync(d_ids, eid, (size_t)n_used * sizeof(int32_t), cudaMemcpyHostToDevice, stream()), "ids H2D");
    BenchCtx c = {d_w, d_ids, d_aq, d_ad, d_out, blocks, rows, n_used};
    return bench_loop(iters, ms_out, [](void *p) {
        BenchCtx *c = (BenchCtx *)p;
        llamd_fwd_matvec_grouped(c->w, c->ids, c->aq, c->ad, c->out, c->blocks, c->rows, c->n_used);
    }, &c);
}

int llamd_cuda_quantize_q8k(const float *x, int nblocks, int8_t *qs, float *d, int16_t *bsums) {
    if (!x || !qs || !d || nblocks <= 0) return -1;
    float *d_x = (float *)scratch(4, (size_t)nblocks * 256 * sizeof(float));
    int8_t *d_q = (int8_t *)scratch(0, (size_t)nblocks * 256);
    float *d_d = (float *)scratch(1, (size_t)nblocks * sizeof(float));
    int16_t *d_b = (int16_t *)scratch(5, (size_t)nblocks * 16 * sizeof(int16_t));
    if (!d_x || !d_q || !d_d || !d_b) return -1;
    LLAMD_TRY(cudaMemcpyAsync(d_x, x, (size_t)nblocks * 256 * sizeof(float), cudaMemcpyHostToDevice, stream()), "x H2D");
    llamd_fwd_quantize_bsums(d_x, d_q, d_d, d_b, nblocks);
    LLAMD_TRY(cudaMemcpyAsync(qs, d_q, (size_t)nblocks * 256, cudaMemcpyDeviceToHost, stream()), "qs D2H");
    LLAMD_TRY(cudaMemcpyAsync(d, d_d, (size_t)nblocks * sizeof(float), cudaMemcpyDeviceToHost, stream()), "d D2H");
    if (bsums) LLAMD_TRY(cudaMemcpyAsync(bsums, d_b, (size_t)nblocks * 16 * sizeof(int16_t), cudaMemcpyDeviceToHost, stream()), "bsums D2H");
    return llamd_fwd_sync();
}

int llamd_cuda_matvec_q6k_f32(const void *d_w, const float *x, float *out, int blocks, int rows, int nseq) {
    if (!d_w || !x || !out || blocks <= 0 || rows <= 0 || nseq < 1 || nseq > LLAMD_MAX_SEQ) return -1;
    const size_t k = (size_t)blocks * 256;
    float *d_x = (float *)scratch(4, nseq * k * sizeof(float));
    int8_t *d_q = (int8_t *)scratch(0, nseq * k);
    float *d_d = (float *)scratch(1, (size_t)nseq * blocks * sizeof(float));
    float *d_out = (float *)scratch(2, (size_t)nseq * rows * sizeof(float));
    if (!d_x || !d_q || !d_d || !d_out) return -1;
    LLAMD_TRY(cudaMemcpyAsync(d_x, x, nseq * k * sizeof(float), cudaMemcpyHostToDevice, stream()), "x H2D");
    llamd_fwd_quantize(d_x, d_q, d_d, nseq * blocks);
    llamd_fwd_matvec_batch(d_w, d_q, d_d, d_out, blocks, rows, nseq);
    LLAMD_TRY(cudaMemcpyAsync(out, d_out, (size_t)nseq * rows * sizeof(float), cudaMemcpyDeviceToHost, stream()), "out D2H");
    return llamd_fwd_sync();
}

int llamd_cuda_matvec_q8_0_f32(const void *d_w, const float *x, float *out, int blocks32, int rows, int nseq) {
    if (!d_w || !x || !out || blocks32 <= 0 || rows <= 0 || nseq < 1 || nseq > LLAMD_MAX_SEQ) return -1;
    const size_t k = (size_t)blocks32 * 32;
    float *d_x = (float *)scratch(4, nseq * k * sizeof(float));
    float *d_out = (float *)scratch(2, (size_t)nseq * rows * sizeof(float));
    if (!d_x || !d_out) return -1;
    LLAMD_TRY(cudaMemcpyAsync(d_x, x, nseq * k * sizeof(float), cudaMemcpyHostToDevice, stream()), "x H2D");
    llamd_fwd_matvec_q8_0(d_w, d_x, d_out, blocks32, rows, nseq);
    LLAMD_TRY(cudaMemcpyAsync(out, d_out, (size_t)nseq * rows * sizeof(float), cudaMemcpyDeviceToHost, stream()), "out D2H");
    if (llamd_fwd_sync() != 0) return -1;
    if (llamd_fwd_matvec_q8_0_status() != 0) {
        set_error_msg("matvec_q8_0: a bulk copy of the weights did not arrive within its limit; rows are missing");
        return -1;
    }
    return 0;
}

}  // extern "C"
