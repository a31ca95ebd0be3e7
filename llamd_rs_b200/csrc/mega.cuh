// Interface of the resident decode kernel (mega.cu) for the model that launches it (model.cu).
#pragma once
#include "common.cuh"
#include "../../include/llamd_cuda_model.h"

namespace llamd {

struct MegaLayer {
    const uint8_t *attn_q, *attn_k, *attn_v, *attn_out, *gate, *up, *down;  // tiled Q6_K
    const float *attn_norm, *q_norm, *k_norm, *ffn_norm, *router;           // f32 (q_norm / k_norm may be null)
    float *kc, *vc;                                                          // [max_kv][kv_dim] f32, or binary16 when MegaParams::kv16
};

struct MegaParams {
    int n_layer, E, H, HKV, hd, n_expert, nu, ffe, max_kv;
    float eps;
    const MegaLayer *layers;
    const uint8_t *tok_embd;
    const float *output_norm, *rope_tab;
    const int32_t *meta;
    float *scores;  // [n_head][max_kv] scaled attention logits of this token
    float *q, *k, *v, *attn, *xb2, *logits, *e_gate, *e_up, *e_down, *x_out, *expert_w;
    int32_t *expert_ids;
    int8_t *aq_out;
    float *ad_out;
    float *trace_x;      // [n_layer][E] or null
    int32_t *trace_ids;  // [n_layer][nu] or null
    unsigned int *bar;
    unsigned long long *prof;  // [32] nanoseconds per phase, accumulated by CTA 0 (null: off)
    int *status;
    unsigned int spin_limit;
    int act_blocks;      // blocks the activation image must hold
    int sl_floats;       // padded max_kv
    int ktile_rows;      // cached positions one CTA scores: ceil(max_kv / (SMs / n_head_kv))
    int kv16;            // 1: the caches hold binary16 values (rounded at the store, widened exactly at the load)
    int fast;            // bit mask: tree reductions in place of the long ordered f32 sums of 1 the norms, 2 the router's dots, 4 attention
};

size_t mega_smem_bytes(const llamd_hparams &hp, int max_kv, int *act_blocks, int *sl_floats, int *ktile_rows_out);
bool mega_supported(const llamd_hparams &hp, int max_kv);
void launch_decode_mega(MegaParams p, const llamd_hparams &hp);

}  // namespace llamd
