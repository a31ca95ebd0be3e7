// The routing decision of one token, shared by the router kernels and the resident decode kernel.
#pragma once
#include <math.h>

#include "quant.cuh"

namespace llamd {

#define WEIGHT_SUM_FLOOR 6.103515625e-5f  // 2^-14, crates/llamd-models/src/moe.rs:50
constexpr int kMaxUsed = 64;

// ---- route: crates/llamd-models/src/moe.rs:73-113 --------------------------
// One CTA. s_p holds the n_expert logits on entry and the probabilities on
// exit. (NaN logits break the order: slots they would have taken then name expert 0 with weight 0.) Works for any blockDim that is a multiple of 32.
static __device__ void route_block(float *s_p, float *s_red, int *s_redi, int n_expert, int n_used, int32_t *__restrict__ ids,
                            float *__restrict__ weights, float *__restrict__ probs) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = (blockDim.x + 31) >> 5;
    // max is order-free
    float m = -INFINITY;
    for (int i = tid; i < n_expert; i += blockDim.x) m = fmaxf(m, s_p[i]);
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = s_red[0];
    for (int w = 1; w < nwarps; w++) m = fmaxf(m, s_red[w]);
    __syncthreads();
    for (int i = tid; i < n_expert; i += blockDim.x) s_p[i] = ref_expf(__fsub_rn(s_p[i], m));
    __syncthreads();
    // probs.iter().sum(): left to right from -0.0
    if (tid == 0) s_red[32] = chain_sum(s_p, n_expert, -0.0f);
    __syncthreads();
    const float total = s_red[32];
    for (int i = tid; i < n_expert; i += blockDim.x) {
        const float p = __fdiv_rn(s_p[i], total);
        s_p[i] = p;
        if (probs) probs[i] = p;
    }
    for (int k = tid; k < n_used; k += blockDim.x) {  // (defined slots even if a NaN probability breaks the order below)
        s_redi[40 + k] = 0;
        s_red[40 + k] = 0.0f;
    }
    __syncthreads();
    // The n_used best by (probability descending, index ascending) -- the reference's stable sort -- found by rank:
    // every expert counts the experts that come before it in that order, and those of rank < n_used write themselves
    // into place. One pass over shared memory and one barrier, where n_used rounds of block-wide arg-max took two
    // barriers each (~4 us of an ~18 us router launch).
    for (int i = tid; i < n_expert; i += blockDim.x) {
        const float mine = s_p[i];
        int rank = 0;
        for (int j = 0; j < n_expert; j++) {
            const float o = s_p[j];
            rank += (o > mine || (o == mine && j < i)) ? 1 : 0;
        }
        if (rank < n_used) {
            s_redi[40 + rank] = i;
            s_red[40 + rank] = mine;
        }
    }
    __syncthreads();
    if (tid == 0) {
        float sum = -0.0f;
        for (int k = 0; k < n_used; k++) sum = __fadd_rn(sum, s_red[40 + k]);
        s_red[33] = fmaxf(sum, WEIGHT_SUM_FLOOR);
    }
    __syncthreads();
    for (int k = tid; k < n_used; k += blockDim.x) {
        ids[k] = s_redi[40 + k];
        weights[k] = __fdiv_rn(s_red[40 + k], s_red[33]);
    }
}

}  // namespace llamd
