// The routing decision of one token, shared by the router kernels and the resident decode kernel.
#pragma once
#include <math.h>

#include "quant.cuh"

namespace llamd {

#define WEIGHT_SUM_FLOOR 6.103515625e-5f  // 2^-14, crates/llamd-models/src/moe.rs:50
constexpr int kMaxUsed = 64;

// ---- route: crates/llamd-models/src/moe.rs:73-113 --------------------------
// One CTA. s_p holds the n_expert logits on entry and the probabilities on
// exit. Works for any blockDim that is a multiple of 32.
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
    __syncthreads();
    // n_used rounds of arg-max: probability descending, index ascending.
    // A taken expert is marked with -1 (probabilities are never negative).
    for (int k = 0; k < n_used; k++) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = tid; i < n_expert; i += blockDim.x) {
            const float v = s_p[i];
            if (v > bv || (v == bv && i < bi)) {
                bv = v;
                bi = i;
            }
        }
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (lane == 0) {
            s_red[warp] = bv;
            s_redi[warp] = bi;
        }
        __syncthreads();
        if (tid == 0) {
            float v = s_red[0];
            int ix = s_redi[0];
            for (int w = 1; w < nwarps; w++)
                if (s_red[w] > v || (s_red[w] == v && s_redi[w] < ix)) {
                    v = s_red[w];
                    ix = s_redi[w];
                }
            s_redi[40 + k] = ix;
            s_red[40 + k] = v;
            s_p[ix] = -1.0f;  // taken: cannot win again
        }
        __syncthreads();
    }
    if (tid == 0) {
        float sum = -0.0f;
        for (int k = 0; k < n_used; k++) sum = __fadd_rn(sum, s_red[40 + k]);
        sum = fmaxf(sum, WEIGHT_SUM_FLOOR);
        for (int k = 0; k < n_used; k++) {
            ids[k] = s_redi[40 + k];
            weights[k] = __fdiv_rn(s_red[40 + k], sum);
        }
    }
}

}  // namespace llamd
