// Device helpers shared by the quantizing kernels: the exponential, the Q8_K
// block quantizer and SiLU(gate)*up, each in the reference's operation order.
#pragma once
#include "common.cuh"

namespace llamd {

// The reference calls Rust's f32::exp, i.e. the host libm's expf. Here the
// exponential is evaluated in double and rounded once to f32.
__device__ __forceinline__ float ref_expf(float x) { return __double2float_rn(exp((double)x)); }

// ---- Q8_K: crates/llamd-quant/src/dot.rs:88-128 ---------------------------
// One warp per 256-element block; lane l owns elements 8l..8l+7.
// Produces qs[256] (natural order), d and optionally bsums[16].
__device__ __forceinline__ void q8k_quantize_block(const float v[8], int lane, int8_t *__restrict__ qs, float *__restrict__ d_out,
                                                   int16_t *__restrict__ bsums) {
    // the SIGNED value at the largest magnitude, first such element
    float amax = 0.0f, mx = 0.0f;
    int idx = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const float a = fabsf(v[i]);
        if (a > amax) {
            amax = a;
            mx = v[i];
            idx = lane * 8 + i;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float oa = __shfl_xor_sync(0xffffffffu, amax, off);
        const float om = __shfl_xor_sync(0xffffffffu, mx, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (oa > amax || (oa == amax && oi < idx)) {
            amax = oa;
            mx = om;
            idx = oi;
        }
    }
    int q[8];
    float dd = 0.0f;
    if (amax == 0.0f) {
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = 0;
    } else {
        const float iscale = __fdiv_rn(-127.0f, mx);
#pragma unroll
        for (int i = 0; i < 8; i++) q[i] = min(127, __float2int_rn(__fmul_rn(iscale, v[i])));
        dd = __fdiv_rn(1.0f, iscale);
    }
    uint32_t w0 = 0, w1 = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        w0 |= ((uint32_t)q[i] & 0xFFu) << (8 * i);
        w1 |= ((uint32_t)q[4 + i] & 0xFFu) << (8 * i);
    }
    *reinterpret_cast<uint2 *>(qs + lane * 8) = make_uint2(w0, w1);
    if (lane == 0) *d_out = dd;
    if (bsums) {
        int s = 0;
#pragma unroll
        for (int i = 0; i < 8; i++) s += q[i];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if ((lane & 1) == 0) bsums[lane >> 1] = (int16_t)s;
    }
}

// silu(gate) * up (crates/llamd-cpu/src/lib.rs:103-114, layer.rs:252):
// v / (1 + exp(-v)), then the elementwise product.
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float s = __fdiv_rn(g, __fadd_rn(1.0f, ref_expf(-g)));
    return __fmul_rn(s, u);
}

}  // namespace llamd
