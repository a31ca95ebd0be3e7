// Device helpers shared by the quantizing kernels: the exponential, the Q8_K
// block quantizer and SiLU(gate)*up, each in the reference's operation order.
#pragma once
#include "common.cuh"

namespace llamd {

// The reference calls Rust's f32::exp, i.e. the host libm's expf. Here the exponential is evaluated in double and
// rounded once to f32, which is the correctly rounded result; the host's expf is not always (glibc's differs by one
// ulp on roughly one input in 12000). Routing decisions and Q8_K roundings downstream amplify such a bit, so the
// library makes the two agree exactly: when it starts it evaluates this very expression on the device for EVERY
// float in the range where exp is neither 1, 0 nor infinite, compares with the host's expf, and keeps the inputs
// that differ in a hash table (runtime.cu: build_exp_table). ref_expf looks its argument up there: one probe of a
// sparsely filled table in L2, a hit only for the listed inputs. Each translation unit has its own copy of the two
// pointers (constant memory), set through the binder it registers below.
static __constant__ const uint32_t *c_exp_keys = nullptr;  // [mask + 1] input bit patterns, 0 = empty slot
static __constant__ const uint32_t *c_exp_vals = nullptr;  // [mask + 1] the host expf's result bits
static __constant__ uint32_t c_exp_mask = 0;
static __constant__ uint32_t c_exp_window = 0;  // see exp_needs_lookup; 0 = look every input up

// The host's expf can differ from the correctly rounded value only where exp(x) lies very close to the midpoint of
// two neighbouring floats (its error before the final rounding is a few thousandths of an ulp). The 29 bits of the
// double result below float precision say how close: the table is consulted only within `window` (in units of
// 2^-29 ulp) of the midpoint. The window is measured when the table is built: the largest distance over every listed
// input, on the device, plus one; an input outside it is therefore not in the table. Results that are subnormal as
// floats round at another bit position and are always looked up.
__device__ __forceinline__ bool exp_needs_lookup(float x, double yd, uint32_t window) {
    if (window == 0 || x < -87.0f) return true;
    const uint32_t frac = (uint32_t)__double_as_longlong(yd) & 0x1FFFFFFFu;
    return frac - (0x10000000u - window) < 2u * window;  // |frac - 2^28| < window
}

__device__ __forceinline__ float ref_expf(float x) {
    const double yd = exp((double)x);
    float y = __double2float_rn(yd);
    const uint32_t *keys = c_exp_keys;
    if (keys && exp_needs_lookup(x, yd, c_exp_window)) {
        const uint32_t b = __float_as_uint(x), mask = c_exp_mask;
        uint32_t h = (b * 2654435761u) >> 8 & mask;
        for (int probe = 0; probe < 64; probe++) {  // (a table at most a quarter full: runs are short)
            const uint32_t k = __ldg(keys + h);
            if (k == 0) break;
            if (k == b) {
                y = __uint_as_float(__ldg(c_exp_vals + h));
                break;
            }
            h = (h + 1) & mask;
        }
    }
    return y;
}

void register_exp_binder(void (*bind)(const uint32_t *, const uint32_t *, uint32_t, uint32_t));
namespace {
inline void bind_exp_table_here(const uint32_t *keys, const uint32_t *vals, uint32_t mask, uint32_t window) {
    cudaMemcpyToSymbol(c_exp_keys, &keys, sizeof keys);
    cudaMemcpyToSymbol(c_exp_vals, &vals, sizeof vals);
    cudaMemcpyToSymbol(c_exp_mask, &mask, sizeof mask);
    cudaMemcpyToSymbol(c_exp_window, &window, sizeof window);
}
struct ExpBinderRegistration {
    ExpBinderRegistration() { register_exp_binder(bind_exp_table_here); }
};
static ExpBinderRegistration s_exp_binder_registration;
}  // namespace

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
