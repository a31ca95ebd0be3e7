// Q8_K activation quantizer and the small f32 ops that feed it.
//
// Everything here reproduces the reference's scalar f32 arithmetic in its
// order (no FMA contraction, no reassociation), because each value ends up in
// an int8 quant or a routing decision where the last bit is observable.
#include "quant.cuh"

namespace llamd {

__global__ void __launch_bounds__(256) q8k_quantize_kernel(const float *__restrict__ x, int8_t *__restrict__ qs, float *__restrict__ d,
                                                           int16_t *__restrict__ bsums, int nblocks) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= nblocks) return;
    const float4 *p = reinterpret_cast<const float4 *>(x + (size_t)warp * 256 + lane * 8);
    const float4 a = p[0], b = p[1];
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    q8k_quantize_block(v, lane, qs + (size_t)warp * 256, d + warp, bsums ? bsums + (size_t)warp * 16 : nullptr);
}

// ---- rms_norm: crates/llamd-cpu/src/lib.rs:55-75, then `* w` --------------
// The sum of squares is a left-to-right f32 chain in the reference; thread 0
// walks it from shared memory while the other threads wait. One CTA per row.
// ssq holds the squares x[i]*x[i] (computed by all threads); n % 4 == 0.
__device__ __forceinline__ float rms_scale_sequential(const float *__restrict__ ssq, int n, float eps) {
    const float sum = chain_sum(ssq, n, 0.0f);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)n), eps)));
}

// out = (x*scale)*w ; optionally Q8_K of out. Dynamic smem: 2n floats.
// Before the norm, x may first receive
//   - `residual`: x := x + residual (the attention residual,
//     crates/llamd-runtime/src/layer.rs:170), or
//   - `down`/`cw`: x := x + sum_e cw[e]*down[e] with e in routing order and the
//     expert sum started from 0 (moe_ffn, layer.rs:243-258, then :281-287),
// and the updated x is written to sum_out.
template <int kMaxV>  // float4 groups per thread: rows of up to 1024 * kMaxV elements
__global__ void __launch_bounds__(256) rms_norm_kernel(const float *__restrict__ x, const float *__restrict__ residual,
                                                       const float *__restrict__ down, const float *__restrict__ cw, int n_used,
                                                       float *__restrict__ sum_out, const float *__restrict__ w, float *__restrict__ out,
                                                       int8_t *__restrict__ qs, float *__restrict__ d, int n, float eps, const WaitPlan wait, int fast) {
    extern __shared__ __align__(16) float sx[];  // [n] values, then [n] squares
    float *ssq = sx + n;
    __shared__ float s_scale;
    __shared__ float s_tree[32];
    pdl_trigger();
    const int seq = blockIdx.x, tid = threadIdx.x;
    // Thread t owns the float4 groups t, t+256, ...: every global load of the
    // kernel is issued before anything waits on one.
    // (kMaxV = 2 for rows of up to 2048: a third of the registers of the widest form, so three CTAs share an SM where a
    // tile of 512 rows had one, each waiting on its own chain)
    const int n4 = n / 4;
    float4 wv[kMaxV], xv[kMaxV];
#pragma unroll
    for (int u = 0; u < kMaxV; u++) {
        const int j = tid + u * 256;
        wv[u] = j < n4 ? __ldg(reinterpret_cast<const float4 *>(w) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    if (wait.counter) {
        // Expert parallelism: the expert outputs read below are stored by other GPUs. Wait (bounded) for all of their
        // arrivals, then clear the counter: nothing more arrives before this rank has passed its next dispatch.
        if (tid == 0) {
            if (bounded_wait(wait.counter, wait.target, false, wait.status, 1, wait.limit)) {
                *wait.counter = 0;
                __threadfence();
            }
        }
        __syncthreads();
    }
    const float4 *x4 = reinterpret_cast<const float4 *>(x + (size_t)seq * n);
#pragma unroll
    for (int u = 0; u < kMaxV; u++) {
        const int j = tid + u * 256;
        xv[u] = j < n4 ? x4[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (down) {
        float4 acc[kMaxV];
#pragma unroll
        for (int u = 0; u < kMaxV; u++) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        const float *cws = cw + (size_t)seq * n_used;
        for (int e0 = 0; e0 < n_used; e0 += 4) {
            float4 dv[4][kMaxV];
            float we[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int e = e0 + q;
                we[q] = e < n_used ? cws[e] : 0.0f;
                const float4 *d4 = reinterpret_cast<const float4 *>(down + ((size_t)seq * n_used + (e < n_used ? e : 0)) * n);
#pragma unroll
                for (int u = 0; u < kMaxV; u++) {
                    const int j = tid + u * 256;
                    dv[q][u] = (j < n4 && e < n_used) ? __ldcg(d4 + j) : make_float4(0.f, 0.f, 0.f, 0.f);  // L2: may come from a peer
                }
            }
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if (e0 + q < n_used) {
#pragma unroll
                    for (int u = 0; u < kMaxV; u++) {
                        acc[u].x = __fadd_rn(acc[u].x, __fmul_rn(we[q], dv[q][u].x));
                        acc[u].y = __fadd_rn(acc[u].y, __fmul_rn(we[q], dv[q][u].y));
                        acc[u].z = __fadd_rn(acc[u].z, __fmul_rn(we[q], dv[q][u].z));
                        acc[u].w = __fadd_rn(acc[u].w, __fmul_rn(we[q], dv[q][u].w));
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kMaxV; u++) {
            xv[u].x = __fadd_rn(xv[u].x, acc[u].x);
            xv[u].y = __fadd_rn(xv[u].y, acc[u].y);
            xv[u].z = __fadd_rn(xv[u].z, acc[u].z);
            xv[u].w = __fadd_rn(xv[u].w, acc[u].w);
        }
    } else if (residual) {
        const float4 *r4 = reinterpret_cast<const float4 *>(residual + (size_t)seq * n);
#pragma unroll
        for (int u = 0; u < kMaxV; u++) {
            const int j = tid + u * 256;
            if (j < n4) {
                const float4 r = r4[j];
                xv[u].x = __fadd_rn(xv[u].x, r.x);
                xv[u].y = __fadd_rn(xv[u].y, r.y);
                xv[u].z = __fadd_rn(xv[u].z, r.z);
                xv[u].w = __fadd_rn(xv[u].w, r.w);
            }
        }
    }
#pragma unroll
    for (int u = 0; u < kMaxV; u++) {
        const int j = tid + u * 256;
        if (j < n4) {
            if (down || residual) reinterpret_cast<float4 *>(sum_out + (size_t)seq * n)[j] = xv[u];
            reinterpret_cast<float4 *>(sx)[j] = xv[u];
            reinterpret_cast<float4 *>(ssq)[j] =
                make_float4(__fmul_rn(xv[u].x, xv[u].x), __fmul_rn(xv[u].y, xv[u].y), __fmul_rn(xv[u].z, xv[u].z), __fmul_rn(xv[u].w, xv[u].w));
        }
    }
    __syncthreads();
    float scale;
    if (fast & 1) {  // the sum of squares as a reduction tree (the `fast` arithmetic)
        float part = 0.0f;
        for (int i = tid; i < n; i += 256) part = __fadd_rn(part, ssq[i]);
        const float sum = block_tree_sum(part, s_tree);
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)n), eps)));
    } else {
        if (tid == 0) s_scale = rms_scale_sequential(ssq, n, eps);
        __syncthreads();
        scale = s_scale;
    }
#pragma unroll
    for (int u = 0; u < kMaxV; u++) {
        const int j = tid + u * 256;
        if (j < n4) {
            const float4 o = make_float4(__fmul_rn(__fmul_rn(xv[u].x, scale), wv[u].x), __fmul_rn(__fmul_rn(xv[u].y, scale), wv[u].y),
                                         __fmul_rn(__fmul_rn(xv[u].z, scale), wv[u].z), __fmul_rn(__fmul_rn(xv[u].w, scale), wv[u].w));
            reinterpret_cast<float4 *>(sx)[j] = o;
            if (out) reinterpret_cast<float4 *>(out + (size_t)seq * n)[j] = o;
        }
    }
    if (!qs) return;
    __syncthreads();
    const int warp = tid >> 5, lane = tid & 31, nwarps = blockDim.x >> 5;
    for (int b = warp; b < n / 256; b += nwarps) {
        float v[8];
        const float4 a = reinterpret_cast<const float4 *>(sx + b * 256 + lane * 8)[0], c = reinterpret_cast<const float4 *>(sx + b * 256 + lane * 8)[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
        q8k_quantize_block(v, lane, qs + (size_t)seq * n + (size_t)b * 256, d + (size_t)seq * (n / 256) + b, nullptr);
    }
}

// Per-head norm (crates/llamd-runtime/src/layer.rs:62-79): one warp per head,
// lane 0 walks the chain.
__global__ void head_rms_norm_mul_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ out, int n_head,
                                         int hd, float eps) {
    const int head = blockIdx.x;
    if (head >= n_head) return;
    extern __shared__ __align__(16) float sx[];
    float *ssq = sx + hd;
    __shared__ float s_scale;
    for (int i = threadIdx.x; i < hd; i += blockDim.x) {
        const float v = x[(size_t)head * hd + i];
        sx[i] = v;
        ssq[i] = __fmul_rn(v, v);
    }
    __syncthreads();
    if (threadIdx.x == 0) s_scale = rms_scale_sequential(ssq, hd, eps);
    __syncthreads();
    for (int i = threadIdx.x; i < hd; i += blockDim.x)
        out[(size_t)head * hd + i] = __fmul_rn(__fmul_rn(sx[i], s_scale), w[i]);
}

__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(a[i], b[i]);
}

__global__ void silu_mul_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ out, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = silu_mul(gate[i], up[i]);
}
// One warp per 256-element block: act = silu(gate)*up, then Q8_K of act.
__global__ void __launch_bounds__(256) silu_mul_quant_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                             float *__restrict__ out, int8_t *__restrict__ qs, float *__restrict__ d,
                                                             int nblocks) {
    pdl_trigger();
    pdl_wait();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= nblocks) return;
    const size_t base = (size_t)warp * 256 + lane * 8;
    const float4 g0 = *reinterpret_cast<const float4 *>(gate + base), g1 = *reinterpret_cast<const float4 *>(gate + base + 4);
    const float4 u0 = *reinterpret_cast<const float4 *>(up + base), u1 = *reinterpret_cast<const float4 *>(up + base + 4);
    float v[8] = {silu_mul(g0.x, u0.x), silu_mul(g0.y, u0.y), silu_mul(g0.z, u0.z), silu_mul(g0.w, u0.w),
                  silu_mul(g1.x, u1.x), silu_mul(g1.y, u1.y), silu_mul(g1.z, u1.z), silu_mul(g1.w, u1.w)};
    if (out) {
        *reinterpret_cast<float4 *>(out + base) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(out + base + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
    q8k_quantize_block(v, lane, qs + (size_t)warp * 256, d + warp, nullptr);
}

// The same for a handful of blocks (a decode token: 8 experts x 3 blocks): a CTA per block, one element per thread, so
// that the eight dependent exp evaluations a lane would walk one after the other run side by side; warp 0 quantizes
// from shared memory. Same operations per element, same bits.
__global__ void __launch_bounds__(256) silu_mul_quant_small_kernel(const float *__restrict__ gate, const float *__restrict__ up,
                                                                   float *__restrict__ out, int8_t *__restrict__ qs, float *__restrict__ d,
                                                                   int nblocks) {
    __shared__ __align__(16) float s_v[256];
    pdl_trigger();
    pdl_wait();
    const int blk = blockIdx.x, tid = threadIdx.x;
    const size_t i = (size_t)blk * 256 + tid;
    const float v = silu_mul(gate[i], up[i]);
    if (out) out[i] = v;
    s_v[tid] = v;
    __syncthreads();
    if (tid < 32) {
        const float4 a = reinterpret_cast<const float4 *>(s_v + tid * 8)[0], b = reinterpret_cast<const float4 *>(s_v + tid * 8)[1];
        const float w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        q8k_quantize_block(w, tid, qs + (size_t)blk * 256, d + blk, nullptr);
    }
}

// out[i] = residual[i] + sum_e w[e]*down[e][i], e in routing order
// (crates/llamd-runtime/src/layer.rs:243-258 then :281-287): the expert sum
// starts from 0 and the residual is added last.
__global__ void moe_combine_kernel(const float *__restrict__ down, const float *__restrict__ weights, const float *__restrict__ residual,
                                   float *__restrict__ out, int n_used, int n_embd) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int seq = blockIdx.y;
    if (i >= n_embd) return;
    down += (size_t)seq * n_used * n_embd;
    weights += (size_t)seq * n_used;
    float acc = 0.0f;
    for (int e = 0; e < n_used; e++) acc = __fadd_rn(acc, __fmul_rn(weights[e], down[(size_t)e * n_embd + i]));
    if (residual) acc = __fadd_rn(residual[(size_t)seq * n_embd + i], acc);
    out[(size_t)seq * n_embd + i] = acc;
}

}  // namespace llamd

using namespace llamd;

template <typename... Args>
static void launch_rms_norm(const char *what, int nseq, int n, Args... args) {
    if (n <= 2048)
        launch_kc(PDL_NORM, what, rms_norm_kernel<2>, dim3(nseq), dim3(256), 2 * n * sizeof(float), args...);
    else
        launch_kc(PDL_NORM, what, rms_norm_kernel<6>, dim3(nseq), dim3(256), 2 * n * sizeof(float), args...);
}

// `wait`: with expert parallelism the rows of `down` are stored by other GPUs; the launch first waits for their arrivals.
void llamd::combine_rms_norm_quant_wait(const WaitPlan &wait, const float *x, const float *down, const float *weights, int n_used,
                                        float *sum_out, const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq, int flags) {
    if (n % 256 || (size_t)n * 8 > 48 * 1024) {
        set_error_msg("combine_rms_norm_quant: n must be a multiple of 256 and at most 6144");
        return;
    }
    launch_rms_norm("combine_rms_norm_quant", nseq, n, x, (const float *)nullptr, down, weights, n_used, sum_out, w, out, qs, d, n, eps, wait,
                    flags);
}
// llamd_fwd_rms_norm_quant / llamd_fwd_add_rms_norm_quant with a decode pass's flags (kPass... in common.cuh).
void llamd::rms_norm_quant_flags(const float *x, const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq, int flags) {
    if (n % 256 || (size_t)n * 8 > 48 * 1024) {
        set_error_msg("rms_norm_quant: n must be a multiple of 256 and at most 6144");
        return;
    }
    launch_rms_norm("rms_norm_quant", nseq, n, x, (const float *)nullptr, (const float *)nullptr, (const float *)nullptr, 0, (float *)nullptr, w, out,
                    qs, d, n, eps, WaitPlan{}, flags);
}
void llamd::add_rms_norm_quant_flags(const float *x, const float *residual, float *sum_out, const float *w, float *out, int8_t *qs, float *d,
                                     int n, float eps, int nseq, int flags) {
    if (n % 256 || (size_t)n * 8 > 48 * 1024) {
        set_error_msg("add_rms_norm_quant: n must be a multiple of 256 and at most 6144");
        return;
    }
    launch_rms_norm("add_rms_norm_quant", nseq, n, x, residual, (const float *)nullptr, (const float *)nullptr, 0, sum_out, w, out, qs, d, n, eps,
                    WaitPlan{}, flags);
}

extern "C" {

void llamd_fwd_quantize_bsums(const float *x, int8_t *qs, float *d, int16_t *bsums, int nblocks) {
    if (nblocks <= 0) return;
    launch_kc(PDL_SMALL, "q8k_quantize", q8k_quantize_kernel, dim3((nblocks + 7) / 8), dim3(256), 0, x, qs, d, bsums, nblocks);
}
void llamd_fwd_quantize(const float *x, int8_t *qs, float *d, int nblocks) {
    llamd_fwd_quantize_bsums(x, qs, d, nullptr, nblocks);
}

void llamd_fwd_rms_norm_mul(const float *x, const float *w, float *out, int n, float eps, int nseq) {
    if (n % 4 || (size_t)n * 8 > 48 * 1024) {
        set_error_msg("rms_norm: n must be a multiple of 4 and at most 6144");
        return;
    }
    launch_rms_norm("rms_norm_mul", nseq, n, x, (const float *)nullptr, (const float *)nullptr, (const float *)nullptr, 0, (float *)nullptr, w, out,
                    (int8_t *)nullptr, (float *)nullptr, n, eps, WaitPlan{}, 0);
}
void llamd_fwd_rms_norm_quant(const float *x, const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq) {
    rms_norm_quant_flags(x, w, out, qs, d, n, eps, nseq, 0);
}
// x + residual -> sum_out, then norm*w and its Q8_K form. Fuses the residual
// add of layer.rs:170 into the norm of :173-174.
void llamd_fwd_add_rms_norm_quant(const float *x, const float *residual, float *sum_out, const float *w, float *out, int8_t *qs,
                                  float *d, int n, float eps, int nseq) {
    add_rms_norm_quant_flags(x, residual, sum_out, w, out, qs, d, n, eps, nseq, 0);
}
// x + sum_e weights[e]*down[e] -> sum_out (the MoE combine and residual,
// forward.rs:586), then norm*w and its Q8_K form: the tail of one layer fused
// with the attention norm of the next (or with the output norm).
void llamd_fwd_combine_rms_norm_quant(const float *x, const float *down, const float *weights, int n_used, float *sum_out,
                                      const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq) {
    combine_rms_norm_quant_wait(WaitPlan{}, x, down, weights, n_used, sum_out, w, out, qs, d, n, eps, nseq, 0);
}
void llamd_fwd_head_rms_norm_mul(const float *x, const float *w, float *out, int n_head, int hd, float eps) {
    if (hd % 4) {
        set_error_msg("head_rms_norm: head_dim must be a multiple of 4");
        return;
    }
    head_rms_norm_mul_kernel<<<n_head, 128, 2 * hd * sizeof(float), stream()>>>(x, w, out, n_head, hd, eps);
    LLAMD_CHECK_LAUNCH("head_rms_norm_mul");
}
void llamd_fwd_add(const float *a, const float *b, float *out, int n) {
    add_kernel<<<(n + 255) / 256, 256, 0, stream()>>>(a, b, out, n);
    LLAMD_CHECK_LAUNCH("add");
}
void llamd_fwd_silu_mul(const float *gate, const float *up, float *out, int n) {
    silu_mul_kernel<<<(n + 255) / 256, 256, 0, stream()>>>(gate, up, out, n);
    LLAMD_CHECK_LAUNCH("silu_mul");
}
void llamd_fwd_silu_mul_quant(const float *gate, const float *up, float *out, int8_t *qs, float *d, int n) {
    if (n % 256) {
        set_error_msg("silu_mul_quant: n must be a multiple of 256");
        return;
    }
    const int nblocks = n / 256;
    if (nblocks <= 592) {  // (four CTAs per SM: beyond that the warp-per-block form's throughput wins)
        launch_kc(PDL_SMALL, "silu_mul_quant_small", silu_mul_quant_small_kernel, dim3(nblocks), dim3(256), 0, gate, up, out, qs, d, nblocks);
        return;
    }
    launch_kc(PDL_SMALL, "silu_mul_quant", silu_mul_quant_kernel, dim3((nblocks + 7) / 8), dim3(256), 0, gate, up, out, qs, d, nblocks);
}
void llamd_fwd_moe_combine(const float *down, const float *weights, float *out, int n_used, int n_embd) {
    moe_combine_kernel<<<dim3((n_embd + 255) / 256, 1), 256, 0, stream()>>>(down, weights, nullptr, out, n_used, n_embd);
    LLAMD_CHECK_LAUNCH("moe_combine");
}
void llamd_fwd_moe_combine_add(const float *down, const float *weights, const float *residual, float *out, int n_used, int n_embd,
                               int nseq) {
    launch_k("moe_combine_add", moe_combine_kernel, dim3((n_embd + 255) / 256, nseq), dim3(256), 0, down, weights, residual, out, n_used,
             n_embd);
}

}  // extern "C"
