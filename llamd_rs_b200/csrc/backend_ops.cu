// The ten operations of `llamd_tensor::Backend` (crates/llamd-tensor/src/lib.rs:148-174) as device kernels with
// the arithmetic of the reference's CpuBackend (crates/llamd-cpu/src/lib.rs:55-225): f32 throughout, every sum one
// in-order chain from +0.0 with an unfused multiply and add; exp is evaluated in double and rounded once (the reference
// calls the host libm's expf, which is within one ulp of that). These are the general
// row-wise forms (any row length, any number of rows); the decode and prefill passes use the fused, shape-specific
// kernels of ops.cu / quantize.cu, which compute the same values.
#include "common.cuh"
#include "quant.cuh"

namespace llamd {
namespace {

constexpr int kRowThreads = 256;
constexpr int kChunk = 2048;  // floats of a row staged per step

// One CTA per row. The sum of squares is walked in order by thread 0 over squares that all threads staged in
// shared memory (the chain is the cost: ~4 cycles per element; the staging hides the loads).
__global__ void __launch_bounds__(kRowThreads) rms_norm_rows_kernel(const float *__restrict__ x, float *__restrict__ out, int n, float eps) {
    __shared__ float s_sq[kChunk];
    __shared__ float s_scale;
    pdl_trigger();
    pdl_wait();
    const float *src = x + (size_t)blockIdx.x * n;
    float *dst = out + (size_t)blockIdx.x * n;
    float sum = 0.0f;
    for (int c0 = 0; c0 < n; c0 += kChunk) {
        const int len = min(kChunk, n - c0);
        for (int i = threadIdx.x; i < len; i += kRowThreads) {
            const float v = src[c0 + i];
            s_sq[i] = __fmul_rn(v, v);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int i = 0;
            for (; i + 8 <= len; i += 8) {
                const float4 a = *reinterpret_cast<const float4 *>(s_sq + i), b = *reinterpret_cast<const float4 *>(s_sq + i + 4);
                sum = __fadd_rn(sum, a.x); sum = __fadd_rn(sum, a.y); sum = __fadd_rn(sum, a.z); sum = __fadd_rn(sum, a.w);
                sum = __fadd_rn(sum, b.x); sum = __fadd_rn(sum, b.y); sum = __fadd_rn(sum, b.z); sum = __fadd_rn(sum, b.w);
            }
            for (; i < len; i++) sum = __fadd_rn(sum, s_sq[i]);
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)n), eps)));
    __syncthreads();
    const float scale = s_scale;
    for (int i = threadIdx.x; i < n; i += kRowThreads) dst[i] = __fmul_rn(src[i], scale);
}

// One CTA per row: max (order-free), e = exp(x - max) stored, the sum of e walked in order, then e * (1 / sum).
__global__ void __launch_bounds__(kRowThreads) softmax_rows_kernel(const float *__restrict__ x, float *__restrict__ out, int n) {
    __shared__ float s_e[kChunk];
    __shared__ float s_red[kRowThreads / 32];
    __shared__ float s_bcast;
    pdl_trigger();
    pdl_wait();
    const float *src = x + (size_t)blockIdx.x * n;
    float *dst = out + (size_t)blockIdx.x * n;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < n; i += kRowThreads) mx = fmaxf(mx, src[i]);
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0) {
        float m = s_red[0];
        for (int w = 1; w < kRowThreads / 32; w++) m = fmaxf(m, s_red[w]);
        s_bcast = m;
    }
    __syncthreads();
    mx = s_bcast;
    float sum = 0.0f;
    for (int c0 = 0; c0 < n; c0 += kChunk) {
        const int len = min(kChunk, n - c0);
        for (int i = threadIdx.x; i < len; i += kRowThreads) {
            const float e = ref_expf(__fsub_rn(src[c0 + i], mx));
            s_e[i] = e;
            dst[c0 + i] = e;
        }
        __syncthreads();
        if (threadIdx.x == 0)
            for (int i = 0; i < len; i++) sum = __fadd_rn(sum, s_e[i]);
        __syncthreads();
    }
    if (threadIdx.x == 0) s_bcast = __fdiv_rn(1.0f, sum);
    __syncthreads();
    const float inv = s_bcast;
    for (int i = threadIdx.x; i < n; i += kRowThreads) dst[i] = __fmul_rn(dst[i], inv);  // each thread rereads what it wrote
}

enum { EW_SILU, EW_MUL, EW_SCALE, EW_EXP };
template <int OP>
__global__ void elementwise_kernel(const float *__restrict__ a, const float *__restrict__ b, float by, float *__restrict__ out, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const float v = a[i];
        if (OP == EW_SILU) out[i] = __fdiv_rn(v, __fadd_rn(1.0f, ref_expf(-v)));
        if (OP == EW_MUL) out[i] = __fmul_rn(v, b[i]);
        if (OP == EW_SCALE) out[i] = __fmul_rn(v, by);
        if (OP == EW_EXP) out[i] = ref_expf(v);
    }
}

// out[j][i] = fold(+0.0, +) of w[i][t] * x[j][t], t ascending: one thread per output element, any k. 32 rows of w
// by 8 rows of x per CTA; both operands staged through shared memory 32 columns at a time.
constexpr int kMmW = 32, kMmX = 8, kMmK = 32;
__global__ void __launch_bounds__(kMmW *kMmX) matmul_f32_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ out, int k,
                                                                int m, int n) {
    __shared__ float s_w[kMmW][kMmK + 1], s_x[kMmX][kMmK + 1];
    pdl_trigger();
    pdl_wait();
    const int ti = threadIdx.x % kMmW, tj = threadIdx.x / kMmW;
    const int i0 = blockIdx.x * kMmW, j0 = blockIdx.y * kMmX;
    float acc = 0.0f;
    for (int k0 = 0; k0 < k; k0 += kMmK) {
        const int len = min(kMmK, k - k0);
        for (int e = threadIdx.x; e < kMmW * kMmK; e += kMmW * kMmX) {
            const int r = e / kMmK, c = e % kMmK;
            s_w[r][c] = (i0 + r < m && c < len) ? w[(size_t)(i0 + r) * k + k0 + c] : 0.0f;
        }
        {
            const int r = threadIdx.x / kMmK, c = threadIdx.x % kMmK;  // 8 x 32 = one element per thread
            s_x[r][c] = (j0 + r < n && c < len) ? x[(size_t)(j0 + r) * k + k0 + c] : 0.0f;
        }
        __syncthreads();
        for (int c = 0; c < len; c++) acc = __fadd_rn(acc, __fmul_rn(s_w[ti][c], s_x[tj][c]));  // no padding terms enter the chain
        __syncthreads();
    }
    if (i0 + ti < m && j0 + tj < n) out[(size_t)(j0 + tj) * m + i0 + ti] = acc;
}

// NeoX pairing (i, i + d/2) with the caller's sin/cos per row: sincos[row][i] = (sin, cos) of theta(row, i).
__global__ void rope_rows_kernel(const float *__restrict__ x, float *__restrict__ out, int row_len, int head_dim, const float2 *__restrict__ sincos) {
    pdl_trigger();
    pdl_wait();
    const int half = head_dim / 2, pairs = row_len / 2;
    const float *src = x + (size_t)blockIdx.x * row_len;
    float *dst = out + (size_t)blockIdx.x * row_len;
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int h = p / half, i = p - h * half, base = h * head_dim;
        const float2 sc = sincos[(size_t)blockIdx.x * half + i];
        const float a = src[base + i], b = src[base + i + half];
        dst[base + i] = __fsub_rn(__fmul_rn(a, sc.y), __fmul_rn(b, sc.x));
        dst[base + i + half] = __fadd_rn(__fmul_rn(a, sc.x), __fmul_rn(b, sc.y));
    }
}

__global__ void get_rows_kernel(const float *__restrict__ table, const uint32_t *__restrict__ ids, float *__restrict__ out, int row_len) {
    pdl_trigger();
    pdl_wait();
    const float *src = table + (size_t)ids[blockIdx.x] * row_len;
    float *dst = out + (size_t)blockIdx.x * row_len;
    for (int i = threadIdx.x; i < row_len; i += blockDim.x) dst[i] = src[i];
}

int ew_grid(size_t n) {
    const size_t g = (n + 255) / 256;
    return (int)(g < 148 * 16 ? (g ? g : 1) : 148 * 16);
}

}  // namespace
}  // namespace llamd

using namespace llamd;

extern "C" {

void llamd_fwd_rms_norm_rows(const float *x, float *out, int n, int rows, float eps) {
    if (n <= 0 || rows <= 0) return;
    launch_k("rms_norm_rows", rms_norm_rows_kernel, dim3(rows), dim3(kRowThreads), 0, x, out, n, eps);
}
void llamd_fwd_softmax_rows(const float *x, float *out, int n, int rows) {
    if (n <= 0 || rows <= 0) return;
    launch_k("softmax_rows", softmax_rows_kernel, dim3(rows), dim3(kRowThreads), 0, x, out, n);
}
// The exponential every kernel of the library uses (quant.cuh: ref_expf), elementwise: what the reference's
// f32::exp, i.e. the host libm's expf, returns for the same input. For parity checks.
void llamd_fwd_expf(const float *x, float *out, size_t n) {
    if (n) launch_k("expf", elementwise_kernel<EW_EXP>, dim3(ew_grid(n)), dim3(256), 0, x, (const float *)nullptr, 0.0f, out, n);
}
void llamd_fwd_silu(const float *x, float *out, size_t n) {
    if (n) launch_k("silu", elementwise_kernel<EW_SILU>, dim3(ew_grid(n)), dim3(256), 0, x, (const float *)nullptr, 0.0f, out, n);
}
void llamd_fwd_mul(const float *a, const float *b, float *out, size_t n) {
    if (n) launch_k("mul", elementwise_kernel<EW_MUL>, dim3(ew_grid(n)), dim3(256), 0, a, b, 0.0f, out, n);
}
void llamd_fwd_scale(const float *x, float by, float *out, size_t n) {
    if (n) launch_k("scale", elementwise_kernel<EW_SCALE>, dim3(ew_grid(n)), dim3(256), 0, x, (const float *)nullptr, by, out, n);
}
void llamd_fwd_matmul_f32(const float *w, const float *x, float *out, int k, int m, int n) {
    if (m <= 0 || n <= 0) return;
    if (k < 0 || (n + kMmX - 1) / kMmX > 65535) {
        set_error_msg("matmul_f32: k must be non-negative and n at most 524280");
        return;
    }
    launch_k("matmul_f32", matmul_f32_kernel, dim3((m + kMmW - 1) / kMmW, (n + kMmX - 1) / kMmX), dim3(kMmW * kMmX), 0, w, x, out, k, m, n);
}
void llamd_fwd_rope_rows(const float *x, float *out, int row_len, int rows, int head_dim, const float *sincos) {
    if (rows <= 0 || row_len <= 0) return;
    if (head_dim <= 0 || head_dim % 2 || row_len % head_dim) {
        set_error_msg("rope_rows: head_dim must be even and divide the row length");
        return;
    }
    launch_k("rope_rows", rope_rows_kernel, dim3(rows), dim3(128), 0, x, out, row_len, head_dim, reinterpret_cast<const float2 *>(sincos));
}
void llamd_fwd_get_rows_f32(const float *table, const uint32_t *ids, float *out, int row_len, int n_ids) {
    if (n_ids <= 0 || row_len <= 0) return;
    launch_k("get_rows_f32", get_rows_kernel, dim3(n_ids), dim3(256), 0, table, ids, out, row_len);
}

}  // extern "C"
