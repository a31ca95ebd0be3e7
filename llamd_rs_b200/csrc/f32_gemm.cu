// out[t][row] = fold(-0.0, +) of w[row][i] * x[t][i], i ascending: the f32 matvec of
// crates/llamd-models/src/model.rs:253-263 for the ntok tokens of a prefill tile at once.
//
// The sum over i is one chain per output element and stays one: a thread owns a 2x2 patch of
// outputs (two tokens x two rows) and walks i in order for its four private accumulators with an
// unfused multiply and add. Tiling only shares the operand fetches: a CTA stages 64 columns of 16
// tokens and 32 rows in shared memory (double-buffered with cp.async) and every staged value feeds
// two chains. The router logits of a tile (128 experts x 2048 columns x up to 512 tokens) are the
// user; the chains are as long as in the one-token kernel but 16k of them now run side by side.
#include "common.cuh"

namespace llamd {
namespace {

__device__ __forceinline__ void cp_async16(void *dst, const void *src, int bytes) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kFT = 16;       // tokens per CTA
constexpr int kFR = 32;       // rows per CTA
constexpr int kFK = 64;       // columns per staged chunk
constexpr int kFS = kFK + 4;  // shared-memory row stride: 16-byte aligned, neighbouring rows in different bank groups

// grid (row tiles, token tiles), 128 threads. Thread (ty, tx) = (tid / 16, tid % 16) owns tokens 2ty, 2ty+1 and rows tx, tx+16.
__global__ void __launch_bounds__(128) matmul_f32_tokens_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
                                                                int k, int rows, int ntok) {
    __shared__ __align__(16) float sX[2][kFT][kFS];
    __shared__ __align__(16) float sW[2][kFR][kFS];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int r0 = blockIdx.x * kFR, t0 = blockIdx.y * kFT;
    auto stage = [&](int k0, int buf) {
        // 16-byte pieces: (16 + 32) rows x 16 pieces = 768, six per thread
        for (int idx = tid; idx < (kFT + kFR) * (kFK / 4); idx += 128) {
            const int r = idx >> 4, c = idx & 15;
            const int col = k0 + 4 * c;
            const int bytes = col < k ? 16 : 0;  // k is a multiple of 4
            if (r < kFT) {
                const int t = t0 + r;
                cp_async16(&sX[buf][r][4 * c], x + (size_t)min(t, ntok - 1) * k + min(col, k - 4), t < ntok ? bytes : 0);
            } else {
                const int row = r0 + r - kFT;
                cp_async16(&sW[buf][r - kFT][4 * c], w + (size_t)min(row, rows - 1) * k + min(col, k - 4), row < rows ? bytes : 0);
            }
        }
        cp_async_commit();
    };
    float acc[2][2] = {{-0.0f, -0.0f}, {-0.0f, -0.0f}};
    const int n_chunks = (k + kFK - 1) / kFK;
    stage(0, 0);
    for (int ch = 0; ch < n_chunks; ch++) {
        const int buf = ch & 1;
        if (ch + 1 < n_chunks) {
            stage((ch + 1) * kFK, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int n4 = min(kFK, k - ch * kFK) >> 2;  // no padding terms: a chain holds exactly its k products
#pragma unroll 4
        for (int c4 = 0; c4 < n4; c4++) {
            float4 a[2], b[2];
#pragma unroll
            for (int i = 0; i < 2; i++) a[i] = *reinterpret_cast<const float4 *>(&sX[buf][2 * ty + i][4 * c4]);
#pragma unroll
            for (int j = 0; j < 2; j++) b[j] = *reinterpret_cast<const float4 *>(&sW[buf][tx + 16 * j][4 * c4]);
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    float s = acc[i][j];
                    s = __fadd_rn(s, __fmul_rn(b[j].x, a[i].x));
                    s = __fadd_rn(s, __fmul_rn(b[j].y, a[i].y));
                    s = __fadd_rn(s, __fmul_rn(b[j].z, a[i].z));
                    s = __fadd_rn(s, __fmul_rn(b[j].w, a[i].w));
                    acc[i][j] = s;
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int t = t0 + 2 * ty + i;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int row = r0 + tx + 16 * j;
            if (t < ntok && row < rows) out[(size_t)t * rows + row] = acc[i][j];
        }
    }
}

}  // namespace
}  // namespace llamd

using namespace llamd;

extern "C" void llamd_fwd_matmul_f32_tokens(const float *w, const float *x, float *out, int k, int rows, int ntok) {
    if (ntok <= 0 || rows <= 0) return;
    if (k < 4 || k % 4) {
        set_error_msg("matmul_f32_tokens: k must be a positive multiple of 4");
        return;
    }
    launch_k("matmul_f32_tokens", matmul_f32_tokens_kernel, dim3((rows + kFR - 1) / kFR, (ntok + kFT - 1) / kFT), dim3(128), 0, w, x, out, k, rows,
             ntok);
}
