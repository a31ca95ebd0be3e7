// Attention for the tokens of one prefill tile, as three register-tiled kernels.
//
// The arithmetic is that of `attend` (crates/llamd-cpu/src/lib.rs, the per-head
// loop: dot = sum_d q[d]*k[t][d] from 0.0 in d order, logit = dot*scale,
// softmax with an ordered sum, out[d] = sum_t (e[t]*inv)*v[t][d] from 0.0 in t
// order), one query per token, every token seeing positions 0..pos of the ONE
// cache the tile has already stored into. Nothing is re-associated: each
// output element is one thread-private accumulator that walks its reduction
// index in order with an unfused multiply and add. What changes against the
// per-token kernels is only WHO holds the chains: a thread owns a 4x4 (scores)
// or 4x8 (output) patch of independent chains, so operands fetched from shared
// memory are reused 4-8 times and the FP32 pipe, not memory, sets the pace.
//
//   tile_scores_kernel   S[t][p] = scale * (q_t . k_p)        64 tokens x 64 positions x one head per CTA
//   tile_softmax_kernel  W[t][p] = exp(S - max) / sum          one warp per (token, head) row, in place
//   tile_pv_kernel       out[t][d] = sum_p W[t][p] * v_p[d]    32 tokens x head_dim x one head per CTA
//
// A weight beyond a token's own position is staged as +0.0, and 0*v added to
// an accumulator that started at +0.0 leaves it unchanged, so every token's
// chain is exactly the chain over its own positions.
#include "common.cuh"
#include "quant.cuh"

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

constexpr int kST = 64;  // tokens per CTA of the score kernel
constexpr int kSP = 64;  // positions per CTA of the score kernel

// grid (position tiles, token tiles, heads), 256 threads.
// Thread (ty, tx) = (tid / 16, tid % 16) owns tokens 4ty..4ty+3 and positions tx, tx+16, tx+32, tx+48 of the tile.
__global__ void __launch_bounds__(256) tile_scores_kernel(const float *__restrict__ q, const float *__restrict__ kc, float *__restrict__ scores,
                                                          int n_head, int n_head_kv, int hd, const int32_t *__restrict__ meta, int max_kv,
                                                          int ntok) {
    extern __shared__ __align__(16) float sm[];
    __shared__ int s_pos[kST];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int p0 = blockIdx.x * kSP, t0 = blockIdx.y * kST, h = blockIdx.z;
    if (tid < kST) s_pos[tid] = (t0 + tid < ntok) ? meta[2 * (t0 + tid) + 1] : -1;
    __syncthreads();
    int maxpos = -1;
    for (int i = 0; i < kST; i++) maxpos = max(maxpos, s_pos[i]);
    if (p0 > maxpos) return;
    const int S = hd + 4;  // row stride: 16-byte aligned, rows 4 apart fall into different bank groups
    float *sQ = sm, *sK = sm + kST * S;
    const int hd4 = hd >> 2, kv_dim = n_head_kv * hd, kvh = h / (n_head / n_head_kv);
    for (int idx = tid; idx < kST * hd4; idx += 256) {
        const int r = idx / hd4, c = idx - r * hd4;
        const int t = t0 + r, p = p0 + r;
        cp_async16(sQ + r * S + 4 * c, q + ((size_t)min(t, ntok - 1) * n_head + h) * hd + 4 * c, t < ntok ? 16 : 0);
        cp_async16(sK + r * S + 4 * c, kc + (size_t)min(p, maxpos) * kv_dim + (size_t)kvh * hd + 4 * c, p <= maxpos ? 16 : 0);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    const float *qb = sQ + (ty * 4) * S, *kb = sK + tx * S;
#pragma unroll 2
    for (int d4 = 0; d4 < hd4; d4++) {
        float4 a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; i++) a[i] = *reinterpret_cast<const float4 *>(qb + i * S + 4 * d4);
#pragma unroll
        for (int j = 0; j < 4; j++) b[j] = *reinterpret_cast<const float4 *>(kb + j * 16 * S + 4 * d4);
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i].x, b[j].x));
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i].y, b[j].y));
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i].z, b[j].z));
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i].w, b[j].w));
    }
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i, pos = s_pos[ty * 4 + i];
        float *row = scores + ((size_t)t * n_head + h) * max_kv;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int p = p0 + j * 16 + tx;
            if (p <= pos) row[p] = __fmul_rn(acc[i][j], scale);
        }
    }
}

// One warp per (token, head) row: the logits become the softmax weights e*inv in place.
// Dynamic shared memory: [warps][n_cap] floats, n_cap a multiple of 4 that bounds every row's length.
__global__ void tile_softmax_kernel(float *__restrict__ scores, const int32_t *__restrict__ meta, int n_head, int max_kv, int ntok, int n_cap) {
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int row = blockIdx.x * warps + warp;
    if (row >= ntok * n_head) return;
    const int n = min(meta[2 * (row / n_head) + 1] + 1, n_cap);
    float *sl = sm + (size_t)warp * n_cap;
    float *g = scores + (size_t)row * max_kv;
    float lmax = -INFINITY;
    for (int p = lane; p < n; p += 32) {
        const float l = g[p];
        sl[p] = l;
        lmax = fmaxf(lmax, l);
    }
    for (int off = 16; off > 0; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
    for (int p = lane; p < n; p += 32) sl[p] = ref_expf(__fsub_rn(sl[p], lmax));
    __syncwarp();
    float inv = 0.0f;
    if (lane == 0) inv = __fdiv_rn(1.0f, chain_sum(sl, n, 0.0f));
    inv = __shfl_sync(0xffffffffu, inv, 0);
    for (int p = lane; p < n; p += 32) g[p] = __fmul_rn(sl[p], inv);
}

constexpr int kOT = 32;  // tokens per CTA of the output kernel
constexpr int kOP = 32;  // positions per staged tile
constexpr int kWS = kOP + 4;

// grid (token tiles, heads), 128 threads. Thread (ty, tx) = (tid / 16, tid % 16) owns tokens 4ty..4ty+3 and the
// output columns 64g + 4tx .. +3 for g < HD/64.
template <int HD>
__global__ void __launch_bounds__(128) tile_pv_kernel(const float *__restrict__ w, const float *__restrict__ vc, float *__restrict__ out, int n_head,
                                                      int n_head_kv, const int32_t *__restrict__ meta, int max_kv, int ntok) {
    constexpr int G = HD / 64, HD4 = HD / 4;
    __shared__ __align__(16) float sW[2][kOT][kWS];
    __shared__ __align__(16) float sV[2][kOP][HD];
    __shared__ int s_pos[kOT];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const int t0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * kOT, h = blockIdx.y;  // the longest tiles start first
    if (tid < kOT) s_pos[tid] = (t0 + tid < ntok) ? meta[2 * (t0 + tid) + 1] : -1;
    __syncthreads();
    int maxpos = -1;
    for (int i = 0; i < kOT; i++) maxpos = max(maxpos, s_pos[i]);
    const int kv_dim = n_head_kv * HD, kvh = h / (n_head / n_head_kv);
    const float *vb = vc + (size_t)kvh * HD;
    auto stage = [&](int pt, int buf) {
        for (int idx = tid; idx < kOT * (kOP / 4); idx += 128) {
            const int r = idx / (kOP / 4), c = idx - r * (kOP / 4);
            const int p = pt * kOP + 4 * c;
            const int valid = max(0, min(4, s_pos[r] - p + 1));
            const float *src = valid ? w + ((size_t)(t0 + r) * n_head + h) * max_kv + p : w;
            cp_async16(&sW[buf][r][4 * c], src, 4 * valid);
        }
        for (int idx = tid; idx < kOP * HD4; idx += 128) {
            const int r = idx / HD4, c = idx - r * HD4;
            const int p = pt * kOP + r;
            cp_async16(&sV[buf][r][4 * c], vb + (size_t)min(p, maxpos) * kv_dim + 4 * c, p <= maxpos ? 16 : 0);
        }
        cp_async_commit();
    };
    float acc[4][G * 4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int c = 0; c < G * 4; c++) acc[i][c] = 0.0f;
    const int n_pt = maxpos / kOP + 1;  // maxpos >= 0: the tile holds at least one token
    stage(0, 0);
    for (int pt = 0; pt < n_pt; pt++) {
        const int buf = pt & 1;
        if (pt + 1 < n_pt) {
            stage(pt + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
#pragma unroll 2
        for (int p4 = 0; p4 < kOP / 4; p4++) {
            float4 wv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) wv[i] = *reinterpret_cast<const float4 *>(&sW[buf][ty * 4 + i][4 * p4]);
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float4 v[G];
#pragma unroll
                for (int g = 0; g < G; g++) v[g] = *reinterpret_cast<const float4 *>(&sV[buf][4 * p4 + c][64 * g + 4 * tx]);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float wi = c == 0 ? wv[i].x : c == 1 ? wv[i].y : c == 2 ? wv[i].z : wv[i].w;
#pragma unroll
                    for (int g = 0; g < G; g++) {
                        acc[i][4 * g + 0] = __fadd_rn(acc[i][4 * g + 0], __fmul_rn(wi, v[g].x));
                        acc[i][4 * g + 1] = __fadd_rn(acc[i][4 * g + 1], __fmul_rn(wi, v[g].y));
                        acc[i][4 * g + 2] = __fadd_rn(acc[i][4 * g + 2], __fmul_rn(wi, v[g].z));
                        acc[i][4 * g + 3] = __fadd_rn(acc[i][4 * g + 3], __fmul_rn(wi, v[g].w));
                    }
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = t0 + ty * 4 + i;
        if (t < ntok) {
#pragma unroll
            for (int g = 0; g < G; g++)
                *reinterpret_cast<float4 *>(out + ((size_t)t * n_head + h) * HD + 64 * g + 4 * tx) =
                    make_float4(acc[i][4 * g], acc[i][4 * g + 1], acc[i][4 * g + 2], acc[i][4 * g + 3]);
        }
    }
}

}  // namespace
}  // namespace llamd

using namespace llamd;

extern "C" {
// The tiled form of llamd_fwd_attention_tile. n_kv_max bounds pos+1 over the tile's tokens (the host knows it:
// base position + token count); the kernels read each token's own position from meta[2i+1].
// Shapes the tiled kernels do not cover (head_dim other than 64 or 128, max_kv not a multiple of 4, a context
// beyond one row of shared memory) go to the per-token kernels, which compute the same bits.
void llamd_fwd_attention_prefill(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                                 int hd, const int32_t *meta, int max_kv, int ntok, int n_kv_max) {
    if (ntok <= 0) return;
    const int n_cap = (n_kv_max + 3) & ~3;
    const bool tiled = scores && (hd == 64 || hd == 128) && max_kv % 4 == 0 && n_kv_max > 0 && n_kv_max <= max_kv && n_head_kv > 0 &&
                       n_head % n_head_kv == 0 && (size_t)n_cap * 4 <= 200 * 1024;
    if (!tiled) {
        llamd_fwd_attention_tile(q, kc, vc, out, scores, n_head, n_head_kv, hd, meta, max_kv, ntok);
        return;
    }
    const size_t smem_s = (size_t)(kST + kSP) * (hd + 4) * sizeof(float);
    static size_t conf_s = 0;
    if (smem_s > 48 * 1024 && smem_s > conf_s) {
        cudaFuncSetAttribute(tile_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_s);
        conf_s = smem_s;
    }
    launch_k("tile_scores", tile_scores_kernel, dim3((n_kv_max + kSP - 1) / kSP, (ntok + kST - 1) / kST, n_head), dim3(256), smem_s, q, kc, scores,
             n_head, n_head_kv, hd, meta, max_kv, ntok);
    int warps = (int)((200 * 1024) / ((size_t)n_cap * 4));
    warps = warps > 8 ? 8 : warps;
    const size_t smem_m = (size_t)warps * n_cap * sizeof(float);
    static size_t conf_m = 0;
    if (smem_m > 48 * 1024 && smem_m > conf_m) {
        cudaFuncSetAttribute(tile_softmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_m);
        conf_m = smem_m;
    }
    const int rows = ntok * n_head;
    launch_k("tile_softmax", tile_softmax_kernel, dim3((rows + warps - 1) / warps), dim3(32 * warps), smem_m, scores, meta, n_head, max_kv, ntok, n_cap);
    const dim3 grid((ntok + kOT - 1) / kOT, n_head);
    if (hd == 64)
        launch_k("tile_pv", tile_pv_kernel<64>, grid, dim3(128), 0, (const float *)scores, vc, out, n_head, n_head_kv, meta, max_kv, ntok);
    else
        launch_k("tile_pv", tile_pv_kernel<128>, grid, dim3(128), 0, (const float *)scores, vc, out, n_head, n_head_kv, meta, max_kv, ntok);
}
}
