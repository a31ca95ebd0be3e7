// The f32 ops around the quantized matvecs: router, f32 and Q8_0 matvec,
// QK-norm + RoPE + KV store, attention, argmax and the expert scatter plan.
//
// Reductions whose order is observable in the reference (sequential f32 sums)
// are walked in that order by one thread; everything that is order-free (max,
// integer counts) is done in parallel.
#include <cooperative_groups.h>
#include <cuda_fp16.h>
#include <math.h>

#include <vector>

#include "q6k_layout.cuh"
#include "quant.cuh"
#include "route.cuh"

namespace llamd {


// ---- f32 matvec: crates/llamd-models/src/model.rs:253-263 -----------------
// y[row] = fold(-0.0, +) of w[row][t]*x[t], t ascending; w is [rows][k]. One
// warp per row: the independent products go to shared memory with coalesced
// loads, lane 0 walks the ordered sum from there.
__device__ __forceinline__ float row_dot_sequential(const float *__restrict__ wrow, const float *__restrict__ x, int k, float *prod, int lane) {
    const float4 *wr = reinterpret_cast<const float4 *>(wrow);
    const float4 *xr = reinterpret_cast<const float4 *>(x);
    // the weight row does not depend on the previous kernel: park it in shared
    // memory before waiting for the activation
    // (16 loads in flight per lane: the row comes from cold HBM)
    const int k4 = k / 4;
    for (int i0 = 0; i0 < k4; i0 += 512) {
        float4 r[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int idx = i0 + j * 32 + lane;
            r[j] = idx < k4 ? __ldg(wr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int idx = i0 + j * 32 + lane;
            if (idx < k4) reinterpret_cast<float4 *>(prod)[idx] = r[j];
        }
    }
    pdl_wait();
    for (int i0 = 0; i0 < k4; i0 += 512) {
        float4 r[16];
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int idx = i0 + j * 32 + lane;
            r[j] = idx < k4 ? __ldg(xr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int j = 0; j < 16; j++) {
            const int idx = i0 + j * 32 + lane;
            if (idx < k4) {
                const float4 a = reinterpret_cast<float4 *>(prod)[idx], b = r[j];
                reinterpret_cast<float4 *>(prod)[idx] =
                    make_float4(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y), __fmul_rn(a.z, b.z), __fmul_rn(a.w, b.w));
            }
        }
    }
    __syncwarp();
    float acc = -0.0f;  // Rust's f32 Sum folds from -0.0
    if (lane == 0) acc = chain_sum(prod, k, acc);
    return acc;
}

__global__ void __launch_bounds__(128) matvec_f32_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
                                                         int k, int rows) {
    extern __shared__ __align__(16) float sm[];  // [4][k]
    pdl_trigger();
    const int seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row >= rows) {
        pdl_wait();
        return;
    }
    const float acc = row_dot_sequential(w + (size_t)row * k, x + (size_t)seq * k, k, sm + (size_t)warp * k, lane);
    if (lane == 0) out[(size_t)seq * rows + row] = acc;
}

__global__ void router_kernel(const float *__restrict__ logits, int n_expert, int n_used, int32_t *__restrict__ ids,
                              float *__restrict__ weights, float *__restrict__ probs) {
    extern __shared__ float s_p[];
    __shared__ float s_red[40 + kMaxUsed];
    __shared__ int s_redi[40 + kMaxUsed];
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x;
    for (int i = threadIdx.x; i < n_expert; i += blockDim.x) s_p[i] = logits[(size_t)seq * n_expert + i];
    __syncthreads();
    route_block(s_p, s_red, s_redi, n_expert, n_used, ids + (size_t)seq * n_used, weights + (size_t)seq * n_used,
                probs ? probs + (size_t)seq * n_expert : nullptr);
}

// Router logits and routing in one launch.
//
// The logit of expert e is a 2048-long left-to-right f32 sum, a chain no
// reordering may touch. The products w[e][t]*x[t] are independent, so a warp
// computes them for its row with coalesced loads and parks them in shared
// memory; lane 0 then walks the chain from there at the speed of dependent
// adds. Four rows per CTA run their chains side by side on different SMs. The
// CTA that finishes last (device-wide counter) has every logit and routes.
// w is the router matrix as the file holds it, [n_expert][k].
__global__ void __launch_bounds__(128) router_rows_kernel(const float *__restrict__ w, const float *__restrict__ x, int k, int n_expert,
                                                          int n_used, float *__restrict__ logits, int32_t *__restrict__ ids,
                                                          float *__restrict__ weights, float *__restrict__ probs,
                                                          unsigned int *__restrict__ done_counter) {
    extern __shared__ __align__(16) float sm[];  // [4][k] products, reused as the route scratch
    __shared__ float s_red[40 + kMaxUsed];
    __shared__ int s_redi[40 + kMaxUsed];
    __shared__ bool s_last;
    pdl_trigger();
    const int seq = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;
    if (row < n_expert) {
        const float acc = row_dot_sequential(w + (size_t)row * k, x + (size_t)seq * k, k, sm + (size_t)warp * k, lane);
        if (lane == 0) {
            logits[(size_t)seq * n_expert + row] = acc;
            __threadfence();
        }
    } else {
        pdl_wait();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicInc(done_counter + seq, gridDim.x - 1);  // wraps to 0 after the last CTA
        s_last = prev == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float *s_p = sm;
    for (int i = threadIdx.x; i < n_expert; i += blockDim.x) s_p[i] = __ldcg(logits + (size_t)seq * n_expert + i);
    __syncthreads();
    route_block(s_p, s_red, s_redi, n_expert, n_used, ids + (size_t)seq * n_used, weights + (size_t)seq * n_used,
                probs ? probs + (size_t)seq * n_expert : nullptr);
}

// The FFN norm and the router in ONE launch (decode): x_out = x + residual; xn = rms_norm(x_out) * w_norm; the Q8_K form
// of xn for the experts; the 128 router logits over xn; the routing decision. Every CTA repeats the cheap norm (one
// 2048-add chain, which sits in front of the router's chains whichever kernel walks it) and then does its four router
// rows as router_rows_kernel does; CTA 0 also writes x_out, the Q8_K bytes and scales (and xn, if asked). One launch
// boundary fewer per layer than norm -> router, the same operations in the same order, hence the same bits.
// x_out must not alias x or residual: the other CTAs still read them.
__global__ void __launch_bounds__(128) norm_router_kernel(const float *__restrict__ w, const float *__restrict__ x, const float *__restrict__ residual,
                                                          float *__restrict__ x_out, const float *__restrict__ w_norm, float *__restrict__ xn_out,
                                                          int8_t *__restrict__ qs, float *__restrict__ d, int k, float eps, int n_expert, int n_used,
                                                          float *__restrict__ logits, int32_t *__restrict__ ids, float *__restrict__ weights,
                                                          float *__restrict__ probs, unsigned int *__restrict__ done_counter, int fast) {
    extern __shared__ __align__(16) float sm[];  // [4][k] router rows / products, [k] x then xn, [k] squares
    __shared__ float s_tree[32];
    __shared__ float s_red[40 + kMaxUsed];
    __shared__ int s_redi[40 + kMaxUsed];
    __shared__ float s_scale;
    __shared__ bool s_last;
    pdl_trigger();
    const int seq = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row = blockIdx.x * 4 + warp, k4 = k / 4;
    float *prod = sm + (size_t)warp * k, *sx = sm + (size_t)4 * k, *ssq = sx + k;
    // the router rows and the norm weights do not depend on the previous kernel: they travel before the wait
    if (row < n_expert) {
        const float4 *wr = reinterpret_cast<const float4 *>(w + (size_t)row * k);
        for (int i0 = 0; i0 < k4; i0 += 512) {
            float4 r[16];
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int idx = i0 + j * 32 + lane;
                r[j] = idx < k4 ? __ldg(wr + idx) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const int idx = i0 + j * 32 + lane;
                if (idx < k4) reinterpret_cast<float4 *>(prod)[idx] = r[j];
            }
        }
    }
    constexpr int kWn = 4;  // (k <= 2048: one register set; a longer row reads the rest where it is used)
    float4 wn_r[kWn];
#pragma unroll
    for (int u = 0; u < kWn; u++) {
        const int j = tid + u * 128;
        wn_r[u] = j < k4 ? __ldg(reinterpret_cast<const float4 *>(w_norm) + j) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    // x + residual, its squares (crates/llamd-cpu/src/lib.rs:55-75 after the add of layer.rs:281-287)
    const float4 *x4 = reinterpret_cast<const float4 *>(x + (size_t)seq * k), *r4 = reinterpret_cast<const float4 *>(residual + (size_t)seq * k);
    for (int j = tid; j < k4; j += 128) {
        const float4 a = x4[j], b = r4[j];
        const float4 v = make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
        reinterpret_cast<float4 *>(sx)[j] = v;
        reinterpret_cast<float4 *>(ssq)[j] = make_float4(__fmul_rn(v.x, v.x), __fmul_rn(v.y, v.y), __fmul_rn(v.z, v.z), __fmul_rn(v.w, v.w));
        if (blockIdx.x == 0) reinterpret_cast<float4 *>(x_out + (size_t)seq * k)[j] = v;
    }
    __syncthreads();
    float scale;
    if (fast & 1) {  // the `fast` arithmetic: the sum of squares as a reduction tree
        float part = 0.0f;
        for (int i = tid; i < k; i += 128) part = __fadd_rn(part, ssq[i]);
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(block_tree_sum(part, s_tree), (float)k), eps)));
    } else {
        if (tid == 0) s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(chain_sum(ssq, k, 0.0f), (float)k), eps)));
        __syncthreads();
        scale = s_scale;
    }
    auto weigh = [&](int j, const float4 wn) {
        const float4 v = reinterpret_cast<const float4 *>(sx)[j];
        const float4 o = make_float4(__fmul_rn(__fmul_rn(v.x, scale), wn.x), __fmul_rn(__fmul_rn(v.y, scale), wn.y),
                                     __fmul_rn(__fmul_rn(v.z, scale), wn.z), __fmul_rn(__fmul_rn(v.w, scale), wn.w));
        reinterpret_cast<float4 *>(sx)[j] = o;
        if (blockIdx.x == 0 && xn_out) reinterpret_cast<float4 *>(xn_out + (size_t)seq * k)[j] = o;
    };
#pragma unroll
    for (int u = 0; u < kWn; u++)
        if (tid + u * 128 < k4) weigh(tid + u * 128, wn_r[u]);
    for (int j = tid + kWn * 128; j < k4; j += 128) weigh(j, __ldg(reinterpret_cast<const float4 *>(w_norm) + j));
    __syncthreads();
    if (blockIdx.x == 0) {  // the Q8_K form for the experts (dot.rs:88-128): a warp per 256-element block
        for (int b = warp; b < k / 256; b += 4) {
            const float4 a = reinterpret_cast<const float4 *>(sx + b * 256 + lane * 8)[0], c = reinterpret_cast<const float4 *>(sx + b * 256 + lane * 8)[1];
            const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
            q8k_quantize_block(v, lane, qs + (size_t)seq * k + (size_t)b * 256, d + (size_t)seq * (k / 256) + b, nullptr);
        }
    }
    // the router rows: y = fold(-0.0, +) of w[r][t] * xn[t], t ascending (crates/llamd-models/src/model.rs:253-263)
    if (row < n_expert && (fast & 2)) {  // the `fast` arithmetic: the same products, summed by a tree over the warp
        float part = 0.0f;
        for (int j = lane; j < k4; j += 32) {
            const float4 a = reinterpret_cast<const float4 *>(prod)[j], b = reinterpret_cast<const float4 *>(sx)[j];
            part = __fadd_rn(part, __fmul_rn(a.x, b.x));
            part = __fadd_rn(part, __fmul_rn(a.y, b.y));
            part = __fadd_rn(part, __fmul_rn(a.z, b.z));
            part = __fadd_rn(part, __fmul_rn(a.w, b.w));
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, off));
        if (lane == 0) {
            logits[(size_t)seq * n_expert + row] = part;
            __threadfence();
        }
    } else if (row < n_expert) {
        for (int j = lane; j < k4; j += 32) {
            const float4 a = reinterpret_cast<const float4 *>(prod)[j], b = reinterpret_cast<const float4 *>(sx)[j];
            reinterpret_cast<float4 *>(prod)[j] = make_float4(__fmul_rn(a.x, b.x), __fmul_rn(a.y, b.y), __fmul_rn(a.z, b.z), __fmul_rn(a.w, b.w));
        }
        __syncwarp();
        if (lane == 0) {
            logits[(size_t)seq * n_expert + row] = chain_sum(prod, k, -0.0f);
            __threadfence();
        }
    }
    __syncthreads();
    if (tid == 0) {
        const unsigned int prev = atomicInc(done_counter + seq, gridDim.x - 1);  // wraps to 0 after the last CTA
        s_last = prev == gridDim.x - 1;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    float *s_p = sm;
    for (int i = tid; i < n_expert; i += blockDim.x) s_p[i] = __ldcg(logits + (size_t)seq * n_expert + i);
    __syncthreads();
    route_block(s_p, s_red, s_redi, n_expert, n_used, ids + (size_t)seq * n_used, weights + (size_t)seq * n_used,
                probs ? probs + (size_t)seq * n_expert : nullptr);
}

// ---- Q8_0 matvec: dequantize (d*q) then the sequential f32 dot -------------
// (crates/llamd-quant/src/lib.rs:154-162 + crates/llamd-models/src/model.rs:253-263)
template <int NSEQ>
__global__ void __launch_bounds__(128) matvec_q8_0_kernel(const uint8_t *__restrict__ tiled, const float *__restrict__ x,
                                                          float *__restrict__ out, int blocks, int rows) {
    extern __shared__ float sx[];  // [NSEQ][k]
    pdl_trigger();
    pdl_wait();
    const int k = blocks * 32;
    for (int i = threadIdx.x; i < NSEQ * k; i += blockDim.x) sx[i] = x[i];
    __syncthreads();
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= rows) return;
    const int lane = row & 31;
    float acc[NSEQ];
#pragma unroll
    for (int s = 0; s < NSEQ; s++) acc[s] = -0.0f;
    const uint8_t *t = tiled + q80_tile_offset(row, 0, blocks);
    uint4 q0 = __ldg(reinterpret_cast<const uint4 *>(t) + lane), q1 = __ldg(reinterpret_cast<const uint4 *>(t + 512) + lane);
    uint16_t db = __ldg(reinterpret_cast<const uint16_t *>(t + 1024) + lane);
    for (int b = 0; b < blocks; b++) {
        const uint4 c0 = q0, c1 = q1;
        const float d = f16_bits_to_f32(db);
        if (b + 1 < blocks) {
            t += kQ80TileBytes;
            q0 = __ldg(reinterpret_cast<const uint4 *>(t) + lane);
            q1 = __ldg(reinterpret_cast<const uint4 *>(t + 512) + lane);
            db = __ldg(reinterpret_cast<const uint16_t *>(t + 1024) + lane);
        }
        const uint32_t ws[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
        for (int j = 0; j < 32; j++) {
            const float w = __fmul_rn(d, (float)(int8_t)(ws[j >> 2] >> (8 * (j & 3))));
#pragma unroll
            for (int s = 0; s < NSEQ; s++) acc[s] = __fadd_rn(acc[s], __fmul_rn(w, sx[s * k + b * 32 + j]));
        }
    }
#pragma unroll
    for (int s = 0; s < NSEQ; s++) out[(size_t)s * rows + row] = acc[s];
}

// The same result with the row's work spread over a CTA. Above, one thread unpacks, converts, multiplies and adds
// every element of its row alone and is bound by its own instruction latency (~20 cycles per element). Here a CTA owns
// 32 rows: seven producer warps turn 8 blocks (256 columns) of the 32 rows into f32 weights d*q in shared memory,
// [column][row] so that a lane per row reads without bank conflicts, while one chain warp per sequence (lane = row)
// walks acc = acc + w*x over the previous 256 columns: only the add is on the dependent chain (~4 cycles per element).
// Raw blocks are loaded two chunks ahead into registers, converted one chunk ahead, double-buffered in shared memory.
constexpr int kQ80ChunkBlocks = 8;
constexpr int kQ80Producers = 224;  // 7 warps
template <int NSEQ>
__global__ void __launch_bounds__(kQ80Producers + 32 * NSEQ) matvec_q8_0_rows_kernel(const uint8_t *__restrict__ tiled, const float *__restrict__ x,
                                                                                     float *__restrict__ out, int blocks, int rows) {
    extern __shared__ __align__(16) float smem_f[];
    float *s_w = smem_f;                                      // [2][kQ80ChunkBlocks * 32 columns][32 rows]
    float *sx = smem_f + 2 * kQ80ChunkBlocks * 32 * 32;       // [NSEQ][k]
    pdl_trigger();
    pdl_wait();
    const int k = blocks * 32, tid = threadIdx.x;
    const bool producer = tid < kQ80Producers;
    const int n_chunks = (blocks + kQ80ChunkBlocks - 1) / kQ80ChunkBlocks;
    const uint8_t *tile0 = tiled + (size_t)blockIdx.x * blocks * kQ80TileBytes;  // this CTA's 32 rows, block 0
    constexpr int kItems = kQ80ChunkBlocks * 64;                                 // (block, half, row): 16 weights each
    constexpr int kPer = (kItems + kQ80Producers - 1) / kQ80Producers;           // 3
    uint4 raw[kPer];
    uint16_t rawd[kPer];
    auto load_chunk = [&](int ch) {
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int item = tid + u * kQ80Producers;
            const int bl = item >> 6, h = (item >> 5) & 1, r = item & 31;
            raw[u] = make_uint4(0, 0, 0, 0);
            rawd[u] = 0;
            if (item < kItems && ch * kQ80ChunkBlocks + bl < blocks) {
                const uint8_t *t = tile0 + (size_t)(ch * kQ80ChunkBlocks + bl) * kQ80TileBytes;
                raw[u] = __ldg(reinterpret_cast<const uint4 *>(t + 512 * h) + r);
                rawd[u] = __ldg(reinterpret_cast<const uint16_t *>(t + 1024) + r);
            }
        }
    };
    auto store_chunk = [&](int buf) {
        float *dst = s_w + buf * (kQ80ChunkBlocks * 32 * 32);
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int item = tid + u * kQ80Producers;
            if (item < kItems) {
                const int bl = item >> 6, h = (item >> 5) & 1, r = item & 31;
                const float d = f16_bits_to_f32(rawd[u]);
                const uint32_t ws[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
                for (int j = 0; j < 16; j++)
                    dst[(bl * 32 + h * 16 + j) * 32 + r] = __fmul_rn(d, (float)(int8_t)(ws[j >> 2] >> (8 * (j & 3))));
            }
        }
    };
    if (producer) load_chunk(0);
    for (int i = tid; i < NSEQ * k; i += blockDim.x) sx[i] = x[i];
    if (producer) {
        store_chunk(0);
        if (n_chunks > 1) load_chunk(1);
    }
    __syncthreads();
    const int seq = (tid - kQ80Producers) >> 5, lane = tid & 31;  // chain warps
    float acc = -0.0f;
    for (int ch = 0; ch < n_chunks; ch++) {
        if (producer) {
            if (ch + 1 < n_chunks) store_chunk((ch + 1) & 1);
            if (ch + 2 < n_chunks) load_chunk(ch + 2);
        } else {
            const float *w = s_w + (ch & 1) * (kQ80ChunkBlocks * 32 * 32) + lane;
            const float *xs = sx + (size_t)seq * k + ch * kQ80ChunkBlocks * 32;
            const int ncol = min(kQ80ChunkBlocks, blocks - ch * kQ80ChunkBlocks) * 32;
            // 16 columns at a time, the next 16 loaded while these are added: the loads and the multiplies stay off
            // the chain, which is then the 16 dependent adds (ncol is a multiple of 32)
            float wv[16], xv[16];
            auto fetch = [&](int c0) {
#pragma unroll
                for (int j = 0; j < 16; j++) wv[j] = w[(c0 + j) * 32];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float4 v = *reinterpret_cast<const float4 *>(xs + c0 + 4 * j);
                    xv[4 * j] = v.x, xv[4 * j + 1] = v.y, xv[4 * j + 2] = v.z, xv[4 * j + 3] = v.w;
                }
            };
            fetch(0);
            for (int c0 = 0; c0 < ncol; c0 += 16) {
                float pr[16];
#pragma unroll
                for (int j = 0; j < 16; j++) pr[j] = __fmul_rn(wv[j], xv[j]);
                if (c0 + 16 < ncol) fetch(c0 + 16);
#pragma unroll
                for (int j = 0; j < 16; j++) acc = __fadd_rn(acc, pr[j]);
            }
        }
        __syncthreads();
    }
    const int row = blockIdx.x * 32 + lane;
    if (!producer && row < rows) out[(size_t)seq * rows + row] = acc;
}

// The same arithmetic again, fed by bulk copies. The form above keeps ONE chunk of raw blocks in flight per CTA (8.7 KB
// per SM against an HBM round trip of ~2 us: 0.5 TB/s over the whole GPU, which is what it measured). Here one thread
// asks for the CTA's WHOLE slice of the matrix -- 32 rows x all blocks, one contiguous run of the tiled layout -- as one
// bulk copy per 256-column chunk (cp.async.bulk, each completing on its own mbarrier) before anything else happens, so
// the memory latency is paid once and the producers then convert from shared memory. With one sequence the producers
// store the products (d*q)*x, so the chain warp's loop is a shared load and the dependent add alone.
// Every mbarrier wait is bounded; a wait that runs out sets *status and the CTA leaves its outputs unwritten.
__device__ __forceinline__ uint32_t q80_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool q80_mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t a = q80_smem_u32(bar);
    for (int it = 0; it < (1 << 14); it++) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(a), "r"(parity), "r"(20000u)
            : "memory");
        if (done) return true;
    }
    return false;
}
constexpr int kQ80MaxChunks = 32;  // k <= 8192
template <int NSEQ>
__global__ void __launch_bounds__(kQ80Producers + 32 * NSEQ) matvec_q8_0_bulk_kernel(const uint8_t *__restrict__ tiled, const float *__restrict__ x,
                                                                                     float *__restrict__ out, int blocks, int rows, int *status) {
    extern __shared__ __align__(16) float smem_f[];
    __shared__ __align__(8) uint64_t s_bar[kQ80MaxChunks];
    __shared__ int s_fail;
    constexpr bool kProd = NSEQ == 1;                         // the ring holds products w*x instead of weights
    // ring: [2][64 column quads][32 rows][4]: a lane (= row) reads four consecutive columns with one 16-byte load, and the
    // 32 lanes' loads are one conflict-free 512-byte run (a scalar load per column cost the chain warp 16 issue slots per
    // 16 adds and ran at ~7 cycles per add instead of ~4.4)
    float *s_w = smem_f;
    float *sx = smem_f + 2 * kQ80ChunkBlocks * 32 * 32;       // [NSEQ][k]
    const int k = blocks * 32, tid = threadIdx.x;
    uint8_t *s_raw = reinterpret_cast<uint8_t *>(sx + (size_t)NSEQ * k);  // [blocks][1088]: the tiles as they lie in memory
    const bool producer = tid < kQ80Producers;
    const int n_chunks = (blocks + kQ80ChunkBlocks - 1) / kQ80ChunkBlocks;
    const uint8_t *tile0 = tiled + (size_t)blockIdx.x * blocks * kQ80TileBytes;  // this CTA's 32 rows, block 0
    if (tid == 0) {
        s_fail = 0;
        for (int ch = 0; ch < n_chunks; ch++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(q80_smem_u32(&s_bar[ch])) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // the weights do not depend on the previous kernel: their copies start before the dependency wait
        for (int ch = 0; ch < n_chunks; ch++) {
            const int nb = min(kQ80ChunkBlocks, blocks - ch * kQ80ChunkBlocks);
            const uint32_t bytes = (uint32_t)nb * kQ80TileBytes;  // (1088 = 68 x 16)
            const uint32_t bar = q80_smem_u32(&s_bar[ch]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             q80_smem_u32(s_raw + (size_t)ch * kQ80ChunkBlocks * kQ80TileBytes)),
                         "l"(tile0 + (size_t)ch * kQ80ChunkBlocks * kQ80TileBytes), "r"(bytes), "r"(bar)
                         : "memory");
        }
    }
    pdl_trigger();
    pdl_wait();
    for (int i = tid; i < NSEQ * k; i += blockDim.x) sx[i] = x[i];
    __syncthreads();  // (the barriers are initialised, the activations staged)
    constexpr int kItems = kQ80ChunkBlocks * 64;                        // (block, half, row): 16 weights each
    constexpr int kPer = (kItems + kQ80Producers - 1) / kQ80Producers;  // 3
    auto convert_chunk = [&](int ch) -> bool {
        if (!q80_mbar_wait(&s_bar[ch], 0)) return false;
        float4 *dst = reinterpret_cast<float4 *>(s_w + (ch & 1) * (kQ80ChunkBlocks * 32 * 32));
#pragma unroll
        for (int u = 0; u < kPer; u++) {
            const int item = tid + u * kQ80Producers;
            const int bl = item >> 6, h = (item >> 5) & 1, r = item & 31;
            if (item < kItems && ch * kQ80ChunkBlocks + bl < blocks) {
                const uint8_t *t = s_raw + (size_t)(ch * kQ80ChunkBlocks + bl) * kQ80TileBytes;
                const uint4 raw = *(reinterpret_cast<const uint4 *>(t + 512 * h) + r);
                const float d = f16_bits_to_f32(*(reinterpret_cast<const uint16_t *>(t + 1024) + r));
                const uint32_t ws[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
                const float4 *xs = reinterpret_cast<const float4 *>(sx + (ch * kQ80ChunkBlocks + bl) * 32 + h * 16);
#pragma unroll
                for (int g = 0; g < 4; g++) {
                    // q as f32 without the converter unit: the byte q + 128 dropped into the mantissa of 2^23 is 2^23 + 128 + q
                    float q[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) q[j] = __fsub_rn(__uint_as_float(__byte_perm(ws[g], 0x4B000000u, 0x7650 + j)), 8388736.0f);
                    float4 o = make_float4(__fmul_rn(d, q[0]), __fmul_rn(d, q[1]), __fmul_rn(d, q[2]), __fmul_rn(d, q[3]));
                    if (kProd) {
                        const float4 xv = xs[g];
                        o = make_float4(__fmul_rn(o.x, xv.x), __fmul_rn(o.y, xv.y), __fmul_rn(o.z, xv.z), __fmul_rn(o.w, xv.w));
                    }
                    dst[(bl * 8 + h * 4 + g) * 32 + r] = o;
                }
            }
        }
        return true;
    };
    if (producer && !convert_chunk(0)) s_fail = 1;
    __syncthreads();
    const int seq = (tid - kQ80Producers) >> 5, lane = tid & 31;  // chain warps
    float acc = -0.0f;
#define Q80_ADD4(v) acc = __fadd_rn(acc, v.x), acc = __fadd_rn(acc, v.y), acc = __fadd_rn(acc, v.z), acc = __fadd_rn(acc, v.w)
    for (int ch = 0; ch < n_chunks; ch++) {
        if (producer) {
            if (ch + 1 < n_chunks && !s_fail && !convert_chunk(ch + 1)) s_fail = 1;
        } else {
            const float4 *w = reinterpret_cast<const float4 *>(s_w + (ch & 1) * (kQ80ChunkBlocks * 32 * 32)) + lane;
            const int nq = min(kQ80ChunkBlocks, blocks - ch * kQ80ChunkBlocks) * 8;  // column quads: a multiple of 8
            if (kProd) {
                // two register sets of 16 products alternate; a set is re-loaded right after it has been added
                float4 a0 = w[0], a1 = w[32], a2 = w[64], a3 = w[96], b0 = w[128], b1 = w[160], b2 = w[192], b3 = w[224];
                for (int q0 = 0; q0 < nq; q0 += 8) {
                    Q80_ADD4(a0), Q80_ADD4(a1), Q80_ADD4(a2), Q80_ADD4(a3);
                    const int qa = min(q0 + 8, nq - 8) * 32;
                    a0 = w[qa], a1 = w[qa + 32], a2 = w[qa + 64], a3 = w[qa + 96];
                    Q80_ADD4(b0), Q80_ADD4(b1), Q80_ADD4(b2), Q80_ADD4(b3);
                    const int qb = min(q0 + 12, nq - 4) * 32;
                    b0 = w[qb], b1 = w[qb + 32], b2 = w[qb + 64], b3 = w[qb + 96];
                }
            } else {
                const float4 *xs = reinterpret_cast<const float4 *>(sx + (size_t)seq * k + ch * kQ80ChunkBlocks * 32);
                float4 wv[4], xv[4];
                auto fetch = [&](int q0) {
#pragma unroll
                    for (int j = 0; j < 4; j++) wv[j] = w[(q0 + j) * 32], xv[j] = xs[q0 + j];
                };
                fetch(0);
                for (int q0 = 0; q0 < nq; q0 += 4) {
                    float4 pr[4];
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        pr[j] = make_float4(__fmul_rn(wv[j].x, xv[j].x), __fmul_rn(wv[j].y, xv[j].y), __fmul_rn(wv[j].z, xv[j].z), __fmul_rn(wv[j].w, xv[j].w));
                    if (q0 + 4 < nq) fetch(q0 + 4);
                    Q80_ADD4(pr[0]), Q80_ADD4(pr[1]), Q80_ADD4(pr[2]), Q80_ADD4(pr[3]);
                }
            }
        }
        __syncthreads();
    }
#undef Q80_ADD4
    if (s_fail) {
        // a copy did not arrive within the limit: wait (bounded again) for the ones still in flight before this CTA's shared
        // memory is given up, record it, write nothing
        if (tid == 0) {
            for (int ch = 0; ch < n_chunks; ch++) q80_mbar_wait(&s_bar[ch], 0);
            atomicExch(status, 1 + (int)blockIdx.x);
        }
        return;
    }
    const int row = blockIdx.x * 32 + lane;
    if (!producer && row < rows) out[(size_t)seq * rows + row] = acc;
}

// ---- QK-norm + RoPE (+ KV store) -----------------------------------------
// The KV cache's element type. The reference's caches are f32 (crates/llamd-runtime/src/kv.rs:27-170) and that is the
// default; with binary16 elements (model option "kv_f16": the benchmark configuration names an f16 cache) a K or V value
// is rounded to nearest-even once, when it is stored, and widened exactly when it is read: every other operation is
// unchanged, so the results are those of the f32 arithmetic over a cache of f16-representable values.
template <class T>
struct KvIo;
template <>
struct KvIo<float> {
    static __device__ __forceinline__ float4 ld4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
    static __device__ __forceinline__ void st(float *p, float v) { *p = v; }
};
template <>
struct KvIo<__half> {
    static __device__ __forceinline__ float4 ld4(const __half *p) {
        const uint2 u = __ldg(reinterpret_cast<const uint2 *>(p));
        const __half2 a = *reinterpret_cast<const __half2 *>(&u.x), b = *reinterpret_cast<const __half2 *>(&u.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void st(__half *p, float v) { *p = __float2half_rn(v); }
};

// crates/llamd-runtime/src/layer.rs:120-153, crates/llamd-cpu/src/lib.rs:158-209.
// One CTA of hd/2 threads per head; thread 0 walks the sum of squares. The
// sin/cos come from a table the host built with its own libm, which is what
// the reference's CPU path calls (powf, sin, cos).
template <class KVT>
__global__ void norm_rope_kernel(float *__restrict__ xq, const float *__restrict__ wq, float *__restrict__ xk, const float *__restrict__ wk,
                                 const float *__restrict__ v_src, KVT *__restrict__ kc, KVT *__restrict__ vc, int n_head_q,
                                 int n_head_k, int hd, const int32_t *__restrict__ meta, int pos_imm, const float *__restrict__ rope_tab,
                                 float eps, int kv_stride) {
    extern __shared__ float sx[];
    __shared__ float s_scale;
    pdl_trigger();
    pdl_wait();
    // blocks [0, n_head_q) are query heads, [n_head_q, n_head_q + n_head_k) key heads
    const bool is_k = (int)blockIdx.x >= n_head_q;
    const int head = is_k ? blockIdx.x - n_head_q : blockIdx.x;
    const int n_head = is_k ? n_head_k : n_head_q;
    float *x = is_k ? xk : xq;
    const float *w = is_k ? wk : wq;
    const int seq = blockIdx.y, half = hd / 2, i = threadIdx.x;
    const int pos = meta ? meta[2 * seq + 1] : pos_imm;
    float *xh = x + ((size_t)seq * n_head + head) * hd;
    sx[i] = xh[i];
    sx[i + half] = xh[i + half];
    __syncthreads();
    float scale = 1.0f;
    if (w) {
        if (i == 0) {
            float sum = 0.0f;
#pragma unroll 8
            for (int t = 0; t < hd; t++) sum = __fadd_rn(sum, __fmul_rn(sx[t], sx[t]));
            s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)hd), eps)));
        }
        __syncthreads();
        scale = s_scale;
    }
    float a = sx[i], b = sx[i + half];
    if (w) {
        a = __fmul_rn(__fmul_rn(a, scale), w[i]);
        b = __fmul_rn(__fmul_rn(b, scale), w[i + half]);
    }
    const float2 sc = *reinterpret_cast<const float2 *>(rope_tab + ((size_t)pos * half + i) * 2);
    const float o0 = __fsub_rn(__fmul_rn(a, sc.y), __fmul_rn(b, sc.x));
    const float o1 = __fadd_rn(__fmul_rn(a, sc.x), __fmul_rn(b, sc.y));
    xh[i] = o0;
    xh[i + half] = o1;
    if (is_k && kc) {
        const int kv_dim = n_head * hd;
        // kv_stride: positions between two sequences' caches; 0 when every row of
        // the launch is a position of ONE sequence (a prefill tile)
        KVT *kdst = kc + ((size_t)seq * kv_stride + pos) * kv_dim + (size_t)head * hd;
        KVT *vdst = vc + ((size_t)seq * kv_stride + pos) * kv_dim + (size_t)head * hd;
        const float *vs = v_src + ((size_t)seq * n_head + head) * hd;
        KvIo<KVT>::st(kdst + i, o0);
        KvIo<KVT>::st(kdst + i + half, o1);
        KvIo<KVT>::st(vdst + i, vs[i]);
        KvIo<KVT>::st(vdst + i + half, vs[i + half]);
    }
}

__global__ void kv_store_kernel(float *__restrict__ kc, float *__restrict__ vc, const float *__restrict__ k, const float *__restrict__ v,
                                int pos, int kv_dim) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kv_dim) {
        kc[(size_t)pos * kv_dim + i] = k[i];
        vc[(size_t)pos * kv_dim + i] = v[i];
    }
}

// ---- attention: crates/llamd-runtime/src/attention.rs:62-125 ---------------
// One CTA of 256 threads per (query head, sequence).
//   logit[t] = (sum_d q[d]*k[t][d], d ascending) * scale
//   max (order-free), e[t] = exp(logit[t]-max), sum e[t] t ascending
//   out[d] = sum_t (e[t]*inv) * v[t][d], t ascending
// The three sums are left-to-right chains. K and V are staged through shared
// memory in tiles of 64 positions, fetched by all threads with many loads in
// flight and prefetched one tile ahead, so the chains read shared memory only:
// thread t walks d for its position (tile rows padded to hd+1 words, no bank
// conflicts), thread d walks t for its output column.
constexpr int kAttTile = 64;

__global__ void __launch_bounds__(256) attention_kernel(const float *__restrict__ q, const float *__restrict__ kc,
                                                        const float *__restrict__ vc, float *__restrict__ out, int n_head, int n_head_kv,
                                                        int hd, const int32_t *__restrict__ meta, int n_kv_imm, int max_kv, int kv_stride) {
    extern __shared__ __align__(16) float sm[];
    const int stride = hd + 1;
    float *sq = sm;                       // [hd]
    float *sl = sm + hd;                  // [n_kv] scores
    const int n_kv_cap = meta ? max_kv : n_kv_imm;
    float *tile = sl + ((n_kv_cap + 3) & ~3);  // [2][kAttTile][stride]
    __shared__ float s_red[16];
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
    const int n_kv = meta ? meta[2 * seq + 1] + 1 : n_kv_imm;
    const int kv_dim = n_head_kv * hd, kvh = h / (n_head / n_head_kv);
    const float *kb = kc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd;
    const float *vb = vc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd;
    const float *qh = q + ((size_t)seq * n_head + h) * hd;
    for (int i = tid; i < hd; i += blockDim.x) sq[i] = qh[i];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const int hd4 = hd / 4, per_tile4 = kAttTile * hd4;  // float4s per tile
    const int n_tiles = (n_kv + kAttTile - 1) / kAttTile;
    constexpr int kMaxLd = 8;  // float4 loads in flight per thread (hd 128: 64*32/256)

    // fetch tile `ti` of `base` into registers
    float4 reg[kMaxLd];
    auto fetch = [&](const float *base, int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / hd4, c = idx - r * hd4;
            const int t = ti * kAttTile + r;
            reg[j] = (idx < per_tile4 && t < n_kv) ? __ldg(reinterpret_cast<const float4 *>(base + (size_t)t * kv_dim) + c)
                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](float *dst) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            if (idx < per_tile4) {
                const int r = idx / hd4, c = idx - r * hd4;
                float *p = dst + r * stride + 4 * c;
                p[0] = reg[j].x;
                p[1] = reg[j].y;
                p[2] = reg[j].z;
                p[3] = reg[j].w;
            }
        }
    };

    // ---- scores ----
    fetch(kb, 0);
    float lmax = -INFINITY;
    for (int ti = 0; ti < n_tiles; ti++) {
        float *cur = tile + (ti & 1) * kAttTile * stride;
        stash(cur);
        __syncthreads();
        if (ti + 1 < n_tiles) fetch(kb, ti + 1);
        const int t = ti * kAttTile + tid;
        if (tid < kAttTile && t < n_kv) {
            const float *kr = cur + tid * stride;
            float dot = 0.0f;
            if ((hd & 15) == 0) {
                // blocks of 16 products, the next block fetched while this one is added
                float pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(sq[i], kr[i]);
                for (int d0 = 0; d0 < hd; d0 += 16) {
                    const int dn = (d0 + 16 < hd) ? d0 + 16 : d0;
#pragma unroll
                    for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(sq[dn + i], kr[dn + i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) dot = __fadd_rn(dot, pa[i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) pa[i] = pb[i];
                }
            } else {
                for (int d = 0; d < hd; d++) dot = __fadd_rn(dot, __fmul_rn(sq[d], kr[d]));
            }
            const float l = __fmul_rn(dot, scale);
            sl[t] = l;
            lmax = fmaxf(lmax, l);
        }
        // the buffer written two iterations from now is this one: the barrier
        // at the top of the next iteration orders those writes after this read
    }
    for (int off = 16; off > 0; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = lmax;
    __syncthreads();
    lmax = s_red[0];
    for (int w = 1; w < 8; w++) lmax = fmaxf(lmax, s_red[w]);
    // ---- softmax ----
    fetch(vb, 0);  // V tile 0 travels while the exponentials and the sum run
    for (int t = tid; t < n_kv; t += blockDim.x) sl[t] = ref_expf(__fsub_rn(sl[t], lmax));
    __syncthreads();
    if (tid == 0) s_red[8] = __fdiv_rn(1.0f, chain_sum(sl, n_kv, 0.0f));
    __syncthreads();
    const float inv = s_red[8];
    // ---- weighted values ----
    float acc = 0.0f;
    for (int ti = 0; ti < n_tiles; ti++) {
        float *cur = tile + (ti & 1) * kAttTile * stride;
        stash(cur);
        __syncthreads();
        if (ti + 1 < n_tiles) fetch(vb, ti + 1);
        if (tid < hd) {
            const int t0 = ti * kAttTile, cnt = min(kAttTile, n_kv - t0);
            if (cnt == kAttTile) {
                float pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(__fmul_rn(sl[t0 + i], inv), cur[i * stride + tid]);
#pragma unroll
                for (int r0 = 0; r0 < kAttTile; r0 += 16) {
                    const int rn = (r0 + 16 < kAttTile) ? r0 + 16 : r0;
#pragma unroll
                    for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(__fmul_rn(sl[t0 + rn + i], inv), cur[(rn + i) * stride + tid]);
#pragma unroll
                    for (int i = 0; i < 16; i++) acc = __fadd_rn(acc, pa[i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) pa[i] = pb[i];
                }
            } else {
#pragma unroll 4
                for (int r = 0; r < cnt; r++) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(sl[t0 + r], inv), cur[r * stride + tid]));
            }
        }
    }
    if (tid < hd) out[((size_t)seq * n_head + h) * hd + tid] = acc;
}

// ---- attention, split over CTAs ---------------------------------------------
// The same arithmetic as attention_kernel, cut so that more SMs pull K and V:
//   attn_scores_kernel  grid (head, kSplitT, seq): CTA c takes the 64-position
//                       tiles ti with ti % kSplitT == c and writes the scaled
//                       logits to the global `scores` buffer;
//   attn_out_kernel     grid (head, kSplit, seq): every CTA redoes the (cheap)
//                       softmax over all positions, then walks t for its own
//                       hd/kSplit output columns.
// Each position's dot and each output column's sum is still one left-to-right
// chain, so the result is bit-identical to the single-CTA kernel.
constexpr int kSplit = 4;    // output-column split of attn_out_kernel
constexpr int kSplitT = 8;   // position-tile split of attn_scores_kernel

template <class KVT>
__global__ void __launch_bounds__(256) attn_scores_kernel(const float *__restrict__ q, const KVT *__restrict__ kc, float *__restrict__ scores,
                                                          int n_head, int n_head_kv, int hd, const int32_t *__restrict__ meta,
                                                          int n_kv_imm, int max_kv, int kv_stride) {
    extern __shared__ __align__(16) float sm[];
    const int stride = hd + 1;
    float *sq = sm;          // [hd]
    float *tile = sm + hd;   // [2][kAttTile][stride]
    pdl_trigger();
    pdl_wait();
    const int h = blockIdx.x, c = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
    const int n_kv = meta ? meta[2 * seq + 1] + 1 : n_kv_imm;
    const int kv_dim = n_head_kv * hd, kvh = h / (n_head / n_head_kv);
    const KVT *kb = kc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd;
    const float *qh = q + ((size_t)seq * n_head + h) * hd;
    float *sc = scores + ((size_t)seq * n_head + h) * max_kv;
    for (int i = tid; i < hd; i += blockDim.x) sq[i] = qh[i];
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const int hd4 = hd / 4, per_tile4 = kAttTile * hd4;
    const int n_tiles = (n_kv + kAttTile - 1) / kAttTile;
    constexpr int kMaxLd = 8;
    float4 reg[kMaxLd];
    auto fetch = [&](int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / hd4, cc = idx - r * hd4;
            const int t = ti * kAttTile + r;
            reg[j] = (idx < per_tile4 && t < n_kv) ? KvIo<KVT>::ld4(kb + (size_t)t * kv_dim + 4 * cc) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](float *dst) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            if (idx < per_tile4) {
                const int r = idx / hd4, cc = idx - r * hd4;
                float *p = dst + r * stride + 4 * cc;
                p[0] = reg[j].x; p[1] = reg[j].y; p[2] = reg[j].z; p[3] = reg[j].w;
            }
        }
    };
    if (c < n_tiles) fetch(c);
    int buf = 0;
    for (int ti = c; ti < n_tiles; ti += kSplitT, buf ^= 1) {
        float *cur = tile + buf * kAttTile * stride;
        stash(cur);
        __syncthreads();
        if (ti + kSplitT < n_tiles) fetch(ti + kSplitT);
        const int t = ti * kAttTile + tid;
        if (tid < kAttTile && t < n_kv) {
            const float *kr = cur + tid * stride;
            float dot = 0.0f;
            if ((hd & 15) == 0) {
                float pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(sq[i], kr[i]);
                for (int d0 = 0; d0 < hd; d0 += 16) {
                    const int dn = (d0 + 16 < hd) ? d0 + 16 : d0;
#pragma unroll
                    for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(sq[dn + i], kr[dn + i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) dot = __fadd_rn(dot, pa[i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) pa[i] = pb[i];
                }
            } else {
                for (int d = 0; d < hd; d++) dot = __fadd_rn(dot, __fmul_rn(sq[d], kr[d]));
            }
            sc[t] = __fmul_rn(dot, scale);
        }
    }
}

// attn_scores_kernel with the launch in front of it folded in (decode): QK-norm, RoPE and the K/V store of the token's
// own position (norm_rope_kernel). Every CTA of head h norms and ropes h's query itself (a 128-add chain, repeated by the
// kSplitT CTAs of the head); the CTA whose tiles contain the token's position does the same for the kv head's new key
// and scores it from shared memory instead of from the cache; of the query heads that share a kv head the first one's
// such CTA stores the K and V rows for later tokens (and for attn_out_kernel, which follows in the stream). The same
// operations on the same values as the two launches: with a binary16 cache the new key is scored as the cache will
// hold it, rounded.
template <class KVT>
__global__ void __launch_bounds__(256) attn_rope_scores_kernel(const float *__restrict__ q_raw, const float *__restrict__ wq,
                                                               const float *__restrict__ k_raw, const float *__restrict__ wk,
                                                               const float *__restrict__ v_raw, KVT *__restrict__ kc, KVT *__restrict__ vc,
                                                               float *__restrict__ scores, int n_head, int n_head_kv, int hd,
                                                               const int32_t *__restrict__ meta, int max_kv, int kv_stride,
                                                               const float *__restrict__ rope_tab, float eps, int flags) {
    extern __shared__ __align__(16) float sm[];
    const int stride = hd + 1, half = hd / 2;
    float *sq = sm;                 // [hd] the roped query
    float *tile = sm + hd;          // [2][kAttTile][stride]
    float *s_raw = tile + 2 * kAttTile * stride;  // [2][hd] raw q, raw k
    float *sk = s_raw + 2 * hd;     // [hd] the roped new key, as the cache holds it
    __shared__ float s_scale[2];
    pdl_trigger();
    // kPassEarlyLoads: the positions and the cached rows of earlier positions were complete before this pass began (its
    // first launch waits for everything in front of it), so they are read before the wait, while the projections that
    // produce q, k and v are still running.
    const bool early = (flags & kPassEarlyLoads) != 0;
    if (!early) pdl_wait();
    const int h = blockIdx.x, c = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
    const int pos = meta[2 * seq + 1], n_kv = pos + 1;
    const int ratio = n_head / n_head_kv, kv_dim = n_head_kv * hd, kvh = h / ratio;
    const int ti_pos = pos / kAttTile;
    const bool need_k = (ti_pos % kSplitT) == c;        // this CTA scores the new key
    const bool storer = need_k && (h % ratio) == 0;     // ... and writes the K and V rows of the position
    KVT *krow = kc + ((size_t)seq * kv_stride + pos) * kv_dim + (size_t)kvh * hd;
    KVT *vrow = vc + ((size_t)seq * kv_stride + pos) * kv_dim + (size_t)kvh * hd;
    const KVT *kb = kc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd;
    float *sc = scores + ((size_t)seq * n_head + h) * max_kv;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const int hd4 = hd / 4, per_tile4 = kAttTile * hd4;
    const int n_tiles = (n_kv + kAttTile - 1) / kAttTile;
    constexpr int kMaxLd = 8;
    float4 reg[kMaxLd];
    auto fetch = [&](int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / hd4, cc = idx - r * hd4;
            const int t = ti * kAttTile + r;
            // (the token's own row is not in the cache yet: it comes from shared memory below)
            reg[j] = (idx < per_tile4 && t < pos) ? KvIo<KVT>::ld4(kb + (size_t)t * kv_dim + 4 * cc) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](float *dst, int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / hd4, cc = idx - r * hd4;
            if (idx < per_tile4 && ti * kAttTile + r != pos) {  // (the token's own row is written below, by other threads)
                float *p = dst + r * stride + 4 * cc;
                p[0] = reg[j].x; p[1] = reg[j].y; p[2] = reg[j].z; p[3] = reg[j].w;
            }
        }
    };
    if (c < n_tiles) fetch(c);  // the cached rows travel while the query is prepared
    // the norm weights and the rotation of this position do not depend on the launch in front either
    float w_lo = 1.0f, w_hi = 1.0f;
    float2 cs_r = make_float2(0.f, 1.f);
    {
        const int idx = tid;
        const bool is_k = idx >= half;
        const int i = is_k ? idx - half : idx;
        const float *w = is_k ? wk : wq;
        if (idx < 2 * half && idx < (int)blockDim.x) {
            if (w) {
                w_lo = __ldg(w + i);
                w_hi = __ldg(w + i + half);
            }
            cs_r = __ldg(reinterpret_cast<const float2 *>(rope_tab + ((size_t)pos * half + i) * 2));
        }
    }
    if (early) {
        // the CTA's later tiles: asked into L2 now, read from there in the loop below
        const int lpr = hd * (int)sizeof(KVT) / 128;  // 128-byte lines per cached row of this head
        if (lpr > 0)
            for (int ti = c + kSplitT; ti < n_tiles; ti += kSplitT)
                for (int i = tid; i < kAttTile * lpr; i += blockDim.x) {
                    const int r = i / lpr, l = i - r * lpr, t = ti * kAttTile + r;
                    if (t < pos) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(kb + (size_t)t * kv_dim) + l * 128));
                }
        pdl_wait();
    }
    // ---- QK-norm (crates/llamd-runtime/src/layer.rs:62-79) and RoPE (crates/llamd-cpu/src/lib.rs:158-209) ----
    const float *qh = q_raw + ((size_t)seq * n_head + h) * hd, *kh = k_raw + ((size_t)seq * n_head_kv + kvh) * hd;
    for (int i = tid; i < hd; i += blockDim.x) {
        s_raw[i] = qh[i];
        if (need_k) s_raw[hd + i] = kh[i];
    }
    __syncthreads();
    if ((tid == 0 && wq) || (tid == 32 && wk && need_k)) {  // each sum of squares walked in order, the two side by side
        const float *sx = s_raw + (tid ? hd : 0);
        float sum = 0.0f;
#pragma unroll 8
        for (int t = 0; t < hd; t++) sum = __fadd_rn(sum, __fmul_rn(sx[t], sx[t]));
        s_scale[tid ? 1 : 0] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)hd), eps)));
    }
    __syncthreads();
    for (int idx = tid; idx < (need_k ? 2 : 1) * half; idx += blockDim.x) {
        const bool is_k = idx >= half;
        const int i = is_k ? idx - half : idx;
        const float *sx = s_raw + (is_k ? hd : 0);
        const float *w = is_k ? wk : wq;
        const bool first = idx == tid;  // (the first round's weights and rotation are in registers)
        float a = sx[i], b = sx[i + half];
        if (w) {
            const float nsc = s_scale[is_k ? 1 : 0];
            a = __fmul_rn(__fmul_rn(a, nsc), first ? w_lo : w[i]);
            b = __fmul_rn(__fmul_rn(b, nsc), first ? w_hi : w[i + half]);
        }
        const float2 cs = first ? cs_r : *reinterpret_cast<const float2 *>(rope_tab + ((size_t)pos * half + i) * 2);
        const float o0 = __fsub_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x));
        const float o1 = __fadd_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
        if (!is_k) {
            sq[i] = o0;
            sq[i + half] = o1;
        } else {
            // as the cache holds it (a binary16 cache rounds here, once); the storer writes the rows
            KVT t0, t1;
            KvIo<KVT>::st(&t0, o0);
            KvIo<KVT>::st(&t1, o1);
            sk[i] = (float)t0;
            sk[i + half] = (float)t1;
            if (storer) {
                krow[i] = t0;
                krow[i + half] = t1;
                const float *vs = v_raw + ((size_t)seq * n_head_kv + kvh) * hd;
                KvIo<KVT>::st(vrow + i, vs[i]);
                KvIo<KVT>::st(vrow + i + half, vs[i + half]);
            }
        }
    }
    __syncthreads();
    // ---- scores, as attn_scores_kernel ----
    int buf = 0;
    for (int ti = c; ti < n_tiles; ti += kSplitT, buf ^= 1) {
        float *cur = tile + buf * kAttTile * stride;
        stash(cur, ti);
        if (ti == ti_pos)
            for (int i = tid; i < hd; i += blockDim.x) cur[(pos - ti * kAttTile) * stride + i] = sk[i];
        __syncthreads();
        if (ti + kSplitT < n_tiles) fetch(ti + kSplitT);
        const int t = ti * kAttTile + tid;
        if (tid < kAttTile && t < n_kv) {
            const float *kr = cur + tid * stride;
            float dot = 0.0f;
            if ((hd & 15) == 0) {
                float pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(sq[i], kr[i]);
                for (int d0 = 0; d0 < hd; d0 += 16) {
                    const int dn = (d0 + 16 < hd) ? d0 + 16 : d0;
#pragma unroll
                    for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(sq[dn + i], kr[dn + i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) dot = __fadd_rn(dot, pa[i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) pa[i] = pb[i];
                }
            } else {
                for (int d = 0; d < hd; d++) dot = __fadd_rn(dot, __fmul_rn(sq[d], kr[d]));
            }
            sc[t] = __fmul_rn(dot, scale);
        }
    }
}

constexpr int kPvTile = 256;  // positions per V tile

// With a TailPlan the CTA that finishes a sequence last also writes the Q8_K form of that sequence's whole
// attention output (what llamd_fwd_quantize would do one launch later).
template <class KVT>
__global__ void __launch_bounds__(256) attn_out_kernel(const float *__restrict__ scores, const KVT *__restrict__ vc, float *__restrict__ out,
                                                       int n_head, int n_head_kv, int hd, const int32_t *__restrict__ meta, int n_kv_imm,
                                                       int max_kv, int kv_stride, const TailPlan tail, int fast) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float s_red[16];
    __shared__ float s_tree[32];
    __shared__ float s_part[256];
    pdl_trigger();
    const bool clusters = !tail.counter && tail.qs;  // launched as clusters that quantize the result (below); uniform
    // (a CTA's shared memory may be written by its cluster only once it runs: every CTA says so here, and waits for the
    // others' word just before it writes theirs)
    if (clusters) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    const bool early = (fast & kPassEarlyLoads) != 0 && meta;  // (see attn_rope_scores_kernel)
    if (!early) pdl_wait();
    const int h = blockIdx.x, c = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
    const int n_kv = meta ? meta[2 * seq + 1] + 1 : n_kv_imm;
    const int n_kv_cap = meta ? max_kv : n_kv_imm;
    const int cols = hd / kSplit, cols4 = cols / 4;  // this CTA's output columns [c*cols, (c+1)*cols)
    float *sl = sm;                                  // [n_kv]
    float *tile = sm + ((n_kv_cap + 3) & ~3);        // [2][kPvTile][cols]
    const int kv_dim = n_head_kv * hd, kvh = h / (n_head / n_head_kv);
    const KVT *vb = vc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd + (size_t)c * cols;
    const float *sc = scores + ((size_t)seq * n_head + h) * max_kv;
    const int per_tile4 = kPvTile * cols4;
    const int n_tiles = (n_kv + kPvTile - 1) / kPvTile;
    constexpr int kMaxLd = 8;  // 256 rows x 32 cols / 4 / 256
    float4 reg[kMaxLd];
    auto fetch = [&](int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / cols4, cc = idx - r * cols4;
            const int t = ti * kPvTile + r;
            reg[j] = (idx < per_tile4 && t < n_kv) ? KvIo<KVT>::ld4(vb + (size_t)t * kv_dim + 4 * cc) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](float *dst) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            if (idx < per_tile4) reinterpret_cast<float4 *>(dst)[idx] = reg[j];
        }
    };
    if (early) {
        // this CTA's slice of every cached value row, asked into L2 while the scores are still being made (the row of the
        // token's own position is written by the launch in front: a hint for it is harmless, its load comes after the wait)
        for (int t = tid; t < n_kv; t += blockDim.x)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(vb + (size_t)t * kv_dim)));
        pdl_wait();
    }
    fetch(0);  // V tile 0 travels while the softmax runs
    float lmax = -INFINITY;
    for (int t = tid; t < n_kv; t += blockDim.x) {
        const float l = sc[t];
        sl[t] = l;
        lmax = fmaxf(lmax, l);
    }
    for (int off = 16; off > 0; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
    if ((tid & 31) == 0) s_red[tid >> 5] = lmax;
    __syncthreads();
    lmax = s_red[0];
    for (int w = 1; w < 8; w++) lmax = fmaxf(lmax, s_red[w]);
    for (int t = tid; t < n_kv; t += blockDim.x) sl[t] = ref_expf(__fsub_rn(sl[t], lmax));
    __syncthreads();
    float inv;
    if (fast & 4) {  // the `fast` arithmetic: the softmax sum as a reduction tree
        float part = 0.0f;
        for (int t = tid; t < n_kv; t += blockDim.x) part = __fadd_rn(part, sl[t]);
        inv = __fdiv_rn(1.0f, block_tree_sum(part, s_tree));
    } else {
        if (tid == 0) s_red[8] = __fdiv_rn(1.0f, chain_sum(sl, n_kv, 0.0f));
        __syncthreads();
        inv = s_red[8];
    }
    float acc = 0.0f;
    for (int ti = 0; ti < n_tiles; ti++) {
        float *cur = tile + (ti & 1) * kPvTile * cols;
        stash(cur);
        __syncthreads();
        if (ti + 1 < n_tiles) fetch(ti + 1);
        if (fast & 4) {
            // ... and the weighted values by 256 / cols groups of positions per column, joined in group order below
            const int t0 = ti * kPvTile, cnt = min(kPvTile, n_kv - t0);
            const int g = tid / cols, dcol = tid - g * cols, ng = 256 / cols;
            for (int r = g; r < cnt; r += ng) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(sl[t0 + r], inv), cur[r * cols + dcol]));
        } else if (tid < cols) {
            const int t0 = ti * kPvTile, cnt = min(kPvTile, n_kv - t0);
            int r = 0;
            if (cnt >= 16) {
                float pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(__fmul_rn(sl[t0 + i], inv), cur[i * cols + tid]);
                for (; r + 16 <= cnt; r += 16) {
                    const int rn = (r + 32 <= cnt) ? r + 16 : r;
#pragma unroll
                    for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(__fmul_rn(sl[t0 + rn + i], inv), cur[(rn + i) * cols + tid]);
#pragma unroll
                    for (int i = 0; i < 16; i++) acc = __fadd_rn(acc, pa[i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) pa[i] = pb[i];
                }
            }
            for (; r < cnt; r++) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(sl[t0 + r], inv), cur[r * cols + tid]));
        }
    }
    if (fast & 4) {
        s_part[tid] = acc;  // [group][column]
        __syncthreads();
        if (tid < cols) {
            acc = s_part[tid];
            for (int g = 1; g < 256 / cols; g++) acc = __fadd_rn(acc, s_part[g * cols + tid]);
        }
    }
    if (tid < cols) out[((size_t)seq * n_head + h) * hd + (size_t)c * cols + tid] = acc;
    if (clusters) {
        // Launched as clusters of the 256 / hd heads x kSplit column slices that make up one 256-element block of the
        // attention output (hd == 128, 32 columns per CTA: the block's eight 32-element runs, one per CTA): the Q8_K form
        // of the block (dot.rs:88-128) is made here, what llamd_fwd_quantize would do one launch later. Each CTA finds
        // the first largest magnitude of its run and leaves it, with its signed value, in every CTA's table at the run's
        // place; behind the cluster barrier each CTA walks the eight in element order and quantizes its own run.
        __shared__ float s_ca[8], s_cm[8];
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        const int e0 = (h * hd + c * cols) & 255;  // this run's place in its block
        const int run = e0 / cols;                 // 0..7
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");  // every CTA of the cluster has started
        if (tid < 32) {
            float amax = fabsf(acc), mx = acc;
            int idx = e0 + tid;
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
            if (tid < 8) {  // lane r writes CTA r's table
                *cluster.map_shared_rank(&s_ca[run], tid) = amax;
                *cluster.map_shared_rank(&s_cm[run], tid) = mx;
            }
        }
        cluster.sync();
        if (tid < 32) {
            float amax = 0.0f, mx = 0.0f;
#pragma unroll
            for (int r = 0; r < 8; r++)
                if (s_ca[r] > amax) {  // (runs in element order: an equal magnitude later in the block does not replace)
                    amax = s_ca[r];
                    mx = s_cm[r];
                }
            int q = 0;
            float dd = 0.0f;
            if (amax != 0.0f) {
                const float iscale = __fdiv_rn(-127.0f, mx);
                q = min(127, __float2int_rn(__fmul_rn(iscale, acc)));
                dd = __fdiv_rn(1.0f, iscale);
            }
            // four lanes' bytes into one word
            uint32_t w = (uint32_t)q & 0xFFu;
            w |= __shfl_down_sync(0xffffffffu, w, 1) << 8;
            w |= __shfl_down_sync(0xffffffffu, w, 2) << 16;
            const size_t blk = ((size_t)seq * n_head * hd + (size_t)h * hd + (size_t)c * cols) >> 8;
            if ((tid & 3) == 0) *reinterpret_cast<uint32_t *>(tail.qs + blk * 256 + e0 + tid) = w;
            if (run == 0 && tid == 0) tail.d[blk] = dd;
        }
    }
    if (tail.counter) {  // uniform over the launch
        __shared__ bool s_last;
        const unsigned per_seq = gridDim.x * gridDim.y;
        __threadfence();  // this CTA's columns are visible before its arrival is
        __syncthreads();
        if (tid == 0) s_last = atomicInc(tail.counter + seq, per_seq - 1) == per_seq - 1;  // wraps to 0
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int n = n_head * hd, nblk = n >> 8, lane = tid & 31;
            for (int blk = tid >> 5; blk < nblk; blk += 8) {
                const float *src = out + (size_t)seq * n + (size_t)blk * 256 + lane * 8;
                const float4 a = __ldcg(reinterpret_cast<const float4 *>(src)), b = __ldcg(reinterpret_cast<const float4 *>(src + 4));
                float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                q8k_quantize_block(v, lane, tail.qs + ((size_t)seq * nblk + blk) * 256, tail.d + (size_t)seq * nblk + blk, nullptr);
            }
        }
    }
}

// ---- the same two launches for a batch of sequences -----------------------------------------------------------------
// With several sequences per pass the grids above are many small CTAs in which a quarter (scores) or an eighth (values) of
// the threads walk chains while the rest wait, several waves of them. Here a CTA serves ALL the query heads that share
// a kv head: the cached tile is read once for them instead of once each, every thread has a chain to walk, and the grid is
// one wave. The same operations on the same values in the same order per (head, position) and per (head, column), hence
// the same bits as the per-head kernels.
constexpr int kGqaMax = 8;  // query heads per kv head these kernels hold

template <class KVT>
__global__ void __launch_bounds__(256) attn_rope_scores_gqa_kernel(const float *__restrict__ q_raw, const float *__restrict__ wq,
                                                                   const float *__restrict__ k_raw, const float *__restrict__ wk,
                                                                   const float *__restrict__ v_raw, KVT *__restrict__ kc, KVT *__restrict__ vc,
                                                                   float *__restrict__ scores, int n_head, int n_head_kv, int hd,
                                                                   const int32_t *__restrict__ meta, int max_kv, int kv_stride,
                                                                   const float *__restrict__ rope_tab, float eps, int flags) {
    extern __shared__ __align__(16) float sm[];
    const int stride = hd + 1, half = hd / 2, ratio = n_head / n_head_kv;
    float *sq = sm;                               // [ratio][hd] the roped queries
    float *tile = sq + ratio * hd;                // [2][kAttTile][stride]
    float *s_raw = tile + 2 * kAttTile * stride;  // [ratio + 1][hd] raw queries, raw key
    float *sk = s_raw + (ratio + 1) * hd;         // [hd] the roped new key, as the cache holds it
    __shared__ float s_scale[kGqaMax + 1];
    pdl_trigger();
    const bool early = (flags & kPassEarlyLoads) != 0;  // (see attn_rope_scores_kernel)
    if (!early) pdl_wait();
    const int kvh = blockIdx.x, c = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
    const int pos = meta[2 * seq + 1], n_kv = pos + 1;
    const int kv_dim = n_head_kv * hd, h0 = kvh * ratio;
    const int ti_pos = pos / kAttTile;
    const bool need_k = (ti_pos % kSplitT) == c;  // this CTA scores the new key, and stores the K and V rows of the position
    KVT *krow = kc + ((size_t)seq * kv_stride + pos) * kv_dim + (size_t)kvh * hd;
    KVT *vrow = vc + ((size_t)seq * kv_stride + pos) * kv_dim + (size_t)kvh * hd;
    const KVT *kb = kc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd;
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    const int hd4 = hd / 4, per_tile4 = kAttTile * hd4;
    const int n_tiles = (n_kv + kAttTile - 1) / kAttTile;
    constexpr int kMaxLd = 8;
    float4 reg[kMaxLd];
    auto fetch = [&](int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / hd4, cc = idx - r * hd4;
            const int t = ti * kAttTile + r;
            reg[j] = (idx < per_tile4 && t < pos) ? KvIo<KVT>::ld4(kb + (size_t)t * kv_dim + 4 * cc) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](float *dst, int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / hd4, cc = idx - r * hd4;
            if (idx < per_tile4 && ti * kAttTile + r != pos) {  // (the token's own row is written below, by other threads)
                float *p = dst + r * stride + 4 * cc;
                p[0] = reg[j].x; p[1] = reg[j].y; p[2] = reg[j].z; p[3] = reg[j].w;
            }
        }
    };
    if (c < n_tiles) fetch(c);
    if (early) {
        const int lpr = hd * (int)sizeof(KVT) / 128;
        if (lpr > 0)
            for (int ti = c + kSplitT; ti < n_tiles; ti += kSplitT)
                for (int i = tid; i < kAttTile * lpr; i += blockDim.x) {
                    const int r = i / lpr, l = i - r * lpr, t = ti * kAttTile + r;
                    if (t < pos) asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(kb + (size_t)t * kv_dim) + l * 128));
                }
        pdl_wait();
    }
    // ---- QK-norm (crates/llamd-runtime/src/layer.rs:62-79) and RoPE (crates/llamd-cpu/src/lib.rs:158-209) of the kv head's
    // query heads (adjacent in q_raw) and, where needed, of the new key
    const int n_vec = ratio + (need_k ? 1 : 0);
    for (int i = tid; i < ratio * hd; i += blockDim.x) s_raw[i] = q_raw[((size_t)seq * n_head + h0) * hd + i];
    if (need_k)
        for (int i = tid; i < hd; i += blockDim.x) s_raw[ratio * hd + i] = k_raw[((size_t)seq * n_head_kv + kvh) * hd + i];
    __syncthreads();
    {
        // vector v's sum of squares is walked in order by lane v / 8 of warp v % 8: the chains run side by side
        const int warp = tid >> 5, lane = tid & 31, v = lane * 8 + warp;
        if (lane < 2 && v < n_vec && (v < ratio ? wq != nullptr : wk != nullptr)) {
            const float *sx = s_raw + v * hd;
            float sum = 0.0f;
#pragma unroll 8
            for (int t = 0; t < hd; t++) sum = __fadd_rn(sum, __fmul_rn(sx[t], sx[t]));
            s_scale[v] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)hd), eps)));
        }
    }
    __syncthreads();
    for (int idx = tid; idx < n_vec * half; idx += blockDim.x) {
        const int v = idx / half, i = idx - v * half;
        const bool is_k = v == ratio;
        const float *sx = s_raw + v * hd;
        const float *w = is_k ? wk : wq;
        float a = sx[i], b = sx[i + half];
        if (w) {
            const float nsc = s_scale[v];
            a = __fmul_rn(__fmul_rn(a, nsc), w[i]);
            b = __fmul_rn(__fmul_rn(b, nsc), w[i + half]);
        }
        const float2 cs = *reinterpret_cast<const float2 *>(rope_tab + ((size_t)pos * half + i) * 2);
        const float o0 = __fsub_rn(__fmul_rn(a, cs.y), __fmul_rn(b, cs.x));
        const float o1 = __fadd_rn(__fmul_rn(a, cs.x), __fmul_rn(b, cs.y));
        if (!is_k) {
            sq[v * hd + i] = o0;
            sq[v * hd + i + half] = o1;
        } else {
            KVT t0, t1;  // as the cache holds it (a binary16 cache rounds here, once)
            KvIo<KVT>::st(&t0, o0);
            KvIo<KVT>::st(&t1, o1);
            sk[i] = (float)t0;
            sk[i + half] = (float)t1;
            krow[i] = t0;
            krow[i + half] = t1;
            const float *vs = v_raw + ((size_t)seq * n_head_kv + kvh) * hd;
            KvIo<KVT>::st(vrow + i, vs[i]);
            KvIo<KVT>::st(vrow + i + half, vs[i + half]);
        }
    }
    __syncthreads();
    // ---- scores: (query head, position) pairs of the tile over the threads ----
    int buf = 0;
    for (int ti = c; ti < n_tiles; ti += kSplitT, buf ^= 1) {
        float *cur = tile + buf * kAttTile * stride;
        stash(cur, ti);
        if (ti == ti_pos)
            for (int i = tid; i < hd; i += blockDim.x) cur[(pos - ti * kAttTile) * stride + i] = sk[i];
        __syncthreads();
        if (ti + kSplitT < n_tiles) fetch(ti + kSplitT);
        for (int idx = tid; idx < ratio * kAttTile; idx += blockDim.x) {
            const int j = idx / kAttTile, r = idx - j * kAttTile;
            const int t = ti * kAttTile + r;
            if (t >= n_kv) continue;
            const float *kr = cur + r * stride, *q = sq + j * hd;
            float dot = 0.0f;
            if ((hd & 15) == 0) {
                float pa[16], pb[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(q[i], kr[i]);
                for (int d0 = 0; d0 < hd; d0 += 16) {
                    const int dn = (d0 + 16 < hd) ? d0 + 16 : d0;
#pragma unroll
                    for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(q[dn + i], kr[dn + i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) dot = __fadd_rn(dot, pa[i]);
#pragma unroll
                    for (int i = 0; i < 16; i++) pa[i] = pb[i];
                }
            } else {
                for (int d = 0; d < hd; d++) dot = __fadd_rn(dot, __fmul_rn(q[d], kr[d]));
            }
            scores[((size_t)seq * n_head + h0 + j) * max_kv + t] = __fmul_rn(dot, scale);
        }
    }
}

// Softmax and weighted values for the query heads of one kv head: warp j is head j (ratio * hd / kSplit == 256 threads).
template <class KVT>
__global__ void __launch_bounds__(256) attn_out_gqa_kernel(const float *__restrict__ scores, const KVT *__restrict__ vc, float *__restrict__ out,
                                                           int n_head, int n_head_kv, int hd, const int32_t *__restrict__ meta, int max_kv,
                                                           int kv_stride, int flags) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float s_inv[kGqaMax];
    pdl_trigger();
    const bool early = (flags & kPassEarlyLoads) != 0;
    if (!early) pdl_wait();
    const int kvh = blockIdx.x, c = blockIdx.y, seq = blockIdx.z, tid = threadIdx.x;
    const int ratio = n_head / n_head_kv, h0 = kvh * ratio;
    const int n_kv = meta[2 * seq + 1] + 1, cap = (max_kv + 3) & ~3;
    const int cols = hd / kSplit, cols4 = cols / 4;
    float *sl = sm;                 // [ratio][cap]
    float *tile = sm + ratio * cap;  // [2][kPvTile][cols]
    const int kv_dim = n_head_kv * hd;
    const KVT *vb = vc + (size_t)seq * kv_stride * kv_dim + (size_t)kvh * hd + (size_t)c * cols;
    const int per_tile4 = kPvTile * cols4;
    const int n_tiles = (n_kv + kPvTile - 1) / kPvTile;
    constexpr int kMaxLd = 8;
    float4 reg[kMaxLd];
    auto fetch = [&](int ti) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            const int r = idx / cols4, cc = idx - r * cols4;
            const int t = ti * kPvTile + r;
            reg[j] = (idx < per_tile4 && t < n_kv) ? KvIo<KVT>::ld4(vb + (size_t)t * kv_dim + 4 * cc) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto stash = [&](float *dst) {
#pragma unroll
        for (int j = 0; j < kMaxLd; j++) {
            const int idx = tid + j * 256;
            if (idx < per_tile4) reinterpret_cast<float4 *>(dst)[idx] = reg[j];
        }
    };
    if (early) {
        for (int t = tid; t < n_kv; t += blockDim.x)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const char *>(vb + (size_t)t * kv_dim)));
        pdl_wait();
    }
    fetch(0);
    const int j = tid >> 5, lane = tid & 31;  // (ratio == 8 warps: warp j is query head h0 + j)
    {
        const float *sc = scores + ((size_t)seq * n_head + h0 + j) * max_kv;
        float *slj = sl + (size_t)j * cap;
        float lmax = -INFINITY;
        for (int t = lane; t < n_kv; t += 32) {
            const float l = sc[t];
            slj[t] = l;
            lmax = fmaxf(lmax, l);
        }
        for (int off = 16; off > 0; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
        for (int t = lane; t < n_kv; t += 32) slj[t] = ref_expf(__fsub_rn(slj[t], lmax));
        __syncwarp();
        if (lane == 0) s_inv[j] = __fdiv_rn(1.0f, chain_sum(slj, n_kv, 0.0f));
    }
    __syncthreads();
    const float inv = s_inv[j];
    const float *slj = sl + (size_t)j * cap;
    float acc = 0.0f;
    for (int ti = 0; ti < n_tiles; ti++) {
        float *cur = tile + (ti & 1) * kPvTile * cols;
        stash(cur);
        __syncthreads();
        if (ti + 1 < n_tiles) fetch(ti + 1);
        const int t0 = ti * kPvTile, cnt = min(kPvTile, n_kv - t0);
        int r = 0;
        if (cnt >= 16) {
            float pa[16], pb[16];
#pragma unroll
            for (int i = 0; i < 16; i++) pa[i] = __fmul_rn(__fmul_rn(slj[t0 + i], inv), cur[i * cols + lane]);
            for (; r + 16 <= cnt; r += 16) {
                const int rn = (r + 32 <= cnt) ? r + 16 : r;
#pragma unroll
                for (int i = 0; i < 16; i++) pb[i] = __fmul_rn(__fmul_rn(slj[t0 + rn + i], inv), cur[(rn + i) * cols + lane]);
#pragma unroll
                for (int i = 0; i < 16; i++) acc = __fadd_rn(acc, pa[i]);
#pragma unroll
                for (int i = 0; i < 16; i++) pa[i] = pb[i];
            }
        }
        for (; r < cnt; r++) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(slj[t0 + r], inv), cur[r * cols + lane]));
    }
    out[((size_t)seq * n_head + h0 + j) * hd + (size_t)c * cols + lane] = acc;
}

// The attention-output launch with a cluster per 256-element block of its result (attn_out_kernel's quantizing tail).
template <class KVT>
static void attn_out_cluster_launch(size_t smem, const float *scores, const KVT *vc, float *out, int n_head, int n_head_kv, int hd,
                                    const int32_t *meta, int max_kv, int nseq, int8_t *qs, float *d, int flags) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_head, kSplit, nseq);
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 256 / hd;
    attr[0].val.clusterDim.y = kSplit;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_pdl & PDL_ATTN) ? 2 : 1;
    g_launches++;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, attn_out_kernel<KVT>, scores, vc, out, n_head, n_head_kv, hd, meta, 0, max_kv, max_kv,
                                             TailPlan{nullptr, qs, d}, flags);
    if (e != cudaSuccess) set_error(e, "attn_out (clusters)");
}
// whether the attention output can leave its launch quantized: one cluster = one block
static bool attn_out_cluster_ok(int n_head, int hd) {
    return hd == 128 && hd / kSplit == 32 && (256 / hd) * kSplit <= 8 && n_head % (256 / hd) == 0;
}

// order[] = the slots sorted by (expert id, slot): every slot counts the slots that come before it (a few hundred slots:
// one CTA, no scratch memory).
__global__ void __launch_bounds__(256) slot_order_kernel(const int32_t *__restrict__ ids, int n_slots, int32_t *__restrict__ order) {
    extern __shared__ int32_t s_ids[];
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) s_ids[i] = ids[i];
    __syncthreads();
    for (int i = threadIdx.x; i < n_slots; i += blockDim.x) {
        const int mine = s_ids[i];
        int rank = 0;
        for (int j = 0; j < n_slots; j++) {
            const int o = s_ids[j];
            rank += (o < mine || (o == mine && j < i)) ? 1 : 0;
        }
        order[rank] = i;
    }
}

// ---- argmax, lowest index on a tie (llamd_forward.hip:353-389) -------------
__device__ __forceinline__ void argmax_combine(float &v, int &i, float ov, int oi) {
    if (ov > v || (ov == v && oi < i)) {
        v = ov;
        i = oi;
    }
}
__global__ void argmax_partial_kernel(const float *__restrict__ x, int n, float *__restrict__ pv, int32_t *__restrict__ pi) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    x += (size_t)seq * n;
    float v = -INFINITY;
    int ix = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) argmax_combine(v, ix, x[i], i);
    __shared__ float sv[32];
    __shared__ int si[32];
    for (int off = 16; off > 0; off >>= 1) argmax_combine(v, ix, __shfl_xor_sync(0xffffffffu, v, off), __shfl_xor_sync(0xffffffffu, ix, off));
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = v;
        si[threadIdx.x >> 5] = ix;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) argmax_combine(v, ix, sv[w], si[w]);
        pv[(size_t)seq * gridDim.x + blockIdx.x] = v;
        pi[(size_t)seq * gridDim.x + blockIdx.x] = ix;
    }
}
__global__ void argmax_final_kernel(const float *__restrict__ pv, const int32_t *__restrict__ pi, int nblocks, int32_t *__restrict__ out) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x;
    float v = -INFINITY;
    int ix = 0x7fffffff;
    for (int i = threadIdx.x; i < nblocks; i += blockDim.x) argmax_combine(v, ix, pv[(size_t)seq * nblocks + i], pi[(size_t)seq * nblocks + i]);
    __shared__ float sv[32];
    __shared__ int si[32];
    for (int off = 16; off > 0; off >>= 1) argmax_combine(v, ix, __shfl_xor_sync(0xffffffffu, v, off), __shfl_xor_sync(0xffffffffu, ix, off));
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = v;
        si[threadIdx.x >> 5] = ix;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); w++) argmax_combine(v, ix, sv[w], si[w]);
        out[seq] = ix == 0x7fffffff ? 0 : ix;
    }
}

// ---- expert scatter plan (crates/llamd-vulkan/shaders/moe_group.comp:40-82) --
// Counting sort of the (token, slot) pairs by expert, stable: pairs of one
// expert come out in ascending pair order (the shader leaves that order
// unspecified; a fixed order makes runs reproducible).
// One CTA of 32 warps. Warp w owns the contiguous pairs [w*chunk, (w+1)*chunk):
// it histograms them by expert into its own row of s_hist, each pair keeping
// its rank among the warp's earlier pairs of the same expert (match_any finds
// the lanes of a 32-pair step that share an expert). A scan over (expert, warp)
// turns the counts into output positions.
// Also emits the work list the expert-major matvec walks: entries of up to 8
// pairs of one expert, (expert, first, count), and their number.
constexpr int kGroupMaxPerLane = 40;  // pairs per lane: 32 warps x 32 lanes x 40 = 40960 pairs
// Pairs whose expert lies outside [own_lo, own_hi) are left out of the plan (expert parallelism: they belong to
// another GPU; an id outside the tensor is left out the same way).
__global__ void __launch_bounds__(1024) moe_group_kernel(const int32_t *__restrict__ ids, int n_expert, int npair, int n_used,
                                                         int32_t *__restrict__ gstart, int32_t *__restrict__ gcount,
                                                         int32_t *__restrict__ ptoken, int32_t *__restrict__ pslot, int32_t *__restrict__ work,
                                                         int32_t *__restrict__ n_work, int own_lo, int own_hi) {
    extern __shared__ int s_hist[];  // [32 warps][n_expert]
    __shared__ int s_count[1024];
    __shared__ int s_start[1024];
    __shared__ int s_wstart[1024];
    __shared__ int s_warp_tot[32], s_warp_wtot[32];
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < 32 * n_expert; i += 1024) s_hist[i] = 0;
    __syncthreads();
    const int chunk = ((npair + 32 * 32 - 1) / (32 * 32)) * 32;  // pairs per warp, a multiple of 32
    const int steps = chunk / 32;
    int *hist = s_hist + warp * n_expert;
    int my_rank[kGroupMaxPerLane];  // rank << 10 | expert
#pragma unroll
    for (int s = 0; s < kGroupMaxPerLane; s++) {
        if (s < steps) {
            const int p = warp * chunk + s * 32 + lane;
            int e = p < npair ? ids[p] : -1;
            const bool live = e >= own_lo && e < own_hi;
            if (!live) e = -1 - lane;  // dead lanes match nobody
            const unsigned same = __match_any_sync(0xffffffffu, e);
            const int before = __popc(same & ((1u << lane) - 1u));
            int base = 0;
            if (live) base = hist[e];
            __syncwarp();
            if (live && before == 0) hist[e] = base + __popc(same);
            __syncwarp();
            my_rank[s] = live ? (((base + before) << 10) | (e & 1023)) : -1;
        }
    }
    __syncthreads();
    // expert e: total, then its start among all experts, then each warp's first position
    int total = 0;
    for (int e = tid; e < n_expert; e += 1024) {  // n_expert <= 1024: at most one expert per thread
        for (int w = 0; w < 32; w++) total += s_hist[w * n_expert + e];
        s_count[e] = total;
    }
    int incl = total, wincl = (total + 7) / 8;
    for (int off = 1; off < 32; off <<= 1) {
        const int a = __shfl_up_sync(0xffffffffu, incl, off), b = __shfl_up_sync(0xffffffffu, wincl, off);
        if (lane >= off) {
            incl += a;
            wincl += b;
        }
    }
    if (lane == 31) {
        s_warp_tot[warp] = incl;
        s_warp_wtot[warp] = wincl;
    }
    __syncthreads();
    int run = 0, wrun = 0;
    for (int w = 0; w < warp; w++) {
        run += s_warp_tot[w];
        wrun += s_warp_wtot[w];
    }
    if (tid < n_expert) {
        const int start = run + incl - total, wstart = wrun + wincl - (total + 7) / 8;
        s_start[tid] = start;
        s_wstart[tid] = wstart;
        int at = start;
        for (int w = 0; w < 32; w++) {
            const int c = s_hist[w * n_expert + tid];
            s_hist[w * n_expert + tid] = at;
            at += c;
        }
        gstart[tid] = start;
        gcount[tid] = total;
    }
    if (tid == 1023 && n_work) *n_work = wrun + wincl;  // threads beyond n_expert carry zero totals
    __syncthreads();
#pragma unroll
    for (int s = 0; s < kGroupMaxPerLane; s++) {
        if (s < steps) {
            const int p = warp * chunk + s * 32 + lane;
            if (my_rank[s] >= 0) {
                const int dst = hist[my_rank[s] & 1023] + (my_rank[s] >> 10);
                ptoken[dst] = p / n_used;
                pslot[dst] = p;
            }
        }
    }
    if (work) {
        for (int e = warp; e < n_expert; e += 32) {
            const int start = s_start[e], count = s_count[e], wi0 = s_wstart[e];
            for (int f = lane * 8; f < count; f += 256) {
                const int wi = wi0 + f / 8;
                work[3 * wi + 0] = e;
                work[3 * wi + 1] = start + f;
                work[3 * wi + 2] = min(8, count - f);
            }
        }
    }
}

}  // namespace llamd

using namespace llamd;

extern "C" {

void llamd_fwd_matvec_f32_batch(const float *w, const float *x, float *out, int k, int rows, int nseq) {
    const size_t smem = (size_t)4 * k * sizeof(float);
    if (k % 4 || smem > 200 * 1024) {
        set_error_msg("matvec_f32: k must be a multiple of 4 and at most 12800");
        return;
    }
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaFuncSetAttribute(matvec_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = smem;
    }
    launch_k("matvec_f32", matvec_f32_kernel, dim3((rows + 3) / 4, nseq), dim3(128), smem, w, x, out, k, rows);
}
void llamd_fwd_matvec_f32(const float *w, const float *x, float *out, int k, int rows) {
    llamd_fwd_matvec_f32_batch(w, x, out, k, rows, 1);
}

void llamd_fwd_router(const float *logits, int n_expert, int n_used, int32_t *ids, float *weights, float *probs, int nseq) {
    if (n_expert < 1 || n_expert > 1024 || n_used < 1 || n_used > n_expert || n_used > kMaxUsed) {
        set_error_msg("router: n_expert must be 1..1024 and n_used 1..min(n_expert,64)");
        return;
    }
    const int threads = ((n_expert + 31) / 32) * 32;
    launch_k("router", router_kernel, dim3(nseq), dim3(threads), n_expert * sizeof(float), logits, n_expert, n_used, ids, weights, probs);
}
// The router's f32 matvec (forward.rs:340) and routing (:317) in one launch.
// w is [n_expert][k] as uploaded; `counter` is nseq zero-initialised words the
// kernel leaves at zero again.
void llamd_fwd_router_matvec(const float *w, const float *x, int k, int n_expert, int n_used, float *logits, int32_t *ids,
                             float *weights, float *probs, unsigned int *counter, int nseq) {
    if (n_expert < 1 || n_expert > 1024 || n_used < 1 || n_used > n_expert || n_used > kMaxUsed || k % 4 || !logits || !counter) {
        set_error_msg("router: n_expert must be 1..1024, n_used 1..min(n_expert,64), k a multiple of 4, logits and counter given");
        return;
    }
    const size_t smem = (size_t)4 * k * sizeof(float);
    if (smem > 200 * 1024 || (size_t)n_expert * sizeof(float) > smem) {
        set_error_msg("router: k too large (or smaller than n_expert/4) for the shared-memory staging");
        return;
    }
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaFuncSetAttribute(router_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = smem;
    }
    launch_kc(PDL_ROUTER, "router_matvec", router_rows_kernel, dim3((n_expert + 3) / 4, nseq), dim3(128), smem, w, x, k, n_expert, n_used, logits, ids,
             weights, probs, counter);
}

// The FFN norm fused in front (see norm_router_kernel). x_out: the new residual stream, a buffer other than x / residual.
void llamd_fwd_norm_router(const float *w, const float *x, const float *residual, float *x_out, const float *w_norm, float *xn_out,
                           int8_t *qs, float *d, int k, float eps, int n_expert, int n_used, float *logits, int32_t *ids, float *weights,
                           float *probs, unsigned int *counter, int nseq) {
    norm_router_flags(w, x, residual, x_out, w_norm, xn_out, qs, d, k, eps, n_expert, n_used, logits, ids, weights, probs, counter, nseq, 0);
}
}  // extern "C"
// (flags: what a model's decode pass asks of the kernel, see kPass... in common.cuh; 0 = the exact arithmetic)
void llamd::norm_router_flags(const float *w, const float *x, const float *residual, float *x_out, const float *w_norm, float *xn_out,
                              int8_t *qs, float *d, int k, float eps, int n_expert, int n_used, float *logits, int32_t *ids, float *weights,
                              float *probs, unsigned int *counter, int nseq, int flags) {
    const size_t smem = (size_t)6 * k * sizeof(float);
    if (k % 256 || n_expert < 1 || n_used < 1 || n_used > kMaxUsed || n_used > n_expert || (size_t)4 * k < (size_t)n_expert || smem > 200 * 1024 ||
        x_out == x || x_out == residual) {
        set_error_msg("norm_router: k a multiple of 256 that fits shared memory, 1 <= n_used <= n_expert <= 4k, x_out a buffer of its own");
        return;
    }
    static size_t configured = 0;
    if (smem > 44 * 1024 && smem > configured) {
        const cudaError_t e = cudaFuncSetAttribute(norm_router_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error(e, "norm_router smem attribute");
            return;
        }
        configured = smem;
    }
    launch_kc(PDL_ROUTER, "norm_router", norm_router_kernel, dim3((n_expert + 3) / 4, nseq), dim3(128), smem, w, x, residual, x_out, w_norm, xn_out, qs, d,
              k, eps, n_expert, n_used, logits, ids, weights, probs, counter, flags);
}
extern "C" {

static int g_q80_rows_max_ctas = 148 * 4;
static int *g_q80_status = nullptr;
static int *q80_status_word() {
    if (!g_q80_status) {
        if (cudaMalloc(&g_q80_status, sizeof(int)) != cudaSuccess || cudaMemsetAsync(g_q80_status, 0, sizeof(int), stream()) != cudaSuccess) {
            cudaGetLastError();
            g_q80_status = nullptr;
        }
    }
    return g_q80_status;
}
// 0 while every bulk copy of the Q8_0 matvec has arrived within its limit; otherwise 1 + the CTA whose wait ran out (its
// 32 rows were not written). Synchronises the stream.
int llamd_fwd_matvec_q8_0_status(void) {
    if (!g_q80_status) return 0;
    int h = 0;
    if (cudaMemcpyAsync(&h, g_q80_status, sizeof(int), cudaMemcpyDeviceToHost, stream()) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(stream()) != cudaSuccess) return -1;
    return h;
}
void llamd_fwd_matvec_q8_0(const void *w, const float *x, float *out, int blocks32, int rows, int nseq) {
    const size_t smem = (size_t)nseq * blocks32 * 32 * sizeof(float);
    if (nseq < 1 || nseq > LLAMD_MAX_SEQ || smem > 200 * 1024 || rows <= 0 || blocks32 <= 0) {
        set_error_msg("matvec_q8_0: nseq 1..8, rows and blocks positive, nseq*k*4 <= 200 KiB");
        return;
    }
    const uint8_t *t = (const uint8_t *)w;
    // the CTA-per-32-rows form needs 64 KiB of staged weights beside the activations; the thread-per-row form takes the rest
    const size_t smem_rows = smem + 2 * kQ80ChunkBlocks * 32 * 32 * sizeof(float);
    // measured: it wins while its CTAs fit one wave (attn_q 40 -> 10s of us); beyond that the thread-per-row form's
    // deeper occupancy does (lm_head)
    const bool by_rows = smem_rows <= 220 * 1024 && (rows + 31) / 32 <= g_q80_rows_max_ctas;
    // ... and with the CTA's whole slice of the matrix brought in by bulk copies, where that fits beside the rest
    const size_t smem_bulk = smem_rows + (size_t)blocks32 * kQ80TileBytes;
    const bool by_bulk = by_rows && smem_bulk <= 226 * 1024 && (blocks32 + kQ80ChunkBlocks - 1) / kQ80ChunkBlocks <= kQ80MaxChunks &&
                         ((uintptr_t)w & 15) == 0 && q80_status_word() != nullptr;
    const dim3 grid(by_rows ? (rows + 31) / 32 : (rows + 127) / 128);
#define Q80_CASE(N)                                                                                                   \
    case N: {                                                                                                          \
        static size_t configured = 0, configured_rows = 0;                                                             \
        if (by_bulk) {                                                                                                 \
            static size_t configured_bulk = 0;                                                                         \
            if (smem_bulk > configured_bulk) {                                                                         \
                if (cudaFuncSetAttribute(matvec_q8_0_bulk_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bulk) != cudaSuccess) { \
                    set_error_msg("matvec_q8_0: shared memory attribute");                                             \
                    return;                                                                                            \
                }                                                                                                      \
                configured_bulk = smem_bulk;                                                                           \
            }                                                                                                          \
            launch_kc(PDL_OTHER, "matvec_q8_0_bulk", matvec_q8_0_bulk_kernel<N>, grid, dim3(kQ80Producers + 32 * N), smem_bulk, t, x, out, blocks32, rows, q80_status_word()); \
            break;                                                                                                     \
        }                                                                                                              \
        if (by_rows) {                                                                                                 \
            if (smem_rows > configured_rows) {                                                                         \
                cudaFuncSetAttribute(matvec_q8_0_rows_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows); \
                configured_rows = smem_rows;                                                                           \
            }                                                                                                          \
            launch_k("matvec_q8_0_rows", matvec_q8_0_rows_kernel<N>, grid, dim3(kQ80Producers + 32 * N), smem_rows, t, x, out, blocks32, rows); \
            break;                                                                                                     \
        }                                                                                                              \
        if (smem > 48 * 1024 && smem > configured) {                                                                   \
            cudaFuncSetAttribute(matvec_q8_0_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
            configured = smem;                                                                                         \
        }                                                                                                              \
        launch_k("matvec_q8_0", matvec_q8_0_kernel<N>, grid, dim3(128), smem, t, x, out, blocks32, rows);                \
    } break;
    switch (nseq) {
        Q80_CASE(1) Q80_CASE(2) Q80_CASE(3) Q80_CASE(4) Q80_CASE(5) Q80_CASE(6) Q80_CASE(7) Q80_CASE(8)
    }
#undef Q80_CASE

}

// sin/cos for every (pos, i), computed with the host libm exactly as the
// reference's CPU rope does (crates/llamd-cpu/src/lib.rs:196-200).
int llamd_cuda_rope_table(float *host_out, int max_pos, int hd, float freq_base) {
    if (!host_out || max_pos <= 0 || hd <= 0 || hd % 2) return -1;
    const int half = hd / 2;
    for (int p = 0; p < max_pos; p++) {
        const float pos = (float)(uint32_t)p * 1.0f;
        for (int i = 0; i < half; i++) {
            const float exponent = 2.0f * (float)i / (float)hd;
            const float theta = pos / powf(freq_base, exponent);
            host_out[((size_t)p * half + i) * 2 + 0] = sinf(theta);
            host_out[((size_t)p * half + i) * 2 + 1] = cosf(theta);
        }
    }
    return 0;
}

void llamd_fwd_rope(float *x, int pos, int n_head, int hd, const float *rope_tab) {
    launch_k("rope", norm_rope_kernel<float>, dim3(n_head, 1), dim3(hd / 2), hd * sizeof(float), x, nullptr, nullptr, nullptr, nullptr, nullptr,
             nullptr, n_head, 0, hd, nullptr, pos, rope_tab, 0.0f, 0);
}
void llamd_fwd_norm_rope(float *x, const float *w, int n_head, int hd, const int32_t *meta, const float *rope_tab, float eps, int nseq) {
    launch_k("norm_rope", norm_rope_kernel<float>, dim3(n_head, nseq), dim3(hd / 2), hd * sizeof(float), x, w, nullptr, nullptr, nullptr, nullptr,
             nullptr, n_head, 0, hd, meta, 0, rope_tab, eps, 0);
}
void llamd_fwd_k_norm_rope_store(float *k, const float *w, const float *v, float *kc, float *vc, int n_head_kv, int hd, int kv_dim,
                                 const int32_t *meta, const float *rope_tab, float eps, int nseq, int max_kv) {
    if (kv_dim != n_head_kv * hd) {
        set_error_msg("k_norm_rope_store: kv_dim != n_head_kv*hd");
        return;
    }
    launch_k("k_norm_rope_store", norm_rope_kernel<float>, dim3(n_head_kv, nseq), dim3(hd / 2), hd * sizeof(float), nullptr, nullptr, k, w, v, kc,
             vc, 0, n_head_kv, hd, meta, 0, rope_tab, eps, max_kv);
}
// Query heads and key heads in one launch: QK-norm, RoPE, and the KV store.
void llamd_fwd_qk_norm_rope_store(float *q, const float *wq, float *k, const float *wk, const float *v, float *kc, float *vc, int n_head,
                                  int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int nseq, int max_kv) {
    launch_kc(PDL_SMALL, "qk_norm_rope_store", norm_rope_kernel<float>, dim3(n_head + n_head_kv, nseq), dim3(hd / 2), hd * sizeof(float), q, wq, k, wk, v, kc, vc,
             n_head, n_head_kv, hd, meta, 0, rope_tab, eps, max_kv);
}
// The same for the ntok tokens of a prefill tile: all rows go into ONE cache.
void llamd_fwd_qk_norm_rope_store_tile(float *q, const float *wq, float *k, const float *wk, const float *v, float *kc, float *vc,
                                       int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int ntok) {
    launch_k("qk_norm_rope_store_tile", norm_rope_kernel<float>, dim3(n_head + n_head_kv, ntok), dim3(hd / 2), hd * sizeof(float), q, wq, k, wk, v, kc,
             vc, n_head, n_head_kv, hd, meta, 0, rope_tab, eps, 0);
}
void llamd_fwd_kv_store(float *kc, float *vc, const float *k, const float *v, int pos, int kv_dim) {
    launch_k("kv_store", kv_store_kernel, dim3((kv_dim + 255) / 256), dim3(256), 0, kc, vc, k, v, pos, kv_dim);
}
// The same three with a binary16 cache (kc, vc: [..][n_head_kv*hd] halves): values rounded to nearest-even at the store.
void llamd_fwd_qk_norm_rope_store_kv16(float *q, const float *wq, float *k, const float *wk, const float *v, void *kc, void *vc, int n_head,
                                       int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int nseq, int max_kv) {
    launch_kc(PDL_SMALL, "qk_norm_rope_store_kv16", norm_rope_kernel<__half>, dim3(n_head + n_head_kv, nseq), dim3(hd / 2), hd * sizeof(float), q, wq, k,
              wk, v, (__half *)kc, (__half *)vc, n_head, n_head_kv, hd, meta, 0, rope_tab, eps, max_kv);
}
void llamd_fwd_qk_norm_rope_store_tile_kv16(float *q, const float *wq, float *k, const float *wk, const float *v, void *kc, void *vc,
                                            int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int ntok) {
    launch_k("qk_norm_rope_store_tile_kv16", norm_rope_kernel<__half>, dim3(n_head + n_head_kv, ntok), dim3(hd / 2), hd * sizeof(float), q, wq, k, wk, v,
             (__half *)kc, (__half *)vc, n_head, n_head_kv, hd, meta, 0, rope_tab, eps, 0);
}
// rows [0, n_pos) of a binary16 cache widened (exactly) to f32: what the tiled prefill attention reads
__global__ void kv_expand_kernel(const __half *__restrict__ src, float *__restrict__ dst, size_t n4) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x)
        reinterpret_cast<float4 *>(dst)[i] = KvIo<__half>::ld4(src + 4 * i);
}
void llamd_fwd_kv16_expand(const void *kc16, const void *vc16, float *kc32, float *vc32, int n_pos, int kv_dim) {
    const size_t n4 = (size_t)n_pos * kv_dim / 4;
    if (!n4 || kv_dim % 4) return;
    const unsigned grid = (unsigned)((n4 + 255) / 256 < 1184 ? (n4 + 255) / 256 : 1184);
    launch_k("kv16_expand", kv_expand_kernel, dim3(grid), dim3(256), 0, (const __half *)kc16, kc32, n4);
    launch_k("kv16_expand", kv_expand_kernel, dim3(grid), dim3(256), 0, (const __half *)vc16, vc32, n4);
}

static void attention_split_launch(const float *q, const void *kc, const void *vc, float *out, float *scores, int n_head,
                                   int n_head_kv, int hd, const int32_t *meta, int n_kv, int max_kv, int nseq, int kv_stride,
                                   const TailPlan &tail_in, bool kv16 = false, int flags = 0) {
    const size_t smem_a = (size_t)(hd + 2 * kAttTile * (hd + 1)) * sizeof(float);
    const size_t smem_b = (size_t)(((max_kv + 3) & ~3) + 2 * kPvTile * (hd / kSplit)) * sizeof(float);
    // (the library runs on one device per process: llamd_cuda_set_device is refused once the stream exists, so a
    // per-process record of the configured size is a per-device one)
    static size_t conf_a[2] = {0, 0}, conf_b[2] = {0, 0};
    if (smem_a > 48 * 1024 && smem_a > conf_a[kv16]) {
        const cudaError_t e = kv16 ? cudaFuncSetAttribute(attn_scores_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a)
                                   : cudaFuncSetAttribute(attn_scores_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
        if (e != cudaSuccess) {
            set_error(e, "attention (scores) smem attribute");
            return;
        }
        conf_a[kv16] = smem_a;
    }
    if (smem_b > 48 * 1024 && smem_b > conf_b[kv16]) {
        const cudaError_t e = kv16 ? cudaFuncSetAttribute(attn_out_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b)
                                   : cudaFuncSetAttribute(attn_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b);
        if (e != cudaSuccess) {
            set_error(e, "attention (output) smem attribute");
            return;
        }
        conf_b[kv16] = smem_b;
    }
    if (kv16)
        launch_kc(PDL_ATTN, "attn_scores", attn_scores_kernel<__half>, dim3(n_head, kSplitT, nseq), dim3(256), smem_a, q, (const __half *)kc, scores, n_head,
                  n_head_kv, hd, meta, n_kv, max_kv, kv_stride);
    else
    launch_kc(PDL_ATTN, "attn_scores", attn_scores_kernel<float>, dim3(n_head, kSplitT, nseq), dim3(256), smem_a, q, (const float *)kc, scores, n_head, n_head_kv, hd, meta, n_kv,
             max_kv, kv_stride);
    TailPlan tail = tail_in;
    if (tail.counter && (n_head * hd) % 256 != 0) {
        set_error_msg("attention: a quantize tail needs n_head * head_dim to be whole Q8_K blocks");
        tail = TailPlan{};
    }
    if (kv16)
        launch_kc(PDL_ATTN, "attn_out", attn_out_kernel<__half>, dim3(n_head, kSplit, nseq), dim3(256), smem_b, (const float *)scores, (const __half *)vc, out,
                  n_head, n_head_kv, hd, meta, n_kv, max_kv, kv_stride, tail, flags);
    else
    launch_kc(PDL_ATTN, "attn_out", attn_out_kernel<float>, dim3(n_head, kSplit, nseq), dim3(256), smem_b, (const float *)scores, (const float *)vc, out, n_head, n_head_kv, hd,
             meta, n_kv, max_kv, kv_stride, tail, flags);
}

static void attention_launch(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv, int hd,
                             const int32_t *meta, int n_kv, int max_kv, int nseq, int kv_stride, const TailPlan &tail = TailPlan{},
                             bool kv16 = false, int flags = 0) {
    const size_t smem = (size_t)(hd + ((max_kv + 3) & ~3) + 2 * kAttTile * (hd + 1)) * sizeof(float);
    if (hd % 4 || hd > 256 || kAttTile * (hd / 4) > 8 * 256 || n_head_kv <= 0 || n_head % n_head_kv || smem > 200 * 1024) {
        set_error_msg("attention: head_dim % 4, grouping, or context beyond the shared-memory score buffer");
        return;
    }
    // With a scores buffer ([nseq][n_head][max_kv] floats) and a head_dim the
    // column split divides, the work is cut over 4x more CTAs.
    if (scores && hd % (4 * kSplit) == 0 && kPvTile * (hd / kSplit) / 4 <= 8 * 256) {
        attention_split_launch(q, kc, vc, out, scores, n_head, n_head_kv, hd, meta, n_kv, max_kv, nseq, kv_stride, tail, kv16, flags);
        return;
    }
    if (kv16) {
        set_error_msg("attention: a binary16 cache needs the scores buffer and a head_dim the column split divides");
        return;
    }
    if (tail.counter) {
        set_error_msg("attention: a quantize tail was planned for the single-CTA kernel, which does not carry it");
        return;
    }
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error(e, "attention smem attribute");
            return;
        }
        configured = smem;
    }
    launch_k("attention", attention_kernel, dim3(n_head, nseq), dim3(256), smem, q, kc, vc, out, n_head, n_head_kv, hd, meta, n_kv, max_kv,
             kv_stride);
}
// `scores` (as in the reference's signature) is scratch for the scaled logits,
// [n_head][n_kv] floats; when it is NULL a single-CTA-per-head kernel keeps
// them in shared memory instead.
void llamd_fwd_attention(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv, int hd,
                         int n_kv) {
    attention_launch(q, kc, vc, out, scores, n_head, n_head_kv, hd, nullptr, n_kv, n_kv, 1, n_kv);
}
// One query per token of a prefill tile: token i (meta[2i+1] = its position)
// attends positions 0..pos_i of the ONE cache at kc/vc. No mask is needed:
// every token of the tile has stored its K and V before this launch.
// scores: [ntok][n_head][max_kv] floats.
void llamd_fwd_attention_tile(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                              int hd, const int32_t *meta, int max_kv, int ntok) {
    attention_launch(q, kc, vc, out, scores, n_head, n_head_kv, hd, meta, 0, max_kv, ntok, 0);
}
// llamd_fwd_attention_meta followed by llamd_fwd_quantize of the result, in the attention's own two launches:
// the CTA that finishes a sequence last writes qs [nseq][n_head*hd] and d [nseq][n_head*hd/256]. counter: nseq
// zero-initialised words the launch leaves at zero again. Needs the scores buffer (the split kernels).
void llamd_fwd_attention_meta_quant(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                                    int hd, const int32_t *meta, int max_kv, int nseq, unsigned int *counter, int8_t *qs, float *d) {
    if (!scores || !counter || !qs || !d) {
        set_error_msg("attention_meta_quant: scores, counter, qs and d must be given");
        return;
    }
    attention_launch(q, kc, vc, out, scores, n_head, n_head_kv, hd, meta, 0, max_kv, nseq, max_kv, TailPlan{counter, qs, d});
}
void llamd_fwd_attention_meta_kv16(const float *q, const void *kc, const void *vc, float *out, float *scores, int n_head, int n_head_kv,
                                   int hd, const int32_t *meta, int max_kv, int nseq) {
    attention_launch(q, (const float *)kc, (const float *)vc, out, scores, n_head, n_head_kv, hd, meta, 0, max_kv, nseq, max_kv, TailPlan{}, true);
}
// QK-norm + RoPE + KV store + attention of one decode token per sequence in TWO launches (scores with the preparation
// folded in, then softmax and weighted values) instead of three; q, k, v are the projections as the matvec left them
// (they are not modified). kv16: the caches hold binary16. Same bits as llamd_fwd_qk_norm_rope_store followed by
// llamd_fwd_attention_meta.
static void attention_rope_launch(const float *q, const float *wq, const float *k, const float *wk, const float *v, void *kc, void *vc,
                                  float *out, float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab,
                                  float eps, int max_kv, int nseq, bool kv16, int8_t *qs = nullptr, float *qd = nullptr, int flags = 0) {
    const size_t smem_a = (size_t)(hd + 2 * kAttTile * (hd + 1) + 3 * hd) * sizeof(float);
    const size_t smem_b = (size_t)(((max_kv + 3) & ~3) + 2 * kPvTile * (hd / kSplit)) * sizeof(float);
    if (!scores || !meta || hd % (4 * kSplit) || hd > 256 || hd / 2 > 256 || kAttTile * (hd / 4) > 8 * 256 || kPvTile * (hd / kSplit) / 4 > 8 * 256 ||
        n_head_kv <= 0 || n_head % n_head_kv || smem_a > 200 * 1024 || smem_b > 200 * 1024) {
        set_error_msg("attention (with the rope folded in): needs the scores buffer, positions on the device, and a head_dim the kernels divide");
        return;
    }
    static size_t conf_a[2] = {0, 0}, conf_b[2] = {0, 0};
    if (smem_a > 48 * 1024 && smem_a > conf_a[kv16]) {
        const cudaError_t e = kv16 ? cudaFuncSetAttribute(attn_rope_scores_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a)
                                   : cudaFuncSetAttribute(attn_rope_scores_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_a);
        if (e != cudaSuccess) {
            set_error(e, "attention (rope + scores) smem attribute");
            return;
        }
        conf_a[kv16] = smem_a;
    }
    if (smem_b > 48 * 1024 && smem_b > conf_b[kv16]) {
        const cudaError_t e = kv16 ? cudaFuncSetAttribute(attn_out_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b)
                                   : cudaFuncSetAttribute(attn_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_b);
        if (e != cudaSuccess) {
            set_error(e, "attention (output) smem attribute");
            return;
        }
        conf_b[kv16] = smem_b;
    }
    // A batch of sequences: one CTA per (kv head, ...) for all the query heads that share it (the decode pass asks for it)
    const int ratio = n_head / n_head_kv, cap = (max_kv + 3) & ~3;
    const size_t smem_ga = (size_t)(ratio * hd + 2 * kAttTile * (hd + 1) + (ratio + 1) * hd + hd) * sizeof(float);
    const size_t smem_gb = (size_t)((size_t)ratio * cap + 2 * kPvTile * (hd / kSplit)) * sizeof(float);
    // (measured, 48 layers at position ~520: 8 sequences 814.7 -> 1044.8 tok/s, 4 sequences 641.8 -> 717.2, 2 sequences 456.2 -> 439.7,
    // so from four sequences on)
    if ((flags & kPassAttnGqa) && !(flags & 4) && nseq >= 4 && ratio == kGqaMax && hd / kSplit == 32 && smem_ga <= 200 * 1024 &&
        smem_gb <= 200 * 1024) {
        static size_t conf_ga[2] = {0, 0}, conf_gb[2] = {0, 0};
        if (smem_ga > conf_ga[kv16]) {
            const cudaError_t e = kv16 ? cudaFuncSetAttribute(attn_rope_scores_gqa_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_ga)
                                       : cudaFuncSetAttribute(attn_rope_scores_gqa_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_ga);
            if (e != cudaSuccess) {
                set_error(e, "attention (rope + scores, per kv head) smem attribute");
                return;
            }
            conf_ga[kv16] = smem_ga;
        }
        if (smem_gb > conf_gb[kv16]) {
            const cudaError_t e = kv16 ? cudaFuncSetAttribute(attn_out_gqa_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_gb)
                                       : cudaFuncSetAttribute(attn_out_gqa_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_gb);
            if (e != cudaSuccess) {
                set_error(e, "attention (output, per kv head) smem attribute");
                return;
            }
            conf_gb[kv16] = smem_gb;
        }
        if (kv16) {
            launch_kc(PDL_ATTN, "attn_rope_scores_gqa", attn_rope_scores_gqa_kernel<__half>, dim3(n_head_kv, kSplitT, nseq), dim3(256), smem_ga, q, wq, k,
                      wk, v, (__half *)kc, (__half *)vc, scores, n_head, n_head_kv, hd, meta, max_kv, max_kv, rope_tab, eps, flags);
            launch_kc(PDL_ATTN, "attn_out_gqa", attn_out_gqa_kernel<__half>, dim3(n_head_kv, kSplit, nseq), dim3(256), smem_gb, (const float *)scores,
                      (const __half *)vc, out, n_head, n_head_kv, hd, meta, max_kv, max_kv, flags);
        } else {
            launch_kc(PDL_ATTN, "attn_rope_scores_gqa", attn_rope_scores_gqa_kernel<float>, dim3(n_head_kv, kSplitT, nseq), dim3(256), smem_ga, q, wq, k,
                      wk, v, (float *)kc, (float *)vc, scores, n_head, n_head_kv, hd, meta, max_kv, max_kv, rope_tab, eps, flags);
            launch_kc(PDL_ATTN, "attn_out_gqa", attn_out_gqa_kernel<float>, dim3(n_head_kv, kSplit, nseq), dim3(256), smem_gb, (const float *)scores,
                      (const float *)vc, out, n_head, n_head_kv, hd, meta, max_kv, max_kv, flags);
        }
        if (qs && qd) llamd_fwd_quantize(out, qs, qd, nseq * (n_head * hd / 256));
        return;
    }
    const bool clusters = qs && qd && attn_out_cluster_ok(n_head, hd);
    if (kv16) {
        launch_kc(PDL_ATTN, "attn_rope_scores", attn_rope_scores_kernel<__half>, dim3(n_head, kSplitT, nseq), dim3(256), smem_a, q, wq, k, wk, v,
                  (__half *)kc, (__half *)vc, scores, n_head, n_head_kv, hd, meta, max_kv, max_kv, rope_tab, eps, flags);
        if (clusters)
            attn_out_cluster_launch<__half>(smem_b, scores, (const __half *)vc, out, n_head, n_head_kv, hd, meta, max_kv, nseq, qs, qd, flags);
        else
            launch_kc(PDL_ATTN, "attn_out", attn_out_kernel<__half>, dim3(n_head, kSplit, nseq), dim3(256), smem_b, (const float *)scores,
                      (const __half *)vc, out, n_head, n_head_kv, hd, meta, 0, max_kv, max_kv, TailPlan{}, flags);
    } else {
        launch_kc(PDL_ATTN, "attn_rope_scores", attn_rope_scores_kernel<float>, dim3(n_head, kSplitT, nseq), dim3(256), smem_a, q, wq, k, wk, v,
                  (float *)kc, (float *)vc, scores, n_head, n_head_kv, hd, meta, max_kv, max_kv, rope_tab, eps, flags);
        if (clusters)
            attn_out_cluster_launch<float>(smem_b, scores, (const float *)vc, out, n_head, n_head_kv, hd, meta, max_kv, nseq, qs, qd, flags);
        else
            launch_kc(PDL_ATTN, "attn_out", attn_out_kernel<float>, dim3(n_head, kSplit, nseq), dim3(256), smem_b, (const float *)scores,
                      (const float *)vc, out, n_head, n_head_kv, hd, meta, 0, max_kv, max_kv, TailPlan{}, flags);
    }
    if (qs && qd && !clusters) llamd_fwd_quantize(out, qs, qd, nseq * (n_head * hd / 256));
}
} // extern "C"
namespace llamd {
// The decode pass's attention with the Q8_K form of its result: three launches' work in two where the head size lets a
// cluster cover a block (the quantize launch otherwise). Same bits as llamd_fwd_attention_rope_meta + llamd_fwd_quantize.
void attention_rope_quant(const float *q, const float *wq, const float *k, const float *wk, const float *v, void *kc, void *vc, float *out,
                          float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int max_kv,
                          int nseq, bool kv16, int8_t *qs, float *d, int flags) {
    attention_rope_launch(q, wq, k, wk, v, kc, vc, out, scores, n_head, n_head_kv, hd, meta, rope_tab, eps, max_kv, nseq, kv16, qs, d, flags);
}
// llamd_fwd_attention_meta / _kv16 with a decode pass's flags.
void attention_meta_flags(const float *q, const void *kc, const void *vc, float *out, float *scores, int n_head, int n_head_kv, int hd,
                          const int32_t *meta, int max_kv, int nseq, bool kv16, int flags) {
    attention_launch(q, (const float *)kc, (const float *)vc, out, scores, n_head, n_head_kv, hd, meta, 0, max_kv, nseq, max_kv, TailPlan{}, kv16,
                     flags);
}
}  // namespace llamd
extern "C" {
void llamd_fwd_attention_rope_meta(const float *q, const float *wq, const float *k, const float *wk, const float *v, float *kc, float *vc,
                                   float *out, float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab,
                                   float eps, int max_kv, int nseq) {
    attention_rope_launch(q, wq, k, wk, v, kc, vc, out, scores, n_head, n_head_kv, hd, meta, rope_tab, eps, max_kv, nseq, false);
}
void llamd_fwd_attention_rope_meta_kv16(const float *q, const float *wq, const float *k, const float *wk, const float *v, void *kc, void *vc,
                                        float *out, float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta,
                                        const float *rope_tab, float eps, int max_kv, int nseq) {
    attention_rope_launch(q, wq, k, wk, v, kc, vc, out, scores, n_head, n_head_kv, hd, meta, rope_tab, eps, max_kv, nseq, true);
}
void llamd_fwd_attention_meta(const float *q, const float *kc, const float *vc, float *out, float *scores, int n_head, int n_head_kv,
                              int hd, const int32_t *meta, int max_kv, int nseq) {
    attention_launch(q, kc, vc, out, scores, n_head, n_head_kv, hd, meta, 0, max_kv, nseq, max_kv);
}

// ---- attention for callers that must not allocate ---------------------------
// Some hosts of this library cannot obtain device memory at call time: an
// inference server that hands all of the GPU's memory to its own pool at
// start-up and forbids any later cudaMalloc, or a real-time loop in which the
// implicit device synchronisation of the CUDA allocator is not acceptable.
// For them the score scratch that llamd_fwd_attention takes from its caller
// lives in this array instead. Every GPU that loads the library carries it
// (1 MiB) until the process exits.
constexpr int kStaticScoreFloats = 64 * 4096;  // n_head * n_kv may not exceed this
static __device__ __align__(256) float g_static_scores[kStaticScoreFloats];
// In host code `g_static_scores` is only a handle for the runtime, not an
// address a kernel can use: the device address is looked up once per device.
constexpr int kMaxDevices = 64;
static float *g_static_scores_dev[kMaxDevices] = {};

int llamd_fwd_attention_noalloc(const float *q, const float *kc, const float *vc, float *out, int n_head, int n_head_kv, int hd,
                                int n_kv) {
    if (!q || !kc || !vc || !out || n_head <= 0 || hd <= 0 || n_kv <= 0) {
        set_error_msg("attention_noalloc: null pointer or empty shape");
        return -1;
    }
    if (error_code() != 0) {
        // an earlier failure nobody has read yet: this call could not tell its own failure from that one
        return -1;
    }
    if ((long long)n_head * n_kv > kStaticScoreFloats) {
        set_error_msg("attention_noalloc: n_head * n_kv exceeds the built-in scratch of 262144 floats (64 heads x 4096 positions)");
        return -1;
    }
    // the kernels keep one head's scores in shared memory beside their K/V tiles
    if (((size_t)hd + (size_t)((n_kv + 3) & ~3) + 2 * (size_t)kAttTile * (hd + 1)) * sizeof(float) > 200 * 1024) {
        set_error_msg("attention_noalloc: n_kv too long for the shared-memory score row: (hd + n_kv + 128 (hd + 1)) * 4 bytes "
                      "must not exceed 200 KiB (34560 positions at head_dim 128)");
        return -1;
    }
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_error(e == cudaSuccess ? cudaErrorInvalidDevice : e, "attention_noalloc: cudaGetDevice");
        return -1;
    }
    if (!g_static_scores_dev[dev]) {
        // first call on this device (it is the current one): resolve the symbol
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_static_scores);
        if (e != cudaSuccess || !p) {
            set_error(e == cudaSuccess ? cudaErrorInvalidSymbol : e, "attention_noalloc: cudaGetSymbolAddress");
            return -1;
        }
        g_static_scores_dev[dev] = p;
    }
    if (!stream()) return -1;
    // Nothing in the scratch has to start at zero: each launch writes the
    // n_head * n_kv scores it later reads, so the previous call's contents are
    // simply overwritten.
    attention_launch(q, kc, vc, out, g_static_scores_dev[dev], n_head, n_head_kv, hd, nullptr, n_kv, n_kv, 1, n_kv);
    return error_code() != 0 ? -1 : 0;  // the sticky error was clear on entry, so a set one is this call's
}

void llamd_fwd_argmax(const float *x, int n, float *scratch_v, int32_t *scratch_i, int32_t *out, int nblocks, int nseq) {
    if (nblocks < 1) nblocks = 1;
    launch_k("argmax_partial", argmax_partial_kernel, dim3(nblocks, nseq), dim3(256), 0, x, n, scratch_v, scratch_i);
    launch_k("argmax_final", argmax_final_kernel, dim3(nseq), dim3(256), 0, (const float *)scratch_v, (const int32_t *)scratch_i, nblocks, out);
}

void llamd_fwd_moe_group_work(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart, int32_t *gcount,
                              int32_t *ptoken, int32_t *pslot, int32_t *work, int32_t *n_work) {
    moe_group_owned(ids, n_expert, n_used, nseq, gstart, gcount, ptoken, pslot, work, n_work, 0, n_expert);
}
}  // extern "C"

// The plan over the pairs whose expert this GPU holds, [own_lo, own_hi) (all of them without expert parallelism).
void llamd::moe_group_owned(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart, int32_t *gcount, int32_t *ptoken,
                            int32_t *pslot, int32_t *work, int32_t *n_work, int own_lo, int own_hi) {
    const int npair = n_used * nseq;
    if (n_expert < 1 || n_expert > 1024 || npair < 0 || npair > 32 * 32 * kGroupMaxPerLane) {
        set_error_msg("moe_group: n_expert 1..1024 and at most 40960 pairs per call");
        return;
    }
    const int threads = 1024;  // 32 warps, each owning a contiguous run of pairs
    const size_t smem = (size_t)32 * n_expert * sizeof(int);
    static size_t configured = 0;
    if (smem > 36 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(moe_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error(e, "moe_group smem attribute");
            return;
        }
        configured = smem;
    }
    launch_k("moe_group", moe_group_kernel, dim3(1), dim3(threads), smem, ids, n_expert, npair, n_used, gstart, gcount, ptoken, pslot, work,
             n_work, own_lo < 0 ? 0 : own_lo, own_hi > n_expert ? n_expert : own_hi);
}

extern "C" {
void llamd_fwd_moe_group(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart, int32_t *gcount, int32_t *ptoken,
                         int32_t *pslot) {
    llamd_fwd_moe_group_work(ids, n_expert, n_used, nseq, gstart, gcount, ptoken, pslot, nullptr, nullptr);
}

}  // extern "C"

void llamd::slot_order_launch(const int32_t *ids, int n_slots, int32_t *order) {
    if (n_slots < 1 || n_slots > 8192) {
        set_error_msg("slot_order: 1..8192 slots");
        return;
    }
    launch_kc(PDL_SMALL, "slot_order", slot_order_kernel, dim3(1), dim3(256), (size_t)n_slots * sizeof(int32_t), ids, n_slots, order);
}
