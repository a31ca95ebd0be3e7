// The resident decode pass: every layer of one token in ONE cooperative kernel.
//
// The per-op pass (model.cu: queue_token) spends most of a token between kernels: a dozen dependent launches per
// layer, each paying a launch boundary and a cold start, around ~7 us of weight streaming and ~16 us of ordered f32
// chains. Here one CTA per SM stays resident for the whole token; the layer's phases are separated by grid barriers
// (an arrive counter in L2, ~1 us) instead of launches, small per-token vectors are recomputed by every CTA from L2
// instead of being produced by a one-CTA kernel and re-read, the residual stream lives in shared memory, and the
// weights of the next phase are requested before the barrier that precedes it is waited for.
//
// Arithmetic is the per-op pass's, operation for operation (the same device functions and the same chains in the same
// order), so tokens, expert ids and logits are bit-identical to it and hence to the CPU path
// (crates/llamd-runtime/src/layer.rs:85-304).
//
// Phases of a layer (G CTAs of kMegaThreads threads; "every CTA" = redundantly):
//   A  every CTA: x += sum_e w_e down_e (previous layer, routing order), attention norm, Q8_K  | its rows of Q, K, V
//   B  item (head, column quarter): QK-norm, RoPE, KV store, scores, softmax, weighted values of its columns
//   C  every CTA: Q8_K of the attention output                                               | its rows of attn_out
//   D  every CTA: x += attn_out, FFN norm, Q8_K (kept for E)                                  | router logit of expert r
//   E  every CTA: route (softmax, top-n_used, weights)                                        | its rows of gate, up
//   F  every CTA: silu(gate) * up and Q8_K for the slots its rows touch                       | its rows of down
// then, after the last layer, the combine + output norm + Q8_K, which the lm_head matvec (a separate launch) reads.
//
// Every wait is bounded: a barrier that is not completed within the poll limit sets a status word and the CTA leaves
// the kernel; the others then run out at their next barrier. The launch is cooperative, so all CTAs are resident and
// a barrier can only fail through a bug, but nothing spins for ever.
#include <cooperative_groups.h>

#include "q6k_layout.cuh"
#include "quant.cuh"
#include "route.cuh"
#include <cuda_fp16.h>

#include "mega.cuh"

namespace llamd {

constexpr int kMegaThreads = 768;
constexpr int kMegaExStride = kMegaThreads + 1;
constexpr int kMegaActWords = 132;   // words per activation block image (matvec_q6k.cu: kActBlockWords)
constexpr int kMegaSplit = 4;        // output-column parts per head

// shared memory carve-up (floats unless noted), the same on host and device
struct MegaSmem {
    size_t x, xn, sq, act, nat, adv, ex, sl, tile, misc, total;
};
__host__ __device__ inline MegaSmem mega_smem(int E, int qd, int hd, int act_blocks, int sl_floats, int n_expert, int ktile_rows, int ratio) {
    MegaSmem s;
    size_t o = 0;
    auto take = [&](size_t bytes) {
        const size_t at = o;
        o += (bytes + 15) & ~(size_t)15;
        return at;
    };
    s.x = take((size_t)E * 4);
    s.xn = take((size_t)E * 4);
    const size_t sqn = (size_t)(E > n_expert ? E : n_expert);
    s.sq = take(sqn * 4);
    s.act = take((size_t)act_blocks * kMegaActWords * 4);
    s.nat = take((size_t)act_blocks * 256);
    s.adv = take((size_t)act_blocks * 4);
    s.ex = take((size_t)8 * kMegaExStride * 4);
    s.sl = take((size_t)sl_floats * 4);
    // B1: the K rows of this CTA's position chunk (rows of hd + 4 words) after the group's q heads, raw and roped;
    // B2: a V tile of kMegaThreads positions x hd / kMegaSplit columns
    const size_t ktile = (size_t)ktile_rows * (hd + 4) + 2 * (size_t)ratio * hd, vtile = (size_t)kMegaThreads * (hd / kMegaSplit);
    s.tile = take((ktile > vtile ? ktile : vtile) * 4);
    s.misc = take((size_t)(4 * hd + 512) * 4);
    (void)qd;
    s.total = o;
    return s;
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Four consecutive cache elements as f32: the cache holds f32, or binary16 values that widen exactly.
__device__ __forceinline__ float4 kv_ld4(const float *base, size_t elem, bool kv16, bool through_l2) {
    if (kv16) {
        const uint2 *p = reinterpret_cast<const uint2 *>(reinterpret_cast<const __half *>(base) + elem);
        const uint2 u = through_l2 ? __ldcg(p) : __ldg(p);
        const __half2 a = *reinterpret_cast<const __half2 *>(&u.x), b = *reinterpret_cast<const __half2 *>(&u.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    const float4 *p = reinterpret_cast<const float4 *>(base + elem);
    return through_l2 ? __ldcg(p) : __ldg(p);
}
// Store one element; returns the value as the cache now holds it.
__device__ __forceinline__ float kv_st(float *base, size_t elem, float v, bool kv16) {
    if (kv16) {
        const __half h = __float2half_rn(v);
        reinterpret_cast<__half *>(base)[elem] = h;
        return __half2float(h);
    }
    base[elem] = v;
    return v;
}

// All CTAs arrive, all leave; false (for the whole CTA) when the wait ran out.
__device__ __forceinline__ bool grid_barrier(const MegaParams &p, unsigned int &target, bool *s_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        target += gridDim.x;
        __threadfence();
        atomicAdd(p.bar, 1u);
        bool ok = false;
        for (unsigned int it = 0; it < p.spin_limit; it++) {
            if ((int)(ld_acquire_gpu(p.bar) - target) >= 0) {
                ok = true;
                break;
            }
            if (it > 64) __nanosleep(32);
        }
        if (!ok) atomicExch(p.status, 1);
        *s_flag = ok;
    }
    __syncthreads();
    return *s_flag;
}

// ---- one (row, block) unit of a Q6_K matvec, as matvec_q6k_kernel does it ---------------------------------------
struct MvUnit {
    uint32_t S[48];
    uint4 scw;
    uint16_t dbits;
};
__device__ __forceinline__ void mv_load(MvUnit &u, const uint8_t *w, size_t unit) {
    const uint8_t *tile = w + (unit >> 5) * kTileBytes;
    const int sl = (int)(unit & 31);
    const uint4 *cp = reinterpret_cast<const uint4 *>(tile) + sl;
#pragma unroll
    for (int c = 0; c < 12; c++) {
        const uint4 v = __ldg(cp + c * 32);
        u.S[4 * c + 0] = v.x;
        u.S[4 * c + 1] = v.y;
        u.S[4 * c + 2] = v.z;
        u.S[4 * c + 3] = v.w;
    }
    u.scw = __ldg(reinterpret_cast<const uint4 *>(tile + kTileScaleOff) + sl);
    u.dbits = __ldg(reinterpret_cast<const uint16_t *>(tile + kTileDOff) + sl);
}
// the unit's eight (d_w * d_a) * aux products into the exchange buffer, column `col`
__device__ __forceinline__ void mv_compute(const MvUnit &u, const uint32_t *s_act_blk, float adv, float *s_ex, int col) {
    int sc[16];
    {
        const uint32_t ws[4] = {u.scw.x, u.scw.y, u.scw.z, u.scw.w};
#pragma unroll
        for (int i = 0; i < 16; i++) sc[i] = (int)(int8_t)(ws[i >> 2] >> (8 * (i & 3)));
    }
    int aux[8];
#pragma unroll
    for (int r = 0; r < 8; r++) aux[r] = 0;
#pragma unroll
    for (int r = 0; r < 8; r++) {
#pragma unroll
        for (int m = 0; m < 2; m++) {
            uint32_t w4[4];
            unpack_quad(u.S[6 * r + 3 * m], u.S[6 * r + 3 * m + 1], u.S[6 * r + 3 * m + 2], w4);
            const uint4 *ap = reinterpret_cast<const uint4 *>(s_act_blk + r * 16 + m * 8);
            const uint4 a01 = ap[0], a23 = ap[1];
            int acc = aux[r];
            acc += sc[8 * m + 0] * __dp4a((int)w4[0], (int)a01.x, 0);
            acc += sc[8 * m + 1] * __dp4a((int)w4[0], (int)a01.y, 0);
            acc += sc[8 * m + 2] * __dp4a((int)w4[1], (int)a01.z, 0);
            acc += sc[8 * m + 3] * __dp4a((int)w4[1], (int)a01.w, 0);
            acc += sc[8 * m + 4] * __dp4a((int)w4[2], (int)a23.x, 0);
            acc += sc[8 * m + 5] * __dp4a((int)w4[2], (int)a23.y, 0);
            acc += sc[8 * m + 6] * __dp4a((int)w4[3], (int)a23.z, 0);
            acc += sc[8 * m + 7] * __dp4a((int)w4[3], (int)a23.w, 0);
            aux[r] = acc;
        }
    }
    const float dsc = __fmul_rn(f16_bits_to_f32(u.dbits), adv);
#pragma unroll
    for (int r = 0; r < 8; r++) s_ex[r * kMegaExStride + col] = __fmul_rn(dsc, (float)(aux[r] >> 2));
}

// natural-order Q8_K bytes of `nblk` blocks -> the residue-major (lo, hi) image the units read
__device__ __forceinline__ void build_act_image(const int8_t *s_nat, uint32_t *s_act, int nblk) {
    for (int i = threadIdx.x; i < nblk * 64; i += kMegaThreads) {
        const int jj = i & 7, r = (i >> 3) & 7, sb = i >> 6;
        const int8_t *src = s_nat + sb * 256;
        const uint32_t b0 = (uint8_t)src[t32_element(r, jj, 0)], b1 = (uint8_t)src[t32_element(r, jj, 1)];
        const uint32_t b2 = (uint8_t)src[t32_element(r, jj, 2)], b3 = (uint8_t)src[t32_element(r, jj, 3)];
        uint32_t *dst = s_act + sb * kMegaActWords + r * 16 + jj * 2;
        dst[0] = b0 | (b1 << 8);
        dst[1] = (b2 << 16) | (b3 << 24);
    }
}

// A virtual row of a phase: where its weights are, which activation it reads, where its result goes.
struct RowRef {
    const uint8_t *w;
    size_t unit0;  // index of the row's first block in w
    int act;       // activation index in the image (blocks act*nb ..)
    float *out;
};

// The rows [row_lo, row_hi) of a phase, `nb` blocks each, in chunks of floor(T / nb) rows. ROWMAP(row) -> RowRef.
// The weights come from L2 (the phase before asked for them); nothing is held in registers outside a chunk's
// load -> dot -> exchange sequence, which at 80 registers per thread is what keeps the 53 loaded words out of local memory.
template <class RowMap>
__device__ __forceinline__ void mv_rows(const RowMap &map, int nb, int row_lo, int row_hi, const uint32_t *s_act, const float *s_adv, float *s_ex) {
    const int tid = threadIdx.x, row_l = tid / nb, b = tid - row_l * nb;
    const int cap = kMegaThreads / nb;
    for (int base = row_lo; base < row_hi; base += cap) {
        const int rows_here = min(cap, row_hi - base);
        if (row_l < rows_here) {
            const RowRef rr = map(base + row_l);
            MvUnit u;
            mv_load(u, rr.w, rr.unit0 + b);
            mv_compute(u, s_act + (size_t)(rr.act * nb + b) * kMegaActWords, s_adv[rr.act * nb + b], s_ex, tid);
        }
        __syncthreads();
        const int n_out = rows_here * 8;
        for (int o0 = 0; o0 < n_out; o0 += kMegaThreads) {
            const int idx = o0 + tid;
            const bool on = idx < n_out;
            const int rl = idx >> 3, r = idx & 7;
            float acc = 0.0f;
            if (on) {
                const float *ex = s_ex + r * kMegaExStride + rl * nb;
                for (int bb = 0; bb < nb; bb++) acc = __fadd_rn(acc, ex[bb]);
            }
            const int lane0 = (tid & 31) & ~7;
            float total = __shfl_sync(0xffffffffu, acc, lane0);
#pragma unroll
            for (int q = 1; q < 8; q++) total = __fadd_rn(total, __shfl_sync(0xffffffffu, acc, lane0 + q));
            if (on && r == 0) *map(base + rl).out = total;
        }
        __syncthreads();
    }
}

// Hints to L2 (nothing waits on them): a byte range, cut into pieces that the CTA's threads each ask for; the tiles that
// hold blocks [unit_lo, unit_hi) of a tiled Q6_K matrix; a phase's rows [lo, hi) as far as they fall into the matrix
// that holds virtual rows [first, first + rows).
__device__ __forceinline__ void l2_prefetch_bytes(const uint8_t *base, size_t bytes) {
    // one 128-byte line per instruction, the CTA's threads striding over the range: a hint that costs the issuing thread
    // nothing (the bulk form, cp.async.bulk.prefetch.L2, held its issuing thread for ~1 us per instruction)
    for (size_t off = (size_t)threadIdx.x * 128; off < bytes; off += (size_t)kMegaThreads * 128)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base + off));
}
__device__ __forceinline__ void l2_prefetch_units(const uint8_t *w, size_t unit_lo, size_t unit_hi) {
    if (unit_hi <= unit_lo) return;
    const size_t t0 = unit_lo >> 5, t1 = (unit_hi - 1) >> 5;
    l2_prefetch_bytes(w + t0 * kTileBytes, (t1 - t0 + 1) * kTileBytes);
}
__device__ __forceinline__ void l2_prefetch_rows(const uint8_t *w, int lo, int hi, int first, int rows, int nb) {
    const int a = max(lo, first), b = min(hi, first + rows);
    if (b > a) l2_prefetch_units(w, (size_t)(a - first) * nb, (size_t)(b - first) * nb);
}

constexpr int kMegaElems = 4;  // elements of an n_embd-long vector per thread per sweep (n_embd <= 3072 in one sweep)

// Sum of one value per thread over the CTA, the same on every thread and from run to run: xor-shuffle tree inside a warp,
// then the warps' sums added in warp order. Used by the `fast` arithmetic only. s_red: kMegaThreads / 32 floats.
__device__ __forceinline__ float block_sum(float v, float *s_red) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = s_red[0];
#pragma unroll
    for (int w = 1; w < kMegaThreads / 32; w++) t = __fadd_rn(t, s_red[w]);
    __syncthreads();
    return t;
}

// rms norm of s_x (n floats): squares by all threads, the ordered sum by thread 0, out = (x * scale) * w into s_out,
// then Q8_K of s_out into s_nat / s_adv (n / 256 blocks). crates/llamd-cpu/src/lib.rs:55-75, dot.rs:88-128.
// The weight vector is read before the chain is walked, so that its latency is hidden behind it.
template <class Stamp>
__device__ __forceinline__ void norm_quant(const float *s_x, const float *__restrict__ w, float *s_sq, float *s_out, int8_t *s_nat, float *s_adv,
                                           int n, float eps, float *s_scalar, const Stamp &stamp, bool fast, float *s_red) {
    const int tid = threadIdx.x;
    float wv[kMegaElems];
#pragma unroll
    for (int u = 0; u < kMegaElems; u++) {
        const int i = tid + u * kMegaThreads;
        wv[u] = i < n ? __ldg(w + i) : 0.0f;
    }
    float scale;
    if (fast) {
        float part = 0.0f;
        for (int i = tid; i < n; i += kMegaThreads) part = __fadd_rn(part, __fmul_rn(s_x[i], s_x[i]));
        const float sum = block_sum(part, s_red);
        scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)n), eps)));
        stamp(1);
    } else {
        for (int i = tid; i < n; i += kMegaThreads) s_sq[i] = __fmul_rn(s_x[i], s_x[i]);
        __syncthreads();
        stamp(0);
        if (tid == 0) {
            const float sum = chain_sum(s_sq, n, 0.0f);
            *s_scalar = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)n), eps)));
        }
        __syncthreads();
        stamp(1);
        scale = *s_scalar;
    }
#pragma unroll
    for (int u = 0; u < kMegaElems; u++) {
        const int i = tid + u * kMegaThreads;
        if (i < n) s_out[i] = __fmul_rn(__fmul_rn(s_x[i], scale), wv[u]);
    }
    for (int i = tid + kMegaElems * kMegaThreads; i < n; i += kMegaThreads) s_out[i] = __fmul_rn(__fmul_rn(s_x[i], scale), __ldg(w + i));
    __syncthreads();
    stamp(2);
    const int warp = tid >> 5, lane = tid & 31;
    for (int b = warp; b < n / 256; b += kMegaThreads / 32) {
        const float4 a = reinterpret_cast<const float4 *>(s_out + b * 256 + lane * 8)[0], c = reinterpret_cast<const float4 *>(s_out + b * 256 + lane * 8)[1];
        const float v[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
        q8k_quantize_block(v, lane, s_nat + b * 256, s_adv + b, nullptr);
    }
    __syncthreads();
}

// route (crates/llamd-models/src/moe.rs:73-113), called by the whole CTA: the same operations as route_block -- max,
// exp(l - max), the sum walked in index order from -0.0, p / sum, the n_used best by (probability descending, index
// ascending), the chosen weights summed in choice order from -0.0, the 2^-14 floor, the division. The stable sort is
// done by rank: thread i counts the experts that come before expert i in that order, and the experts of rank < n_used
// write themselves into place (one pass over shared memory instead of n_used arg-max rounds). n_expert <= kMegaThreads.
// s_p: logits in (overwritten with the probabilities). s_red: 40 floats.
__device__ __forceinline__ void route_cta(float *s_p, int n_expert, int n_used, int32_t *ids, float *weights, float *s_red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float m = tid < n_expert ? s_p[tid] : -INFINITY;
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    m = s_red[0];
    for (int w = 1; w < kMegaThreads / 32; w++) m = fmaxf(m, s_red[w]);
    if (tid < n_expert) s_p[tid] = ref_expf(__fsub_rn(s_p[tid], m));
    __syncthreads();
    if (tid == 0) s_red[32] = chain_sum(s_p, n_expert, -0.0f);
    __syncthreads();
    const float mine = tid < n_expert ? __fdiv_rn(s_p[tid], s_red[32]) : 0.0f;
    __syncthreads();
    if (tid < n_expert) s_p[tid] = mine;
    __syncthreads();
    if (tid < n_expert) {
        int rank = 0;
        for (int j = 0; j < n_expert; j++) {
            const float o = s_p[j];
            rank += (o > mine || (o == mine && j < tid)) ? 1 : 0;
        }
        if (rank < n_used) {
            ids[rank] = tid;
            weights[rank] = mine;
        }
    }
    __syncthreads();
    if (tid == 0) {
        float sum = -0.0f;
        for (int k = 0; k < n_used; k++) sum = __fadd_rn(sum, weights[k]);
        s_red[33] = fmaxf(sum, WEIGHT_SUM_FLOOR);
    }
    __syncthreads();
    if (tid < n_used) weights[tid] = __fdiv_rn(weights[tid], s_red[33]);
    __syncthreads();
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Phase clock, usable inside the phase functions: thread 0 of CTA 0 adds the time since the previous stamp to slot k.
// The sums and the previous stamp live in shared memory (a stamp costs a few dozen cycles; kept in global memory each one
// put a ~1 us read-modify-write into the interval after it) and go to p.prof when the kernel ends.
__shared__ unsigned long long s_mega_prof[33];  // [32]: the previous stamp
__device__ __forceinline__ void mega_stamp(const MegaParams &p, int k) {
    if (p.prof && blockIdx.x == 0 && threadIdx.x == 0) {
        const unsigned long long t = global_ns();
        s_mega_prof[k] += t - s_mega_prof[32];
        s_mega_prof[32] = t;
    }
}

// What a CTA knows for the whole token: its shared-memory regions, the model's dimensions, its share of every phase.
// One copy per CTA in shared memory; the phase functions below are separate functions (not inlined) so that each gets
// a register allocation of its own -- inside one 2000-line kernel body at 80 registers per thread the ordered-sum loops
// and the attention loops were spilling.
struct MegaCtx {
    uint32_t o_x, o_xn, o_sq, o_act, o_nat, o_adv, o_ex, o_sl, o_tile, o_misc;  // byte offsets into the dynamic shared memory
    int E, H, HKV, hd, nu, ffe, ne, qd, kvd, eb, qb, fb;
    int cta, G, pos, n_kv;
    int a_lo, a_hi, c_lo, c_hi, e_lo, e_hi, f_lo, f_hi, slot_lo, slot_hi;
    int ratio, half, cols, b1_kvh, t_lo, t_hi, b1_has_pos;
};

// The CTA's shared-memory regions as typed pointers. Built from the `extern __shared__` base inside every phase function
// (not stored in MegaCtx): a pointer read back from memory is a generic pointer to the compiler, every access through it
// a generic load or store, and the ordered sums then walk at the generic path's latency (measured: 6.3 cycles per add
// instead of 4.3).
struct MegaPtrs {
    float *s_x, *s_xn, *s_sq, *s_adv, *s_ex, *s_sl, *s_tile, *s_k, *s_v, *s_tmp, *s_red, *s_w, *s_scalar;
    uint32_t *s_act;
    int8_t *s_nat;
    int32_t *s_ids;
    __device__ __forceinline__ explicit MegaPtrs(const MegaCtx &c) {
        extern __shared__ __align__(16) uint8_t smem[];
        s_x = reinterpret_cast<float *>(smem + c.o_x);
        s_xn = reinterpret_cast<float *>(smem + c.o_xn);
        s_sq = reinterpret_cast<float *>(smem + c.o_sq);
        s_act = reinterpret_cast<uint32_t *>(smem + c.o_act);
        s_nat = reinterpret_cast<int8_t *>(smem + c.o_nat);
        s_adv = reinterpret_cast<float *>(smem + c.o_adv);
        s_ex = reinterpret_cast<float *>(smem + c.o_ex);
        s_sl = reinterpret_cast<float *>(smem + c.o_sl);
        s_tile = reinterpret_cast<float *>(smem + c.o_tile);
        float *s_misc = reinterpret_cast<float *>(smem + c.o_misc);
        s_k = s_misc + c.hd, s_v = s_misc + 2 * c.hd, s_tmp = s_misc + 3 * c.hd;  // [hd] each
        s_red = s_misc + 4 * c.hd;                                          // [128] reduction scratch
        s_ids = reinterpret_cast<int32_t *>(s_red + 256);                   // [64]
        s_w = s_red + 320;                                                  // [64]
        s_scalar = s_red + 384;                                             // a few broadcast scalars
    }
};

__device__ __noinline__ void mega_prefetch_attn_side(const MegaCtx &c, const MegaLayer &w) {
    l2_prefetch_rows(w.attn_q, c.a_lo, c.a_hi, 0, c.qd, c.eb);
    l2_prefetch_rows(w.attn_k, c.a_lo, c.a_hi, c.qd, c.kvd, c.eb);
    l2_prefetch_rows(w.attn_v, c.a_lo, c.a_hi, c.qd + c.kvd, c.kvd, c.eb);
    l2_prefetch_rows(w.attn_out, c.c_lo, c.c_hi, 0, c.E, c.qb);
    for (int r = c.cta; r < c.ne; r += c.G) l2_prefetch_bytes(reinterpret_cast<const uint8_t *>(w.router + (size_t)r * c.E), (size_t)c.E * 4);
}

// ---- phase A: (combine) + norm + Q8_K | Q, K, V rows. Returns after the tail's output when `tail`. ----
__device__ __noinline__ void mega_phase_a(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly, int il, bool tail) {
    const MegaPtrs S(c);
    const int tid = threadIdx.x, E = c.E, nu = c.nu, eb = c.eb, qd = c.qd, kvd = c.kvd;
    if (!tail && c.n_kv > 1) {
        // this layer's cached K and V rows (evicted since the last token): every CTA asks L2 for a slice of each
        const size_t kv_bytes = (size_t)(c.n_kv - 1) * kvd * (p.kv16 ? 2 : 4);
        const size_t per = ((kv_bytes + c.G - 1) / c.G + 15) & ~(size_t)15, off = per * c.cta;
        if (off < kv_bytes) {
            const size_t n = kv_bytes - off < per ? kv_bytes - off : per;
            l2_prefetch_bytes(reinterpret_cast<const uint8_t *>(ly.kc) + off, n);
            l2_prefetch_bytes(reinterpret_cast<const uint8_t *>(ly.vc) + off, n);
        }
    }
    if (il > 0) {
        // x += sum_e w_e * down_e, e in routing order, the expert sum started from 0 (layer.rs:243-258, 281-287).
        // All of a sweep's loads are issued before the first is used.
        for (int base = 0; base < E; base += kMegaElems * kMegaThreads) {
            float acc[kMegaElems];
#pragma unroll
            for (int q = 0; q < kMegaElems; q++) acc[q] = 0.0f;
            for (int e0 = 0; e0 < nu; e0 += 8) {
                float dv[8][kMegaElems];
#pragma unroll
                for (int e = 0; e < 8; e++)
#pragma unroll
                    for (int q = 0; q < kMegaElems; q++) {
                        const int i = base + tid + q * kMegaThreads;
                        dv[e][q] = (e0 + e < nu && i < E) ? __ldcg(p.e_down + (size_t)(e0 + e) * E + i) : 0.0f;
                    }
#pragma unroll
                for (int e = 0; e < 8; e++)
                    if (e0 + e < nu) {
                        const float we = S.s_w[e0 + e];
#pragma unroll
                        for (int q = 0; q < kMegaElems; q++) acc[q] = __fadd_rn(acc[q], __fmul_rn(we, dv[e][q]));
                    }
            }
#pragma unroll
            for (int q = 0; q < kMegaElems; q++) {
                const int i = base + tid + q * kMegaThreads;
                if (i < E) S.s_x[i] = __fadd_rn(S.s_x[i], acc[q]);
            }
        }
        __syncthreads();
        if (c.cta == 0 && p.trace_x)
            for (int i = tid; i < E; i += kMegaThreads) p.trace_x[(size_t)(il - 1) * E + i] = S.s_x[i];
    }
    mega_stamp(p, 14);
    norm_quant(S.s_x, tail ? p.output_norm : ly.attn_norm, S.s_sq, S.s_xn, S.s_nat, S.s_adv, E, p.eps, S.s_scalar, [&](int k) { mega_stamp(p, 22 + k); }, (p.fast & 1) != 0, S.s_red);
    if (tail) {
        if (c.cta == 0) {
            for (int i = tid; i < E; i += kMegaThreads) {
                p.x_out[i] = S.s_x[i];
                p.aq_out[i] = S.s_nat[i];
            }
            if (tid < eb) p.ad_out[tid] = S.s_adv[tid];
        }
        return;
    }
    mega_stamp(p, 15);
    auto map_a = [&](int row) -> RowRef {
        if (row < qd) return RowRef{ly.attn_q, (size_t)row * eb, 0, p.q + row};
        if (row < qd + kvd) return RowRef{ly.attn_k, (size_t)(row - qd) * eb, 0, p.k + (row - qd)};
        return RowRef{ly.attn_v, (size_t)(row - qd - kvd) * eb, 0, p.v + (row - qd - kvd)};
    };
    build_act_image(S.s_nat, S.s_act, eb);
    __syncthreads();
    mv_rows(map_a, eb, c.a_lo, c.a_hi, S.s_act, S.s_adv, S.s_ex);
}

// ---- phase B1: QK-norm, RoPE, KV store, scores of (kv head, chunk of positions) ----
__device__ __noinline__ void mega_phase_b1(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly) {
    const MegaPtrs S(c);
    if (!(c.b1_kvh < c.HKV && c.t_hi > c.t_lo)) return;
    const int tid = threadIdx.x, hd = c.hd, ratio = c.ratio, half = c.half, kvd = c.kvd, pos = c.pos, t_lo = c.t_lo;
    float *s_qraw = S.s_tile, *s_qr = S.s_tile + ratio * hd, *s_kt = S.s_tile + 2 * ratio * hd;  // [ratio][hd] x2, [chunk][hd + 4]
    const int stride = hd + 4, hd4 = hd / 4, cnt = c.t_hi - t_lo;
    const bool kv16 = p.kv16 != 0;
    const size_t kb = (size_t)c.b1_kvh * hd;  // element offset of this kv head inside a cache row
    // the chunk's cached K rows start their trip first (the row of this very position is made below)
    constexpr int kLd = 4;
    for (int i0 = 0; i0 < cnt * hd4; i0 += kLd * kMegaThreads) {
        float4 reg[kLd];
#pragma unroll
        for (int j = 0; j < kLd; j++) {
            const int idx = i0 + tid + j * kMegaThreads;
            const int r = idx / hd4, cc = idx - r * hd4;
            reg[j] = (idx < cnt * hd4 && t_lo + r != pos) ? kv_ld4(ly.kc, kb + (size_t)(t_lo + r) * kvd + 4 * cc, kv16, false)
                                                          : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (i0 == 0) {  // the group's q heads and this token's k, v head, raw
            for (int i = tid; i < ratio * hd; i += kMegaThreads) s_qraw[i] = __ldcg(p.q + (size_t)c.b1_kvh * ratio * hd + i);
            for (int i = tid; i < hd; i += kMegaThreads) {
                S.s_k[i] = __ldcg(p.k + (size_t)c.b1_kvh * hd + i);
                S.s_v[i] = __ldcg(p.v + (size_t)c.b1_kvh * hd + i);
            }
        }
#pragma unroll
        for (int j = 0; j < kLd; j++) {
            const int idx = i0 + tid + j * kMegaThreads;
            if (idx < cnt * hd4) {
                const int r = idx / hd4, cc = idx - r * hd4;
                *reinterpret_cast<float4 *>(s_kt + r * stride + 4 * cc) = reg[j];
            }
        }
    }
    __syncthreads();
    // per-head norm (layer.rs:62-79): each sum of squares walked in order by its own thread
    if ((tid & 31) == 0 && (tid >> 5) <= ratio) {
        const int j = tid >> 5;  // 0..ratio-1: q heads, ratio: the k head
        const float *sx = j < ratio ? s_qraw + j * hd : S.s_k;
        const float *w = j < ratio ? ly.q_norm : ly.k_norm;
        float scale = 1.0f;
        if (w) {
            float sum = 0.0f;
#pragma unroll 8
            for (int t = 0; t < hd; t++) sum = __fadd_rn(sum, __fmul_rn(sx[t], sx[t]));
            scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sum, (float)hd), p.eps)));
        }
        S.s_scalar[8 + j] = scale;
    }
    __syncthreads();
    // NeoX RoPE on (i, i + half) pairs, angles from the host-built table
    for (int idx = tid; idx < (ratio + 1) * half; idx += kMegaThreads) {
        const int j = idx / half, i = idx - j * half;
        const bool is_k = j == ratio;
        const float *sx = is_k ? S.s_k : s_qraw + j * hd;
        const float *w = is_k ? ly.k_norm : ly.q_norm;
        const float scale = S.s_scalar[8 + j];
        float a = sx[i], b = sx[i + half];
        if (w) {
            a = __fmul_rn(__fmul_rn(a, scale), __ldg(w + i));
            b = __fmul_rn(__fmul_rn(b, scale), __ldg(w + i + half));
        }
        const float2 sc = *reinterpret_cast<const float2 *>(p.rope_tab + ((size_t)pos * half + i) * 2);
        const float o0 = __fsub_rn(__fmul_rn(a, sc.y), __fmul_rn(b, sc.x));
        const float o1 = __fadd_rn(__fmul_rn(a, sc.x), __fmul_rn(b, sc.y));
        float *dst = is_k ? S.s_tmp : s_qr + j * hd;
        dst[i] = o0;
        dst[i + half] = o1;
    }
    __syncthreads();
    if (c.b1_has_pos) {  // this position's K (roped) and V go into the cache and into the chunk
        for (int i = tid; i < hd; i += kMegaThreads) {
            const float kept = kv_st(ly.kc, (size_t)pos * kvd + kb + i, S.s_tmp[i], kv16);
            kv_st(ly.vc, (size_t)pos * kvd + kb + i, S.s_v[i], kv16);
            s_kt[(pos - t_lo) * stride + i] = kept;  // (what a later token will read from the cache)
        }
        __syncthreads();
    }
    // logit[h][t] = (sum_d q[d] * k[t][d], d ascending) * scale (attention.rs:99-106): one thread per (head, position)
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn((float)hd));
    for (int idx = tid; idx < ratio * cnt; idx += kMegaThreads) {
        const int j = idx / cnt, r = idx - j * cnt;
        const float4 *kr = reinterpret_cast<const float4 *>(s_kt + r * stride);
        const float4 *q4 = reinterpret_cast<const float4 *>(s_qr + j * hd);
        float dot = 0.0f;
        float pa[16];  // four 16-byte reads ahead of the adds: the chain is then the dependent adds alone
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const float4 kv = kr[jj], qv = q4[jj];
            pa[4 * jj] = __fmul_rn(qv.x, kv.x), pa[4 * jj + 1] = __fmul_rn(qv.y, kv.y), pa[4 * jj + 2] = __fmul_rn(qv.z, kv.z), pa[4 * jj + 3] = __fmul_rn(qv.w, kv.w);
        }
        for (int d4 = 0; d4 < hd4; d4 += 4) {
            float pb[16];
            const int n4 = d4 + 4 < hd4 ? d4 + 4 : d4;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                const float4 kv = kr[n4 + jj], qv = q4[n4 + jj];
                pb[4 * jj] = __fmul_rn(qv.x, kv.x), pb[4 * jj + 1] = __fmul_rn(qv.y, kv.y), pb[4 * jj + 2] = __fmul_rn(qv.z, kv.z), pb[4 * jj + 3] = __fmul_rn(qv.w, kv.w);
            }
#pragma unroll
            for (int jj = 0; jj < 16; jj++) dot = __fadd_rn(dot, pa[jj]);
#pragma unroll
            for (int jj = 0; jj < 16; jj++) pa[jj] = pb[jj];
        }
        p.scores[(size_t)(c.b1_kvh * ratio + j) * p.max_kv + t_lo + r] = __fmul_rn(dot, scale);
    }
}

// ---- phase B2: softmax and weighted values of (head, column part) ----
__device__ __noinline__ void mega_phase_b2(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly) {
    const MegaPtrs S(c);
    if (c.cta >= c.H * kMegaSplit) return;
    const int tid = threadIdx.x, hd = c.hd, cols = c.cols, kvd = c.kvd, n_kv = c.n_kv, pos = c.pos;
    const int h = c.cta / kMegaSplit, cpart = c.cta - h * kMegaSplit, kvh = h / c.ratio;
    constexpr int kLd = 8;
    const bool kv16 = p.kv16 != 0;
    const size_t vb = (size_t)kvh * hd + (size_t)cpart * cols;  // element offset of this item's columns inside a cache row
    const int cols4 = cols / 4;
    float acc = 0.0f;
    for (int t0 = 0; t0 < n_kv; t0 += kMegaThreads) {
        const int cnt = min(kMegaThreads, n_kv - t0);
        // the V rows of this item's columns start their trip first
        float4 reg[kLd];
#pragma unroll
        for (int j = 0; j < kLd; j++) {
            const int idx = tid + j * kMegaThreads;
            const int r = idx / cols4, cc = idx - r * cols4;
            const int t = t0 + r;
            // (this position's row was stored by another CTA before the barrier: read it from L2)
            reg[j] = idx >= cnt * cols4 ? make_float4(0.f, 0.f, 0.f, 0.f)
                                        : kv_ld4(ly.vc, vb + (size_t)t * kvd + 4 * cc, kv16, t == pos);
        }
        if (t0 == 0) {
            // max (order-free), e[t] = exp(l - max), the sum walked in order (attention.rs:107-115)
            float lmax = -INFINITY;
            for (int t = tid; t < n_kv; t += kMegaThreads) {
                const float l = __ldcg(p.scores + (size_t)h * p.max_kv + t);
                S.s_sl[t] = l;
                lmax = fmaxf(lmax, l);
            }
            for (int off = 16; off > 0; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
            if ((tid & 31) == 0) S.s_red[tid >> 5] = lmax;
            __syncthreads();
            lmax = S.s_red[0];
            for (int w = 1; w < kMegaThreads / 32; w++) lmax = fmaxf(lmax, S.s_red[w]);
            for (int t = tid; t < n_kv; t += kMegaThreads) S.s_sl[t] = ref_expf(__fsub_rn(S.s_sl[t], lmax));
        }
        __syncthreads();  // (the exponentials are in place; a previous V tile is dead)
#pragma unroll
        for (int j = 0; j < kLd; j++) {
            const int idx = tid + j * kMegaThreads;
            if (idx < cnt * cols4) reinterpret_cast<float4 *>(S.s_tile)[idx] = reg[j];
        }
        if (p.fast & 4) {
            // the softmax sum by the CTA's reduction tree; the weighted values by kMegaThreads / cols groups of positions
            // per column, whose partial sums are added in group order after the last tile
            __syncthreads();
            if (t0 == 0) {
                float part = 0.0f;
                for (int t = tid; t < n_kv; t += kMegaThreads) part = __fadd_rn(part, S.s_sl[t]);
                const float total = block_sum(part, S.s_red);
                if (tid == 0) S.s_scalar[3] = __fdiv_rn(1.0f, total);
                __syncthreads();
            }
            const float inv = S.s_scalar[3];
            const int g = tid / cols, d = tid - g * cols, ng = min(kMegaThreads, c.E) / cols;  // (the partial sums go to s_sq: n_embd floats)
            const float *sl = S.s_sl + t0;
            if (g < ng)
                for (int r = g; r < cnt; r += ng) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(sl[r], inv), S.s_tile[r * cols + d]));
            __syncthreads();
            continue;
        }
        if (t0 == 0 && tid == 0) S.s_scalar[3] = __fdiv_rn(1.0f, chain_sum(S.s_sl, n_kv, 0.0f));
        __syncthreads();
        // out[d] = sum_t (e[t] * inv) * v[t][d], t ascending (:116-121)
        if (tid < cols) {
            const float inv = S.s_scalar[3];
            const float *sl = S.s_sl + t0, *tile = S.s_tile + tid;
            int r = 0;
            if (cnt >= 16) {
                float pa[16], pb[16];
#pragma unroll
                for (int j = 0; j < 16; j++) pa[j] = __fmul_rn(__fmul_rn(sl[j], inv), tile[j * cols]);
                for (; r + 16 <= cnt; r += 16) {
                    const int rn = (r + 32 <= cnt) ? r + 16 : r;
#pragma unroll
                    for (int j = 0; j < 16; j++) pb[j] = __fmul_rn(__fmul_rn(sl[rn + j], inv), tile[(rn + j) * cols]);
#pragma unroll
                    for (int j = 0; j < 16; j++) acc = __fadd_rn(acc, pa[j]);
#pragma unroll
                    for (int j = 0; j < 16; j++) pa[j] = pb[j];
                }
            }
            for (; r < cnt; r++) acc = __fadd_rn(acc, __fmul_rn(__fmul_rn(sl[r], inv), tile[r * cols]));
        }
        __syncthreads();
    }
    if (p.fast & 4) {
        const int ng = min(kMegaThreads, c.E) / cols;
        if (tid < ng * cols) S.s_sq[tid] = acc;  // [group][column]
        __syncthreads();
        if (tid < cols) {
            acc = S.s_sq[tid];
            for (int g = 1; g < ng; g++) acc = __fadd_rn(acc, S.s_sq[g * cols + tid]);
        }
    }
    if (tid < cols) p.attn[(size_t)h * hd + (size_t)cpart * cols + tid] = acc;
}

// ---- phase C: Q8_K of the attention output | attn_out rows ----
__device__ __noinline__ void mega_phase_c(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly) {
    const MegaPtrs S(c);
    const int tid = threadIdx.x, qb = c.qb;
    auto map_c = [&](int row) -> RowRef { return RowRef{ly.attn_out, (size_t)row * qb, 0, p.xb2 + row}; };
    const int warp = tid >> 5, lane = tid & 31;
    for (int b = warp; b < qb; b += kMegaThreads / 32) {
        const float4 a = __ldcg(reinterpret_cast<const float4 *>(p.attn + b * 256 + lane * 8)), c4 = __ldcg(reinterpret_cast<const float4 *>(p.attn + b * 256 + lane * 8) + 1);
        const float v[8] = {a.x, a.y, a.z, a.w, c4.x, c4.y, c4.z, c4.w};
        q8k_quantize_block(v, lane, S.s_nat + b * 256, S.s_adv + b, nullptr);
    }
    __syncthreads();
    build_act_image(S.s_nat, S.s_act, qb);
    __syncthreads();
    mv_rows(map_c, qb, c.c_lo, c.c_hi, S.s_act, S.s_adv, S.s_ex);
}

// ---- phase D: x += attn_out, FFN norm, Q8_K (kept for E) | router logits ----
__device__ __noinline__ void mega_phase_d(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly) {
    const MegaPtrs S(c);
    const int tid = threadIdx.x, E = c.E;
    // the router row this CTA dots (asked of L2 a layer ago) and attn_out's result, read before the norm's chain
    float wr_pre[kMegaElems], rv[kMegaElems];
#pragma unroll
    for (int q = 0; q < kMegaElems; q++) {
        const int i = tid + q * kMegaThreads;
        rv[q] = i < E ? __ldcg(p.xb2 + i) : 0.0f;
        wr_pre[q] = (c.cta < c.ne && i < E) ? __ldg(ly.router + (size_t)c.cta * E + i) : 0.0f;
    }
#pragma unroll
    for (int q = 0; q < kMegaElems; q++) {
        const int i = tid + q * kMegaThreads;
        if (i < E) S.s_x[i] = __fadd_rn(S.s_x[i], rv[q]);
    }
    for (int i = tid + kMegaElems * kMegaThreads; i < E; i += kMegaThreads) S.s_x[i] = __fadd_rn(S.s_x[i], __ldcg(p.xb2 + i));
    __syncthreads();
    norm_quant(S.s_x, ly.ffn_norm, S.s_sq, S.s_xn, S.s_nat, S.s_adv, E, p.eps, S.s_scalar, [](int) {}, (p.fast & 1) != 0, S.s_red);
    build_act_image(S.s_nat, S.s_act, c.eb);  // kept for phase E
    mega_stamp(p, 17);
    if (p.fast & 2) {
        // the same products, summed by the CTA's reduction tree
        for (int r = c.cta; r < c.ne; r += c.G) {
            const float *wr = ly.router + (size_t)r * E;
            float part = 0.0f;
            if (r == c.cta) {
#pragma unroll
                for (int q = 0; q < kMegaElems; q++) {
                    const int i = tid + q * kMegaThreads;
                    if (i < E) part = __fadd_rn(part, __fmul_rn(wr_pre[q], S.s_xn[i]));
                }
                for (int i = tid + kMegaElems * kMegaThreads; i < E; i += kMegaThreads) part = __fadd_rn(part, __fmul_rn(__ldg(wr + i), S.s_xn[i]));
            } else {
                for (int i = tid; i < E; i += kMegaThreads) part = __fadd_rn(part, __fmul_rn(__ldg(wr + i), S.s_xn[i]));
            }
            const float y = block_sum(part, S.s_red);
            if (tid == 0) p.logits[r] = y;
        }
        return;
    }
    for (int r = c.cta; r < c.ne; r += c.G) {
        // y = fold(-0.0, +) of w[r][t] * x[t], t ascending (crates/llamd-models/src/model.rs:253-263)
        const float *wr = ly.router + (size_t)r * E;
        __syncthreads();
        if (r == c.cta) {
#pragma unroll
            for (int q = 0; q < kMegaElems; q++) {
                const int i = tid + q * kMegaThreads;
                if (i < E) S.s_sq[i] = __fmul_rn(wr_pre[q], S.s_xn[i]);
            }
            for (int i = tid + kMegaElems * kMegaThreads; i < E; i += kMegaThreads) S.s_sq[i] = __fmul_rn(__ldg(wr + i), S.s_xn[i]);
        } else {
            for (int i = tid; i < E; i += kMegaThreads) S.s_sq[i] = __fmul_rn(__ldg(wr + i), S.s_xn[i]);
        }
        __syncthreads();
        if (tid == 0) p.logits[r] = chain_sum(S.s_sq, E, -0.0f);
    }
}

__device__ __forceinline__ int mega_expert_of(const MegaCtx &c, int slot) {
    const MegaPtrs S(c);
    const int ex = S.s_ids[slot];
    return (ex < 0 || ex >= c.ne) ? 0 : ex;
}

// ---- phase E: route | gate and up rows of the routed experts ----
__device__ __noinline__ void mega_phase_e(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly, int il) {
    const MegaPtrs S(c);
    const int tid = threadIdx.x, ne = c.ne, nu = c.nu, ffe = c.ffe, eb = c.eb, E = c.E, fb = c.fb;
    for (int i = tid; i < ne; i += kMegaThreads) S.s_sq[i] = __ldcg(p.logits + i);
    __syncthreads();
    mega_stamp(p, 18);
    route_cta(S.s_sq, ne, nu, S.s_ids, S.s_w, S.s_red);
    mega_stamp(p, 19);
    if (c.cta == 0 && tid < nu) {
        p.expert_ids[tid] = S.s_ids[tid];
        p.expert_w[tid] = S.s_w[tid];
        if (p.trace_ids) p.trace_ids[(size_t)il * nu + tid] = S.s_ids[tid];
    }
    auto map_e = [&](int row) -> RowRef {
        const int slot = row / (2 * ffe), rem = row - slot * 2 * ffe, mat = rem / ffe, r = rem - mat * ffe;
        return RowRef{mat ? ly.up : ly.gate, ((size_t)mega_expert_of(c, slot) * ffe + r) * eb, 0, (mat ? p.e_up : p.e_gate) + (size_t)slot * ffe + r};
    };
    // the down projection's rows are known too (the ids are): ask L2 for them now, they are needed a phase later
    for (int seg = c.f_lo; seg < c.f_hi;) {
        const int slot = seg / E, seg_hi = min(c.f_hi, (slot + 1) * E);
        const size_t row0 = (size_t)mega_expert_of(c, slot) * E;
        l2_prefetch_units(ly.down, (row0 + (seg - slot * E)) * fb, (row0 + (seg_hi - slot * E)) * fb);
        seg = seg_hi;
    }
    mega_stamp(p, 20);
    mv_rows(map_e, eb, c.e_lo, c.e_hi, S.s_act, S.s_adv, S.s_ex);  // the activation image is phase D's
}

// ---- phase F: silu(gate) * up, Q8_K, for the slots of this CTA's rows | down rows ----
__device__ __noinline__ void mega_phase_f(const MegaParams &p, const MegaCtx &c, const MegaLayer &ly) {
    const MegaPtrs S(c);
    const int tid = threadIdx.x, ffe = c.ffe, fb = c.fb, E = c.E, slot_lo = c.slot_lo;
    auto map_f = [&](int row) -> RowRef {
        const int slot = row / E, r = row - slot * E;
        return RowRef{ly.down, ((size_t)mega_expert_of(c, slot) * E + r) * fb, slot - slot_lo, p.e_down + (size_t)slot * E + r};
    };
    if (c.f_hi > c.f_lo) {
        const int warp = tid >> 5, lane = tid & 31, nslot = c.slot_hi - slot_lo + 1;
        if (nslot * ffe <= E) {
            // silu(gate) * up of the slots' elements, one or two per thread (a warp per block would leave most of the CTA idle
            // behind eight dependent exponentials per lane), then a warp per block quantizes from shared memory
            const size_t base = (size_t)slot_lo * ffe;
            for (int i = tid; i < nslot * ffe; i += kMegaThreads) S.s_xn[i] = silu_mul(__ldcg(p.e_gate + base + i), __ldcg(p.e_up + base + i));
            __syncthreads();
            for (int blk = warp; blk < nslot * fb; blk += kMegaThreads / 32) {
                const float4 a = reinterpret_cast<const float4 *>(S.s_xn + blk * 256 + lane * 8)[0], b4 = reinterpret_cast<const float4 *>(S.s_xn + blk * 256 + lane * 8)[1];
                const float v[8] = {a.x, a.y, a.z, a.w, b4.x, b4.y, b4.z, b4.w};
                q8k_quantize_block(v, lane, S.s_nat + blk * 256, S.s_adv + blk, nullptr);
            }
        } else
            for (int blk = warp; blk < nslot * fb; blk += kMegaThreads / 32) {
                const int sl_ = slot_lo + blk / fb, b = blk - (blk / fb) * fb;
                const size_t base = (size_t)sl_ * ffe + (size_t)b * 256 + lane * 8;
                const float4 g0 = __ldcg(reinterpret_cast<const float4 *>(p.e_gate + base)), g1 = __ldcg(reinterpret_cast<const float4 *>(p.e_gate + base) + 1);
                const float4 u0 = __ldcg(reinterpret_cast<const float4 *>(p.e_up + base)), u1 = __ldcg(reinterpret_cast<const float4 *>(p.e_up + base) + 1);
                const float v[8] = {silu_mul(g0.x, u0.x), silu_mul(g0.y, u0.y), silu_mul(g0.z, u0.z), silu_mul(g0.w, u0.w),
                                    silu_mul(g1.x, u1.x), silu_mul(g1.y, u1.y), silu_mul(g1.z, u1.z), silu_mul(g1.w, u1.w)};
                q8k_quantize_block(v, lane, S.s_nat + blk * 256, S.s_adv + blk, nullptr);
            }
        __syncthreads();
        build_act_image(S.s_nat, S.s_act, nslot * fb);
        __syncthreads();
    }
    mega_stamp(p, 21);
    mv_rows(map_f, fb, c.f_lo, c.f_hi, S.s_act, S.s_adv, S.s_ex);
}

__global__ void __launch_bounds__(kMegaThreads, 1) decode_mega_kernel(const __grid_constant__ MegaParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ MegaCtx ctx;
    __shared__ bool s_flag;
    const int tid = threadIdx.x, cta = blockIdx.x, G = gridDim.x;
    if (tid == 0) {
        MegaCtx c;
        c.E = p.E, c.H = p.H, c.HKV = p.HKV, c.hd = p.hd, c.nu = p.nu, c.ffe = p.ffe, c.ne = p.n_expert;
        c.qd = c.H * c.hd, c.kvd = c.HKV * c.hd, c.eb = c.E / 256, c.qb = c.qd / 256, c.fb = c.ffe / 256;
        c.ratio = c.H / c.HKV, c.half = c.hd / 2, c.cols = c.hd / kMegaSplit;
        const MegaSmem L = mega_smem(c.E, c.qd, c.hd, p.act_blocks, p.sl_floats, c.ne, p.ktile_rows, c.ratio);
        c.o_x = (uint32_t)L.x, c.o_xn = (uint32_t)L.xn, c.o_sq = (uint32_t)L.sq, c.o_act = (uint32_t)L.act, c.o_nat = (uint32_t)L.nat;
        c.o_adv = (uint32_t)L.adv, c.o_ex = (uint32_t)L.ex, c.o_sl = (uint32_t)L.sl, c.o_tile = (uint32_t)L.tile, c.o_misc = (uint32_t)L.misc;
        c.cta = cta, c.G = G, c.pos = p.meta[1], c.n_kv = c.pos + 1;
        // row ranges of the phases (the same every layer)
        const int rows_a = c.qd + 2 * c.kvd, rpc_a = (rows_a + G - 1) / G;
        c.a_lo = min(cta * rpc_a, rows_a), c.a_hi = min(c.a_lo + rpc_a, rows_a);
        const int rpc_c = (c.E + G - 1) / G;
        c.c_lo = min(cta * rpc_c, c.E), c.c_hi = min(c.c_lo + rpc_c, c.E);
        const int rows_e = c.nu * 2 * c.ffe, rpc_e = (rows_e + G - 1) / G;
        c.e_lo = min(cta * rpc_e, rows_e), c.e_hi = min(c.e_lo + rpc_e, rows_e);
        const int rows_f = c.nu * c.E, rpc_f = (rows_f + G - 1) / G;
        c.f_lo = min(cta * rpc_f, rows_f), c.f_hi = min(c.f_lo + rpc_f, rows_f);
        c.slot_lo = c.f_lo / c.E, c.slot_hi = c.f_hi > c.f_lo ? (c.f_hi - 1) / c.E : c.slot_lo;
        // attention, first half: CTA -> (kv head, chunk of positions); second half: CTA -> (head, column part)
        const int ncp = G / c.HKV;  // position chunks per kv head
        c.b1_kvh = cta / ncp;
        const int chunk = cta - c.b1_kvh * ncp, ppc = (c.n_kv + ncp - 1) / ncp;
        c.t_lo = min(chunk * ppc, c.n_kv);
        c.t_hi = c.b1_kvh < c.HKV ? min(c.t_lo + ppc, c.n_kv) : c.t_lo;
        c.b1_has_pos = c.b1_kvh < c.HKV && c.pos >= c.t_lo && c.pos < c.t_hi;
        ctx = c;
    }
    __syncthreads();
    const int token = p.meta[0];
    unsigned int bar_target = 0;
    long long prof_c0 = 0;
    unsigned long long prof_t0 = 0;
    if (p.prof && cta == 0 && tid == 0) {
        for (int k = 0; k < 32; k++) s_mega_prof[k] = 0;
        prof_c0 = clock64();
        prof_t0 = s_mega_prof[32] = global_ns();
    }
#define MEGA_STAMP(k) mega_stamp(p, k)
#define MEGA_BARRIER(k)                                       \
    do {                                                      \
        if (!grid_barrier(p, bar_target, &s_flag)) return;    \
        MEGA_STAMP(k);                                        \
    } while (0)

    // ---- embed: one row of token_embd, d * sc * q (crates/llamd-quant/src/lib.rs:181-226) ----
    {
        const int E = p.E, eb = E / 256;
        float *sx0 = reinterpret_cast<float *>(smem + ctx.o_x);
        for (int i = tid; i < E; i += kMegaThreads) {
            const size_t unit = (size_t)token * eb + (i >> 8);
            const int e = i & 255;
            const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(p.tok_embd + t32_d_offset(unit)));
            const float sc = (float)(int8_t)p.tok_embd[t32_scale_offset(unit) + (e >> 4)];
            sx0[i] = __fmul_rn(__fmul_rn(d, sc), (float)t32_weight(p.tok_embd, unit, e));
        }
    }
    mega_prefetch_attn_side(ctx, p.layers[0]);
    __syncthreads();

    for (int il = 0; il <= p.n_layer; il++) {
        const bool tail = il == p.n_layer;  // after the last layer: combine + output norm only
        const MegaLayer &ly = p.layers[tail ? p.n_layer - 1 : il];
        mega_phase_a(p, ctx, ly, il, tail);
        if (tail) break;
        MEGA_STAMP(0);
        MEGA_BARRIER(1);
        mega_phase_b1(p, ctx, ly);
        MEGA_STAMP(2);
        MEGA_BARRIER(3);
        mega_phase_b2(p, ctx, ly);
        MEGA_STAMP(4);
        MEGA_BARRIER(5);
        mega_phase_c(p, ctx, ly);
        MEGA_STAMP(6);
        MEGA_BARRIER(7);
        mega_phase_d(p, ctx, ly);
        MEGA_STAMP(8);
        MEGA_BARRIER(9);
        mega_phase_e(p, ctx, ly, il);
        if (il + 1 < p.n_layer) mega_prefetch_attn_side(ctx, p.layers[il + 1]);  // streams behind the expert weights
        MEGA_STAMP(10);
        MEGA_BARRIER(11);
        mega_phase_f(p, ctx, ly);
        MEGA_STAMP(12);
        MEGA_BARRIER(13);
    }
    if (p.prof && cta == 0 && tid == 0) {
        s_mega_prof[30] = (unsigned long long)(clock64() - prof_c0);  // SM cycles and nanoseconds of the whole token: their
        s_mega_prof[31] = global_ns() - prof_t0;                      // ratio is the clock the SM really ran at
        for (int k = 0; k < 32; k++) p.prof[k] += s_mega_prof[k];
    }
#undef MEGA_BARRIER
#undef MEGA_STAMP
}

}  // namespace llamd

using namespace llamd;

namespace llamd {

// Shared memory the kernel needs for these dimensions, or 0 when they do not fit it.
size_t mega_smem_bytes(const llamd_hparams &hp, int max_kv, int *act_blocks, int *sl_floats, int *ktile_rows_out) {
    const int E = hp.n_embd, qd = hp.n_head * hp.head_dim, ffe = hp.n_ff_expert;
    int ab = E / 256;
    if (qd / 256 > ab) ab = qd / 256;
    if (2 * (ffe / 256) > ab) ab = 2 * (ffe / 256);
    const int sl = (max_kv + 3) & ~3;
    if (act_blocks) *act_blocks = ab;
    if (sl_floats) *sl_floats = sl;
    int dev = 0, sms = 1;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int ncp = sms / hp.n_head_kv > 0 ? sms / hp.n_head_kv : 1;
    const int ktile_rows = (max_kv + ncp - 1) / ncp;
    if (ktile_rows_out) *ktile_rows_out = ktile_rows;
    return mega_smem(E, qd, hp.head_dim, ab, sl, hp.n_expert, ktile_rows, hp.n_head / hp.n_head_kv).total;
}

// Can this model run in the resident kernel on the current device? (dimension and shared-memory limits)
bool mega_supported(const llamd_hparams &hp, int max_kv) {
    const int E = hp.n_embd, qd = hp.n_head * hp.head_dim, ffe = hp.n_ff_expert, hd = hp.head_dim;
    if (E % 256 || qd % 256 || ffe % 256 || hd % (4 * kMegaSplit) || hd > kMegaThreads / 2 || hp.n_head % hp.n_head_kv) return false;
    if (E / 256 > kMegaThreads || qd / 256 > kMegaThreads || hp.n_expert_used > 64 || hp.n_expert > kMegaThreads || hp.n_expert_used > hp.n_expert) return false;
    int dev = 0, sms = 0, optin = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (hp.n_head * kMegaSplit > sms || hp.n_expert_used > sms) return false;  // one attention item per CTA; a CTA's down rows span <= 2 slots
    if (hp.n_head_kv > sms) return false;  // one score chunk per CTA and kv head
    return mega_smem_bytes(hp, max_kv, nullptr, nullptr, nullptr) <= (size_t)optin;
}

// Queue the resident pass for one token (meta = [token, pos] on the device). `bar` and `status` are one word each;
// the barrier word is cleared here, in stream order, before the launch.
void launch_decode_mega(MegaParams p, const llamd_hparams &hp) {
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = mega_smem_bytes(hp, p.max_kv, &p.act_blocks, &p.sl_floats, &p.ktile_rows);
    static size_t configured = 0;
    if (smem > configured) {
        const cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error(e, "resident decode kernel: shared memory attribute");
            return;
        }
        configured = smem;
    }
    static int resident = -1;
    if (resident < 0) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel, kMegaThreads, smem) != cudaSuccess) per_sm = 0;
        resident = per_sm;
    }
    if (resident < 1) {
        set_error_msg("resident decode kernel: a CTA does not fit an SM with these dimensions");
        return;
    }
    if (cudaMemsetAsync(p.bar, 0, sizeof(unsigned int), stream()) != cudaSuccess) {
        set_error(cudaGetLastError(), "resident decode kernel: barrier reset");
        return;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sms);
    cfg.blockDim = dim3(kMegaThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident at once: the grid barriers rely on it
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    g_launches++;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, decode_mega_kernel, p);
    if (e != cudaSuccess) set_error(e, "resident decode kernel");
}

}  // namespace llamd
