// Q6_K x Q8_K for MANY tokens on the integer tensor path: the grouped expert
// GEMM of prefill (and the QKV / attn_out projections of a prefill tile).
//
// The reference's arithmetic (crates/llamd-quant/src/dot.rs:138-196) keeps, per
// (row, token, block b, residue r = element mod 8), the integer
//     aux[r] = sum over 16 groups g, 2 elements s of  scale[g] * w[16g+8s+r] * a[16g+8s+r]
// and then accumulates in f32, in block order:  sums[r] += (f16(d_b) * ad_b) * (float)aux[r].
// That fixes the shape of the tensor-core formulation: each (b, r) is its own
// 32-deep contraction whose result needs its own f32 scaling, so the MMA is
//     D[16 rows x 8 tokens] = A[16 x 32] * B[32 x 8]     (mma.sync m16n8k32, s8 x s8 -> s32)
// with A = scale[g]*w folded per row and B = the token's Q8_K bytes of that
// residue. scale*w needs 13 bits, so A is split exactly into hi = U >> 6 and
// lo = U & 63 (two MMAs, aux = 64*hi + lo). Integer results are exact in any
// order; the f32 tail runs in the reference's order inside each thread (a
// thread owns all eight residues of its four (row, token) outputs), so the
// result is bit-identical to the scalar loop and to the dp4a matvec kernels.
// This mirrors the role of crates/llamd-vulkan/shaders/q6k_expert_cm.comp
// (cooperative-matrix s8 GEMM with f32 scaling per 16-K group).
//
// A CTA owns 16 weight rows of one matrix/expert at a time: it folds and splits
// those rows once into shared memory in MMA fragment order, then each warp walks
// token tiles of 8. Activations are read as residue-major words (one 32-bit word
// = the four bytes of one MMA k-quad) prepared by q8k_residue_major_kernel.
// Two launch shapes share the code:
//   grouped  grid (row tiles, experts), 4 warps: one fold, then all of the expert's tokens;
//   dense    a fixed number of resident CTAs (8 warps) split the (row tile, 64-token chunk)
//            items evenly; a CTA folds a row tile once for the consecutive chunks it owns.
#include "q6k_layout.cuh"

namespace llamd {

constexpr int kGemmRows = 16;
constexpr int kTokStride = 68;  // words per staged token row: 16-byte aligned, conflict-free fragment reads
constexpr int kChunkTiles = 8;  // token tiles per dense work item

struct GemmParams {
    const uint8_t *w[3];  // tiled Q6_K; up to three matrices that share the activations
    float *out[3];
    int rows[3];
    int tile_begin[3];    // first row tile (blockIdx.x) of each matrix
    int njobs;
    int nb;               // blocks per row
    const uint32_t *aq_rm;  // activations, residue-major words: [index][nb][8 residues][8 words]
    const float *ad;        // [index][nb]
    // token groups: group e = pairs [gstart[e], gstart[e]+gcount[e]); pair p reads activation act_map[p] and writes
    // output row block out_map[p]. gstart == null: one group of n_tokens pairs. maps == null: identity.
    const int32_t *gstart, *gcount, *act_map, *out_map;
    int n_tokens;
    long long expert_units;  // blocks between consecutive experts in w
    int prefetch_ahead;      // grouped kernel: CTA i asks L2 for the weights of CTA i + prefetch_ahead (0: off)
    // expert parallelism: output row block o lives on GPU o / out_div, at local row block o % out_div (null: out[j])
    float *const *out_tab;
    int out_div;
    // pre-folded copies of the matrices (grouped kernel; null: fold from w): [expert][row tile] images of fold_tile_bytes,
    // each exactly what fold_row_tile leaves in shared memory (A fragments, then the 16 x nb block scales)
    const uint8_t *folded[3];
    long long fold_tile_bytes;
};

// Ask L2 for the tiles that hold the 16 x nb blocks starting at block `unit0` (a hint: nothing waits on it).
__device__ __forceinline__ void prefetch_row_tile(const uint8_t *w, size_t unit0, int live_rows, int nb) {
    const size_t t_lo = unit0 >> 5, t_hi = (unit0 + (size_t)min(live_rows, kGemmRows) * nb - 1) >> 5;
    const uint8_t *src = w + t_lo * kTileBytes;
    const uint32_t bytes = (uint32_t)((t_hi - t_lo + 1) * kTileBytes);  // 6720 = 16 * 420
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mma_s8(int (&c)[4], const uint4 &a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "r"(0));
}

// Natural-order Q8_K quants -> residue-major words (t32_element order), one thread per word.
__global__ void q8k_residue_major_kernel(const int8_t *__restrict__ aq, uint32_t *__restrict__ rm, size_t nblocks) {
    pdl_trigger();
    pdl_wait();
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= nblocks * 64) return;
    const size_t blk = i >> 6;
    const int r = (int)(i >> 3) & 7, j = (int)i & 7;
    const uint8_t *src = reinterpret_cast<const uint8_t *>(aq) + blk * 256;
    rm[i] = (uint32_t)src[t32_element(r, j, 0)] | ((uint32_t)src[t32_element(r, j, 1)] << 8) | ((uint32_t)src[t32_element(r, j, 2)] << 16) |
            ((uint32_t)src[t32_element(r, j, 3)] << 24);
}

// ---- fold the scales into the weights, split hi/lo, store in fragment order ----
// One thread per (row, block, half): residues 4h..4h+3 of the block are 6 of its 12 code chunks, fetched with
// coalesced 16-byte loads (consecutive threads = consecutive blocks of the tile), all issued before any is used.
//
// Two weights of one scale group are folded by ONE 32-bit multiply-add: with q = w + 32 in [0, 63],
//     (q0 | q1 << 16) * sc + (C | C << 16),  C = 16384 - 32*sc
// is, as an integer, sum_i (sc*(q_i - 32) + 16384) << 16i, and every term lies in [12288, 20480], so the two 16-bit
// fields hold V_i = U_i + 16384 with no carry between them. 16384 is a multiple of 64*256: V & 63 = U & 63 and the
// low byte of V >> 6 is the two's-complement byte of U >> 6.
struct FoldItem {
    uint32_t S[24];  // six 16-byte code chunks: residues 4h..4h+3 of one block
    uint4 scw;       // its 16 scales
    float d;
    int rb, half;    // row_local * nb + block, which half; rb < 0: nothing to do
};

__device__ __forceinline__ void fold_load(FoldItem &f, const uint8_t *__restrict__ w, size_t unit0, int live_rows, int nb, int it) {
    const int n_units = kGemmRows * nb;
    f.rb = -1;
    if (it >= 2 * n_units) return;
    f.half = it >= n_units ? 1 : 0;
    f.rb = it - f.half * n_units;
    f.scw = make_uint4(0, 0, 0, 0);
    f.d = 0.0f;
    if (f.rb / nb < live_rows) {
        const size_t unit = unit0 + f.rb;
        const uint8_t *tile = w + (unit >> 5) * kTileBytes;
        const int sl = (int)(unit & 31);
        const uint4 *cp = reinterpret_cast<const uint4 *>(tile) + sl + f.half * 6 * 32;
#pragma unroll
        for (int c = 0; c < 6; c++) {
            const uint4 v = __ldg(cp + c * 32);
            f.S[4 * c + 0] = v.x; f.S[4 * c + 1] = v.y; f.S[4 * c + 2] = v.z; f.S[4 * c + 3] = v.w;
        }
        f.scw = __ldg(reinterpret_cast<const uint4 *>(tile + kTileScaleOff) + sl);
        f.d = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(tile + kTileDOff) + sl));
    } else {
        // a row past the matrix: with zero scales the fold below yields hi = lo = 0 whatever the codes
#pragma unroll
        for (int c = 0; c < 24; c++) f.S[c] = 0;
    }
}

__device__ __forceinline__ void fold_store(const FoldItem &f, int nb, uint4 *s_frag, float *s_d) {
    if (f.rb < 0) return;
    const int row_l = f.rb / nb, b = f.rb - row_l * nb;
    if (f.half == 0) s_d[f.rb] = f.d;
    uint32_t sc[16], crep[16];
    {
        const uint32_t ws[4] = {f.scw.x, f.scw.y, f.scw.z, f.scw.w};
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int v = (int)(int8_t)(ws[i >> 2] >> (8 * (i & 3)));
            sc[i] = (uint32_t)v;
            crep[i] = (uint32_t)(16384 - 32 * v) * 0x00010001u;
        }
    }
#pragma unroll
    for (int rl = 0; rl < 4; rl++) {
        const int r = 4 * f.half + rl;
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const uint32_t s0 = f.S[6 * rl + 3 * m], s1 = f.S[6 * rl + 3 * m + 1], s2 = f.S[6 * rl + 3 * m + 2];
            // the stored byte is (q ^ 0x20) << 2; the fourth word's codes are the low bit pairs of the other three
            uint32_t qb[4];
            qb[0] = ((s0 >> 2) & 0x3F3F3F3Fu) ^ 0x20202020u;
            qb[1] = ((s1 >> 2) & 0x3F3F3F3Fu) ^ 0x20202020u;
            qb[2] = ((s2 >> 2) & 0x3F3F3F3Fu) ^ 0x20202020u;
            qb[3] = (((s0 << 4) & 0x30303030u) | ((s1 << 2) & 0x0C0C0C0Cu) | (s2 & 0x03030303u)) ^ 0x20202020u;
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int jw = 4 * m + i;  // bytes 0,1 of word jw belong to scale group 2jw, bytes 2,3 to 2jw+1
                const uint32_t v01 = __byte_perm(qb[i], 0u, 0x4140) * sc[2 * jw] + crep[2 * jw];
                const uint32_t v23 = __byte_perm(qb[i], 0u, 0x4342) * sc[2 * jw + 1] + crep[2 * jw + 1];
                const uint32_t lo = __byte_perm(v01, v23, 0x6420) & 0x3F3F3F3Fu;
                const uint32_t hi = __byte_perm(v01 >> 6, v23 >> 6, 0x6420);
                // fragment word q of lane L: row = L/4 + 8(q&1), word jw = L%4 + 4(q>>1).
                // Lane L's 16 bytes sit in slot L ^ (L >> 3) ^ (b & 7): the threads of a warp here write the same jw
                // of neighbouring rows and blocks, and the swizzle spreads them over all eight 16-byte bank groups
                // (the readers of one fragment still touch 32 distinct slots).
                const int L = (row_l & 7) * 4 + (jw & 3), q = (row_l >> 3) + 2 * (jw >> 2);
                const int P = L ^ (L >> 3) ^ (b & 7);
                reinterpret_cast<uint32_t *>(s_frag + ((size_t)(b * 8 + r) * 2 + 0) * 32 + P)[q] = hi;
                reinterpret_cast<uint32_t *>(s_frag + ((size_t)(b * 8 + r) * 2 + 1) * 32 + P)[q] = lo;
            }
        }
    }
}

// HOIST: two items per thread and trip, the loads of both in flight before either is folded (more registers).
template <int THREADS, bool HOIST>
__device__ __forceinline__ void fold_row_tile(const uint8_t *__restrict__ w, size_t unit0, int live_rows, int nb, uint4 *s_frag, float *s_d,
                                              int tid) {
    const int n_items = 2 * kGemmRows * nb;
    if (HOIST) {
        for (int base = 0; base < n_items; base += 2 * THREADS) {
            FoldItem fa, fb;
            fold_load(fa, w, unit0, live_rows, nb, base + tid);
            fold_load(fb, w, unit0, live_rows, nb, base + THREADS + tid);
            fold_store(fa, nb, s_frag, s_d);
            fold_store(fb, nb, s_frag, s_d);
        }
    } else {
        for (int base = 0; base < n_items; base += THREADS) {
            FoldItem fa;
            fold_load(fa, w, unit0, live_rows, nb, base + tid);
            fold_store(fa, nb, s_frag, s_d);
        }
    }
}

// ---- token tiles of 8 against the folded row tile ----
// Warp `warp` of `nwarps` takes tiles tile_lo + warp, + nwarps, ... below tile_hi. Per block b the warp copies its
// 8 tokens' 256 activation bytes into its own buffer with coalesced 16-byte loads; the next block's bytes wait in
// registers meanwhile.
template <int DEPTH>
__device__ __forceinline__ void mma_token_tiles(const GemmParams &p, int j, int row0, int rows, int first, int count, int tile_lo, int tile_hi,
                                                const uint4 *s_frag, const float *s_d, uint32_t *s_b, int warp, int nwarps, int lane) {
    const int nb = p.nb;
    const int g4 = lane >> 2, q4 = lane & 3;
    const int m0 = g4, m1 = g4 + 8;
    for (int tn = tile_lo + warp; tn < tile_hi; tn += nwarps) {
        const int n0 = tn * 8;
        // the two tokens whose outputs this lane owns
        const int pa0 = first + min(n0 + 2 * q4, count - 1), pa1 = first + min(n0 + 2 * q4 + 1, count - 1);
        const long long ia0 = p.act_map ? p.act_map[pa0] : pa0, ia1 = p.act_map ? p.act_map[pa1] : pa1;
        // staging: 8 tokens x 16 pieces of 16 bytes = 128 pieces, four per lane
        const uint4 *src[4];
        int dsto[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int chunk = lane + 32 * i;
            const int tok = chunk >> 4, c16 = chunk & 15;
            const int pt = first + min(n0 + tok, count - 1);
            const long long it = p.act_map ? p.act_map[pt] : pt;
            src[i] = reinterpret_cast<const uint4 *>(p.aq_rm + (size_t)it * nb * 64) + c16;
            dsto[i] = tok * kTokStride + c16 * 4;
        }
        float sums[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int r = 0; r < 8; r++) sums[i][r] = 0.0f;
        // The tokens' activation bytes of the next DEPTH blocks wait in registers. (DEPTH 3-4 was measured: no faster than
        // 1 -- the warps wait on the tile's own copy, on shared-memory and MMA latency and on fixed-latency dependencies
        // in equal parts, at 12 warps per SM -- so the kernels use 1 and keep their registers.)
        uint4 st[DEPTH][4];
        float an[DEPTH][2];
#pragma unroll
        for (int s = 0; s < DEPTH; s++) {
            if (s < nb) {
#pragma unroll
                for (int i = 0; i < 4; i++) st[s][i] = __ldg(src[i] + (size_t)s * 16);
                an[s][0] = __ldg(p.ad + ia0 * nb + s);
                an[s][1] = __ldg(p.ad + ia1 * nb + s);
            }
        }
        for (int b0 = 0; b0 < nb; b0 += DEPTH) {
#pragma unroll
            for (int s = 0; s < DEPTH; s++) {
                const int b = b0 + s;
                if (b >= nb) break;
#pragma unroll
                for (int i = 0; i < 4; i++) *reinterpret_cast<uint4 *>(s_b + dsto[i]) = st[s][i];
                __syncwarp();
                const float a0 = an[s][0], a1 = an[s][1];
                if (b + DEPTH < nb) {
#pragma unroll
                    for (int i = 0; i < 4; i++) st[s][i] = __ldg(src[i] + (size_t)(b + DEPTH) * 16);
                    an[s][0] = __ldg(p.ad + ia0 * nb + b + DEPTH);
                    an[s][1] = __ldg(p.ad + ia1 * nb + b + DEPTH);
                }
                const float d0 = s_d[m0 * nb + b], d1 = s_d[m1 * nb + b];
                const float dsc[4] = {__fmul_rn(d0, a0), __fmul_rn(d0, a1), __fmul_rn(d1, a0), __fmul_rn(d1, a1)};
                const uint4 *fr = s_frag + (size_t)b * 8 * 2 * 32 + (lane ^ (lane >> 3) ^ (b & 7));
                const uint32_t *bt = s_b + g4 * kTokStride + q4;
#pragma unroll
                for (int r = 0; r < 8; r++) {
                    const uint4 ah = fr[(r * 2 + 0) * 32], al = fr[(r * 2 + 1) * 32];
                    const uint32_t b0w = bt[r * 8], b1w = bt[r * 8 + 4];
                    int ch[4], cl[4];
                    mma_s8(ch, ah, b0w, b1w);
                    mma_s8(cl, al, b0w, b1w);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        // aux = 64*hi + lo as a float, exactly (|aux| < 2^24). Two routes share the work between pipes:
                        // the int->float converter (a quarter-rate unit), and an arithmetic route for the fourth output:
                        // |hi|, |lo| < 2^22, so adding them to 1.5*2^23 as integers and subtracting the constant as floats
                        // converts each exactly, and 64*fh + fl is exact because the sum is representable.
                        float aux;
                        if (i < 3) {
                            aux = (float)(ch[i] * 64 + cl[i]);
                        } else {
                            const float fh = __fsub_rn(__int_as_float(0x4B400000 + ch[i]), 12582912.0f);
                            const float fl = __fsub_rn(__int_as_float(0x4B400000 + cl[i]), 12582912.0f);
                            aux = __fmaf_rn(fh, 64.0f, fl);
                        }
                        sums[i][r] = __fadd_rn(sums[i][r], __fmul_rn(dsc[i], aux));
                    }
                }
                __syncwarp();
            }
        }
        // y = ((((((s0+s1)+s2)+s3)+s4)+s5)+s6)+s7, then scatter
        float tot[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float t = sums[i][0];
#pragma unroll
            for (int r = 1; r < 8; r++) t = __fadd_rn(t, sums[i][r]);
            tot[i] = t;
        }
        const bool v0 = n0 + 2 * q4 < count, v1 = n0 + 2 * q4 + 1 < count;
        long long o0 = p.out_map ? p.out_map[pa0] : pa0, o1 = p.out_map ? p.out_map[pa1] : pa1;
        float *out0 = p.out[j], *out1 = p.out[j];
        if (p.out_tab) {  // the rows of a pair go to the GPU the pair's token lives on (plain peer stores)
            if (v0) out0 = p.out_tab[o0 / p.out_div];
            if (v1) out1 = p.out_tab[o1 / p.out_div];
            o0 %= p.out_div;
            o1 %= p.out_div;
        }
        if (row0 + m0 < rows) {
            if (v0) out0[o0 * rows + row0 + m0] = tot[0];
            if (v1) out1[o1 * rows + row0 + m0] = tot[1];
        }
        if (row0 + m1 < rows) {
            if (v0) out0[o0 * rows + row0 + m1] = tot[2];
            if (v1) out1[o1 * rows + row0 + m1] = tot[3];
        }
    }
}

// Shared memory: [nb][8 residues][hi, lo][32 lanes] x 16 B of A fragments, [16 rows][nb] f32 of d, one staging
// buffer of 8 x kTokStride words per warp.
__host__ __device__ inline size_t gemm_smem_bytes(int nb, int threads) {
    return (size_t)nb * 8 * 2 * 32 * 16 + (size_t)kGemmRows * nb * 4 + (size_t)(threads / 32) * 8 * kTokStride * 4;
}

__device__ __forceinline__ int job_of_tile(const GemmParams &p, int rt) {
    int j = 0;
    if (p.njobs > 1 && rt >= p.tile_begin[1]) j = 1;
    if (p.njobs > 2 && rt >= p.tile_begin[2]) j = 2;
    return j;
}

// grid (row tiles of all jobs, groups). HOIST (long rows): three CTAs per SM fit anyway, spend registers on loads
// in flight; short rows: keep registers low so that five CTAs fit.
template <bool HOIST>
__global__ void __launch_bounds__(128, HOIST ? 3 : 5) q6k_gemm_grouped_kernel(const GemmParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = p.nb;
    uint4 *s_frag = reinterpret_cast<uint4 *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)nb * 8 * 2 * 32 * 16);
    pdl_trigger();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0 && p.prefetch_ahead > 0) {
        // the weights of the CTA that will take this one's place on the SM start their trip from HBM now
        const long long lin = (long long)blockIdx.y * gridDim.x + blockIdx.x + p.prefetch_ahead;
        if (lin < (long long)gridDim.x * gridDim.y) {
            const int px = (int)(lin % gridDim.x), pe = (int)(lin / gridDim.x);
            const int pj = job_of_tile(p, px);
            const int prow0 = (px - p.tile_begin[pj]) * kGemmRows;
            if (p.folded[pj]) {
                const int tiles_j = (p.rows[pj] + kGemmRows - 1) / kGemmRows;
                const uint8_t *src = p.folded[pj] + ((size_t)pe * tiles_j + (size_t)(px - p.tile_begin[pj])) * (size_t)p.fold_tile_bytes;
                asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"((uint32_t)p.fold_tile_bytes) : "memory");
            } else
            prefetch_row_tile(p.w[pj], (size_t)pe * (size_t)(p.gstart ? p.expert_units : 0) + (size_t)prow0 * nb, p.rows[pj] - prow0, nb);
        }
    }
    pdl_wait();
    const int j = job_of_tile(p, blockIdx.x);
    const int rows = p.rows[j];
    const int row0 = ((int)blockIdx.x - p.tile_begin[j]) * kGemmRows;
    const int e = blockIdx.y;
    const int first = p.gstart ? p.gstart[e] : 0;
    const int count = p.gstart ? p.gcount[e] : p.n_tokens;
    if (count <= 0) return;
    const size_t unit0 = (size_t)e * (size_t)(p.gstart ? p.expert_units : 0) + (size_t)row0 * nb;
    if (p.folded[j]) {
        // the tile was folded when the model was loaded: its image comes straight into place, 16 bytes per request, and
        // the CTA's time goes to the MMAs instead of to turning Q6_K blocks into operands again
        const int tiles_j = (rows + kGemmRows - 1) / kGemmRows;
        const uint8_t *src = p.folded[j] + ((size_t)e * tiles_j + (size_t)(row0 / kGemmRows)) * (size_t)p.fold_tile_bytes;
        const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem);
        const int n16 = (int)(p.fold_tile_bytes >> 4);
        for (int i = tid; i < n16; i += 128)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 16u * (uint32_t)i), "l"(src + 16 * (size_t)i) : "memory");
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
        fold_row_tile<128, HOIST>(p.w[j], unit0, rows - row0, nb, s_frag, s_d, tid);
    }
    __syncthreads();
    uint32_t *s_b = reinterpret_cast<uint32_t *>(s_d + kGemmRows * nb) + (size_t)warp * 8 * kTokStride;
    mma_token_tiles<1>(p, j, row0, rows, first, count, 0, (count + 7) >> 3, s_frag, s_d, s_b, warp, 4, lane);
}

// Folds every (expert, row tile) of one matrix once and keeps the image: grid (row tiles, experts).
__global__ void __launch_bounds__(128) q6k_prefold_kernel(const uint8_t *__restrict__ w, uint8_t *__restrict__ dst, int rows, int nb,
                                                          long long expert_units, long long tile_bytes) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint4 *s_frag = reinterpret_cast<uint4 *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)nb * 8 * 2 * 32 * 16);
    const int tid = threadIdx.x, row0 = blockIdx.x * kGemmRows, e = blockIdx.y;
    for (int i = tid; i < kGemmRows * nb; i += 128) s_d[i] = 0.0f;  // (rows past the matrix: fold_store leaves their scales alone)
    __syncthreads();
    fold_row_tile<128, false>(w, (size_t)e * (size_t)expert_units + (size_t)row0 * nb, rows - row0, nb, s_frag, s_d, tid);
    __syncthreads();
    uint4 *out = reinterpret_cast<uint4 *>(dst + ((size_t)e * gridDim.x + blockIdx.x) * (size_t)tile_bytes);
    const int n16 = (int)(tile_bytes >> 4);
    for (int i = tid; i < n16; i += 128) out[i] = reinterpret_cast<const uint4 *>(smem)[i];
}

// One group of n_tokens tokens; gridDim.x resident CTAs share the (row tile, chunk of kChunkTiles token tiles) items,
// CTA c taking the contiguous range [c*items/grid, (c+1)*items/grid) in row-tile-major order.
__global__ void __launch_bounds__(256, 2) q6k_gemm_dense_kernel(const GemmParams p, int total_row_tiles) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = p.nb;
    uint4 *s_frag = reinterpret_cast<uint4 *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)nb * 8 * 2 * 32 * 16);
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    uint32_t *s_b = reinterpret_cast<uint32_t *>(s_d + kGemmRows * nb) + (size_t)warp * 8 * kTokStride;
    const int n_tiles = (p.n_tokens + 7) >> 3;
    const int n_chunks = (n_tiles + kChunkTiles - 1) / kChunkTiles;
    const long long items = (long long)total_row_tiles * n_chunks;
    const long long it_lo = items * blockIdx.x / gridDim.x, it_hi = items * (blockIdx.x + 1) / gridDim.x;
    int cur_rt = -1, j = 0, row0 = 0;
    for (long long it = it_lo; it < it_hi; it++) {
        const int rt = (int)(it / n_chunks), ch = (int)(it - (long long)rt * n_chunks);
        if (rt != cur_rt) {
            __syncthreads();  // every warp is done with the previous row tile's fragments
            cur_rt = rt;
            j = job_of_tile(p, rt);
            row0 = (rt - p.tile_begin[j]) * kGemmRows;
            if (tid == 0 && (long long)(rt + 1) * n_chunks < it_hi) {  // this CTA's next row tile
                const int nj = job_of_tile(p, rt + 1);
                const int nrow0 = (rt + 1 - p.tile_begin[nj]) * kGemmRows;
                prefetch_row_tile(p.w[nj], (size_t)nrow0 * nb, p.rows[nj] - nrow0, nb);
            }
            fold_row_tile<256, false>(p.w[j], (size_t)row0 * nb, p.rows[j] - row0, nb, s_frag, s_d, tid);
            __syncthreads();
        }
        mma_token_tiles<1>(p, j, row0, p.rows[j], 0, p.n_tokens, ch * kChunkTiles, min(n_tiles, (ch + 1) * kChunkTiles), s_frag, s_d, s_b, warp, 8,
                        lane);
    }
}

}  // namespace llamd

using namespace llamd;

static void gemm_launch(GemmParams &p, int n_groups) {
    const int threads = n_groups > 1 || p.gstart || p.folded[0] ? 128 : 256;  // (a folded matrix: the kernel that copies tiles)
    const size_t smem = gemm_smem_bytes(p.nb, threads);
    if (p.nb < 1 || smem > 220 * 1024) {
        set_error_msg("q6k gemm: blocks per row must be 1..24");
        return;
    }
    int tiles = 0;
    for (int i = 0; i < p.njobs; i++) {
        p.tile_begin[i] = tiles;
        tiles += (p.rows[i] + kGemmRows - 1) / kGemmRows;
    }
    if (threads == 128) {
        if (n_groups > 65535) {
            set_error_msg("q6k gemm: too many groups");
            return;
        }
        const bool hoist = p.nb > 4;
        auto kernel = hoist ? q6k_gemm_grouped_kernel<true> : q6k_gemm_grouped_kernel<false>;
        static size_t configured[2] = {0, 0};
        if (smem > 48 * 1024 && smem > configured[hoist]) {
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            configured[hoist] = smem;
        }
        static int cached_nb = -1, cached_slots = 0;
        if (cached_nb != p.nb) {
            int dev = 0, sms = 0, per_sm = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 128, smem);
            cached_slots = sms * (per_sm > 0 ? per_sm : 1);
            cached_nb = p.nb;
        }
        p.prefetch_ahead = cached_slots;
        launch_k("q6k_gemm_grouped", kernel, dim3(tiles, n_groups), dim3(128), smem, p);
        return;
    }
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaFuncSetAttribute(q6k_gemm_dense_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = smem;
    }
    // as many CTAs as stay resident at once (per shared-memory size: cached)
    static int cached_nb = -1, cached_slots = 0;
    if (cached_nb != p.nb) {
        int dev = 0, sms = 0, per_sm = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, q6k_gemm_dense_kernel, 256, smem);
        cached_slots = sms * (per_sm > 0 ? per_sm : 1);
        cached_nb = p.nb;
    }
    const int n_tiles = (p.n_tokens + 7) / 8, n_chunks = (n_tiles + kChunkTiles - 1) / kChunkTiles;
    const long long items = (long long)tiles * n_chunks;
    const int grid = (int)(items < cached_slots ? items : cached_slots);
    launch_k("q6k_gemm_dense", q6k_gemm_dense_kernel, dim3(grid), dim3(256), smem, p, tiles);
}

extern "C" {

// Q8_K quants [nblocks][256] (natural order) -> the residue-major words the GEMM reads.
void llamd_fwd_q8k_residue_major(const int8_t *aq, void *aq_rm, size_t nblocks) {
    if (!nblocks) return;
    const size_t n = nblocks * 64;
    launch_k("q8k_residue_major", q8k_residue_major_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, aq, (uint32_t *)aq_rm, nblocks);
}

// Up to three matrices (w1/w2 may be NULL) against ntok activations; outputs [ntok][rows_i].
// Same results as llamd_fwd_matvec_tokens, on the integer tensor path.
void llamd_fwd_gemm_tokens(const void *w0, const void *w1, const void *w2, const void *aq_rm, const float *ad, float *o0, float *o1,
                           float *o2, int blocks, int rows0, int rows1, int rows2, int ntok) {
    if (ntok < 1) return;
    GemmParams p = {};
    p.w[0] = (const uint8_t *)w0; p.w[1] = (const uint8_t *)w1; p.w[2] = (const uint8_t *)w2;
    p.out[0] = o0; p.out[1] = o1; p.out[2] = o2;
    p.rows[0] = rows0; p.rows[1] = rows1; p.rows[2] = rows2;
    p.njobs = w2 ? 3 : (w1 ? 2 : 1);
    p.nb = blocks;
    p.aq_rm = (const uint32_t *)aq_rm;
    p.ad = ad;
    p.n_tokens = ntok;
    gemm_launch(p, 1);
}

// Expert-major grouped GEMM over the scatter plan (gstart/gcount per expert, pairs sorted by expert):
// pair p reads activation act_map[p] and writes out[pslot[p]][rows]. wb/ob may be NULL.
// Same results as llamd_fwd_expert_major.
void llamd_fwd_expert_gemm(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount, const int32_t *act_map,
                           const int32_t *pslot, const void *aq_rm, const float *ad, float *oa, float *ob, int blocks, int rows,
                           int n_expert) {
    expert_gemm_scatter(wa, wb, gstart, gcount, act_map, pslot, aq_rm, ad, oa, ob, blocks, rows, n_expert, nullptr, 1, nullptr, nullptr);
}

}  // extern "C"

size_t llamd::expert_fold_tile_bytes(int blocks) { return (size_t)blocks * 8 * 2 * 32 * 16 + (size_t)kGemmRows * blocks * 4; }
size_t llamd::expert_fold_bytes(int blocks, int rows, int n_expert) {
    return expert_fold_tile_bytes(blocks) * (size_t)((rows + kGemmRows - 1) / kGemmRows) * (size_t)n_expert;
}
void llamd::expert_prefold(const void *w, void *dst, int blocks, int rows, int n_expert) {
    const size_t tile_bytes = expert_fold_tile_bytes(blocks);
    static size_t configured = 0;
    if (tile_bytes > 48 * 1024 && tile_bytes > configured) {
        if (cudaFuncSetAttribute(q6k_prefold_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tile_bytes) != cudaSuccess) {
            set_error_msg("expert prefold: shared memory attribute");
            return;
        }
        configured = tile_bytes;
    }
    if (n_expert > 65535 || n_expert < 1 || rows < 1) {
        set_error_msg("expert prefold: 1..65535 experts, rows positive");
        return;
    }
    launch_k("q6k_prefold", q6k_prefold_kernel, dim3((rows + kGemmRows - 1) / kGemmRows, n_expert), dim3(128), tile_bytes, (const uint8_t *)w,
             (uint8_t *)dst, rows, blocks, (long long)rows * blocks, (long long)tile_bytes);
}

void llamd::expert_gemm_scatter(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount, const int32_t *act_map,
                                const int32_t *pslot, const void *aq_rm, const float *ad, float *oa, float *ob, int blocks, int rows,
                                int n_expert, float *const *out_tab, int out_div, const void *fa, const void *fb) {
    if (out_tab && (wb || out_div < 1)) {
        set_error_msg("expert gemm: scattered outputs take one matrix and a positive row-block count per GPU");
        return;
    }
    GemmParams p = {};
    p.out_tab = out_tab;
    p.out_div = out_div;
    p.w[0] = (const uint8_t *)wa; p.w[1] = (const uint8_t *)wb;
    p.folded[0] = (const uint8_t *)fa; p.folded[1] = wb ? (const uint8_t *)fb : nullptr;
    p.fold_tile_bytes = (long long)expert_fold_tile_bytes(blocks);
    p.out[0] = oa; p.out[1] = ob;
    p.rows[0] = rows; p.rows[1] = rows;
    p.njobs = wb ? 2 : 1;
    p.nb = blocks;
    p.aq_rm = (const uint32_t *)aq_rm;
    p.ad = ad;
    p.gstart = gstart; p.gcount = gcount; p.act_map = act_map; p.out_map = pslot;
    p.expert_units = (long long)rows * blocks;
    gemm_launch(p, n_expert);
}

// Up to three matrices kept folded (expert_prefold with one "expert" each) against ntok activations: out_i[ntok][rows_i].
// The grouped kernel with a single group: a CTA copies its row tile's image and multiplies; 2 bytes per weight whatever
// ntok is, where the matvec repeats its integer work per sequence. Same results as llamd_fwd_gemm_tokens.
void llamd::gemm_tokens_folded3(const void *f0, const void *f1, const void *f2, const void *aq_rm, const float *ad, float *o0, float *o1,
                                float *o2, int blocks, int rows0, int rows1, int rows2, int ntok) {
    if (ntok < 1) return;
    GemmParams p = {};
    p.folded[0] = (const uint8_t *)f0; p.folded[1] = (const uint8_t *)f1; p.folded[2] = (const uint8_t *)f2;
    p.fold_tile_bytes = (long long)expert_fold_tile_bytes(blocks);
    p.out[0] = o0; p.out[1] = o1; p.out[2] = o2;
    p.rows[0] = rows0; p.rows[1] = rows1; p.rows[2] = rows2;
    p.njobs = f2 ? 3 : (f1 ? 2 : 1);
    p.nb = blocks;
    p.aq_rm = (const uint32_t *)aq_rm;
    p.ad = ad;
    p.n_tokens = ntok;
    gemm_launch(p, 1);
}
void llamd::gemm_tokens_folded(const void *folded, const void *aq_rm, const float *ad, float *out, int blocks, int rows, int ntok) {
    gemm_tokens_folded3(folded, nullptr, nullptr, aq_rm, ad, out, nullptr, nullptr, blocks, rows, 0, 0, ntok);
}
