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
// A CTA (4 warps) owns 16 weight rows of one matrix/expert for all of that
// expert's tokens: it folds and splits its rows once into shared memory in MMA
// fragment order (amortised over every token tile), then each warp walks token
// tiles of 8. Activations are read as residue-major words (one 32-bit word =
// the four bytes of one MMA k-quad) prepared by q8k_residue_major_kernel.
#include "q6k_layout.cuh"

namespace llamd {

constexpr int kGemmThreads = 128;
constexpr int kGemmRows = 16;

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
};

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

__global__ void __launch_bounds__(kGemmThreads) q6k_gemm_kernel(const GemmParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = p.nb;
    // [nb][8 residues][hi, lo][32 lanes] x 16 B of A fragments, then [16 rows][nb] f32 of d
    uint4 *s_frag = reinterpret_cast<uint4 *>(smem);
    float *s_d = reinterpret_cast<float *>(smem + (size_t)nb * 8 * 2 * 32 * 16);
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int j = 0;
    if (p.njobs > 1 && (int)blockIdx.x >= p.tile_begin[1]) j = 1;
    if (p.njobs > 2 && (int)blockIdx.x >= p.tile_begin[2]) j = 2;
    const int rows = p.rows[j];
    const int row0 = ((int)blockIdx.x - p.tile_begin[j]) * kGemmRows;
    const int e = blockIdx.y;
    const int first = p.gstart ? p.gstart[e] : 0;
    const int count = p.gstart ? p.gcount[e] : p.n_tokens;
    if (count <= 0) return;
    const uint8_t *w = p.w[j];
    const size_t unit0 = (size_t)e * (size_t)(p.gstart ? p.expert_units : 0) + (size_t)row0 * nb;

    // ---- fold the scales into the weights, split hi/lo, store in fragment order ----
    // One thread per (row, block): its 13 coalesced 16-byte loads fetch the whole block (as in the matvec
    // kernel), all issued before any is used.
    for (int rb = tid; rb < kGemmRows * nb; rb += kGemmThreads) {  // rb = row_local * nb + b
        const int row_l = rb / nb, b = rb - row_l * nb;
        const bool live = row0 + row_l < rows;
        uint32_t S[48];
        uint4 scw = make_uint4(0, 0, 0, 0);
        if (live) {
            const size_t unit = unit0 + rb;
            const uint8_t *tile = w + (unit >> 5) * kTileBytes;
            const int sl = (int)(unit & 31);
            const uint4 *cp = reinterpret_cast<const uint4 *>(tile) + sl;
#pragma unroll
            for (int c = 0; c < 12; c++) {
                const uint4 v = __ldg(cp + c * 32);
                S[4 * c + 0] = v.x; S[4 * c + 1] = v.y; S[4 * c + 2] = v.z; S[4 * c + 3] = v.w;
            }
            scw = __ldg(reinterpret_cast<const uint4 *>(tile + kTileScaleOff) + sl);
            s_d[rb] = f16_bits_to_f32(__ldg(reinterpret_cast<const uint16_t *>(tile + kTileDOff) + sl));
        } else {
#pragma unroll
            for (int c = 0; c < 48; c++) S[c] = 0;
            s_d[rb] = 0.0f;
        }
        int sc[16];
        {
            const uint32_t ws[4] = {scw.x, scw.y, scw.z, scw.w};
#pragma unroll
            for (int i = 0; i < 16; i++) sc[i] = (int)(int8_t)(ws[i >> 2] >> (8 * (i & 3)));
        }
#pragma unroll
        for (int r = 0; r < 8; r++) {
#pragma unroll
            for (int m = 0; m < 2; m++) {
                const uint32_t s0 = S[6 * r + 3 * m], s1 = S[6 * r + 3 * m + 1], s2 = S[6 * r + 3 * m + 2];
                uint32_t w4[4];
                w4[0] = s0 & 0xFCFCFCFCu;
                w4[1] = s1 & 0xFCFCFCFCu;
                w4[2] = s2 & 0xFCFCFCFCu;
                w4[3] = ((s0 << 6) & 0xC0C0C0C0u) | ((s1 << 4) & 0x30303030u) | ((s2 << 2) & 0x0C0C0C0Cu);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    uint32_t hi = 0, lo = 0;
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        // byte k of word jw = 4m+i: weight (q-32) = the 6-bit field above bit 2; its group is 2*jw + (k>>1)
                        const int wv = ((int)(w4[i] << (24 - 8 * k))) >> 26;
                        const int u = wv * sc[2 * (4 * m + i) + (k >> 1)];  // 13 bits signed
                        lo |= (uint32_t)(u & 63) << (8 * k);
                        hi |= (uint32_t)((u >> 6) & 0xFF) << (8 * k);
                    }
                    // fragment word q of lane L: row = L/4 + 8(q&1), word jw = L%4 + 4(q>>1)
                    const int jw = 4 * m + i;
                    // Lane L's 16 bytes sit in slot L ^ (L >> 3) ^ (b & 7): a warp here is 4 rows x 8 blocks writing the
                    // same jw, and the swizzle spreads those over all eight 16-byte bank groups (the readers of one
                    // fragment still touch 32 distinct slots).
                    const int L = (row_l & 7) * 4 + (jw & 3), q = (row_l >> 3) + 2 * (jw >> 2);
                    const int P = L ^ (L >> 3) ^ (b & 7);
                    reinterpret_cast<uint32_t *>(s_frag + ((size_t)(b * 8 + r) * 2 + 0) * 32 + P)[q] = hi;
                    reinterpret_cast<uint32_t *>(s_frag + ((size_t)(b * 8 + r) * 2 + 1) * 32 + P)[q] = lo;
                }
            }
        }
    }
    __syncthreads();

    // ---- token tiles of 8, one warp each ----
    // Per block b the warp copies its 8 tokens' 256 activation bytes into its own buffer with coalesced
    // 16-byte loads (rows padded to 68 words so the fragment reads are conflict-free); the next block's
    // bytes wait in registers meanwhile.
    constexpr int kTokStride = 68;  // words
    uint32_t *s_b = reinterpret_cast<uint32_t *>(smem + (size_t)nb * 8 * 2 * 32 * 16 + (size_t)kGemmRows * nb * 4) +
                    (size_t)warp * 8 * kTokStride;
    const int g4 = lane >> 2, q4 = lane & 3;
    const int m0 = g4, m1 = g4 + 8;
    const int n_tiles = (count + 7) >> 3;
    for (int tn = warp; tn < n_tiles; tn += kGemmThreads / 32) {
        const int n0 = tn * 8;
        // the two tokens whose outputs this lane owns
        const int pa0 = first + min(n0 + 2 * q4, count - 1), pa1 = first + min(n0 + 2 * q4 + 1, count - 1);
        const long long ia0 = p.act_map ? p.act_map[pa0] : pa0, ia1 = p.act_map ? p.act_map[pa1] : pa1;
        // staging: lane l copies 16-byte chunk (l & 15) + 16*i of token (l >> 4) + 2*i' ... 8 tokens x 16 chunks = 128 chunks, 4 per lane
        const uint4 *src[4];
        int dsto[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int chunk = lane + 32 * i;  // 0..127
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
        uint4 st[4];
#pragma unroll
        for (int i = 0; i < 4; i++) st[i] = __ldg(src[i]);
        for (int b = 0; b < nb; b++) {
            uint32_t *buf = s_b;
#pragma unroll
            for (int i = 0; i < 4; i++) *reinterpret_cast<uint4 *>(buf + dsto[i]) = st[i];
            __syncwarp();
            if (b + 1 < nb) {
#pragma unroll
                for (int i = 0; i < 4; i++) st[i] = __ldg(src[i] + (size_t)(b + 1) * 16);
            }
            const float a0 = __ldg(p.ad + ia0 * nb + b), a1 = __ldg(p.ad + ia1 * nb + b);
            const float d0 = s_d[m0 * nb + b], d1 = s_d[m1 * nb + b];
            const float dsc[4] = {__fmul_rn(d0, a0), __fmul_rn(d0, a1), __fmul_rn(d1, a0), __fmul_rn(d1, a1)};
            const uint4 *fr = s_frag + (size_t)b * 8 * 2 * 32 + (lane ^ (lane >> 3) ^ (b & 7));
            const uint32_t *bt = buf + g4 * kTokStride + q4;
#pragma unroll
            for (int r = 0; r < 8; r++) {
                const uint4 ah = fr[(r * 2 + 0) * 32], al = fr[(r * 2 + 1) * 32];
                const uint32_t b0 = bt[r * 8], b1 = bt[r * 8 + 4];
                int ch[4], cl[4];
                mma_s8(ch, ah, b0, b1);
                mma_s8(cl, al, b0, b1);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // (float)(64*hi + lo) without the slow int->float pipe: |hi|, |lo| < 2^22, so adding them to
                    // 1.5*2^23 as integers and subtracting the constant as floats converts exactly; 64*fh + fl is
                    // exact too because the sum (|aux| < 2^24) is representable.
                    const float fh = __fsub_rn(__int_as_float(0x4B400000 + ch[i]), 12582912.0f);
                    const float fl = __fsub_rn(__int_as_float(0x4B400000 + cl[i]), 12582912.0f);
                    const float aux = __fmaf_rn(fh, 64.0f, fl);
                    sums[i][r] = __fadd_rn(sums[i][r], __fmul_rn(dsc[i], aux));
                }
            }
            __syncwarp();
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
        float *out = p.out[j];
        const bool v0 = n0 + 2 * q4 < count, v1 = n0 + 2 * q4 + 1 < count;
        const long long o0 = p.out_map ? p.out_map[pa0] : pa0, o1 = p.out_map ? p.out_map[pa1] : pa1;
        if (row0 + m0 < rows) {
            if (v0) out[o0 * rows + row0 + m0] = tot[0];
            if (v1) out[o1 * rows + row0 + m0] = tot[1];
        }
        if (row0 + m1 < rows) {
            if (v0) out[o0 * rows + row0 + m1] = tot[2];
            if (v1) out[o1 * rows + row0 + m1] = tot[3];
        }
    }
}

}  // namespace llamd

using namespace llamd;

static void gemm_launch(GemmParams &p, int n_groups) {
    const size_t smem = (size_t)p.nb * 8 * 2 * 32 * 16 + (size_t)kGemmRows * p.nb * 4 + (size_t)(kGemmThreads / 32) * 8 * 68 * 4;
    if (p.nb < 1 || smem > 200 * 1024) {
        set_error_msg("q6k gemm: blocks per row must be 1..24");
        return;
    }
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaFuncSetAttribute(q6k_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = smem;
    }
    int tiles = 0;
    for (int i = 0; i < p.njobs; i++) {
        p.tile_begin[i] = tiles;
        tiles += (p.rows[i] + kGemmRows - 1) / kGemmRows;
    }
    if (n_groups > 65535) {
        set_error_msg("q6k gemm: too many groups");
        return;
    }
    launch_k("q6k_gemm", q6k_gemm_kernel, dim3(tiles, n_groups), dim3(kGemmThreads), smem, p);
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
    GemmParams p = {};
    p.w[0] = (const uint8_t *)wa; p.w[1] = (const uint8_t *)wb;
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

}  // extern "C"
