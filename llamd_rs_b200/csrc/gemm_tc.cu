// Q6_K x activation GEMM on the 5th-generation tensor cores (tcgen05, accumulators in TMEM):
// the TOLERANCE-LEVEL prefill path (model option prefill_gemm = 2).
//
// The exact path (expert_gemm.cu) must stop after every 32-deep contraction to apply the reference's f32
// scaling in order, which is what keeps it off tcgen05. This kernel gives that up: inside a 256-element block
// ONE f32 accumulator per output runs over all eight residues inside the tensor core, and the block's f16 scale
// d joins afterwards, out += (64 d) * D, once per block. Everything else is kept as precise as the hardware lets:
//   weight  U = scale * (q - 32) is an integer of 13 bits; it enters as TWO exact f16 values, U >> 6 and
//           (U & 63) / 64 (their sum is U / 64)
//   act     x = ad * aq in f32 enters as two f16 terms, B1 = f16(x), B2 = f16(x - B1) (22 bits)
// and all four products are accumulated. What remains against the exact path is the order of the f32 sums
// (outputs agree to ~1e-5 relative: the tensor core's f32 sum is not IEEE-rounded; the reference's bound for a quantized matmul is QUANTIZED_MATMUL = 1e-3,
// crates/llamd-core/src/tolerance.rs:41-66), so a prompt prefilled this way is close to, but not bit-identical
// to, feeding its tokens one by one; that is why it is an option and not the default. (A first version with one
// f16 term per operand, d folded into the weight, measured 1e-2 on outputs of rms 7: outside the bound, whose
// `close` scaling is absolute below 1.)
//
// One CTA (8 warps) = 128 weight rows of one matrix or expert x up to 64 tokens:
//   stage s of 8*nb: residue s%8 of block s/8, 32 contraction elements
//     all threads   fold their half residue (16 weights, two per 32-bit multiply-add) into the stage's A tile and
//                   copy the B tile (cp.async); tiles are K-major, 128-byte rows [32 f16 | 32 f16], with the
//                   128-byte swizzle the matrix descriptors name; the next stage's code words are already in flight
//     one thread    8 x tcgen05.mma (M 128, N n_pad, K 16) accumulating into TMEM, tcgen05.commit -> mbarrier
//   two A buffers (the fold of stage s+1 overlaps the MMAs of stage s), a ring of four B buffers filled two stages
//   ahead, code words loaded two stages ahead
//   blocks alternate between two accumulator tiles in TMEM; one stage into the next block, the finished one is
//   read back: tcgen05.ld (32 lanes x 32 columns per warp), acc += 64 d * D in registers
//   at the end: scatter acc to out[token][row].
// act_f16_rm_kernel writes the activations in the contraction order used here (residue-major inside a block).
// Every wait on an mbarrier is bounded; a timeout raises a flag the host reads (llamd_fwd_gemm_tc_status).
#include <cuda_fp16.h>

#include "q6k_layout.cuh"

namespace llamd {
namespace {

constexpr int kTcM = 128;          // rows per CTA = TMEM lanes
constexpr int kTcN = 64;           // tokens per CTA at most = TMEM columns
constexpr int kTcStageBytes = kTcM * 128;  // 64 f16 per row

struct TcParams {
    const uint8_t *w[3];
    float *out[3];
    int rows[3];
    int tile_begin[3];
    int njobs, nb;
    const __half *act;  // [index][nb][8 residues][64]: 32 first terms, 32 second terms
    const int32_t *gstart, *gcount, *act_map, *out_map;
    int n_tokens;
    long long expert_units;
    int *status;  // device word: 0 ok, else the code of the first wait that gave up
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// try_wait parks the thread in hardware for up to the hinted time per call, so a waiting warp issues almost
// nothing; false after 2^14 calls (tens of milliseconds at the least): the caller records it and unwinds.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
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
// K-major tile with 128-byte rows and the 128-byte swizzle; 8-row groups 1024 bytes apart (matrix descriptor
// format of tcgen05.mma: start address, leading and stride byte offsets in 16-byte units, version 1 at bit 46,
// layout type 2 = SWIZZLE_128B at bits 61-63).
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;             // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;   // stride byte offset: one 8-row group
    d |= (uint64_t)1 << 46;             // descriptor version
    d |= (uint64_t)2 << 61;             // SWIZZLE_128B
    return d;
}

// activations: natural-order Q8_K -> the two f16 terms of ad * aq, per (block, residue) a row of
// [32 x term 1 | 32 x term 2]. One thread per element.
__global__ void act_f16_rm_kernel(const int8_t *__restrict__ aq, const float *__restrict__ ad, __half *__restrict__ out, size_t nblocks) {
    pdl_trigger();
    pdl_wait();
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= nblocks * 256) return;
    const size_t blk = i >> 8;
    const int pos = (int)(i & 255);
    const int r = pos >> 5, j = (pos >> 2) & 7, k = pos & 3;
    const float v = __fmul_rn(ad[blk], (float)aq[blk * 256 + t32_element(r, j, k)]);
    const __half h1 = __float2half_rn(v);
    const __half h2 = __float2half_rn(__fsub_rn(v, __half2float(h1)));
    __half *row = out + (blk * 8 + r) * 64;
    row[j * 4 + k] = h1;
    row[32 + j * 4 + k] = h2;
}

__device__ __forceinline__ int tc_job_of_tile(const TcParams &p, int rt) {
    int j = 0;
    if (p.njobs > 1 && rt >= p.tile_begin[1]) j = 1;
    if (p.njobs > 2 && rt >= p.tile_begin[2]) j = 2;
    return j;
}

// 32 TMEM columns of this warp's 32 lanes -> registers
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// grid (row tiles of all jobs, token groups, experts or 1), 256 threads.
__global__ void __launch_bounds__(256, 2) q6k_gemm_tc_kernel(const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t s_bar[2];  // the MMAs that read stage buffer 0 / 1 are done
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nb = p.nb;
    const int j = tc_job_of_tile(p, blockIdx.x);
    const int rows = p.rows[j];
    const int row0 = ((int)blockIdx.x - p.tile_begin[j]) * kTcM;
    const int e = blockIdx.z;
    const int first_all = p.gstart ? p.gstart[e] : 0;
    const int count_all = p.gstart ? p.gcount[e] : p.n_tokens;
    const int t0 = blockIdx.y * kTcN;
    if (t0 >= count_all) return;  // uniform per CTA, before any barrier or TMEM use
    const int first = first_all + t0, count = min(kTcN, count_all - t0);
    const int n_pad = max(16, (count + 15) & ~15);
    uint8_t *smem = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem, *sB = smem + 2 * kTcStageBytes;  // two A stages of 128 rows, a ring of four B stages of kTcN rows

    if (tid == 0) {
        mbar_init(&s_bar[0], 1);
        mbar_init(&s_bar[1], 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem)), "r"(2 * kTcN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = s_tmem;

    // instruction descriptor: D f32 (bit 4), A and B f16 K-major, N >> 3 at bit 17, M >> 4 at bit 24
    const uint32_t idesc = (1u << 4) | ((uint32_t)(n_pad >> 3) << 17) | ((uint32_t)(kTcM >> 4) << 24);

    if (tid == 0) {
        // The CTA's 128 rows x nb blocks are whole consecutive tiles: ask L2 for all of them now, so that the word loads
        // of the stage loop meet L2 latency, not HBM's (a hint; nothing waits on it).
        const size_t u0 = (size_t)e * (size_t)(p.gstart ? p.expert_units : 0) + (size_t)row0 * nb;
        const size_t u1 = u0 + (size_t)min(kTcM, rows - row0) * nb;
        const size_t t_lo = u0 >> 5, t_hi = (u1 - 1) >> 5;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.w[j] + t_lo * kTileBytes), "r"((uint32_t)((t_hi - t_lo + 1) * kTileBytes))
                     : "memory");
    }
    const int row = tid & 127, m = tid >> 7;  // this thread folds words 3m..3m+2 of the stage's residue for its row
    const bool live = row0 + row < rows;
    const size_t unit_row = (size_t)e * (size_t)(p.gstart ? p.expert_units : 0) + (size_t)(row0 + row) * nb;
    const uint8_t *wj = p.w[j];
    // B copy: kTcN rows x 8 pieces of 16 bytes per stage, two per thread
    const __half *bsrc[2];
    int bdst[2], bbytes[2];
#pragma unroll
    for (int i = 0; i < 2; i++) {
        const int piece = tid + 256 * i;
        const int n = piece >> 3, c16 = piece & 7;
        const int pt = first + min(n, count - 1);
        const long long idx = p.act_map ? p.act_map[pt] : pt;
        bsrc[i] = p.act + (size_t)idx * nb * 512 + c16 * 8;
        bdst[i] = n * 128 + ((c16 ^ (n & 7)) << 4);
        bbytes[i] = n < count ? 16 : 0;  // rows beyond the group's tokens are zero
    }
    // epilogue geometry: warp w reads TMEM lanes 32*(w%4) .. +31 (its rows) and the columns (tokens) [32*(w/4), +32)
    const int lane_grp = warp & 3, col0 = (warp >> 2) * 32;
    const uint32_t taddr = tmem + ((uint32_t)(lane_grp * 32) << 16) + (uint32_t)col0;
    const int e_row = lane_grp * 32 + lane;  // the row this thread accumulates in the epilogue
    float acc[32];
#pragma unroll
    for (int n = 0; n < 32; n++) acc[n] = 0.0f;
    // out += (64 * d[row][b]) * D for the block whose MMAs have completed
    // d of (this thread's epilogue row, block b), requested several stages before the drain that uses it
    uint32_t d_bits = 0;
    auto load_d = [&](int b) {
        if (col0 < n_pad && row0 + e_row < rows) {
            const size_t unit = (size_t)e * (size_t)(p.gstart ? p.expert_units : 0) + (size_t)(row0 + e_row) * nb + b;
            d_bits = __ldg(reinterpret_cast<const uint16_t *>(wj + (unit >> 5) * kTileBytes + kTileDOff) + (unit & 31));
        }
    };
    auto drain_block = [&](int b) {
        if (col0 >= n_pad) return;  // uniform per warp
        const float dscale = (row0 + e_row < rows) ? 64.0f * f16_bits_to_f32((uint16_t)d_bits) : 0.0f;
        uint32_t v[32];
        tmem_ld32(taddr + (uint32_t)((b & 1) * kTcN), v);  // blocks alternate between two accumulator tiles
#pragma unroll
        for (int n = 0; n < 32; n++) acc[n] = fmaf(dscale, __uint_as_float(v[n]), acc[n]);
    };

    // ---- the stage loop: blocks outside, the eight residues of a block unrolled inside, so that every word offset,
    // buffer index and barrier parity below is a compile-time constant ----
    // byte offset of code word wdx inside a tile, for the block in slot 0 (chunk wdx/4 is 512 bytes, a word 4)
#define TC_WOFF(wdx) ((((wdx) >> 2) * 512) + (((wdx) & 3) * 4))
    const uint32_t sA_u = smem_u32(sA), sB_u = smem_u32(sB);
    const int sw = row & 7;
    // the four 16-byte pieces this thread writes in a stage's A tile: row = [U >> 6: words jw 0..7 | (U & 63)/64: words jw 0..7],
    // 8 bytes per word; this thread owns jw = 4m .. 4m+3
    const uint32_t a_off[4] = {(uint32_t)(row * 128 + (((2 * m + 0) ^ sw) << 4)), (uint32_t)(row * 128 + (((2 * m + 1) ^ sw) << 4)),
                               (uint32_t)(row * 128 + (((4 + 2 * m + 0) ^ sw) << 4)), (uint32_t)(row * 128 + (((4 + 2 * m + 1) ^ sw) << 4))};
    const bool bcopy[2] = {n_pad * 8 > tid, n_pad * 8 > tid + 256};
    bool ok = true;
    // where block b of this thread's row sits: tile base + its slot
    auto block_ptr = [&](int b) -> const uint8_t * {
        const size_t unit = unit_row + b;
        return wj + (unit >> 5) * kTileBytes + (unit & 31) * 16;
    };
    const uint8_t *tb = live ? block_ptr(0) : wj;
    // code words of the next stage (Sn) and of the one after it (Sn2): two stages of L2 latency are covered
    uint32_t Sn[3] = {0, 0, 0}, Sn2[3] = {0, 0, 0};
    uint2 scn = make_uint2(0, 0);
    if (live) {
#pragma unroll
        for (int x = 0; x < 3; x++) {
            Sn[x] = __ldg(reinterpret_cast<const uint32_t *>(tb + (m ? TC_WOFF(3 + x) : TC_WOFF(x))));
            Sn2[x] = __ldg(reinterpret_cast<const uint32_t *>(tb + (m ? TC_WOFF(6 + 3 + x) : TC_WOFF(6 + x))));
        }
        scn = __ldg(reinterpret_cast<const uint2 *>(tb + kTileScaleOff + 8 * m));
    }
    // the B tiles of stages 0 and 1 start their trip now; stage s issues the copy for stage s+2
    auto copy_b = [&](int ring) {
#pragma unroll
        for (int i = 0; i < 2; i++) {
            if (bcopy[i])
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sB_u + ring * (kTcN * 128) + bdst[i]), "l"(bsrc[i]), "r"(bbytes[i])
                             : "memory");
            bsrc[i] += 64;  // the next stage's 32 + 32 halves
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    copy_b(0);
    copy_b(1);
    int sc[8];
#pragma unroll
    for (int i = 0; i < 8; i++) sc[i] = 0;
    for (int b = 0; b < nb; b++) {
        const uint8_t *tb_next = (live && b + 1 < nb) ? block_ptr(b + 1) : tb;
#pragma unroll
        for (int r = 0; r < 8; r++) {
            const int buf = r & 1;
            // the MMAs that read this buffer two stages ago: completion number (s >> 1) - 1 of its barrier, and s >> 1 = 4b + r/2
            if (b > 0 || r >= 2) {
                if (!mbar_wait(&s_bar[buf], (uint32_t)(((r >> 1) + 1) & 1))) ok = false;
            }
            if (r == 1 && b > 0) {
                // The wait above covered stage s-2, the last of block b-1: its sum is complete. Block b accumulates into the
                // other tile meanwhile, so nothing here waits for an MMA that was only just issued.
                ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-wide: the warp reads together or not at all
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (ok) drain_block(b - 1);
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            // ring slot (s+2)&3 was read by the MMAs of stage s-2, which the wait above covered
            if (b + 1 < nb || r < 6) copy_b((r + 2) & 3);
            else asm volatile("cp.async.commit_group;" ::: "memory");  // keep one group per stage so that the count below holds

            if (r == 3) load_d(b);  // the previous block's drain (at r == 1) is done with the old value
            // ---- this thread's 16 weights: MMA words jw = 4m .. 4m+3 of residue r of block (row, b) ----
            const uint32_t S0 = Sn[0], S1 = Sn[1], S2 = Sn[2];
            if (r == 0) {
                const uint32_t ws[2] = {scn.x, scn.y};
#pragma unroll
                for (int i = 0; i < 8; i++) sc[i] = (int)(int8_t)(ws[i >> 2] >> (8 * (i & 3)));
            }
            Sn[0] = Sn2[0]; Sn[1] = Sn2[1]; Sn[2] = Sn2[2];
            if (live) {  // the words of stage s+2: two stages of work hide their latency
                if (r < 6) {
#pragma unroll
                    for (int x = 0; x < 3; x++)
                        Sn2[x] = __ldg(reinterpret_cast<const uint32_t *>(tb + (m ? TC_WOFF(6 * (r + 2) + 3 + x) : TC_WOFF(6 * (r + 2) + x))));
                } else if (b + 1 < nb) {
#pragma unroll
                    for (int x = 0; x < 3; x++)
                        Sn2[x] = __ldg(reinterpret_cast<const uint32_t *>(tb_next + (m ? TC_WOFF(6 * (r - 6) + 3 + x) : TC_WOFF(6 * (r - 6) + x))));
                }
                if (r == 4 && b + 1 < nb) scn = __ldg(reinterpret_cast<const uint2 *>(tb_next + kTileScaleOff + 8 * m));  // used from the next block's r == 0
            }
            uint32_t ahi[8], alo[8];
            if (live) {
                // The stored byte is 4*(q-32) mod 256; ^0x80 makes it 4q. The fourth word's codes are the low bit pairs of
                // the other three.
                uint32_t ub[4];
                ub[0] = (S0 & 0xFCFCFCFCu) ^ 0x80808080u;
                ub[1] = (S1 & 0xFCFCFCFCu) ^ 0x80808080u;
                ub[2] = (S2 & 0xFCFCFCFCu) ^ 0x80808080u;
                ub[3] = (((S0 << 6) & 0xC0C0C0C0u) | ((S1 << 4) & 0x30303030u) | ((S2 << 2) & 0x0C0C0C0Cu)) ^ 0x80808080u;
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // Two weights per multiply-add. With the bytes spread into 16-bit fields, x - 0x00800080 is, as an
                    // integer, sum_i 4*(q_i - 32) << 16i, so sc*(x - 0x00800080) + 0x80008000 holds 4*U_i + 32768
                    // (U = sc*(q-32), in [16512, 49152]) in each field with no carry between them: the high byte is
                    // (U >> 6) + 128, the low byte 4*(U & 63). Bytes 0,1 of word i belong to scale group 2i, bytes 2,3 to 2i+1.
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const uint32_t x = __byte_perm(ub[i], 0u, h ? 0x4342 : 0x4140);
                        const uint32_t v = (x - 0x00800080u) * (uint32_t)sc[2 * i + h] + 0x80008000u;
                        // bytes under the exponent of 1024: (1024 + byte) as f16, two per register
                        const uint32_t bh = __byte_perm(v, 0x64646464u, 0x4341), bl = __byte_perm(v, 0x64646464u, 0x4240);
                        const __half2 hh = __hsub2(*reinterpret_cast<const __half2 *>(&bh), __half2half2(__ushort_as_half(0x6480)));  // - 1152: U >> 6
                        const __half2 hl = __hfma2(*reinterpret_cast<const __half2 *>(&bl), __half2half2(__ushort_as_half(0x1C00)),  // * 1/256
                                                   __half2half2(__ushort_as_half(0xC400)));                                     // - 4: (U & 63) / 64
                        ahi[2 * i + h] = *reinterpret_cast<const uint32_t *>(&hh);
                        alo[2 * i + h] = *reinterpret_cast<const uint32_t *>(&hl);
                    }
                }
            } else {
#pragma unroll
                for (int q = 0; q < 8; q++) ahi[q] = alo[q] = 0;
            }
            {
                const uint32_t ab = sA_u + buf * kTcStageBytes;
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ab + a_off[0]), "r"(ahi[0]), "r"(ahi[1]), "r"(ahi[2]), "r"(ahi[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ab + a_off[1]), "r"(ahi[4]), "r"(ahi[5]), "r"(ahi[6]), "r"(ahi[7]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ab + a_off[2]), "r"(alo[0]), "r"(alo[1]), "r"(alo[2]), "r"(alo[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ab + a_off[3]), "r"(alo[4]), "r"(alo[5]), "r"(alo[6]), "r"(alo[7]) : "memory");
            }
            asm volatile("cp.async.wait_group 2;" ::: "memory");  // all but the two newest copies: this stage's B tile has landed
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core's reads
            __syncthreads();
            if (tid == 0 && ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = tc_smem_desc(sA_u + buf * kTcStageBytes);
                const uint64_t db = tc_smem_desc(sB_u + (r & 3) * (kTcN * 128));
                // 32-byte slices of a row (16 contraction elements each, +2 in 16-byte units). A: 0,1 = U >> 6; 2,3 = (U & 63)/64.
                // B: 0,1 = first f16 term of the activation; 2,3 = second term. All four products, both halves of the residue.
                const int sa[8] = {0, 1, 0, 1, 2, 3, 2, 3}, sb[8] = {0, 1, 2, 3, 0, 1, 2, 3};
#pragma unroll
                for (int kk = 0; kk < 8; kk++) {
                    const uint32_t accum = (r > 0 || kk > 0) ? 1u : 0u;  // a block starts its own sum
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem + (uint32_t)((b & 1) * kTcN)), "l"(da + (uint64_t)(2 * sa[kk])), "l"(db + (uint64_t)(2 * sb[kk])), "r"(idesc),
                        "r"(accum)
                        : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s_bar[buf])) : "memory");
            }
        }
        tb = tb_next;
    }
#undef TC_WOFF
    const int n_stages = 8 * nb;
    // the last block
    if (!mbar_wait(&s_bar[(n_stages - 1) & 1], (uint32_t)((n_stages - 1) >> 1) & 1)) ok = false;
    ok = __all_sync(0xffffffffu, ok);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) drain_block(nb - 1);
    if (!ok) {
        s_abort = 1;
        if (p.status) atomicCAS(p.status, 0, 1 + (int)blockIdx.x);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (!s_abort && col0 < n_pad && row0 + e_row < rows) {
        float *out = p.out[j];
#pragma unroll
        for (int n = 0; n < 32; n++) {
            if (col0 + n < count) {
                const int pt = first + col0 + n;
                const long long oi = p.out_map ? p.out_map[pt] : pt;
                out[oi * rows + row0 + e_row] = acc[n];
            }
        }
    }
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * kTcN) : "memory");
}

int *g_tc_status = nullptr;  // device word, allocated on first use

}  // namespace
}  // namespace llamd

using namespace llamd;

static void tc_launch(TcParams &p, int n_groups, int max_count) {
    if (p.nb < 1) return;
    if (!g_tc_status) {
        if (cudaMalloc(&g_tc_status, sizeof(int)) != cudaSuccess) {
            set_error(cudaGetLastError(), "gemm_tc status word");
            return;
        }
        cudaMemsetAsync(g_tc_status, 0, sizeof(int), stream());
    }
    p.status = g_tc_status;
    int tiles = 0;
    for (int i = 0; i < p.njobs; i++) {
        p.tile_begin[i] = tiles;
        tiles += (p.rows[i] + kTcM - 1) / kTcM;
    }
    const int tgroups = (max_count + kTcN - 1) / kTcN;
    if (n_groups > 65535 || tgroups > 65535 || tgroups < 1) {
        set_error_msg("q6k gemm (tcgen05): too many groups");
        return;
    }
    const size_t smem = 2 * (size_t)kTcStageBytes + 4 * (size_t)kTcN * 128 + 1024;  // two A and four B stages, alignment slack
    static size_t configured = 0;
    if (smem > configured) {
        cudaFuncSetAttribute(q6k_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        configured = smem;
    }
    launch_k("q6k_gemm_tc", q6k_gemm_tc_kernel, dim3(tiles, tgroups, n_groups), dim3(256), smem, p);
}

extern "C" {

// Q8_K activations [nblocks] (natural order, scales ad) -> f16 in the order the tcgen05 GEMM contracts over.
void llamd_fwd_act_f16_rm(const int8_t *aq, const float *ad, void *act16, size_t nblocks) {
    if (!nblocks) return;
    const size_t n = nblocks * 256;
    launch_k("act_f16_rm", act_f16_rm_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, aq, ad, (__half *)act16, nblocks);
}

// llamd_fwd_gemm_tokens at tolerance level on tcgen05: up to three matrices against ntok f16 activations.
void llamd_fwd_gemm_tokens_tc(const void *w0, const void *w1, const void *w2, const void *act16, float *o0, float *o1, float *o2,
                              int blocks, int rows0, int rows1, int rows2, int ntok) {
    if (ntok < 1) return;
    TcParams p = {};
    p.w[0] = (const uint8_t *)w0; p.w[1] = (const uint8_t *)w1; p.w[2] = (const uint8_t *)w2;
    p.out[0] = o0; p.out[1] = o1; p.out[2] = o2;
    p.rows[0] = rows0; p.rows[1] = rows1; p.rows[2] = rows2;
    p.njobs = w2 ? 3 : (w1 ? 2 : 1);
    p.nb = blocks;
    p.act = (const __half *)act16;
    p.n_tokens = ntok;
    tc_launch(p, 1, ntok);
}

// llamd_fwd_expert_gemm at tolerance level on tcgen05. max_count bounds the tokens of any one expert (the
// host knows the tile's token count; n_pairs is always a bound).
void llamd_fwd_expert_gemm_tc(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount, const int32_t *act_map,
                              const int32_t *pslot, const void *act16, float *oa, float *ob, int blocks, int rows, int n_expert,
                              int max_count) {
    TcParams p = {};
    p.w[0] = (const uint8_t *)wa; p.w[1] = (const uint8_t *)wb;
    p.out[0] = oa; p.out[1] = ob;
    p.rows[0] = rows; p.rows[1] = rows;
    p.njobs = wb ? 2 : 1;
    p.nb = blocks;
    p.act = (const __half *)act16;
    p.gstart = gstart; p.gcount = gcount; p.act_map = act_map; p.out_map = pslot;
    p.expert_units = (long long)rows * blocks;
    tc_launch(p, n_expert, max_count);
}

// 0 while every wait inside the tcgen05 GEMM has completed; otherwise 1 + the row tile of the first CTA whose
// wait ran out (its outputs, and possibly later ones, were not written). Synchronises the stream.
int llamd_fwd_gemm_tc_status(void) {
    if (!g_tc_status) return 0;
    int h = 0;
    if (cudaMemcpyAsync(&h, g_tc_status, sizeof(int), cudaMemcpyDeviceToHost, stream()) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(stream()) != cudaSuccess) return -1;
    return h;
}

}  // extern "C"
