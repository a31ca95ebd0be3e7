// Q6_K x Q8_K matrix-vector product: the decode hot path.
//
// Arithmetic contract (crates/llamd-quant/src/dot.rs:138-196). For each row:
//   per block b, eight integers  aux[r] = sum_g scale[g] * (a[16g+r]*w[16g+r] + a[16g+8+r]*w[16g+8+r])
//   then  sums[r] += (f16(d_b) * ad_b) * (float)aux[r]   for b = 0, 1, ... in order
//   then  y = ((((((s0+s1)+s2)+s3)+s4)+s5)+s6)+s7
// The integers are exact in any order; the f32 tail is reproduced operation
// for operation (separate multiply and add, no FMA), so y is bit-identical to
// the reference's scalar loop.
//
// Mapping. One thread owns one (row, block) unit of the tiled weight layout
// (q6k_layout.cuh): it streams 13 x 16 B + 2 B from HBM with fully coalesced
// loads, unpacks residue by residue and forms its eight integers with dp4a
// against activations staged in shared memory. A CTA of 256 threads covers
// floor(256/blocks) whole rows. The per-unit f32 products go through shared
// memory to the threads that walk the ordered sums.
//
// Activation staging: for block b and residue r the shared-memory image holds
// eight word pairs (lo, hi): word j carries bytes a[e(r,j,0..3)] and lo / hi
// keep bytes 0-1 / 2-3 only, so dp4a(W4_j, lo) and dp4a(W4_j, hi) are the two
// per-group pair products (times 4, since W4 = 4*(q-32)).
#include "q6k_layout.cuh"
#include "quant.cuh"

namespace llamd {

constexpr int kThreads = 256;
constexpr int kActBlockWords = 132;  // 128 + 4 padding words: conflict-free 16-byte reads across blocks
constexpr int kExStride = 257;

struct MatvecJob {
    const uint8_t *w;  // tiled Q6_K
    float *out;
    int rows;          // rows per matrix (per expert)
    int cta_begin;     // first CTA (within one slot) that works on this job
};

struct MatvecParams {
    MatvecJob job[3];
    int njobs;
    int ctas_per_slot;     // sum over jobs of ceil(rows / rows_per_cta)
    int nb;                // blocks per row
    int rows_per_cta;
    const int32_t *ids;    // [n_slots] expert ids, or null (ungrouped)
    int n_slots;           // 1 when ids is null; nseq*n_used for a batched grouped launch
    int n_expert;          // for the device-side id check
    long long expert_units;  // blocks between consecutive experts in w
    const int8_t *aq;      // activations: [nseq][nb*256] ungrouped, else indexed by slot / act_div
    const float *ad;
    int act_div;           // grouped: activation index = slot / act_div
    // Expert parallelism: this GPU holds experts [own_lo, own_hi) only, stored from local index 0.
    // A slot whose expert lives elsewhere is skipped (its output rows are left untouched).
    int own_lo, own_hi;
    // Many-token ("multi") launches, blockIdx.y = item, NSEQ sequences per item:
    //   work == null: item g covers tokens g*NSEQ .. (of n_tokens), activation
    //                 and output index = token;
    //   work != null: item i = (expert, first, count) of the expert scatter plan;
    //                 sequence s reads activation act_map[first+s] and writes output
    //                 row block out_map[first+s]; items >= *n_work do nothing.
    const int32_t *work, *n_work, *act_map, *out_map;
    int n_tokens;
    // Activation source (template parameter ACT):
    //   ACT_Q8K  aq/ad hold Q8_K activations;
    //   ACT_F32  xf holds f32 activations [index][k], quantized by every CTA in its prologue
    //            (fuses crates/llamd-rocm/src/forward.rs:375 `quantize` into the matvec);
    //   ACT_SILU xf = gate, xu = up, f32 [index][k]: silu(gate)*up, then quantized (fuses :316 too).
    const float *xf, *xu;
    PrefetchPlan pf;  // the weights of the matvec that follows this launch (a hint for L2)
    TailPlan tail;    // gate+up launches: the slot's last CTA also produces the SiLU-gated, quantized activation
    PeerOutPlan peer;  // expert parallelism: a slot's rows go to its home rank's buffer, followed by an arrival
    DispatchWait dwait;  // expert parallelism: the ids / activations are pushed by the peers; wait for all of them first
    NormPlan norm;       // ACT_NORM: the activation is made here from the residual stream (combine + rms norm + Q8_K)
    // Grouped launches: the ids were complete before the launch in front of this one began (see MatvecPlans::ids_early),
    // so they are read, and the weight loads issued, before the dependency wait.
    int ids_early;
    // Grouped launches: the order in which the CTAs take the slots (MatvecPlans::slot_order), or null for 0, 1, 2, ...
    const int32_t *slot_order;
};

//   ACT_NORM the activation is rms_norm(x + combine) * w, quantized, made by every CTA (NormPlan): the norm launch in front
//            of the matvec folded into it.
enum { ACT_Q8K = 0, ACT_F32 = 1, ACT_SILU = 2, ACT_NORM = 3 };

// shared memory: [act image][exchange floats, aliased with the natural-order staging][activation block scales]
__host__ __device__ inline size_t matvec_ad_offset(int nseq, int nb) {
    const size_t act = (size_t)nseq * nb * kActBlockWords * 4;
    const size_t ex = (size_t)nseq * 8 * kExStride * 4;
    const size_t nat = (size_t)nseq * nb * 256;
    return act + (((ex > nat ? ex : nat) + 15) & ~(size_t)15);
}

// One CTA of a launch with peer outputs is done (its stores, if any, fenced at system scope by the caller): count it,
// and let the CTA that completes the count tell every rank that this rank's rows are in place.
__device__ __forceinline__ void peer_arrive(const PeerOutPlan &peer, unsigned int total_ctas, int home) {
    if (!peer.local_done) {  // the per-CTA form: every CTA arrives on its slot's home rank
        atomicAdd_system(peer.arrive_tab[home], 1u);
        return;
    }
    if (atomicInc(peer.local_done, total_ctas - 1) == total_ctas - 1) {  // wraps to 0 for the next launch
        __threadfence_system();  // (orders the counted CTAs' fenced stores before the arrivals below)
        for (int h = 0; h < peer.world; h++) atomicAdd_system(peer.arrive_tab[h], 1u);
    }
}

// EP: the expert-parallel forms (requests pushed by peers, rows stored to peers); kept out of the other instantiations.
// EXTRA: the optional L2 prefetch plan and the SiLU tail. Both are off by default, and their code in the plain kernel
// cost every launch ~0.3 us and lm_head 3 % of its bandwidth, so they too are an instantiation of their own.
template <int NSEQ, bool MULTI, int ACT, bool EP = false, bool EXTRA = false>
__global__ void __launch_bounds__(kThreads, NSEQ == 1 ? 3 : (NSEQ == 2 ? 2 : 1)) matvec_q6k_kernel(const MatvecParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int nb = p.nb;
    // shared memory: [act: NSEQ*nb*132 words][ex: NSEQ*8*257 floats, aliased with the natural-order staging]
    uint32_t *s_act = reinterpret_cast<uint32_t *>(smem);
    float *s_ex = reinterpret_cast<float *>(smem + (size_t)NSEQ * nb * kActBlockWords * 4);
    int8_t *s_nat = reinterpret_cast<int8_t *>(s_ex);
    float *s_ad = reinterpret_cast<float *>(smem + matvec_ad_offset(NSEQ, nb));  // [NSEQ*nb] activation block scales

    // A grouped launch lets its successor start only once it has passed its own wait: whatever starts after it may then
    // take the router's ids as complete (the down projection reads them before ITS wait). The other forms let go at once.
    const bool early = !MULTI && p.ids && p.ids_early;
    const bool late_trigger = !MULTI && p.ids && !early;
    if (!late_trigger) pdl_trigger();
    // ---- which job / slot / rows -------------------------------------
    int slot = blockIdx.x / p.ctas_per_slot;
    const int cta = blockIdx.x - slot * p.ctas_per_slot;
    int j = 0;
    if (p.njobs > 1 && cta >= p.job[1].cta_begin) j = 1;
    if (p.njobs > 2 && cta >= p.job[2].cta_begin) j = 2;
    const MatvecJob job = p.job[j];
    const int row0 = (cta - job.cta_begin) * p.rows_per_cta;
    const int rows_here = min(p.rows_per_cta, job.rows - row0);
    const int tid = threadIdx.x;
    const bool active = tid < rows_here * nb;
    const int row_l = tid / nb, b = tid - row_l * nb;
    // ungrouped launches may be cut into groups of NSEQ sequences, one "slot" per group (small matrices at batch > 1:
    // more CTAs for the same rows; the weights are re-read from L2)
    const int seq0 = (!MULTI && !p.ids) ? slot * NSEQ : 0;

    // expert id of this slot (grouped forms); an id outside the tensor reads
    // expert 0: the host wrappers refuse such ids before any launch.
    long long expert_off = 0;
    __shared__ int s_aidx[NSEQ], s_oidx[NSEQ];
    int count = NSEQ;
    if (MULTI) {
        pdl_wait();
        const int item = blockIdx.y;
        int first;
        if (p.work) {
            if (item >= *p.n_work) return;
            int e = p.work[3 * item];
            if (e < 0 || e >= p.n_expert) e = 0;
            expert_off = (long long)e * p.expert_units;
            first = p.work[3 * item + 1];
            count = min(NSEQ, p.work[3 * item + 2]);
        } else {
            first = item * NSEQ;
            count = min(NSEQ, p.n_tokens - first);
        }
        if (tid < NSEQ) {
            const int sidx = first + (tid < count ? tid : 0);  // unused sequences shadow the first (never stored)
            s_aidx[tid] = p.act_map ? p.act_map[sidx] : sidx;
            s_oidx[tid] = p.out_map ? p.out_map[sidx] : sidx;
        }
        __syncthreads();
    } else if (p.ids) {
        if (!early) pdl_wait();  // the ids come from the router kernel
        if (!EP && p.slot_order) slot = __ldcg(p.slot_order + slot);  // (slots of one expert side by side: its second reader finds it in L2)
        if (EP && p.dwait.counter) {  // ... or from every rank's push: all of this layer's records must have landed
            if (tid == 0) {
                unsigned int ep;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(ep) : "l"(p.dwait.epoch) : "memory");
                bounded_wait(p.dwait.counter, ep * p.dwait.world, true, p.dwait.status, 2, p.dwait.limit);
            }
            __syncthreads();
        }
        if (!early) pdl_trigger();  // (behind the wait for the records too: what starts after this launch may read them)
        if (EXTRA) prefetch_issue(p.pf, blockIdx.x, gridDim.x);
        int e = (EP || early) ? __ldcg(p.ids + slot) : p.ids[slot];
        if (e < 0 || e >= p.n_expert) e = 0;
        if (e < p.own_lo || e >= p.own_hi) {  // another GPU's expert
            // by now this CTA has read everything it needs of the request: the home rank may count it -- but only once
            // the launches in front, which read the same request, are complete (the home rank overwrites it afterwards)
            if (EP && p.peer.out_tab) {
                if (early) pdl_wait();
                if (tid == 0) peer_arrive(p.peer, gridDim.x, slot / p.peer.div);
            }
            return;
        }
        expert_off = (long long)(e - p.own_lo) * p.expert_units;
    }

    // ---- issue the weight loads first: they stay in flight across the staging barrier
    uint32_t S[48];
    uint4 scw = make_uint4(0, 0, 0, 0);
    uint16_t dbits = 0;
    if (active) {
        const size_t unit = (size_t)expert_off + (size_t)(row0 + row_l) * nb + b;
        const uint8_t *tile = job.w + (unit >> 5) * kTileBytes;
        const int sl = (int)(unit & 31);
        const uint4 *cp = reinterpret_cast<const uint4 *>(tile) + sl;
#pragma unroll
        for (int c = 0; c < 12; c++) {
            const uint4 v = __ldg(cp + c * 32);
            S[4 * c + 0] = v.x;
            S[4 * c + 1] = v.y;
            S[4 * c + 2] = v.z;
            S[4 * c + 3] = v.w;
        }
        scw = __ldg(reinterpret_cast<const uint4 *>(tile + kTileScaleOff) + sl);
        dbits = __ldg(reinterpret_cast<const uint16_t *>(tile + kTileDOff) + sl);
    }

    // Ungrouped: the weight loads above do not depend on the previous kernel and
    // are in flight while it finishes; the activations below do.
    if (!MULTI && !p.ids) {
        if (EXTRA && !p.pf.ids) prefetch_issue(p.pf, blockIdx.x, gridDim.x);
        pdl_wait();
        if (EXTRA && p.pf.ids) prefetch_issue(p.pf, blockIdx.x, gridDim.x);
    } else if (early) {
        pdl_wait();  // the activations come from the launch in front
    }
    // ---- stage the activations ----------------------------------------
    // natural order bytes first ...
    if (ACT == ACT_Q8K) {
        // (the block scales are read where they are used, straight from global memory: staging them here put a second
        // dependent round trip in front of the barrier and cost every launch ~0.4 us)
        const int n16 = NSEQ * nb * 16;
        for (int i = tid; i < n16; i += kThreads) {
            const int s = i / (nb * 16), o = i - s * nb * 16;
            const long long a_idx = MULTI ? s_aidx[s] : (p.ids ? slot / p.act_div : seq0 + s);
            const uint4 *src = reinterpret_cast<const uint4 *>(p.aq + a_idx * nb * 256) + o;
            reinterpret_cast<uint4 *>(s_nat)[i] = (EP && p.dwait.counter) ? __ldcg(src) : __ldg(src);  // written by peers: from L2
        }
    } else if (ACT == ACT_NORM) {
        // ... made here from the residual stream: combine, norm (its sum of squares walked in order by one thread), weight,
        // Q8_K (crates/llamd-runtime/src/layer.rs:243-258 and 281-287, crates/llamd-cpu/src/lib.rs:55-75, dot.rs:88-128)
        const NormPlan &np = p.norm;
        const int k = nb * 256, k4 = k / 4;
        float *s_x = reinterpret_cast<float *>(smem + ((matvec_ad_offset(NSEQ, nb) + (size_t)NSEQ * nb * 4 + 15) & ~(size_t)15));
        float *s_sq = s_x + k;
        __shared__ float s_nscale;
        for (int j0 = 0; j0 < k4; j0 += 2 * kThreads) {
            const int ja = j0 + tid, jb = j0 + kThreads + tid;
            float4 xa = ja < k4 ? reinterpret_cast<const float4 *>(np.x)[ja] : make_float4(0.f, 0.f, 0.f, 0.f);
            float4 xb = jb < k4 ? reinterpret_cast<const float4 *>(np.x)[jb] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (np.down) {
                float4 aa = make_float4(0.f, 0.f, 0.f, 0.f), ab = aa;
                for (int e0 = 0; e0 < np.n_used; e0 += 4) {
                    float4 da[4], db[4];
                    float we[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        const int e = e0 + q;
                        we[q] = e < np.n_used ? np.cw[e] : 0.0f;
                        const float4 *d4 = reinterpret_cast<const float4 *>(np.down + (size_t)(e < np.n_used ? e : 0) * k);
                        da[q] = (ja < k4 && e < np.n_used) ? __ldcg(d4 + ja) : make_float4(0.f, 0.f, 0.f, 0.f);
                        db[q] = (jb < k4 && e < np.n_used) ? __ldcg(d4 + jb) : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int q = 0; q < 4; q++)
                        if (e0 + q < np.n_used) {
                            aa.x = __fadd_rn(aa.x, __fmul_rn(we[q], da[q].x)); aa.y = __fadd_rn(aa.y, __fmul_rn(we[q], da[q].y));
                            aa.z = __fadd_rn(aa.z, __fmul_rn(we[q], da[q].z)); aa.w = __fadd_rn(aa.w, __fmul_rn(we[q], da[q].w));
                            ab.x = __fadd_rn(ab.x, __fmul_rn(we[q], db[q].x)); ab.y = __fadd_rn(ab.y, __fmul_rn(we[q], db[q].y));
                            ab.z = __fadd_rn(ab.z, __fmul_rn(we[q], db[q].z)); ab.w = __fadd_rn(ab.w, __fmul_rn(we[q], db[q].w));
                        }
                }
                xa = make_float4(__fadd_rn(xa.x, aa.x), __fadd_rn(xa.y, aa.y), __fadd_rn(xa.z, aa.z), __fadd_rn(xa.w, aa.w));
                xb = make_float4(__fadd_rn(xb.x, ab.x), __fadd_rn(xb.y, ab.y), __fadd_rn(xb.z, ab.z), __fadd_rn(xb.w, ab.w));
            }
            if (ja < k4) {
                reinterpret_cast<float4 *>(s_x)[ja] = xa;
                reinterpret_cast<float4 *>(s_sq)[ja] = make_float4(__fmul_rn(xa.x, xa.x), __fmul_rn(xa.y, xa.y), __fmul_rn(xa.z, xa.z), __fmul_rn(xa.w, xa.w));
                if (blockIdx.x == 0 && np.x_out) reinterpret_cast<float4 *>(np.x_out)[ja] = xa;
            }
            if (jb < k4) {
                reinterpret_cast<float4 *>(s_x)[jb] = xb;
                reinterpret_cast<float4 *>(s_sq)[jb] = make_float4(__fmul_rn(xb.x, xb.x), __fmul_rn(xb.y, xb.y), __fmul_rn(xb.z, xb.z), __fmul_rn(xb.w, xb.w));
                if (blockIdx.x == 0 && np.x_out) reinterpret_cast<float4 *>(np.x_out)[jb] = xb;
            }
        }
        __syncthreads();
        if (tid == 0) s_nscale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(chain_sum(s_sq, k, 0.0f), (float)k), np.eps)));
        __syncthreads();
        const float nscale = s_nscale;
        const int warp = tid >> 5, lane = tid & 31;
        for (int blk = warp; blk < nb; blk += kThreads / 32) {
            const float4 a = reinterpret_cast<const float4 *>(s_x + blk * 256 + lane * 8)[0], c4 = reinterpret_cast<const float4 *>(s_x + blk * 256 + lane * 8)[1];
            const float4 wa = __ldg(reinterpret_cast<const float4 *>(np.w + blk * 256 + lane * 8)), wb = __ldg(reinterpret_cast<const float4 *>(np.w + blk * 256 + lane * 8) + 1);
            const float v[8] = {__fmul_rn(__fmul_rn(a.x, nscale), wa.x), __fmul_rn(__fmul_rn(a.y, nscale), wa.y), __fmul_rn(__fmul_rn(a.z, nscale), wa.z),
                                __fmul_rn(__fmul_rn(a.w, nscale), wa.w), __fmul_rn(__fmul_rn(c4.x, nscale), wb.x), __fmul_rn(__fmul_rn(c4.y, nscale), wb.y),
                                __fmul_rn(__fmul_rn(c4.z, nscale), wb.z), __fmul_rn(__fmul_rn(c4.w, nscale), wb.w)};
            q8k_quantize_block(v, lane, s_nat + blk * 256, s_ad + blk, nullptr);
        }
    } else if (ACT == ACT_SILU) {
        // ... produced here: silu(gate) * up with one or a few elements per thread (a lane walking eight dependent exp
        // evaluations one after the other was most of this prologue), then one warp per 256-element block quantizes
        float *s_f = reinterpret_cast<float *>(smem + ((matvec_ad_offset(NSEQ, nb) + (size_t)NSEQ * nb * 4 + 15) & ~(size_t)15));
        const long long a_idx = p.ids ? slot / p.act_div : seq0;
        const size_t base = (size_t)a_idx * nb * 256;
        for (int i = tid; i < nb * 256; i += kThreads) s_f[i] = silu_mul(p.xf[base + i], p.xu[base + i]);
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31;
        for (int blk = warp; blk < nb; blk += kThreads / 32) {
            const float4 a = reinterpret_cast<const float4 *>(s_f + blk * 256 + lane * 8)[0], c4 = reinterpret_cast<const float4 *>(s_f + blk * 256 + lane * 8)[1];
            const float v[8] = {a.x, a.y, a.z, a.w, c4.x, c4.y, c4.z, c4.w};
            q8k_quantize_block(v, lane, s_nat + blk * 256, s_ad + blk, nullptr);
        }
    } else {
        // ... produced here: one warp per 256-element block quantizes the f32 activation
        const int warp = tid >> 5, lane = tid & 31;
        for (int blk = warp; blk < NSEQ * nb; blk += kThreads / 32) {
            const int s = blk / nb, o = blk - s * nb;
            const long long a_idx = MULTI ? s_aidx[s] : (p.ids ? slot / p.act_div : seq0 + s);
            const size_t base = ((size_t)a_idx * nb + o) * 256 + lane * 8;
            const float4 g0 = *reinterpret_cast<const float4 *>(p.xf + base), g1 = *reinterpret_cast<const float4 *>(p.xf + base + 4);
            float v[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            if (ACT == ACT_SILU) {
                const float4 u0 = *reinterpret_cast<const float4 *>(p.xu + base), u1 = *reinterpret_cast<const float4 *>(p.xu + base + 4);
                const float u[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = silu_mul(v[i], u[i]);
            }
            q8k_quantize_block(v, lane, s_nat + blk * 256, s_ad + blk, nullptr);
        }
    }
    __syncthreads();
    // ... then the residue-major (lo, hi) image
    {
        const int nitems = NSEQ * nb * 64;  // (s, b, r, j)
        for (int i = tid; i < nitems; i += kThreads) {
            const int jj = i & 7, r = (i >> 3) & 7, sb = i >> 6;
            const int8_t *src = s_nat + sb * 256;
            const uint32_t b0 = (uint8_t)src[t32_element(r, jj, 0)], b1 = (uint8_t)src[t32_element(r, jj, 1)];
            const uint32_t b2 = (uint8_t)src[t32_element(r, jj, 2)], b3 = (uint8_t)src[t32_element(r, jj, 3)];
            uint32_t *dst = s_act + sb * kActBlockWords + r * 16 + jj * 2;
            dst[0] = b0 | (b1 << 8);
            dst[1] = (b2 << 16) | (b3 << 24);
        }
    }
    __syncthreads();  // s_nat is dead from here: s_ex may be written

    // ---- integer core -----------------------------------------------------
    if (active) {
        int sc[16];
        {
            const uint32_t ws[4] = {scw.x, scw.y, scw.z, scw.w};
#pragma unroll
            for (int i = 0; i < 16; i++) sc[i] = (int)(int8_t)(ws[i >> 2] >> (8 * (i & 3)));
        }
        int aux[NSEQ][8];
#pragma unroll
        for (int s = 0; s < NSEQ; s++)
#pragma unroll
            for (int r = 0; r < 8; r++) aux[s][r] = 0;
#pragma unroll
        for (int r = 0; r < 8; r++) {
#pragma unroll
            for (int m = 0; m < 2; m++) {
                uint32_t w4[4];
                unpack_quad(S[6 * r + 3 * m], S[6 * r + 3 * m + 1], S[6 * r + 3 * m + 2], w4);
#pragma unroll
                for (int s = 0; s < NSEQ; s++) {
                    const uint4 *ap = reinterpret_cast<const uint4 *>(s_act + (s * nb + b) * kActBlockWords + r * 16 + m * 8);
                    const uint4 a01 = ap[0], a23 = ap[1];
                    int acc = aux[s][r];
                    acc += sc[8 * m + 0] * __dp4a((int)w4[0], (int)a01.x, 0);
                    acc += sc[8 * m + 1] * __dp4a((int)w4[0], (int)a01.y, 0);
                    acc += sc[8 * m + 2] * __dp4a((int)w4[1], (int)a01.z, 0);
                    acc += sc[8 * m + 3] * __dp4a((int)w4[1], (int)a01.w, 0);
                    acc += sc[8 * m + 4] * __dp4a((int)w4[2], (int)a23.x, 0);
                    acc += sc[8 * m + 5] * __dp4a((int)w4[2], (int)a23.y, 0);
                    acc += sc[8 * m + 6] * __dp4a((int)w4[3], (int)a23.z, 0);
                    acc += sc[8 * m + 7] * __dp4a((int)w4[3], (int)a23.w, 0);
                    aux[s][r] = acc;
                }
            }
        }
        const float dw = f16_bits_to_f32(dbits);
#pragma unroll
        for (int s = 0; s < NSEQ; s++) {
            float adv;
            if (ACT == ACT_Q8K) {
                const long long a_idx = MULTI ? s_aidx[s] : (p.ids ? slot / p.act_div : seq0 + s);
                adv = (EP && p.dwait.counter) ? __ldcg(p.ad + a_idx * nb + b) : __ldg(p.ad + a_idx * nb + b);
            } else {
                adv = s_ad[s * nb + b];  // produced by this CTA's quantizer
            }
            const float dsc = __fmul_rn(dw, adv);
#pragma unroll
            for (int r = 0; r < 8; r++)
                s_ex[(s * 8 + r) * kExStride + tid] = __fmul_rn(dsc, (float)(aux[s][r] >> 2));
        }
    }
    __syncthreads();

    // ---- ordered f32 tail ---------------------------------------------------
    // thread (row_l, r) adds the blocks in order; then the eight residues are
    // added in order across the 8 adjacent lanes.
    const int n_out = rows_here * 8;
    for (int base = 0; base < n_out; base += kThreads) {
        const int idx = base + tid;
        const bool on = idx < n_out;
        const int rl = idx >> 3, r = idx & 7;
#pragma unroll
        for (int s = 0; s < NSEQ; s++) {
            float acc = 0.0f;
            if (on) {
                const float *ex = s_ex + (s * 8 + r) * kExStride + rl * nb;
                for (int bb = 0; bb < nb; bb++) acc = __fadd_rn(acc, ex[bb]);
            }
            const int lane0 = (tid & 31) & ~7;
            float total = __shfl_sync(0xffffffffu, acc, lane0);
#pragma unroll
            for (int rr = 1; rr < 8; rr++) total = __fadd_rn(total, __shfl_sync(0xffffffffu, acc, lane0 + rr));
            // ungrouped: out[seq][rows]; grouped: out[slot][rows]
            if (MULTI) {
                if (on && r == 0 && s < count) job.out[(long long)s_oidx[s] * job.rows + row0 + rl] = total;
            } else if (on && r == 0) {
                if (EP && p.peer.out_tab)  // (grouped launches run one sequence per slot: s == 0)
                    p.peer.out_tab[slot / p.peer.div][(size_t)(slot % p.peer.div) * job.rows + row0 + rl] = total;
                else
                    job.out[((long long)s + (p.ids ? slot : seq0)) * job.rows + row0 + rl] = total;
            }
        }
    }
    if (EP && !MULTI && p.peer.out_tab) {  // uniform over the launch; CTAs of slots this rank does not own left above
        __threadfence_system();  // the rows are visible on the home GPU before the rank's arrival is
        __syncthreads();
        if (tid == 0) peer_arrive(p.peer, gridDim.x, slot / p.peer.div);
    }
    // ---- tail of a gate+up launch: silu(gate) * up and its Q8_K form, by the slot's last CTA ----
    if (EXTRA && !MULTI && NSEQ == 1 && p.tail.counter) {  // uniform over the launch
        __shared__ bool s_last;
        __threadfence();  // this CTA's rows are visible before its arrival is
        __syncthreads();
        if (tid == 0) s_last = atomicInc(p.tail.counter + slot, p.ctas_per_slot - 1) == (unsigned)p.ctas_per_slot - 1;  // wraps to 0
        __syncthreads();
        if (s_last) {
            __threadfence();
            const int rows = p.job[0].rows, nblk = rows >> 8, lane = tid & 31;
            const float *gate = p.job[0].out + (size_t)slot * rows, *up = p.job[1].out + (size_t)slot * rows;
            for (int blk = tid >> 5; blk < nblk; blk += kThreads / 32) {
                const size_t base = (size_t)blk * 256 + lane * 8;
                const float4 g0 = __ldcg(reinterpret_cast<const float4 *>(gate + base)), g1 = __ldcg(reinterpret_cast<const float4 *>(gate + base + 4));
                const float4 u0 = __ldcg(reinterpret_cast<const float4 *>(up + base)), u1 = __ldcg(reinterpret_cast<const float4 *>(up + base + 4));
                float v[8] = {silu_mul(g0.x, u0.x), silu_mul(g0.y, u0.y), silu_mul(g0.z, u0.z), silu_mul(g0.w, u0.w),
                              silu_mul(g1.x, u1.x), silu_mul(g1.y, u1.y), silu_mul(g1.z, u1.z), silu_mul(g1.w, u1.w)};
                q8k_quantize_block(v, lane, p.tail.qs + ((size_t)slot * nblk + blk) * 256, p.tail.d + (size_t)slot * nblk + blk, nullptr);
            }
        }
    }
}

static size_t matvec_smem_bytes(int nseq, int nb, int act = ACT_Q8K) {
    const size_t base = matvec_ad_offset(nseq, nb) + (size_t)nseq * nb * 4;
    if (act == ACT_SILU) return ((base + 15) & ~(size_t)15) + (size_t)nb * 256 * 4;  // + the activation as f32
    return act == ACT_NORM ? ((base + 15) & ~(size_t)15) + (size_t)2 * nb * 256 * 4 : base;  // + the residual stream and its squares
}

// sequences per CTA for small ungrouped matrices at batch > 1 (0: never split), and what "small" means
int g_batch_group = 2;  // set through llamd_fwd_set_batch_group
constexpr int kBatchSplitMaxCtas = 512;

template <int NSEQ, bool MULTI = false, int ACT = ACT_Q8K>
static void launch_t(const MatvecParams &p, dim3 grid, const MatvecPlans &plans) {
    const size_t smem = matvec_smem_bytes(NSEQ, p.nb, ACT);
    static size_t configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(matvec_q6k_kernel<NSEQ, MULTI, ACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            set_error(e, "matvec smem attribute");
            return;
        }
        configured = smem;
    }
    MatvecParams q = p;
    q.pf = plans.pf;
    q.norm = plans.norm;
    q.dwait = plans.dwait;
    q.peer = plans.peer;
    q.tail = plans.tail;
    q.ids_early = (plans.ids_early && !MULTI && p.ids && !q.dwait.counter) ? 1 : 0;
    q.slot_order = (!MULTI && p.ids && !q.dwait.counter && !q.peer.out_tab) ? plans.slot_order : nullptr;
    // each plan fits one kind of launch only; a plan given to another kind is refused, not dropped
    if (q.dwait.counter && !(!MULTI && NSEQ == 1 && p.ids)) {
        set_error_msg("matvec: a dispatch wait was planned for a launch that cannot carry it");
        return;
    }
    if (q.peer.out_tab && !(!MULTI && NSEQ == 1 && p.ids && p.njobs == 1)) {
        set_error_msg("matvec: peer outputs were planned for a launch that cannot carry them");
        return;
    }
    // a SiLU tail: only a grouped launch of two matrices whose rows are whole Q8_K blocks can take it
    if (q.tail.counter && !(!MULTI && NSEQ == 1 && p.ids && p.njobs == 2 && p.job[0].rows % 256 == 0 && p.own_lo == 0 && p.own_hi >= p.n_expert)) {
        set_error_msg("matvec: a SiLU tail was planned for a launch that cannot carry it");
        return;
    }
    const bool extra = q.tail.counter || q.pf.ids || q.pf.bytes[0] || q.pf.bytes[1] || q.pf.bytes[2];
    if (NSEQ == 1 && !MULTI && ACT == ACT_Q8K && extra && !(q.peer.out_tab || q.dwait.counter)) {
        launch_kc(p.ids ? PDL_GROUPED : PDL_MATVEC, "matvec_q6k_extra", matvec_q6k_kernel<1, false, ACT_Q8K, false, true>, grid, dim3(kThreads), smem, q);
        return;
    }
    if (NSEQ == 1 && !MULTI && ACT == ACT_Q8K && (q.peer.out_tab || q.dwait.counter)) {
        launch_kc(PDL_GROUPED, "matvec_q6k_ep", matvec_q6k_kernel<1, false, ACT_Q8K, true>, grid, dim3(kThreads), smem, q);
        return;
    }
    if (q.peer.out_tab || q.dwait.counter) {
        set_error_msg("matvec: the expert-parallel forms exist for one sequence of Q8_K activations only");
        return;
    }
    if (extra) {  // the plain instantiations do not carry the optional parts
        q.pf = PrefetchPlan{};
        if (q.tail.counter) {
            set_error_msg("matvec: a SiLU tail needs one sequence of Q8_K activations");
            return;
        }
    }
    launch_kc(MULTI ? PDL_OTHER : (p.ids ? PDL_GROUPED : PDL_MATVEC), "matvec_q6k", matvec_q6k_kernel<NSEQ, MULTI, ACT>, grid, dim3(kThreads), smem, q);
}

// Build the launch. `rows[i]`/`w[i]`/`out[i]` describe up to three matrices
// that share the activation (q,k,v or gate,up). Ungrouped (ids == null): nseq
// activations, outputs [nseq][rows]. Grouped: n_slots expert ids, activation of
// slot s is index s / act_div, outputs [n_slots][rows]; nseq must be 1.
void launch_matvec(int njobs, const void *const *w, float *const *out, const int *rows, int blocks, const int8_t *aq,
                   const float *ad, int nseq, const int32_t *ids, int n_slots, int n_expert, int act_div, int act_mode, const float *xf,
                   const float *xu, int own_lo, int own_hi, const MatvecPlans &plans) {
    if (blocks <= 0 || blocks > kThreads || nseq < 1 || nseq > LLAMD_MAX_BATCH || njobs < 1 || njobs > 3 || (ids && nseq != 1) ||
        (ids && (n_slots < 1 || act_div < 1)) || (nseq > LLAMD_MAX_SEQ && act_mode != ACT_Q8K)) {
        set_error_msg("matvec: blocks must be 1..256, nseq 1..8 (ungrouped Q8_K activations: up to 256), 1..3 matrices");
        return;
    }
    if (nseq > LLAMD_MAX_SEQ) {
        // more sequences than one launch holds: the launch's group size where it splits small matrices over the sequences
        // anyway (below), else one launch per LLAMD_MAX_SEQ sequences (activations and outputs are [nseq][...])
        int ctas = 0;
        for (int i = 0; i < njobs; i++) ctas += rows[i] > 0 ? (rows[i] + kThreads / blocks - 1) / (kThreads / blocks) : 0;
        if (!(g_batch_group > 0 && ctas <= kBatchSplitMaxCtas)) {
            for (int s0 = 0; s0 < nseq; s0 += LLAMD_MAX_SEQ) {
                const int cnt = nseq - s0 < LLAMD_MAX_SEQ ? nseq - s0 : LLAMD_MAX_SEQ;
                float *o[3] = {nullptr, nullptr, nullptr};
                for (int i = 0; i < njobs; i++) o[i] = out[i] + (size_t)s0 * rows[i];
                launch_matvec(njobs, w, o, rows, blocks, aq + (size_t)s0 * blocks * 256, ad + (size_t)s0 * blocks, cnt, ids, n_slots, n_expert,
                              act_div, act_mode, xf, xu, own_lo, own_hi, plans);
            }
            return;
        }
    }
    MatvecParams p = {};
    p.njobs = njobs;
    p.nb = blocks;
    p.rows_per_cta = kThreads / blocks;
    int cta = 0;
    for (int i = 0; i < njobs; i++) {
        if (rows[i] <= 0 || (ids && rows[i] != rows[0])) {
            set_error_msg("matvec: rows must be positive (and equal across a grouped launch)");
            return;
        }
        p.job[i].w = (const uint8_t *)w[i];
        p.job[i].out = out[i];
        p.job[i].rows = rows[i];
        p.job[i].cta_begin = cta;
        cta += (rows[i] + p.rows_per_cta - 1) / p.rows_per_cta;
    }
    p.ctas_per_slot = cta;
    p.ids = ids;
    p.n_slots = ids ? n_slots : 1;
    p.n_expert = n_expert;
    p.expert_units = (long long)rows[0] * blocks;  // experts are `rows` rows apart in the reference order
    p.aq = aq;
    p.ad = ad;
    p.act_div = act_div < 1 ? 1 : act_div;
    p.xf = xf;
    p.xu = xu;
    p.own_lo = own_lo;
    p.own_hi = own_hi;
    // Small matrices at batch > 1: one CTA per 256 (row, block) units leaves most SMs with a single CTA that does nseq
    // times the integer work. Cut the sequences into groups of g (a divisor of nseq): nseq / g times the CTAs.
    if (!ids && nseq > 1 && g_batch_group > 0 && p.ctas_per_slot <= kBatchSplitMaxCtas) {
        int g = g_batch_group < nseq ? g_batch_group : nseq;
        while (nseq % g) g--;
        p.n_slots = nseq / g;
        nseq = g;
    }
    if (nseq > LLAMD_MAX_SEQ || matvec_smem_bytes(nseq, blocks) > 200 * 1024) {
        set_error_msg("matvec: blocks x nseq does not fit a launch");
        return;
    }
    const dim3 grid(p.ctas_per_slot * p.n_slots);
    if (act_mode == ACT_NORM) {
        if (nseq != 1 || ids || !plans.norm.x || !plans.norm.w || plans.norm.x_out == plans.norm.x || (plans.norm.down && (plans.norm.n_used < 1 || !plans.norm.cw)) ||
            matvec_smem_bytes(1, blocks, ACT_NORM) > 200 * 1024) {
            set_error_msg("matvec: a folded norm takes one sequence, ungrouped, with x, w and an x_out other than x");
            return;
        }
        launch_t<1, false, ACT_NORM>(p, grid, plans);
        return;
    }
    if (act_mode == ACT_SILU) {
        if (nseq != 1 || !xf || !xu) {
            set_error_msg("matvec: the silu activation mode takes gate and up, one sequence per slot");
            return;
        }
        launch_t<1, false, ACT_SILU>(p, grid, plans);
        return;
    }
    if (act_mode == ACT_F32) {
        if (!xf) {
            set_error_msg("matvec: f32 activation mode without activations");
            return;
        }
        switch (nseq) {
        case 1: launch_t<1, false, ACT_F32>(p, grid, plans); break;
        case 2: launch_t<2, false, ACT_F32>(p, grid, plans); break;
        case 3: launch_t<3, false, ACT_F32>(p, grid, plans); break;
        case 4: launch_t<4, false, ACT_F32>(p, grid, plans); break;
        case 5: launch_t<5, false, ACT_F32>(p, grid, plans); break;
        case 6: launch_t<6, false, ACT_F32>(p, grid, plans); break;
        case 7: launch_t<7, false, ACT_F32>(p, grid, plans); break;
        default: launch_t<8, false, ACT_F32>(p, grid, plans); break;
        }
        return;
    }
    switch (nseq) {
    case 1: launch_t<1>(p, grid, plans); break;
    case 2: launch_t<2>(p, grid, plans); break;
    case 3: launch_t<3>(p, grid, plans); break;
    case 4: launch_t<4>(p, grid, plans); break;
    case 5: launch_t<5>(p, grid, plans); break;
    case 6: launch_t<6>(p, grid, plans); break;
    case 7: launch_t<7>(p, grid, plans); break;
    default: launch_t<8>(p, grid, plans); break;
    }
}

// Many tokens against shared weights, 8 at a time (the prefill path).
//   work == null: every token 0..n_tokens-1 against the matrices w[i] (QKV, attn_out): out[i][token][rows];
//   work != null: the expert scatter plan's work list (expert, first pair, count<=8): pair p reads activation
//                 act_map[p] and writes out[out_map[p]][rows], expert-major, so an expert's rows are streamed once
//                 for up to 8 of its pairs (crates/llamd-vulkan/shaders/q6k_expert_major[_pa].comp).
void launch_matvec_multi(int njobs, const void *const *w, float *const *out, const int *rows, int blocks, const int8_t *aq,
                         const float *ad, int n_tokens, const int32_t *work, const int32_t *n_work, int max_items, const int32_t *act_map,
                         const int32_t *out_map, int n_expert) {
    constexpr int NS = 8;
    if (blocks <= 0 || blocks > kThreads || njobs < 1 || njobs > 3 || (!work && n_tokens < 1) || (work && (!n_work || max_items < 1))) {
        set_error_msg("matvec_multi: bad arguments");
        return;
    }
    if (matvec_smem_bytes(NS, blocks) > 200 * 1024) {
        set_error_msg("matvec_multi: blocks does not fit shared memory");
        return;
    }
    MatvecParams p = {};
    p.njobs = njobs;
    p.nb = blocks;
    p.rows_per_cta = kThreads / blocks;
    int cta = 0;
    for (int i = 0; i < njobs; i++) {
        if (rows[i] <= 0 || (work && rows[i] != rows[0])) {
            set_error_msg("matvec_multi: rows must be positive (and equal across an expert launch)");
            return;
        }
        p.job[i].w = (const uint8_t *)w[i];
        p.job[i].out = out[i];
        p.job[i].rows = rows[i];
        p.job[i].cta_begin = cta;
        cta += (rows[i] + p.rows_per_cta - 1) / p.rows_per_cta;
    }
    p.ctas_per_slot = cta;
    p.n_slots = 1;
    p.n_expert = n_expert;
    p.expert_units = (long long)rows[0] * blocks;
    p.aq = aq;
    p.ad = ad;
    p.act_div = 1;
    p.work = work;
    p.n_work = n_work;
    p.act_map = act_map;
    p.out_map = out_map;
    p.n_tokens = n_tokens;
    const int items = work ? max_items : (n_tokens + NS - 1) / NS;
    if (items > 65535) {
        set_error_msg("matvec_multi: too many items for one launch");
        return;
    }
    launch_t<NS, true>(p, dim3(cta, items), MatvecPlans{});
}

}  // namespace llamd
