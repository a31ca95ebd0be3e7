// Shared host/device helpers for libllamd_cuda.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/llamd_cuda.h"

namespace llamd {

// One stream for every device-pointer op, as in the reference's device layer
// (crates/llamd-rocm/kernels/llamd_forward.hip:701-716).
cudaStream_t stream();
// Sticky error state: the first failure is kept until read.
void set_error(cudaError_t e, const char *what);
void set_error_msg(const char *what);
int error_code();

// Kernel launches issued through the library since it was loaded (a launch
// recorded into a graph counts once, at capture).
extern unsigned long long g_launches;

#define LLAMD_CHECK_LAUNCH(what)                                   \
    do {                                                           \
        ::llamd::g_launches++;                                     \
        cudaError_t e__ = cudaPeekAtLastError();                   \
        if (e__ != cudaSuccess) ::llamd::set_error(e__, what);     \
    } while (0)

#define LLAMD_TRY(call, what)                                      \
    do {                                                           \
        cudaError_t e__ = (call);                                  \
        if (e__ != cudaSuccess) {                                  \
            ::llamd::set_error(e__, what);                         \
            return -1;                                             \
        }                                                          \
    } while (0)

// Programmatic dependent launch. Every kernel on the decode path is launched
// with the stream-serialization attribute relaxed, calls pdl_trigger() first
// (so the next kernel in the stream may be scheduled while this one runs) and
// pdl_wait() before it touches anything an earlier kernel wrote. What sits
// between the two -- streaming read-only weights into registers -- overlaps
// the tail of the previous kernel. pdl_wait() returns only when the preceding
// kernel has completed and flushed, and every kernel calls it, so completion
// is transitive along the stream. Without the attribute both are no-ops.
extern int g_pdl;
// What a model's decode pass asks of the kernels it launches: an argument of the internal launch functions (..._flags,
// attention_rope_quant, combine_rms_norm_quant_wait) that they hand to the kernels; the extern "C" entry points pass 0.
// Bits 1 | 2 | 4: the `fast` arithmetic (model option arith) -- the norms' sums of squares, the router's dots, attention's
// softmax sum and weighted values as reduction trees instead of the reference's ordered sums. kPassEarlyLoads: the
// attention kernels read the positions and the cached rows of earlier positions before their dependency wait; true only
// inside a pass whose first launch waits for everything in front of it.
constexpr int kPassEarlyLoads = 8;
// kPassAttnGqa: a batch of sequences runs attention as one CTA per kv head for all the query heads that share it.
constexpr int kPassAttnGqa = 16;
extern int g_batch_group;  // matvec_q6k.cu: sequences per CTA for small ungrouped matrices at batch > 1
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Kernel classes for the launch attribute (bits of g_pdl).
enum { PDL_MATVEC = 1, PDL_GROUPED = 2, PDL_ROUTER = 4, PDL_OTHER = 8, PDL_NORM = 16, PDL_ATTN = 32, PDL_SMALL = 64 };

template <typename... KArgs, typename... Args>
inline void launch_kc(int cls, const char *what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (g_pdl & cls) ? 1 : 0;
    g_launches++;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) set_error(e, what);
}
template <typename... KArgs, typename... Args>
inline void launch_k(const char *what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args... args) {
    launch_kc(PDL_OTHER, what, kernel, grid, block, smem, args...);
}

// What the next Q6_K matvec launch should ask L2 to fetch while it runs: the weights of the matvec that follows
// it in the pass. A decode pass alternates short weight-streaming kernels with kernels that are bound by one long
// chain of dependent adds and leave HBM idle; with the next weights already on their way, a matvec finds them in
// L2 instead of starting its stream cold. The plan is a hint: nothing waits on it and it changes no result.
struct PrefetchPlan {
    const uint8_t *base[3];
    unsigned long long bytes[3];  // multiples of 16; 0 = unused. With ids: bytes[0] is the size of ONE expert at base[0]
    const int32_t *ids;           // expert ids on the device (read after the launch's dependency wait), or null
    int n_ids, own_lo, own_hi;    // experts [own_lo, own_hi) are resident, stored from local index 0
};

// CTA `cta` of `n_cta` asks for its share of [base, base + bytes).
__device__ __forceinline__ void l2_prefetch_slice(const uint8_t *base, unsigned long long bytes, int cta, int n_cta) {
    unsigned long long slice = ((bytes / (unsigned long long)n_cta) + 15ull) & ~15ull;
    if (slice == 0) slice = 16;
    const unsigned long long off = slice * (unsigned long long)cta;
    if (off >= bytes) return;
    const unsigned long long n = bytes - off < slice ? bytes - off : slice;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + off), "r"((uint32_t)n) : "memory");
}
__device__ __forceinline__ void prefetch_issue(const PrefetchPlan &pf, int cta, int n_cta) {
    const int tid = threadIdx.x;
    if (!pf.ids) {
        if (tid < 3 && pf.bytes[tid]) l2_prefetch_slice(pf.base[tid], pf.bytes[tid], cta, n_cta);
    } else if (tid < pf.n_ids) {
        const int e = pf.ids[tid];
        if (e >= pf.own_lo && e < pf.own_hi) l2_prefetch_slice(pf.base[0] + (unsigned long long)(e - pf.own_lo) * pf.bytes[0], pf.bytes[0], cta, n_cta);
    }
}

// Work the next grouped gate+up matvec launch finishes itself instead of leaving it to a separate launch: the CTA
// that completes a slot last (a self-resetting arrival counter per slot) computes act = silu(gate) * up for the
// slot's rows and their Q8_K form, i.e. what llamd_fwd_silu_mul_quant would do one launch later.
struct TailPlan {
    unsigned int *counter;  // [n_slots] words, zero before the launch and zero again after it; null = no tail
    int8_t *qs;             // [n_slots][rows]
    float *d;               // [n_slots][rows / 256]
};

// Expert parallelism without the return collective. Each rank maps the other ranks' expert-output buffers (CUDA IPC,
// one process per GPU); the down projection of an owned expert then stores its rows straight into the HOME rank's
// buffer over NVLink and bumps that rank's arrival counter, and the home rank's next kernel (the combine fused into the
// following norm) waits for the expected number of arrivals instead of for an all-to-all.
// Two forms of arrival. Per CTA (the default): each CTA -- of an owned slot after its stores and a system-scope fence, of
// any other slot after it has read the request -- bumps its slot's home rank; the home waits for world x n_used x
// CTAs-per-slot arrivals (1600 at 8 ranks). Per rank (local_done given): every CTA counts itself on a local word and the
// CTA that completes the count fences and bumps every rank's counter once; the home waits for `world` arrivals. The
// second sends 200 x fewer remote atomics and was measured 0.8 % SLOWER at 4 GPUs (its one arrival leaves only after
// the rank's last CTA, where the per-CTA arrivals trickle in behind the rows). Either way a rank has read everything it
// needs of every request by the time a home rank has all its arrivals, so the home may replace its record.
struct PeerOutPlan {
    float *const *out_tab;            // device array [world]: each rank's [n_used][rows] output buffer
    unsigned int *const *arrive_tab;  // device array [world]: each rank's arrival counter
    int div;                          // slots per rank: slot s belongs to rank s / div, local slot s % div
    int world;                        // ranks to signal
    unsigned int *local_done;         // this rank's CTA count of the launch (zero between launches: it wraps); null: the
                                      // per-CTA form, every CTA arriving on its slot's home rank (model option ep_rank_arrive = 0)
};
// What the next norm launch must see before it reads the expert outputs: *counter >= target (then it resets the counter).
// The wait is bounded; when it runs out *status is set and the kernel goes on (the host reports the pass as failed).
// Once *status is set, later waits of the model return at once (the pass has failed; nothing is gained by
// running every later wait out as well) and the counters are left as they are: the model must be recreated.
struct WaitPlan {
    unsigned int *counter;
    unsigned int target;
    int *status;
    unsigned int limit;  // polls before giving up
};
// The request records (expert ids, Q8_K activation) of all ranks are pushed into this rank's buffers by the ranks
// themselves; a grouped launch that reads them first waits until *counter has reached *epoch x world (counter and
// epoch only grow; epoch is bumped by this rank's own push, which precedes the launch in the stream). Bounded.
struct DispatchWait {
    const unsigned int *counter;
    const unsigned int *epoch;
    unsigned int world;
    int *status;
    unsigned int limit;  // polls before giving up
};

// Bounded wait of ONE thread for *counter to reach `target` (wrap-safe when `monotone`, plain >= otherwise).
// Returns false, with *status = code, when `limit` polls have passed or an earlier wait of the model already failed.
__device__ __forceinline__ bool bounded_wait(const unsigned int *counter, unsigned int target, bool monotone, int *status, int code,
                                             unsigned int limit) {
    for (unsigned int it = 0; it < limit; it++) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
        if (monotone ? (int)(v - target) >= 0 : v >= target) return true;
        if (it == 0 && status) {  // not there yet: has an earlier wait of this model already failed? (off the common path)
            int st;
            asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(st) : "l"(status) : "memory");
            if (st != 0) return false;
        }
        if (it > 32) __nanosleep(128);
    }
    if (status) atomicExch(status, code);
    return false;
}

// The norm in front of a matvec, folded into it (one sequence, ungrouped): every CTA computes
//   x' = x (+ sum_e cw[e] * down[e], e ascending: the MoE combine that closes the previous layer),
//   xn = rms_norm(x') * w, and the Q8_K form of xn, which is the activation it multiplies;
// CTA 0 also writes x' to x_out (null: x is not changed, as for the first layer). The operations and their order are
// rms_norm_kernel's. x_out must not alias x or down: the other CTAs still read them.
struct NormPlan {
    const float *x;      // [k] null: no folded norm
    const float *down;   // [n_used][k] or null
    const float *cw;     // [n_used]
    int n_used;
    float *x_out;        // [k] or null
    const float *w;      // [k] norm weights
    float eps;
};
// The optional parts of ONE Q6_K matvec launch, passed by the caller with the launch (all empty by default).
struct MatvecPlans {
    PrefetchPlan pf;
    TailPlan tail;
    PeerOutPlan peer;
    DispatchWait dwait;
    NormPlan norm;
    // A grouped launch may read its expert ids before its dependency wait when they were complete before the launch in
    // front of it could begin. That holds for the down projection of a decode pass: the launch in front of it is the
    // gate+up launch or the SiLU launch behind that one, and a gate+up launch lets nothing start before it has itself
    // waited for the router. The weights then travel while the launch in front still runs. Never set for a launch whose
    // ids are written by the launch directly in front of it.
    int ids_early;
    // A grouped launch over many slots (a batch of sequences): a permutation of the slots, sorted by expert id, in which
    // the CTAs take them. Slots that name the same expert then run side by side and the second finds the expert's bytes in
    // L2 instead of reading them from HBM again. Produced by slot_order_launch; must be complete when the ids are.
    const int32_t *slot_order;
};
// order[] = the slots 0..n_slots-1 sorted by (ids[slot], slot). One small launch.
void slot_order_launch(const int32_t *ids, int n_slots, int32_t *order);

// The decode pass's attention (QK-norm, RoPE and the K/V store inside the scores launch) leaving its result quantized as well.
void attention_rope_quant(const float *q, const float *wq, const float *k, const float *wk, const float *v, void *kc, void *vc, float *out,
                          float *scores, int n_head, int n_head_kv, int hd, const int32_t *meta, const float *rope_tab, float eps, int max_kv,
                          int nseq, bool kv16, int8_t *qs, float *d, int flags);
void attention_meta_flags(const float *q, const void *kc, const void *vc, float *out, float *scores, int n_head, int n_head_kv, int hd,
                          const int32_t *meta, int max_kv, int nseq, bool kv16, int flags);
void norm_router_flags(const float *w, const float *x, const float *residual, float *x_out, const float *w_norm, float *xn_out, int8_t *qs,
                       float *d, int k, float eps, int n_expert, int n_used, float *logits, int32_t *ids, float *weights, float *probs,
                       unsigned int *counter, int nseq, int flags);
void rms_norm_quant_flags(const float *x, const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq, int flags);
void add_rms_norm_quant_flags(const float *x, const float *residual, float *sum_out, const float *w, float *out, int8_t *qs, float *d, int n,
                              float eps, int nseq, int flags);
// Internal launch functions behind the extern "C" entry points of the same names; the model passes its plans here.
void launch_matvec(int njobs, const void *const *w, float *const *out, const int *rows, int blocks, const int8_t *aq,
                   const float *ad, int nseq, const int32_t *ids, int n_slots, int n_expert, int act_div, int act_mode = 0,
                   const float *xf = nullptr, const float *xu = nullptr, int own_lo = 0, int own_hi = 0x7fffffff,
                   const MatvecPlans &plans = MatvecPlans{});
void launch_matvec_multi(int njobs, const void *const *w, float *const *out, const int *rows, int blocks, const int8_t *aq,
                         const float *ad, int n_tokens, const int32_t *work, const int32_t *n_work, int max_items, const int32_t *act_map,
                         const int32_t *out_map, int n_expert);
void matvec_batch(const MatvecPlans &pl, const void *w, const int8_t *aq, const float *ad, float *out, int blocks, int rows, int nseq);
void matvec_x3_batch(const MatvecPlans &pl, const void *w0, const void *w1, const void *w2, const int8_t *aq, const float *ad, float *o0,
                     float *o1, float *o2, int blocks, int rows0, int rows1, int rows2, int nseq);
void matvec_grouped_pa_silu(const MatvecPlans &pl, const void *w, const int32_t *ids, const float *gate, const float *up, float *out, int blocks,
                            int rows, int n_used, int nseq);
void matvec_x3_norm(const MatvecPlans &pl, const void *w0, const void *w1, const void *w2, float *o0, float *o1, float *o2, int blocks,
                    int rows0, int rows1, int rows2);
void matvec_grouped_x2_batch(const MatvecPlans &pl, const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                             float *oa, float *ob, int blocks, int rows, int n_used, int nseq);
void matvec_grouped_pa_batch(const MatvecPlans &pl, const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out,
                             int blocks, int rows, int n_used, int nseq);
void matvec_grouped_x2_owned(const MatvecPlans &pl, const void *wa, const void *wb, const int32_t *ids, const int8_t *aq, const float *ad,
                             float *oa, float *ob, int blocks, int rows, int n_used, int n_slots, int own_lo, int own_hi);
void matvec_grouped_pa_owned(const MatvecPlans &pl, const void *w, const int32_t *ids, const int8_t *aq, const float *ad, float *out,
                             int blocks, int rows, int n_slots, int own_lo, int own_hi);
void moe_group_owned(const int32_t *ids, int n_expert, int n_used, int nseq, int32_t *gstart, int32_t *gcount, int32_t *ptoken,
                     int32_t *pslot, int32_t *work, int32_t *n_work, int own_lo, int own_hi);
// The grouped expert GEMM with its output rows scattered over several GPUs: row block o goes to out_tab[o / out_div],
// local row block o % out_div (out_tab null: everything into oa / ob).
void expert_gemm_scatter(const void *wa, const void *wb, const int32_t *gstart, const int32_t *gcount, const int32_t *act_map,
                         const int32_t *pslot, const void *aq_rm, const float *ad, float *oa, float *ob, int blocks, int rows, int n_expert,
                         float *const *out_tab, int out_div, const void *fa = nullptr, const void *fb = nullptr);
// Pre-folded expert matrices (prefill): every (expert, 16-row tile) folded once into the integer MMA's operand order and
// kept (2 bytes per weight); fa / fb above name such copies of wa / wb.
size_t expert_fold_tile_bytes(int blocks);
size_t expert_fold_bytes(int blocks, int rows, int n_expert);
void expert_prefold(const void *w, void *dst, int blocks, int rows, int n_expert);
void gemm_tokens_folded(const void *folded, const void *aq_rm, const float *ad, float *out, int blocks, int rows, int ntok);
void gemm_tokens_folded3(const void *f0, const void *f1, const void *f2, const void *aq_rm, const float *ad, float *o0, float *o1, float *o2,
                         int blocks, int rows0, int rows1, int rows2, int ntok);
// expert parallelism, a prefill tile (ep.cu)
void ep_push_tile(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *const *ids_tab, float *const *ad_tab,
                  int8_t *const *aq_tab, unsigned int *const *disp_tab, unsigned int *epoch, unsigned int *push_done, int T, int cap,
                  int n_used, int blocks);
void ep_wait_requests(unsigned int *counter, const unsigned int *epoch, int *status, unsigned int limit);
void ep_wait_rows(unsigned int *counter, unsigned int target, int *status, unsigned int limit);
void ep_signal_rows(unsigned int *const *arrive_tab);
void combine_rms_norm_quant_wait(const WaitPlan &wait, const float *x, const float *down, const float *weights, int n_used, float *sum_out,
                                 const float *w, float *out, int8_t *qs, float *d, int n, float eps, int nseq, int flags);

// Grow-only device scratch for the host-facing entry points, the counterpart
// of g_aq/g_ad/g_out in crates/llamd-rocm/kernels/llamd.hip:1027-1051.
void *scratch(int slot, size_t bytes);

constexpr int kTileUnits = 32;
constexpr int kTileBytes = 6720;       // 32 blocks x 210 B
constexpr int kTileCodeBytes = 6144;   // 12 chunks x 32 lanes x 16 B
constexpr int kTileScaleOff = 6144;    // 32 x 16 B
constexpr int kTileDOff = 6656;        // 32 x 2 B

// IEEE binary16 -> binary32, exact (crates/llamd-quant/src/lib.rs:104-108).
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

// One value per thread summed over the CTA, the same on every thread and from run to run: xor-shuffle tree inside a warp,
// then the warps' sums added in warp order. The `fast` arithmetic's replacement for an ordered sum. s_scratch: 32 floats;
// all threads of the CTA must call it.
__device__ __forceinline__ float block_tree_sum(float v, float *s_scratch) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, off));
    const int nwarps = (blockDim.x + 31) >> 5;
    __syncthreads();  // (the scratch may still be read from an earlier call)
    if ((threadIdx.x & 31) == 0) s_scratch[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = s_scratch[0];
    for (int w = 1; w < nwarps; w++) t = __fadd_rn(t, s_scratch[w]);
    return t;
}

// Left-to-right f32 sum of n values in SHARED memory, starting from `acc`:
// acc = (...((acc + s[0]) + s[1]) + ...). The adds form one dependent chain, so the loop is software-pipelined to run
// at the latency of a dependent add (~4.3 cycles, measured): two register sets of 16 values alternate, and a set is
// re-loaded right after it has been added, so that its load latency hides behind the other set's 16 adds. The loads are
// written as ld.shared: through a pointer whose address space the compiler cannot see they become generic loads, whose
// longer latency no longer hides (6.3 cycles per add, measured inside the resident decode kernel). A function of its
// own, so that every caller gets this schedule. s must be 16-byte aligned.
__device__ __forceinline__ float4 chain_lds(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}
#define LLAMD_CHAIN_ADD16(q0, q1, q2, q3)                                                                              \
    acc = __fadd_rn(acc, q0.x); acc = __fadd_rn(acc, q0.y); acc = __fadd_rn(acc, q0.z); acc = __fadd_rn(acc, q0.w);     \
    acc = __fadd_rn(acc, q1.x); acc = __fadd_rn(acc, q1.y); acc = __fadd_rn(acc, q1.z); acc = __fadd_rn(acc, q1.w);     \
    acc = __fadd_rn(acc, q2.x); acc = __fadd_rn(acc, q2.y); acc = __fadd_rn(acc, q2.z); acc = __fadd_rn(acc, q2.w);     \
    acc = __fadd_rn(acc, q3.x); acc = __fadd_rn(acc, q3.y); acc = __fadd_rn(acc, q3.z); acc = __fadd_rn(acc, q3.w)
static __device__ __noinline__ float chain_sum(const float *s, int n, float acc) {
    const uint32_t p = (uint32_t)__cvta_generic_to_shared(s);
    const int nblk = n / 16;
    int i = 0;
    if (nblk >= 2) {
        float4 a0 = chain_lds(p), a1 = chain_lds(p + 16), a2 = chain_lds(p + 32), a3 = chain_lds(p + 48);
        float4 b0 = chain_lds(p + 64), b1 = chain_lds(p + 80), b2 = chain_lds(p + 96), b3 = chain_lds(p + 112);
        for (; i + 2 <= nblk; i += 2) {
            LLAMD_CHAIN_ADD16(a0, a1, a2, a3);
            const uint32_t ja = p + 64u * (uint32_t)min(i + 2, nblk - 1);  // (past the end: a harmless re-load of the last block)
            a0 = chain_lds(ja), a1 = chain_lds(ja + 16), a2 = chain_lds(ja + 32), a3 = chain_lds(ja + 48);
            LLAMD_CHAIN_ADD16(b0, b1, b2, b3);
            const uint32_t jb = p + 64u * (uint32_t)min(i + 3, nblk - 1);
            b0 = chain_lds(jb), b1 = chain_lds(jb + 16), b2 = chain_lds(jb + 32), b3 = chain_lds(jb + 48);
        }
        if (i < nblk) {  // an odd count: the last block is the one set `a` was re-loaded with
            LLAMD_CHAIN_ADD16(a0, a1, a2, a3);
            i++;
        }
    }
    for (int k = i * 16; k < n; k++) acc = __fadd_rn(acc, s[k]);
    return acc;
}
#undef LLAMD_CHAIN_ADD16

}  // namespace llamd
