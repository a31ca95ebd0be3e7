// Expert parallelism: experts sharded over the GPUs of one node, one process
// per GPU, NCCL over NVLink for the per-layer exchange. The reference has no
// distributed code at all; this file is new design.
//
// Every rank decodes its own sequence and holds every non-expert weight, plus
// experts [rank*E/N, (rank+1)*E/N). Per MoE layer:
//   dispatch  all-gather of (expert ids, Q8_K activation) -- 2.1 KB per rank --
//             so every rank sees the routed requests of all N tokens. The Q8_K
//             form is what every expert consumes, so sending it is exact;
//   compute   each rank runs the requested experts it owns;
//   combine   all-to-all of fixed [n_used][n_embd] f32 blocks: rank r returns to
//             rank t the rows it computed for t's token; the home rank then picks
//             each slot's row from the expert's owner and adds them in routing
//             order, as the single-GPU pass does.
// NCCL is loaded with dlopen when expert parallelism is first initialised, so a
// single-GPU process never needs the library.
//
// Second form, after llamd_model_ep_p2p_attach: the same two exchanges as plain
// stores into the other ranks' buffers over NVLink (mapped once through CUDA
// IPC) with arrival counters: ep_push_kernel here for the dispatch, the
// down-projection matvec's own epilogue for the return (matvec_q6k.cu), and
// bounded waits in the consumers (the gate/up matvec, the combining norm).
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <atomic>
#include <chrono>
#include <memory>
#include <thread>

#include "common.cuh"

namespace llamd {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};
static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_ep_rank = 0, g_ep_world = 1;
// How long the host waits for the other ranks (communicator set-up, and each pass that has collectives in it) before it
// aborts the communicator and reports the failure. A rank that never joins, or leaves, then costs its peers this
// long and an error, not a hang.
static int g_ep_timeout_ms = 60000;

static bool nccl_load() {
    if (g_nccl.handle) return true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        set_error_msg("expert parallelism: libnccl.so.2 could not be loaded");
        return false;
    }
#define LOAD(field, name)                                                      \
    g_nccl.field = reinterpret_cast<decltype(g_nccl.field)>(dlsym(h, name));   \
    if (!g_nccl.field) {                                                       \
        set_error_msg("expert parallelism: libnccl lacks " name);              \
        return false;                                                          \
    }
    LOAD(GetUniqueId, "ncclGetUniqueId")
    LOAD(CommInitRank, "ncclCommInitRank")
    LOAD(CommGetAsyncError, "ncclCommGetAsyncError")
    LOAD(CommAbort, "ncclCommAbort")
    LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(AllGather, "ncclAllGather")
    LOAD(Send, "ncclSend")
    LOAD(Recv, "ncclRecv")
    LOAD(GroupStart, "ncclGroupStart")
    LOAD(GroupEnd, "ncclGroupEnd")
    LOAD(GetErrorString, "ncclGetErrorString")
#undef LOAD
    g_nccl.handle = h;
    return true;
}

static bool nccl_ok(ncclResult_t r, const char *what) {
    if (r == ncclSuccess) return true;
    char msg[256];
    snprintf(msg, sizeof msg, "%s: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "nccl error");
    set_error_msg(msg);
    return false;
}

// Give up on the communicator: ncclCommAbort ends its kernels in flight and frees it. The model that used it is dead.
static void comm_abort(const char *why) {
    if (g_comm && g_nccl.CommAbort) g_nccl.CommAbort(g_comm);
    g_comm = nullptr;
    set_error_msg(why);
}

// The host side of a pass with collectives in it: wait for the stream, but not for ever. 0 ok, -1 failed (message set;
// on a time-out, or an asynchronous NCCL error, the communicator has been aborted so that its kernels leave the GPU).
int ep_bounded_sync() {
    if (!g_comm) return llamd_fwd_sync();
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        const cudaError_t q = cudaStreamQuery(stream());
        if (q == cudaSuccess) return llamd_fwd_sync();
        if (q != cudaErrorNotReady) {
            set_error(q, "expert-parallel pass");
            return -1;
        }
        ncclResult_t st = ncclSuccess;
        if (g_nccl.CommGetAsyncError(g_comm, &st) == ncclSuccess && st != ncclSuccess && st != ncclInProgress) {
            comm_abort("expert parallelism: NCCL reported an asynchronous error during the pass; communicator aborted");
            cudaStreamSynchronize(stream());
            return -1;
        }
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > g_ep_timeout_ms) {
            comm_abort("expert parallelism: a pass with collectives did not complete in time (a rank left?); communicator aborted");
            cudaStreamSynchronize(stream());  // the aborted kernels drain
            return -1;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

int ep_rank() { return g_ep_rank; }
int ep_world() { return g_ep_world; }

// Home rank: slot s of my token was computed by the rank that owns expert ids[s];
// its row sits in that rank's block of the receive buffer.
__global__ void ep_pick_kernel(const float *__restrict__ recv, const int32_t *__restrict__ ids, float *__restrict__ down, int n_used, int n_embd,
                               int experts_per_rank) {
    pdl_trigger();
    pdl_wait();
    const int s = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_embd) return;
    const int owner = ids[s] / experts_per_rank;
    down[(size_t)s * n_embd + i] = recv[((size_t)owner * n_used + s) * n_embd + i];
}

// The dispatch without a collective: CTA `dst` of `world` copies this rank's request record (expert ids, activation
// scales, activation quants) into slot `rank` of rank dst's gathered buffers (its own included) over NVLink, then
// counts itself on dst's dispatch counter. CTA 0 also advances this rank's epoch, which the launches that follow
// in the stream multiply by `world` to know how many arrivals to expect.
__global__ void ep_push_kernel(const int32_t *__restrict__ ids, const float *__restrict__ ad, const int8_t *__restrict__ aq,
                               int32_t *const *__restrict__ ids_tab, float *const *__restrict__ ad_tab, int8_t *const *__restrict__ aq_tab,
                               unsigned int *const *__restrict__ disp_tab, unsigned int *__restrict__ epoch, int rank, int n_used, int blocks) {
    pdl_trigger();
    pdl_wait();
    const int dst = blockIdx.x, tid = threadIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(aq);
    uint4 *q = reinterpret_cast<uint4 *>(aq_tab[dst] + (size_t)rank * blocks * 256);
    for (int i = tid; i < blocks * 16; i += blockDim.x) q[i] = src[i];
    if (tid < blocks) ad_tab[dst][(size_t)rank * blocks + tid] = ad[tid];
    if (tid < n_used) ids_tab[dst][(size_t)rank * n_used + tid] = ids[tid];
    __threadfence_system();  // the record is visible on dst before the arrival is
    __syncthreads();
    if (tid == 0) {
        atomicAdd_system(disp_tab[dst], 1u);
        if (dst == 0) *epoch = *epoch + 1;
    }
}

// ---- a prefill tile's exchange over peer memory --------------------------------------------------------------
// Dispatch: every rank copies the Q8_K activations, block scales and routed expert ids of its T tokens into slot
// `rank` of EVERY rank's gathered buffers ([world][cap] token rows; ids beyond T are -1), an all-gather by peer
// stores. blockIdx.y = destination rank, blockIdx.x strides over the rows. The last CTA to finish a destination (a
// local arrival counter that wraps to zero) bumps that rank's dispatch counter: its own fence orders it after the
// stores of the CTAs it saw arrive. The last CTA of destination 0 also advances this rank's epoch.
__global__ void __launch_bounds__(256) ep_push_tile_kernel(const int32_t *__restrict__ ids, const float *__restrict__ ad,
                                                          const int8_t *__restrict__ aq, int32_t *const *__restrict__ ids_tab,
                                                          float *const *__restrict__ ad_tab, int8_t *const *__restrict__ aq_tab,
                                                          unsigned int *const *__restrict__ disp_tab, unsigned int *__restrict__ epoch,
                                                          unsigned int *__restrict__ push_done, int rank, int T, int cap, int n_used,
                                                          int blocks) {
    pdl_trigger();
    pdl_wait();
    const int dst = blockIdx.y, tid = threadIdx.x;
    const size_t row16 = (size_t)blocks * 16;  // uint4 per token row of quants
    const uint4 *src = reinterpret_cast<const uint4 *>(aq);
    uint4 *q = reinterpret_cast<uint4 *>(aq_tab[dst] + (size_t)rank * cap * blocks * 256);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < (size_t)T * row16; i += (size_t)gridDim.x * blockDim.x) q[i] = src[i];
    float *d = ad_tab[dst] + (size_t)rank * cap * blocks;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < (size_t)T * blocks; i += (size_t)gridDim.x * blockDim.x) d[i] = ad[i];
    int32_t *e = ids_tab[dst] + (size_t)rank * cap * n_used;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + tid; i < (size_t)cap * n_used; i += (size_t)gridDim.x * blockDim.x)
        e[i] = i < (size_t)T * n_used ? ids[i] : -1;
    __threadfence_system();  // this CTA's part of the record is visible on dst before its arrival is
    __syncthreads();
    if (tid == 0) {
        const bool last = atomicInc(push_done + dst, gridDim.x - 1) == gridDim.x - 1;  // wraps to 0
        if (last) {
            __threadfence_system();
            atomicAdd_system(disp_tab[dst], 1u);
            if (dst == 0) *epoch = *epoch + 1;
        }
    }
}

// One thread waits (bounded) for a counter other GPUs bump: the requests of all ranks (epoch given: target =
// *epoch x world, the counter only grows) or the arrivals of all ranks' expert rows (target given; the counter is
// cleared once seen). The kernels that follow in the stream read what the peers stored.
__global__ void ep_wait_kernel(unsigned int *counter, const unsigned int *epoch, unsigned int world_or_target, int *status, int code,
                               unsigned int limit) {
    pdl_trigger();
    pdl_wait();
    if (threadIdx.x != 0) return;
    if (epoch) {
        bounded_wait(counter, *epoch * world_or_target, true, status, code, limit);
    } else if (bounded_wait(counter, world_or_target, false, status, code, limit)) {
        *counter = 0;
        __threadfence();
    }
}

// After a kernel whose stores went to other GPUs: tell every rank that this rank's rows have been written. The
// stores belong to an earlier kernel of the stream, hence are ordered before this one; the system-scope fence
// orders them before the arrival for the GPU that observes it.
__global__ void ep_signal_kernel(unsigned int *const *__restrict__ arrive_tab, int world) {
    pdl_trigger();
    pdl_wait();
    if ((int)threadIdx.x < world) {
        __threadfence_system();
        atomicAdd_system(arrive_tab[threadIdx.x], 1u);
    }
}

void ep_push_tile(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *const *ids_tab, float *const *ad_tab,
                  int8_t *const *aq_tab, unsigned int *const *disp_tab, unsigned int *epoch, unsigned int *push_done, int T, int cap,
                  int n_used, int blocks) {
    if (g_ep_world < 2 || T < 1 || T > cap) {
        set_error_msg("ep_push_tile: needs an expert-parallel world and 1..cap tokens");
        return;
    }
    const int ctas = (int)(((size_t)T * blocks * 16 + 255) / 256) < 64 ? (int)(((size_t)T * blocks * 16 + 255) / 256) : 64;
    launch_k("ep_push_tile", ep_push_tile_kernel, dim3(ctas < 1 ? 1 : ctas, g_ep_world), dim3(256), 0, ids, ad, aq, ids_tab, ad_tab, aq_tab,
             disp_tab, epoch, push_done, g_ep_rank, T, cap, n_used, blocks);
}
void ep_wait_requests(unsigned int *counter, const unsigned int *epoch, int *status, unsigned int limit) {
    launch_k("ep_wait_requests", ep_wait_kernel, dim3(1), dim3(32), 0, counter, epoch, (unsigned)g_ep_world, status, 2, limit);
}
void ep_wait_rows(unsigned int *counter, unsigned int target, int *status, unsigned int limit) {
    launch_k("ep_wait_rows", ep_wait_kernel, dim3(1), dim3(32), 0, counter, (const unsigned int *)nullptr, target, status, 1, limit);
}
void ep_signal_rows(unsigned int *const *arrive_tab) {
    launch_k("ep_signal_rows", ep_signal_kernel, dim3(1), dim3(32), 0, arrive_tab, g_ep_world);
}

}  // namespace llamd

using namespace llamd;

extern "C" {

// 128 bytes the ranks must share before llamd_cuda_ep_init (rank 0 makes them).
int llamd_cuda_ep_unique_id(void *out128) {
    if (!out128 || !nccl_load()) return -1;
    ncclUniqueId id;
    if (!nccl_ok(g_nccl.GetUniqueId(&id), "ncclGetUniqueId")) return -1;
    memcpy(out128, &id, sizeof id);
    return 0;
}

// Join the communicator: one process per GPU, the device already selected.
int llamd_cuda_ep_init(int rank, int world, const void *id128) {
    if (world < 1 || rank < 0 || rank >= world || !id128) return -1;
    if (!nccl_load() || !stream()) return -1;
    if (g_comm) {
        g_nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    // A rank that never joins must not hang this one: the (blocking) set-up runs on a helper thread and this thread
    // waits for it with a limit. The communicator stays a blocking one, which is what graph capture of its collectives
    // was verified with. A set-up that timed out is left to its thread; the process should not retry but report.
    struct Init {
        std::atomic<int> done{0};
        ncclComm_t comm = nullptr;
        ncclResult_t rc = ncclSuccess;
    };
    auto st = std::make_shared<Init>();
    int dev = 0;
    cudaGetDevice(&dev);
    std::thread([st, world, id, rank, dev]() {
        cudaSetDevice(dev);
        st->rc = g_nccl.CommInitRank(&st->comm, world, id, rank);
        st->done.store(1, std::memory_order_release);
    }).detach();
    const auto t0 = std::chrono::steady_clock::now();
    while (!st->done.load(std::memory_order_acquire)) {
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > g_ep_timeout_ms) {
            char msg[200];
            snprintf(msg, sizeof msg, "expert parallelism: the communicator was not set up within %d ms (a rank never joined?)", g_ep_timeout_ms);
            set_error_msg(msg);
            return -1;
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    if (!nccl_ok(st->rc, "ncclCommInitRank")) return -1;
    g_comm = st->comm;
    g_ep_rank = rank;
    g_ep_world = world;
    return 0;
}

// Expert parallelism over peer memory only: no communicator is made, so the two NCCL exchanges cannot be used and
// llamd_model_ep_p2p_attach (or _attach_ptrs) must follow model creation. For ranks that share peer pointers some
// other way than through NCCL's bootstrap (and for tests of the bounded waits).
int llamd_cuda_ep_init_local(int rank, int world) {
    if (world < 1 || rank < 0 || rank >= world || !stream()) return -1;
    g_ep_rank = rank;
    g_ep_world = world;
    return 0;
}

// Milliseconds the host waits for other ranks before it aborts the communicator (default 60000).
void llamd_cuda_ep_set_timeout_ms(int ms) { g_ep_timeout_ms = ms < 1 ? 1 : ms; }

// Push this rank's request record to every rank (see ep_push_kernel). The tables are device arrays [world] of the
// ranks' gathered buffers and dispatch counters.
void llamd_fwd_ep_push(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *const *ids_tab, float *const *ad_tab,
                       int8_t *const *aq_tab, unsigned int *const *disp_tab, unsigned int *epoch, int n_used, int blocks) {
    if (g_ep_world < 2 || n_used > 256 || blocks > 256) {
        set_error_msg("ep_push: needs an expert-parallel world, at most 256 experts per token and 256 blocks");
        return;
    }
    launch_k("ep_push", ep_push_kernel, dim3(g_ep_world), dim3(256), 0, ids, ad, aq, ids_tab, ad_tab, aq_tab, disp_tab, epoch, g_ep_rank, n_used,
             blocks);
}

// One rank's handle for a buffer it allocated (64 bytes), and the mapping of a peer's handle into this process.
// Used for the peer-written expert outputs: ranks are separate processes on one node.
int llamd_cuda_ep_ipc_export(const void *dev, void *handle64) {
    if (!dev || !handle64) return -1;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, const_cast<void *>(dev)) != cudaSuccess) {
        set_error(cudaGetLastError(), "cudaIpcGetMemHandle");
        return -1;
    }
    static_assert(sizeof(h) == 64, "ipc handle size");
    memcpy(handle64, &h, 64);
    return 0;
}
void *llamd_cuda_ep_ipc_open(const void *handle64) {
    if (!handle64) return nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *p = nullptr;
    if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        set_error(cudaGetLastError(), "cudaIpcOpenMemHandle");
        return nullptr;
    }
    return p;
}
void llamd_cuda_ep_ipc_close(void *mapped) {
    if (mapped) cudaIpcCloseMemHandle(mapped);
}

void llamd_cuda_ep_finalize(void) {
    if (g_comm && g_nccl.CommDestroy) {
        cudaStreamSynchronize(stream());
        g_nccl.CommDestroy(g_comm);
    }
    g_comm = nullptr;
    g_ep_rank = 0;
    g_ep_world = 1;
}

// dispatch: three all-gathers in one NCCL group (ids, activation scales, activation quants)
void llamd_fwd_ep_dispatch(const int32_t *ids, const float *ad, const int8_t *aq, int32_t *ids_all, float *ad_all, int8_t *aq_all,
                           int n_used, int blocks) {
    if (!g_comm) {
        set_error_msg("ep_dispatch before llamd_cuda_ep_init");
        return;
    }
    bool ok = nccl_ok(g_nccl.GroupStart(), "ncclGroupStart");
    ok = ok && nccl_ok(g_nccl.AllGather(ids, ids_all, (size_t)n_used, ncclInt32, g_comm, stream()), "ncclAllGather ids");
    ok = ok && nccl_ok(g_nccl.AllGather(ad, ad_all, (size_t)blocks, ncclFloat, g_comm, stream()), "ncclAllGather ad");
    ok = ok && nccl_ok(g_nccl.AllGather(aq, aq_all, (size_t)blocks * 256, ncclInt8, g_comm, stream()), "ncclAllGather aq");
    nccl_ok(g_nccl.GroupEnd(), "ncclGroupEnd");
    (void)ok;
}

// combine: block t of `send` ([world][n_used][n_embd]) goes to rank t; block r of `recv` comes from rank r;
// then the home rank picks each slot's row from the owner of its expert into down [n_used][n_embd].
void llamd_fwd_ep_combine(const float *send, float *recv, const int32_t *ids, float *down, int n_used, int n_embd, int n_expert) {
    if (!g_comm) {
        set_error_msg("ep_combine before llamd_cuda_ep_init");
        return;
    }
    const size_t blk = (size_t)n_used * n_embd;
    bool ok = nccl_ok(g_nccl.GroupStart(), "ncclGroupStart");
    for (int peer = 0; ok && peer < g_ep_world; peer++) {
        ok = ok && nccl_ok(g_nccl.Send(send + peer * blk, blk, ncclFloat, peer, g_comm, stream()), "ncclSend");
        ok = ok && nccl_ok(g_nccl.Recv(recv + peer * blk, blk, ncclFloat, peer, g_comm, stream()), "ncclRecv");
    }
    nccl_ok(g_nccl.GroupEnd(), "ncclGroupEnd");
    if (!g_comm) return;
    launch_k("ep_pick", ep_pick_kernel, dim3((n_embd + 255) / 256, n_used), dim3(256), 0, (const float *)recv, ids, down, n_used, n_embd,
             n_expert / g_ep_world);
}

int llamd_cuda_ep_rank(void) { return g_ep_rank; }
int llamd_cuda_ep_world(void) { return g_ep_world; }

}  // extern "C"
