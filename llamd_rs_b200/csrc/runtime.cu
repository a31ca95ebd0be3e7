// Device discovery, raw memory, the library stream, the sticky error and the
// captured graph: the counterpart of the host side of
// crates/llamd-rocm/kernels/llamd_forward.hip:701-916 and
// crates/llamd-rocm/kernels/llamd.hip:1027-1100.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "common.cuh"
#include "quant.cuh"

namespace llamd {

unsigned long long g_launches = 0;
int g_pdl = 7;  // matvec, grouped matvec and router launches: measured best
static cudaStream_t g_stream = nullptr;
static int g_err = 0;
static std::string g_err_msg;
static cudaGraph_t g_graph = nullptr;
static cudaGraphExec_t g_graph_exec = nullptr;
static void *g_scratch[8] = {};
static size_t g_scratch_bytes[8] = {};

// ---- the exponential, made identical to the host libm's expf --------------------------------------------------
// (see quant.cuh: ref_expf). Every translation unit that evaluates exp registers a binder for its constants.
typedef void (*ExpBinder)(const uint32_t *, const uint32_t *, uint32_t, uint32_t);
static std::vector<ExpBinder> &exp_binders() {
    static std::vector<ExpBinder> v;
    return v;
}
void register_exp_binder(ExpBinder bind) { exp_binders().push_back(bind); }

static uint32_t *g_exp_keys_dev = nullptr, *g_exp_vals_dev = nullptr;
static long long g_exp_exceptions = -1;  // -1: no table (switched off, or it could not be built)
static uint32_t g_exp_window = 0;        // the look-up window in use (0: every input is looked up)

// out[i] = bits of (float)exp((double)x) for the float whose bits are first + i: the expression of ref_expf
__global__ void exp_scan_kernel(uint32_t first, uint32_t n, uint32_t *__restrict__ out) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x)
        out[i] = __float_as_uint(__double2float_rn(exp((double)__uint_as_float(first + i))));
}

// dist[i] = how far (in units of 2^-29 ulp) the double result for input bits in[i] lies from the midpoint of two
// floats; 0 for inputs whose float result is subnormal (those are always looked up)
__global__ void exp_window_kernel(const uint32_t *__restrict__ in, uint32_t n, uint32_t *__restrict__ dist) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float x = __uint_as_float(in[i]);
        const uint32_t frac = (uint32_t)__double_as_longlong(exp((double)x)) & 0x1FFFFFFFu;
        dist[i] = x < -87.0f ? 0u : (frac >= 0x10000000u ? frac - 0x10000000u : 0x10000000u - frac);
    }
}

// Inputs below 2^-25 in magnitude give exactly 1.0f on both sides; above 89 both overflow to +inf, below -104 both
// give 0. Everything in between is compared, float by float. LLAMD_EXP_TABLE=0 switches the table off.
static bool build_exp_table(cudaStream_t s) {
    const char *sw = getenv("LLAMD_EXP_TABLE");
    if (sw && !strcmp(sw, "0")) return true;
    const uint32_t ranges[2][2] = {{0x33000000u, 0x42B20000u}, {0xB3000000u, 0xC2D00001u}};
    constexpr uint32_t kChunk = 1u << 25;
    uint32_t *d_out = nullptr;
    if (cudaMalloc(&d_out, (size_t)kChunk * 4) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    std::vector<uint32_t> host(kChunk);
    const unsigned hw = std::thread::hardware_concurrency();
    const int n_threads = (int)(hw < 1 ? 1 : (hw > 64 ? 64 : hw));
    std::vector<std::vector<uint32_t>> found(n_threads);  // (input bits, host result bits) pairs
    bool ok = true;
    for (int r = 0; r < 2 && ok; r++) {
        for (uint64_t first = ranges[r][0]; first < ranges[r][1] && ok; first += kChunk) {
            const uint32_t n = (uint32_t)((ranges[r][1] - first) < kChunk ? (ranges[r][1] - first) : kChunk);
            exp_scan_kernel<<<148 * 8, 256, 0, s>>>((uint32_t)first, n, d_out);
            ok = cudaMemcpyAsync(host.data(), d_out, (size_t)n * 4, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                 cudaStreamSynchronize(s) == cudaSuccess;
            if (!ok) break;
            std::vector<std::thread> pool;
            for (int t = 0; t < n_threads; t++) {
                pool.emplace_back([&, t, first, n]() {
                    const uint32_t lo = (uint32_t)((uint64_t)n * t / n_threads), hi = (uint32_t)((uint64_t)n * (t + 1) / n_threads);
                    for (uint32_t i = lo; i < hi; i++) {
                        const uint32_t bits = (uint32_t)first + i;
                        float x, y;
                        memcpy(&x, &bits, 4);
                        y = expf(x);
                        uint32_t want;
                        memcpy(&want, &y, 4);
                        if (want != host[i]) {
                            found[t].push_back(bits);
                            found[t].push_back(want);
                        }
                    }
                });
            }
            for (auto &th : pool) th.join();
        }
    }
    cudaFree(d_out);
    if (!ok) {
        cudaGetLastError();
        return false;
    }
    size_t n_exc = 0;
    for (auto &v : found) n_exc += v.size() / 2;
    uint32_t slots = 1u << 16;
    while (slots < 4 * n_exc) slots <<= 1;  // at most a quarter full
    std::vector<uint32_t> keys(slots, 0), vals(slots, 0);
    for (auto &v : found)
        for (size_t i = 0; i < v.size(); i += 2) {
            uint32_t h = (v[i] * 2654435761u) >> 8 & (slots - 1);
            while (keys[h]) h = (h + 1) & (slots - 1);
            keys[h] = v[i];
            vals[h] = v[i + 1];
        }
    if (cudaMalloc(&g_exp_keys_dev, (size_t)slots * 4) != cudaSuccess || cudaMalloc(&g_exp_vals_dev, (size_t)slots * 4) != cudaSuccess ||
        cudaMemcpy(g_exp_keys_dev, keys.data(), (size_t)slots * 4, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaMemcpy(g_exp_vals_dev, vals.data(), (size_t)slots * 4, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    // Which inputs need the table at all? The host's expf can only differ from the correctly rounded value where the
    // exact result lies close to the midpoint of two floats. How close is measured here, on the device, over every
    // listed input: the window is the largest distance found plus one, so an input outside it is, by this exhaustive
    // construction, not in the table. (Should the window come out wider than a quarter ulp, it is not worth having.)
    uint32_t window = 0;
    if (n_exc) {
        std::vector<uint32_t> in;
        in.reserve(n_exc);
        for (auto &v : found)
            for (size_t i = 0; i < v.size(); i += 2) in.push_back(v[i]);
        uint32_t *d_in = nullptr, *d_ds = nullptr;
        std::vector<uint32_t> ds(n_exc, 0xFFFFFFFFu);
        if (cudaMalloc(&d_in, n_exc * 4) == cudaSuccess && cudaMalloc(&d_ds, n_exc * 4) == cudaSuccess &&
            cudaMemcpy(d_in, in.data(), n_exc * 4, cudaMemcpyHostToDevice) == cudaSuccess) {
            exp_window_kernel<<<148 * 4, 256, 0, s>>>(d_in, (uint32_t)n_exc, d_ds);
            if (cudaMemcpyAsync(ds.data(), d_ds, n_exc * 4, cudaMemcpyDeviceToHost, s) == cudaSuccess && cudaStreamSynchronize(s) == cudaSuccess) {
                uint32_t worst = 0;
                for (uint32_t d : ds) worst = d > worst ? d : worst;
                if (worst < (1u << 27)) window = worst + 1;
            }
        }
        if (d_in) cudaFree(d_in);
        if (d_ds) cudaFree(d_ds);
        cudaGetLastError();
    }
    g_exp_window = window;
    for (ExpBinder b : exp_binders()) b(g_exp_keys_dev, g_exp_vals_dev, slots - 1, window);
    if (cudaDeviceSynchronize() != cudaSuccess || cudaGetLastError() != cudaSuccess) return false;
    g_exp_exceptions = (long long)n_exc;
    return true;
}

cudaStream_t stream() {
    if (!g_stream) {
        cudaError_t e = cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            set_error(e, "cudaStreamCreate");
            g_stream = nullptr;
        } else if (!build_exp_table(g_stream)) {
            // without the table the exponential is correctly rounded, not the host libm's: refuse rather than drift
            set_error_msg("the table that makes exp identical to the host libm's expf could not be built");
            cudaStreamDestroy(g_stream);
            g_stream = nullptr;
        }
    }
    return g_stream;
}

void set_error(cudaError_t e, const char *what) {
    if (g_err == 0) {
        g_err = (int)e;
        g_err_msg = std::string(what) + ": " + cudaGetErrorString(e);
    }
}
void set_error_msg(const char *what) {
    if (g_err == 0) {
        g_err = -1;
        g_err_msg = what;
    }
}
int error_code() { return g_err; }

void *scratch(int slot, size_t bytes) {
    if (bytes <= g_scratch_bytes[slot] && g_scratch[slot]) return g_scratch[slot];
    if (g_scratch[slot]) {
        cudaStreamSynchronize(stream());
        cudaFree(g_scratch[slot]);
        g_scratch[slot] = nullptr;
        g_scratch_bytes[slot] = 0;
    }
    size_t want = bytes < 4096 ? 4096 : bytes;
    cudaError_t e = cudaMalloc(&g_scratch[slot], want);
    if (e != cudaSuccess) {
        set_error(e, "scratch cudaMalloc");
        return nullptr;
    }
    g_scratch_bytes[slot] = want;
    return g_scratch[slot];
}

}  // namespace llamd

using namespace llamd;

extern "C" {

// How many float inputs the device's exp needed correcting for to equal the host libm's expf (the size of the
// exception table built when the stream was made); -1 when the table is switched off.
long long llamd_cuda_exp_exceptions(void) { return stream() ? g_exp_exceptions : -1; }
// The look-up window in units of 2^-29 ulp: the table is consulted only for results at most this close to the midpoint
// of two floats (the largest distance measured over the listed inputs, plus one); 0 when every input is looked up.
int llamd_cuda_exp_window_on(void) { return stream() ? (int)g_exp_window : 0; }

int llamd_cuda_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int llamd_cuda_device_info(int dev, char *name, int name_len, char *arch, int arch_len,
                           size_t *total_mem, int *sm_count, int *warp_size) {
    cudaDeviceProp p;
    if (cudaGetDeviceProperties(&p, dev) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    if (name && name_len > 0) snprintf(name, (size_t)name_len, "%s", p.name);
    if (arch && arch_len > 0) snprintf(arch, (size_t)arch_len, "sm_%d%d", p.major, p.minor);
    if (total_mem) *total_mem = p.totalGlobalMem;
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (warp_size) *warp_size = p.warpSize;
    return 0;
}

// Select the device every later call of this process uses. Must come before
// the first allocation or launch (the stream is created on first use).
int llamd_cuda_set_device(int dev) {
    if (g_stream) {
        set_error_msg("set_device after the stream was created");
        return -1;
    }
    LLAMD_TRY(cudaSetDevice(dev), "cudaSetDevice");
    return 0;
}

size_t llamd_cuda_free_mem(void) {
    size_t f = 0, t = 0;
    if (cudaMemGetInfo(&f, &t) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return f;
}
size_t llamd_fwd_free_mem(void) { return llamd_cuda_free_mem(); }

const char *llamd_cuda_last_error_string(void) { return g_err_msg.c_str(); }

void *llamd_cuda_upload(const void *host, size_t bytes) {
    void *d = nullptr;
    if (cudaMalloc(&d, bytes ? bytes : 1) != cudaSuccess) {
        set_error(cudaGetLastError(), "upload cudaMalloc");
        return nullptr;
    }
    if (bytes && cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        set_error(cudaGetLastError(), "upload cudaMemcpy");
        cudaFree(d);
        return nullptr;
    }
    return d;
}
void llamd_cuda_release(void *dev) {
    if (dev) cudaFree(dev);
}

void *llamd_fwd_alloc(size_t bytes) {
    void *d = nullptr;
    if (cudaMalloc(&d, bytes ? bytes : 1) != cudaSuccess) {
        set_error(cudaGetLastError(), "alloc cudaMalloc");
        return nullptr;
    }
    return d;
}
void llamd_fwd_free(void *p) {
    if (p) cudaFree(p);
}
int llamd_fwd_upload(void *dst, const void *src, size_t bytes) {
    LLAMD_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, stream()), "upload");
    return 0;
}
int llamd_fwd_download(void *dst, const void *src, size_t bytes) {
    LLAMD_TRY(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, stream()), "download");
    LLAMD_TRY(cudaStreamSynchronize(stream()), "download sync");
    return 0;
}
int llamd_fwd_memset(void *p, int value, size_t bytes) {
    LLAMD_TRY(cudaMemsetAsync(p, value, bytes, stream()), "memset");
    return 0;
}
int llamd_fwd_sync(void) {
    cudaError_t e = cudaStreamSynchronize(stream());
    if (e != cudaSuccess) set_error(e, "sync");
    return g_err == 0 ? 0 : -1;
}
int llamd_fwd_last_error(void) {
    int e = g_err;
    g_err = 0;
    return e;
}
int llamd_fwd_stream_init(void) { return stream() ? 0 : -1; }
unsigned long long llamd_fwd_launch_count(void) { return g_launches; }
// Programmatic dependent launch on (default) or off, for A/B runs. A captured
// graph keeps the mode it was recorded in.
void llamd_fwd_set_pdl(int on) { g_pdl = on == 1 ? 7 : on; }
// Batched decode: sequences per CTA for the small ungrouped matrices (0: one CTA takes all sequences).
void llamd_fwd_set_batch_group(int g) { g_batch_group = g < 0 ? 0 : g; }
void *llamd_fwd_stream(void) { return (void *)stream(); }

// Device-time stopwatch on the library stream (CUDA events).
static cudaEvent_t g_t0 = nullptr, g_t1 = nullptr;
int llamd_fwd_timer_start(void) {
    if (!g_t0) {
        LLAMD_TRY(cudaEventCreate(&g_t0), "event create");
        LLAMD_TRY(cudaEventCreate(&g_t1), "event create");
    }
    LLAMD_TRY(cudaEventRecord(g_t0, stream()), "event record");
    return 0;
}
int llamd_fwd_timer_stop(float *ms_out) {
    if (!g_t0 || !ms_out) return -1;
    LLAMD_TRY(cudaEventRecord(g_t1, stream()), "event record");
    LLAMD_TRY(cudaEventSynchronize(g_t1), "event sync");
    LLAMD_TRY(cudaEventElapsedTime(ms_out, g_t0, g_t1), "event elapsed");
    return 0;
}

int llamd_fwd_begin_capture(void) {
    llamd_fwd_graph_destroy();
    LLAMD_TRY(cudaStreamBeginCapture(stream(), cudaStreamCaptureModeThreadLocal), "begin capture");
    return 0;
}
int llamd_fwd_end_capture(void) {
    cudaGraph_t g = nullptr;
    cudaError_t e = cudaStreamEndCapture(stream(), &g);
    if (e != cudaSuccess || !g) {
        set_error(e, "end capture");
        return -1;
    }
    g_graph = g;
    e = cudaGraphInstantiate(&g_graph_exec, g_graph, 0);
    if (e != cudaSuccess) {
        set_error(e, "graph instantiate");
        cudaGraphDestroy(g_graph);
        g_graph = nullptr;
        g_graph_exec = nullptr;
        return -1;
    }
    return 0;
}
int llamd_fwd_graph_launch(void) {
    if (!g_graph_exec) {
        set_error_msg("graph launch without a captured graph");
        return -1;
    }
    LLAMD_TRY(cudaGraphLaunch(g_graph_exec, stream()), "graph launch");
    return 0;
}
int llamd_fwd_has_graph(void) { return g_graph_exec ? 1 : 0; }
void llamd_fwd_graph_destroy(void) {
    if (g_graph_exec) cudaGraphExecDestroy(g_graph_exec);
    if (g_graph) cudaGraphDestroy(g_graph);
    g_graph_exec = nullptr;
    g_graph = nullptr;
}

}  // extern "C"
