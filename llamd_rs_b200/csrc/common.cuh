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

}  // namespace llamd
