// Weight upload: the reference's 210-byte Q6_K blocks (and 34-byte Q8_0
// blocks) are permuted, bit for bit, into the tiled device layouts; plus the
// inverse and the dequantizers that prove nothing moved wrongly.
#include "q6k_layout.cuh"

namespace llamd {

// One CTA of 64 threads per block.
__global__ void repack_q6k_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t n_units, size_t dst_first) {
    const size_t src_unit = blockIdx.x + (size_t)blockIdx.y * gridDim.x;
    if (src_unit >= n_units) return;
    __shared__ uint8_t blk[LLAMD_Q6K_BLOCK_BYTES];
    for (int i = threadIdx.x; i < LLAMD_Q6K_BLOCK_BYTES; i += blockDim.x)
        blk[i] = src[src_unit * LLAMD_Q6K_BLOCK_BYTES + i];
    __syncthreads();
    const size_t unit = dst_first + src_unit;
    const int t = threadIdx.x;
    if (t < 48) {
        const int r = t / 6, m = (t % 6) / 3, i = t % 3;
        uint32_t word = 0;
        for (int k = 0; k < 4; k++) {
            const uint32_t w4 = ((ggml_q6k_code(blk, t32_element(r, 4 * m + i, k)) ^ 0x20u) << 2) & 0xFFu;
            const uint32_t w3 = ((ggml_q6k_code(blk, t32_element(r, 4 * m + 3, k)) ^ 0x20u) << 2) & 0xFFu;
            const uint32_t byte = (w4 & 0xFCu) | ((w3 >> (6 - 2 * i)) & 3u);
            word |= byte << (8 * k);
        }
        *reinterpret_cast<uint32_t *>(dst + t32_word_offset(unit, t)) = word;
    } else if (t < 52) {
        const int q = t - 48;
        uint32_t word = 0;
        for (int k = 0; k < 4; k++) word |= (uint32_t)blk[192 + 4 * q + k] << (8 * k);
        *reinterpret_cast<uint32_t *>(dst + t32_scale_offset(unit) + 4 * q) = word;
    } else if (t == 52) {
        *reinterpret_cast<uint16_t *>(dst + t32_d_offset(unit)) = (uint16_t)(blk[208] | (blk[209] << 8));
    }
}

// Inverse: tiled -> reference layout. One thread per block (a checking tool,
// not a hot path).
__global__ void unpack_q6k_kernel(const uint8_t *__restrict__ tiled, uint8_t *__restrict__ dst, size_t n_units) {
    const size_t unit = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (unit >= n_units) return;
    uint8_t *blk = dst + unit * LLAMD_Q6K_BLOCK_BYTES;
    for (int half = 0; half < 2; half++) {
        for (int l = 0; l < 32; l++) {
            const int o = half * 128;
            const uint32_t c0 = (uint32_t)(t32_weight(tiled, unit, o + l) + 32);
            const uint32_t c1 = (uint32_t)(t32_weight(tiled, unit, o + l + 32) + 32);
            const uint32_t c2 = (uint32_t)(t32_weight(tiled, unit, o + l + 64) + 32);
            const uint32_t c3 = (uint32_t)(t32_weight(tiled, unit, o + l + 96) + 32);
            blk[half * 64 + l] = (uint8_t)((c0 & 0xF) | ((c2 & 0xF) << 4));
            blk[half * 64 + l + 32] = (uint8_t)((c1 & 0xF) | ((c3 & 0xF) << 4));
            blk[128 + half * 32 + l] = (uint8_t)((c0 >> 4) | ((c1 >> 4) << 2) | ((c2 >> 4) << 4) | ((c3 >> 4) << 6));
        }
    }
    for (int i = 0; i < 16; i++) blk[192 + i] = tiled[t32_scale_offset(unit) + i];
    blk[208] = tiled[t32_d_offset(unit)];
    blk[209] = tiled[t32_d_offset(unit) + 1];
}

// d * sc * q with two f32 multiplies, left to right
// (crates/llamd-quant/src/lib.rs:219-222). One thread per element.
__global__ void dequantize_q6k_kernel(const uint8_t *__restrict__ tiled, size_t first_unit, size_t n_units,
                                      float *__restrict__ out) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= n_units * LLAMD_QK_K) return;
    const size_t unit = first_unit + idx / LLAMD_QK_K;
    const int e = (int)(idx % LLAMD_QK_K);
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(tiled + t32_d_offset(unit)));
    const float sc = (float)(int8_t)tiled[t32_scale_offset(unit) + (e >> 4)];
    const float q = (float)t32_weight(tiled, unit, e);
    out[idx] = __fmul_rn(__fmul_rn(d, sc), q);
}

// Embedding lookup: dequantize row `token` of the table
// (crates/llamd-runtime/src/layer.rs:205-209; the device form reads the token
// from a device-resident meta buffer, crates/llamd-rocm/src/forward.rs:594-599).
__global__ void embed_meta_kernel(const uint8_t *__restrict__ tiled, const int32_t *__restrict__ meta, int token_imm,
                                  float *__restrict__ out, int blocks) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.y;
    const int token = meta ? meta[2 * seq] : token_imm;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= blocks * LLAMD_QK_K) return;
    const size_t unit = (size_t)token * blocks + idx / LLAMD_QK_K;
    const int e = idx % LLAMD_QK_K;
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(tiled + t32_d_offset(unit)));
    const float sc = (float)(int8_t)tiled[t32_scale_offset(unit) + (e >> 4)];
    const float q = (float)t32_weight(tiled, unit, e);
    out[(size_t)seq * blocks * LLAMD_QK_K + idx] = __fmul_rn(__fmul_rn(d, sc), q);
}

// ---- Q8_0 ----------------------------------------------------------------
__global__ void repack_q8_0_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, size_t rows, size_t blocks) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;  // (row, b)
    if (idx >= rows * blocks) return;
    const size_t row = idx / blocks, b = idx % blocks;
    const uint8_t *s = src + idx * LLAMD_Q8_0_BLOCK_BYTES;
    uint8_t *t = dst + q80_tile_offset(row, b, blocks);
    const int lane = (int)(row & 31);
    for (int i = 0; i < 16; i++) {
        t[lane * 16 + i] = s[2 + i];
        t[512 + lane * 16 + i] = s[2 + 16 + i];
    }
    t[1024 + lane * 2] = s[0];
    t[1024 + lane * 2 + 1] = s[1];
}

// crates/llamd-quant/src/lib.rs:154-162
__global__ void dequantize_q8_0_kernel(const uint8_t *__restrict__ tiled, size_t rows, size_t blocks, float *__restrict__ out) {
    const size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (idx >= rows * blocks * 32) return;
    const size_t row = idx / (blocks * 32), b = (idx / 32) % blocks;
    const int j = (int)(idx % 32), lane = (int)(row & 31);
    const uint8_t *t = tiled + q80_tile_offset(row, b, blocks);
    const float d = f16_bits_to_f32(*reinterpret_cast<const uint16_t *>(t + 1024 + lane * 2));
    const int8_t q = (int8_t)t[(j >> 4) * 512 + lane * 16 + (j & 15)];
    out[idx] = __fmul_rn(d, (float)q);
}

// w [rows][k] -> wt [k][rows]
__global__ void transpose_f32_kernel(const float *__restrict__ w, float *__restrict__ wt, int rows, int k) {
    __shared__ float tile[32][33];
    const int x = blockIdx.x * 32 + threadIdx.x, y0 = blockIdx.y * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y)
        if (x < k && y0 + i < rows) tile[i][threadIdx.x] = w[(size_t)(y0 + i) * k + x];
    __syncthreads();
    const int ox = blockIdx.y * 32 + threadIdx.x, oy0 = blockIdx.x * 32;
    for (int i = threadIdx.y; i < 32; i += blockDim.y)
        if (ox < rows && oy0 + i < k) wt[(size_t)(oy0 + i) * rows + ox] = tile[threadIdx.x][i];
}

static dim3 grid_2d(size_t n) {
    const size_t gx = n < 65535 ? (n ? n : 1) : 65535;
    const size_t gy = (n + gx - 1) / gx;
    return dim3((unsigned)gx, (unsigned)(gy ? gy : 1));
}

}  // namespace llamd

using namespace llamd;

extern "C" {

size_t llamd_cuda_q6k_tiled_bytes(size_t n_blocks) {
    return ((n_blocks + kTileUnits - 1) / kTileUnits) * (size_t)kTileBytes;
}

void llamd_fwd_repack_q6k(const void *d_src, void *d_dst, size_t n_blocks) {
    if (n_blocks == 0) return;
    cudaError_t e = cudaMemsetAsync(d_dst, 0, llamd_cuda_q6k_tiled_bytes(n_blocks), stream());
    if (e != cudaSuccess) set_error(e, "repack memset");
    repack_q6k_kernel<<<grid_2d(n_blocks), 64, 0, stream()>>>((const uint8_t *)d_src, (uint8_t *)d_dst, n_blocks, 0);
    LLAMD_CHECK_LAUNCH("repack_q6k");
}

// Repack n_blocks source blocks into blocks [dst_first, dst_first+n) of a tiled
// buffer that was zeroed when it was allocated: lets a large tensor (all the
// experts of a layer) be uploaded piece by piece.
void llamd_fwd_repack_q6k_at(const void *d_src, void *d_dst, size_t n_blocks, size_t dst_first) {
    if (n_blocks == 0) return;
    repack_q6k_kernel<<<grid_2d(n_blocks), 64, 0, stream()>>>((const uint8_t *)d_src, (uint8_t *)d_dst, n_blocks, dst_first);
    LLAMD_CHECK_LAUNCH("repack_q6k_at");
}

void *llamd_cuda_upload_q6k(const void *host_blocks, size_t n_blocks) {
    void *raw = llamd_cuda_upload(host_blocks, n_blocks * LLAMD_Q6K_BLOCK_BYTES);
    if (!raw) return nullptr;
    void *dst = llamd_fwd_alloc(llamd_cuda_q6k_tiled_bytes(n_blocks));
    if (!dst) {
        cudaFree(raw);
        return nullptr;
    }
    llamd_fwd_repack_q6k(raw, dst, n_blocks);
    const int rc = llamd_fwd_sync();
    cudaFree(raw);
    if (rc != 0) {
        cudaFree(dst);
        return nullptr;
    }
    return dst;
}

void llamd_fwd_unpack_q6k(const void *d_tiled, void *d_dst, size_t n_blocks) {
    if (n_blocks == 0) return;
    unpack_q6k_kernel<<<(unsigned)((n_blocks + 127) / 128), 128, 0, stream()>>>((const uint8_t *)d_tiled, (uint8_t *)d_dst, n_blocks);
    LLAMD_CHECK_LAUNCH("unpack_q6k");
}

void llamd_fwd_dequantize_q6k(const void *d_tiled, size_t first_block, size_t n_blocks, float *d_out) {
    if (n_blocks == 0) return;
    const size_t n = n_blocks * LLAMD_QK_K;
    dequantize_q6k_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream()>>>((const uint8_t *)d_tiled, first_block, n_blocks, d_out);
    LLAMD_CHECK_LAUNCH("dequantize_q6k");
}

void llamd_fwd_embed(const void *table, int token, float *out, int blocks) {
    launch_k("embed", embed_meta_kernel, dim3((blocks * LLAMD_QK_K + 255) / 256, 1), dim3(256), 0, (const uint8_t *)table, nullptr, token, out,
             blocks);
}
void llamd_fwd_embed_meta(const void *table, const int32_t *meta, float *out, int blocks, int nseq) {
    // (the first launch of a pass: no programmatic overlap with whatever is in front of it, so that everything the pass
    // launches afterwards starts after the previous pass has completed)
    launch_kc(0, "embed_meta", embed_meta_kernel, dim3((blocks * LLAMD_QK_K + 255) / 256, nseq), dim3(256), 0, (const uint8_t *)table, meta, 0,
             out, blocks);
}

size_t llamd_cuda_q8_0_tiled_bytes(size_t rows, size_t blocks_per_row) {
    return ((rows + 31) / 32) * blocks_per_row * (size_t)kQ80TileBytes;
}
void llamd_fwd_repack_q8_0(const void *d_src, void *d_dst, size_t rows, size_t blocks_per_row) {
    const size_t n = rows * blocks_per_row;
    if (n == 0) return;
    cudaError_t e = cudaMemsetAsync(d_dst, 0, llamd_cuda_q8_0_tiled_bytes(rows, blocks_per_row), stream());
    if (e != cudaSuccess) set_error(e, "repack memset");
    repack_q8_0_kernel<<<(unsigned)((n + 127) / 128), 128, 0, stream()>>>((const uint8_t *)d_src, (uint8_t *)d_dst, rows, blocks_per_row);
    LLAMD_CHECK_LAUNCH("repack_q8_0");
}
void *llamd_cuda_upload_q8_0(const void *host_blocks, size_t rows, size_t blocks_per_row) {
    void *raw = llamd_cuda_upload(host_blocks, rows * blocks_per_row * LLAMD_Q8_0_BLOCK_BYTES);
    if (!raw) return nullptr;
    void *dst = llamd_fwd_alloc(llamd_cuda_q8_0_tiled_bytes(rows, blocks_per_row));
    if (!dst) {
        cudaFree(raw);
        return nullptr;
    }
    llamd_fwd_repack_q8_0(raw, dst, rows, blocks_per_row);
    const int rc = llamd_fwd_sync();
    cudaFree(raw);
    if (rc != 0) {
        cudaFree(dst);
        return nullptr;
    }
    return dst;
}
void llamd_fwd_dequantize_q8_0(const void *d_tiled, size_t rows, size_t blocks_per_row, float *d_out) {
    const size_t n = rows * blocks_per_row * 32;
    if (n == 0) return;
    dequantize_q8_0_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream()>>>((const uint8_t *)d_tiled, rows, blocks_per_row, d_out);
    LLAMD_CHECK_LAUNCH("dequantize_q8_0");
}

void llamd_fwd_transpose_f32(const float *w, float *wt, int rows, int k) {
    dim3 grid((k + 31) / 32, (rows + 31) / 32);
    transpose_f32_kernel<<<grid, dim3(32, 8), 0, stream()>>>(w, wt, rows, k);
    LLAMD_CHECK_LAUNCH("transpose_f32");
}

}  // extern "C"
