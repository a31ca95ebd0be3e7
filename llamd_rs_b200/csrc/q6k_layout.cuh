// The device layout of Q6_K weights ("T32") and the bit-level helpers that
// read it.
//
// A Q6_K block is 256 six-bit codes q, sixteen int8 scales and an f16 d
// (crates/llamd-quant/src/lib.rs:171-180). The reference's dot product keeps
// eight integer accumulators per block, one per residue r = element mod 8
// (crates/llamd-quant/src/dot.rs:175-188), and each accumulator sums
// scale[g] * (a[16g+r]*w[16g+r] + a[16g+8+r]*w[16g+8+r]) over the sixteen
// groups g. The layout below stores a block residue by residue so that one
// thread produces those eight integers without a cross-lane reduction:
//
//   residue r, weight n = 4j+k (j = word 0..7, k = byte 0..3)
//       <-> element e = 16*(2j + (k>>1)) + 8*(k&1) + r
//   byte value  W4 = ((q ^ 0x20) << 2)   i.e. 4*(q-32) as a signed byte
//   four words W4_{4m..4m+3} are stored in three: S_i = (W4_{4m+i} & 0xFC..) |
//       two bits of W4_{4m+3} per byte (bits 7-6, 5-4, 3-2 for i = 0, 1, 2)
//
// so a block's codes take 8 residues x 6 words = 192 bytes, as in the file.
// 32 consecutive blocks form a 6720-byte tile: word-chunk c (16 B, c = 0..11)
// of block slot s sits at c*512 + s*16, which makes every 16-byte load of a
// warp one contiguous 512-byte run; then 32 x 16 scale bytes, then 32 x 2
// bytes of d.
#pragma once
#include "common.cuh"

namespace llamd {

// 6-bit code of element e in a block in the reference's byte layout
// (crates/llamd-quant/src/lib.rs:198-222).
__host__ __device__ __forceinline__ uint32_t ggml_q6k_code(const uint8_t *blk, int e) {
    const int half = e >> 7, w = e & 127, c = w >> 5, l = w & 31;
    const uint8_t lo = blk[64 * half + l + 32 * (c & 1)];
    const uint32_t nib = (c >= 2) ? (uint32_t)(lo >> 4) : (uint32_t)(lo & 0x0F);
    const uint32_t hi = ((uint32_t)blk[128 + 32 * half + l] >> (2 * c)) & 3u;
    return nib | (hi << 4);
}

// element index of (residue r, word j, byte k)
__host__ __device__ __forceinline__ int t32_element(int r, int j, int k) {
    return 16 * (2 * j + (k >> 1)) + 8 * (k & 1) + r;
}

// byte offset of code word wi (0..47) of block `unit` inside the tiled buffer
__host__ __device__ __forceinline__ size_t t32_word_offset(size_t unit, int wi) {
    const size_t tile = unit >> 5, slot = unit & 31;
    return tile * kTileBytes + (size_t)(wi >> 2) * 512 + slot * 16 + (size_t)(wi & 3) * 4;
}
__host__ __device__ __forceinline__ size_t t32_scale_offset(size_t unit) {
    return (unit >> 5) * kTileBytes + kTileScaleOff + (unit & 31) * 16;
}
__host__ __device__ __forceinline__ size_t t32_d_offset(size_t unit) {
    return (unit >> 5) * kTileBytes + kTileDOff + (unit & 31) * 2;
}

// q - 32 of element e of block `unit`, read back from the tiled buffer.
__device__ __forceinline__ int t32_weight(const uint8_t *tiled, size_t unit, int e) {
    const int r = e & 7, s = (e >> 3) & 1, g = e >> 4;
    const int j = g >> 1, k = ((g & 1) << 1) | s;
    const int m = j >> 2, i = j & 3;
    uint32_t c6;
    if (i < 3) {
        c6 = (uint32_t)tiled[t32_word_offset(unit, 6 * r + 3 * m + i) + k] >> 2;
    } else {
        const uint32_t b0 = tiled[t32_word_offset(unit, 6 * r + 3 * m + 0) + k] & 3u;
        const uint32_t b1 = tiled[t32_word_offset(unit, 6 * r + 3 * m + 1) + k] & 3u;
        const uint32_t b2 = tiled[t32_word_offset(unit, 6 * r + 3 * m + 2) + k] & 3u;
        c6 = (b0 << 4) | (b1 << 2) | b2;
    }
    return (int)(c6 ^ 0x20u) - 32;
}

// Unpack the four W4 words of quad m of residue r from the three stored words.
__device__ __forceinline__ void unpack_quad(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t w[4]) {
    w[0] = s0 & 0xFCFCFCFCu;
    w[1] = s1 & 0xFCFCFCFCu;
    w[2] = s2 & 0xFCFCFCFCu;
    const uint32_t u = ((s0 << 6) & 0xC0C0C0C0u) | ((s1 << 4) & 0x30303030u);
    w[3] = u | ((s2 << 2) & 0x0C0C0C0Cu);
}

// Q8_0 device layout: tiles of 32 rows x 1 block (1088 B): two 16-byte halves
// of each row's 32 quants, lane-interleaved, then the 32 f16 scales.
constexpr int kQ80TileBytes = 32 * 34;
__host__ __device__ __forceinline__ size_t q80_tile_offset(size_t row, size_t b, size_t blocks) {
    return ((row >> 5) * blocks + b) * kQ80TileBytes;
}

}  // namespace llamd
