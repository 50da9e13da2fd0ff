// Mask bit-packing for sm_100a: bool bytes [rows, N] -> uint32 words [rows, ceil(N/32)],
// bit j of word w = (byte 32*w + j != 0), bits past column N are zero.
// Bit layout of the reference kernel pack_mask_kernel (csrc/sparse_attention.cu:549-568) and of its
// reader read_mask_bit (csrc/utils.cuh:47-56).
//
// The pass is pure streaming (1 byte read and 1/8 byte written per mask element), so it is built for
// HBM bandwidth: when N is a multiple of 32 the packed array is a flat function of the flat byte
// array and every thread turns one 32-byte vector load (ld.global.v8.b32, sm_100) into one output
// word; a warp reads 1 KB and writes 128 B per step, both fully coalesced.  Other N take the row
// path: one warp per mask row, one byte per lane, a warp ballot per output word.
// On request the flat path also writes an occupancy side-band for the attention kernel (one bit per mask
// row and 64-key tile), which no kernel of the reference has.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sma_common.cuh"

namespace sma {

constexpr int kPackThreads = 256;
// independent 32-byte loads in flight per thread: one without the occupancy side-band (more were slower), two with
// it, so that a warp's side-band store is a whole 32-bit word (a 16-bit store per 32 packed words cost 12 % of the
// kernel's time, the 32-bit store per 64 costs 8 %)
__host__ __device__ constexpr int pack_unroll(bool tiles) { return tiles ? 2 : 1; }
constexpr int kPackBlocksPerSM = 8;

// Four mask bytes -> four bits (bit i = byte i != 0).
__device__ __forceinline__ uint32_t bytes_to_nibble(uint32_t x) {
    // per byte: bit 7 of (x | ((x & 0x7f) + 0x7f)) is set iff the byte is non-zero
    const uint32_t nz = ((x | ((x & 0x7F7F7F7Fu) + 0x7F7F7F7Fu)) >> 7) & 0x01010101u;
    // gather bits 0, 8, 16, 24 into bits 24..27 of the product
    return (nz * 0x01020408u) >> 24;
}

__device__ __forceinline__ uint32_t pack32(const uint32_t (&r)[8]) {
    uint32_t word = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) word |= bytes_to_nibble(r[i]) << (4 * i);
    return word;
}

__device__ __forceinline__ void ld_stream_256(const uint8_t* p, uint32_t (&r)[8]) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "l"(p));
}

// Even bits of x (bits 0, 2, 4, ...) gathered into the low 16 bits.
__device__ __forceinline__ uint32_t even_bits(uint32_t x) {
    x &= 0x55555555u;
    x = (x | (x >> 1)) & 0x33333333u;
    x = (x | (x >> 2)) & 0x0F0F0F0Fu;
    x = (x | (x >> 4)) & 0x00FF00FFu;
    return (x | (x >> 8)) & 0xFFFFu;
}

// Flat path.  Requires: mask 32-byte aligned, total bytes = 32 * n_words.  Launched with one block per
// kPackThreads * pack_unroll words (the grid stride only matters beyond the grid-size limit); a warp takes
// 32 * pack_unroll consecutive words.
//
// kTiles: the kernel also says where the mask keeps anything, for the attention kernel, which skips 64-key
// tiles without a kept key and otherwise has to find them by reading the packed words again.  Per 32 consecutive
// packed words there is one 16-bit word tile_bits[w / 32] whose bit b says that packed words 2b and 2b+1 of those 32
// (64 keys of one mask row when N is a multiple of 64) hold a set bit.  Needs n_words to be a multiple of 64, which
// holds for every N that is a multiple of 64, and tile_bits 4-byte aligned.
template <bool kTiles>
__global__ void __launch_bounds__(kPackThreads, kPackBlocksPerSM)
pack_flat_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ packed, uint16_t* __restrict__ tile_bits,
                 size_t n_words, uint32_t* __restrict__ work_counter) {
    grid_launch_dependents();
    grid_dependency_wait();  // the mask may be the previous kernel's output
    // the attention kernel that follows in the stream starts its work queue at zero (it reads the word only after
    // this grid has completed; the wait above keeps the write behind an earlier kernel that may still use the word)
    if (work_counter != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *work_counter = 0u;
    constexpr int kUnroll = pack_unroll(kTiles);
    const size_t block_words = static_cast<size_t>(kPackThreads) * kUnroll;
    const size_t stride = static_cast<size_t>(gridDim.x) * block_words;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (size_t base = static_cast<size_t>(blockIdx.x) * block_words + warp * (32 * kUnroll) + lane; base < n_words;
         base += stride) {
        uint32_t r[kUnroll][8];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t w = base + 32 * u;
            if (w < n_words) ld_stream_256(mask + 32 * w, r[u]);
        }
        uint32_t bits = 0;
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const size_t w = base + 32 * u;
            if (w < n_words) {
                const uint32_t word = pack32(r[u]);
                packed[w] = word;
                if constexpr (kTiles) {
                    // w - lane is a multiple of 32 and n_words is one too: the whole warp is here
                    const uint32_t nz = __ballot_sync(0xFFFFFFFFu, word != 0u);
                    bits |= even_bits(nz | (nz >> 1)) << (16 * u);
                }
            }
        }
        if constexpr (kTiles) {
            // base - lane is a multiple of 64 and so is n_words: both halves of the 32-bit word are this warp's
            if (lane == 0) *reinterpret_cast<uint32_t*>(tile_bits + (base >> 5)) = bits;
        }
    }
}

// Row path for any N and any alignment: one warp per mask row, grid-stride over rows.
__global__ void __launch_bounds__(kPackThreads)
pack_rows_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ packed, size_t n_rows, int N,
                 uint32_t* __restrict__ work_counter) {
    grid_launch_dependents();
    grid_dependency_wait();
    if (work_counter != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *work_counter = 0u;
    const int lane = threadIdx.x & 31;
    const int nw = (N + 31) >> 5;
    const size_t warps_total = static_cast<size_t>(gridDim.x) * (kPackThreads / 32);
    for (size_t row = static_cast<size_t>(blockIdx.x) * (kPackThreads / 32) + (threadIdx.x >> 5); row < n_rows;
         row += warps_total) {
        const uint8_t* src = mask + row * static_cast<size_t>(N);
        uint32_t* dst = packed + row * static_cast<size_t>(nw);
        uint32_t mine = 0;  // lane l keeps word (w with w % 32 == l) until the group of 32 words is stored
        for (int w = 0; w < nw; ++w) {
            const int col = 32 * w + lane;
            const uint32_t byte = col < N ? src[col] : 0u;
            const uint32_t word = __ballot_sync(0xFFFFFFFFu, byte != 0);
            if ((w & 31) == lane) mine = word;
            if ((w & 31) == 31 || w == nw - 1) {
                const int w_out = (w & ~31) + lane;
                if (w_out <= w) dst[w_out] = mine;
            }
        }
    }
}

}  // namespace sma
