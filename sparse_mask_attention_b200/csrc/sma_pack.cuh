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
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sma_common.cuh"

namespace sma {

constexpr int kPackThreads = 256;
constexpr int kPackUnroll = 1;       // independent 32-byte loads in flight per thread
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

// Flat path.  Requires: mask 32-byte aligned, total bytes = 32 * n_words.  Launched with one block per
// kPackThreads * kPackUnroll words (the grid stride only matters beyond the grid-size limit); kPackUnroll
// independent 32-byte loads in flight per thread.
__global__ void __launch_bounds__(kPackThreads, kPackBlocksPerSM)
pack_flat_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ packed, size_t n_words) {
    grid_launch_dependents();
    grid_dependency_wait();  // the mask may be the previous kernel's output
    const size_t block_words = static_cast<size_t>(kPackThreads) * kPackUnroll;
    const size_t stride = static_cast<size_t>(gridDim.x) * block_words;
    for (size_t base = static_cast<size_t>(blockIdx.x) * block_words + threadIdx.x; base < n_words; base += stride) {
        uint32_t r[kPackUnroll][8];
#pragma unroll
        for (int u = 0; u < kPackUnroll; ++u) {
            const size_t w = base + static_cast<size_t>(u) * kPackThreads;
            if (w < n_words) ld_stream_256(mask + 32 * w, r[u]);
        }
#pragma unroll
        for (int u = 0; u < kPackUnroll; ++u) {
            const size_t w = base + static_cast<size_t>(u) * kPackThreads;
            if (w < n_words) packed[w] = pack32(r[u]);
        }
    }
}

// Row path for any N and any alignment: one warp per mask row, grid-stride over rows.
__global__ void __launch_bounds__(kPackThreads)
pack_rows_kernel(const uint8_t* __restrict__ mask, uint32_t* __restrict__ packed, size_t n_rows, int N) {
    grid_launch_dependents();
    grid_dependency_wait();
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
