// Tile lists ahead of the attention kernel ("plan").
//
// The attention kernel visits, per work item (128 query rows of one batch*head), only the 64-key tiles in which
// some row keeps a key.  Its loader warps can find those tiles themselves, one item ahead, by reading the item's
// packed-mask rows; for long sequences that is 128 rows x N/8 bytes per item through a single warp, which costs
// more than the item's arithmetic when most tiles are empty.  This kernel computes the same lists for all items
// at once, with the whole GPU reading the packed mask at memory speed, into a workspace in global memory that the
// attention kernel's loader warps then copy from.
//
// Workspace layout: item j (the attention kernel's work-item numbering) owns plan_stride_words(N) 32-bit words:
// word 0 = number of non-empty tiles, then that many 16-bit entries in ascending tile order,
// entry = tile index | (row-group flags << 8), flag g set when rows 32g..32g+31 of the item keep something in the
// tile — the in-memory image of a TileList.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "sma_common.cuh"

namespace sma {

constexpr int kPlanRows = 128;  // rows per work item == kBlockM of the attention kernel
constexpr int kPlanTile = 64;   // keys per tile == kBlockN

__host__ __device__ constexpr uint32_t plan_stride_words(int N) {
    const uint32_t tiles = static_cast<uint32_t>((N + kPlanTile - 1) / kPlanTile);
    return (1u + (tiles + 1u) / 2u + 3u) & ~3u;  // count word + 16-bit entries, rounded to 16 bytes
}

// One CTA of 128 threads per work item; warp g takes row group g (rows 32g..32g+31 of the item).
//
// Rows that are whole 16-byte vectors (N % 128 == 0, aligned base) are read the coalesced way: the 32 lanes of a
// warp read 512 consecutive bytes of one row (lane l = vector l = key tiles 2l and 2l+1 of that chunk), eight rows
// in flight, and every lane ORs what it sees over the 32 rows of the group; no cross-lane work inside the loop.
// Other shapes take a simple path (thread r reads row r word by word); they are short or rare.
__global__ void __launch_bounds__(kPlanRows)
build_tile_lists_kernel(const uint32_t* __restrict__ mask_packed, uint32_t* __restrict__ plan, int BH, int N,
                        int num_q_tiles, uint32_t stride_words, uint32_t* __restrict__ work_counter) {
    // Launched the ordinary way (after the previous kernel has completed).  Were its CTAs allowed in early, they
    // would all gather on the few SMs that the previous kernel's first finished CTAs leave, and the attention
    // kernel's CTAs, allowed in behind them, would hold the other SMs idle while this kernel runs on a fifth of
    // the GPU.  The attention kernel may start its set-up only when this CTA's work is done (end of the kernel).
    const int item = blockIdx.x;
    if (work_counter != nullptr && item == 0 && threadIdx.x == 0) *work_counter = 0u;  // the attention kernel's work queue
    const int bh = item % BH;
    const int row0 = (num_q_tiles - 1 - item / BH) * kPlanRows;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nw = (N + 31) >> 5;
    const int num_tiles = (N + kPlanTile - 1) / kPlanTile;
    const uint32_t tail_bits = (N & 31) ? ((1u << (N & 31)) - 1u) : 0xFFFFFFFFu;
    const bool vector_rows = (N & 127) == 0 && (reinterpret_cast<uintptr_t>(mask_packed) & 15u) == 0;
    uint32_t* out = plan + static_cast<size_t>(item) * stride_words;
    uint16_t* entries = reinterpret_cast<uint16_t*>(out + 1);
    constexpr int kMaxPlanTiles = 16384 / kPlanTile;
    __shared__ uint32_t s_group[4][kMaxPlanTiles / 32];  // bit t of row group g: the group keeps something in tile t

    for (int i = threadIdx.x; i < 4 * (kMaxPlanTiles / 32); i += kPlanRows) (&s_group[0][0])[i] = 0u;
    __syncthreads();
    if (vector_rows) {
        const int nvec = nw / 4;
        const uint4* base = reinterpret_cast<const uint4*>(mask_packed + static_cast<size_t>(bh) * N * nw);
        const int grow0 = row0 + 32 * warp;
        for (int c0 = 0; c0 < nvec; c0 += 32) {
            const int vi = c0 + lane;
            uint32_t acc_lo = 0, acc_hi = 0;
            if (vi < nvec) {
                for (int r = 0; r < 32; r += 8) {
                    uint4 x[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        const int row = grow0 + r + u;
                        x[u] = row < N ? __ldg(base + static_cast<size_t>(row) * nvec + vi) : make_uint4(0u, 0u, 0u, 0u);
                    }
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        acc_lo |= x[u].x | x[u].y;
                        acc_hi |= x[u].z | x[u].w;
                    }
                }
            }
            // lane l speaks for tiles 2*vi and 2*vi+1: two ballots give the even and the odd tiles of the chunk
            const uint32_t even = __ballot_sync(0xFFFFFFFFu, acc_lo != 0u);
            const uint32_t odd = __ballot_sync(0xFFFFFFFFu, acc_hi != 0u);
            if (lane < 2) {
                // interleave: tile 2l <- even bit l, tile 2l+1 <- odd bit l; lane 0 writes tiles 0..31 of the chunk's
                // 64, lane 1 tiles 32..63
                const uint32_t e = lane == 0 ? (even & 0xFFFFu) : (even >> 16);
                const uint32_t o = lane == 0 ? (odd & 0xFFFFu) : (odd >> 16);
                uint32_t word = 0;
#pragma unroll
                for (int b = 0; b < 16; ++b) word |= (((e >> b) & 1u) << (2 * b)) | (((o >> b) & 1u) << (2 * b + 1));
                s_group[warp][(2 * c0) / 32 + lane] = word;
            }
        }
    } else {
        const int row = row0 + static_cast<int>(threadIdx.x);
        if (row < N) {
            const uint32_t* mrow = mask_packed + (static_cast<size_t>(bh) * N + row) * nw;
            for (int t = 0; t < num_tiles; ++t) {
                const int i0 = 2 * t, i1 = i0 + 1;
                uint32_t a = i0 < nw ? __ldg(mrow + i0) : 0u;
                uint32_t b = i1 < nw ? __ldg(mrow + i1) : 0u;
                if (i0 == nw - 1) a &= tail_bits;
                if (i1 == nw - 1) b &= tail_bits;
                if ((a | b) != 0u) atomicOr(&s_group[warp][t >> 5], 1u << (t & 31));
            }
        }
    }
    __syncthreads();
    if (warp == 0) {
        uint32_t count = 0;
        for (int t0 = 0; t0 < num_tiles; t0 += 32) {
            const uint32_t b0 = s_group[0][t0 >> 5], b1 = s_group[1][t0 >> 5], b2 = s_group[2][t0 >> 5],
                           b3 = s_group[3][t0 >> 5];
            const uint32_t any = b0 | b1 | b2 | b3;
            if ((any >> lane) & 1u) {
                const uint32_t pos = count + __popc(any & ((1u << lane) - 1u));
                const uint32_t flags = ((b0 >> lane) & 1u) | (((b1 >> lane) & 1u) << 1) | (((b2 >> lane) & 1u) << 2) |
                                       (((b3 >> lane) & 1u) << 3);
                entries[pos] = static_cast<uint16_t>((t0 + lane) | (flags << 8));
            }
            count += __popc(any);
        }
        if (lane == 0) out[0] = count;
    }
    __syncthreads();
    grid_launch_dependents();
}

}  // namespace sma
