// Backward pass of the masked attention for sm_100a: dq, dk, dv from dout, with P recomputed from the saved
// log-sum-exp and the same skipping of key tiles in which no query row keeps a key.
//
// The math is the one the reference's autograd function spells out in PyTorch (python/sparse_attention.py:96-111;
// the CUDA entry point it would call, sparse_attention_bwd_bf16, is only declared: csrc/sparse_attention.h:57-64):
//     P  = exp(scale * q k^T - lse)  where the mask keeps, 0 elsewhere
//     dV = P^T dO
//     dP = dO V^T
//     dS = scale * P o (dP - delta),   delta_i = sum_j P_ij dP_ij = dO_i . O_i
//     dQ = dS K,   dK = dS^T Q
//
// Three kernels:
//   bwd_prepare_kernel  delta = rowsum(dO o O) in fp32 and zeroes of the fp32 dQ accumulator (one warp per row)
//   attn_bwd_kernel     one CTA per (batch*head, block of 128 keys).  It keeps K_j and V_j in shared memory, walks
//                       the blocks of 128 query rows that keep anything in its 128 keys, and per such block issues
//                       five tcgen05 products: S = Q K^T and dP = dO V^T into tensor memory; eight warps (two
//                       threads per query row, 64 keys each) turn them into P and dS, written as 16-bit tiles into
//                       shared memory;
//                       dV += P^T dO and dK += dS^T Q accumulate in tensor memory over the whole walk, dQ_i = dS K
//                       goes to tensor memory and from there, by vector atomics, into the fp32 accumulator (each row
//                       of dQ receives one contribution per key block).  At the end dK_j, dV_j are rounded and stored.
//   bwd_finish_kernel   dq = round(accumulator)
//
// P and dS are the A operands of products that contract over the query rows (P^T, dS^T: "MN-major" operands, read
// from shared memory transposed) and, for dQ, over the keys (K-major): one buffer serves both.  A buffer is two
// panels of [128 query rows][64 keys] 16-bit values, rows of 128 bytes with the 128-byte swizzle, the second panel
// 16 KB behind the first (the leading byte offset of the MN-major descriptor).
//
// dQ is summed by atomics in fp32: its last bits depend on the order in which CTAs arrive, so it is reproducible
// to rounding, not bit for bit.  dK and dV are deterministic.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sma_common.cuh"

namespace sma {

constexpr int kBwdBlock = 128;              // query rows per step, and keys per CTA
constexpr int kBwdDim = 64;                 // head dimension
constexpr int kBwdComputeWarps = 8;         // two threads per query row: 64 keys each
constexpr int kBwdThreads = 32 * (kBwdComputeWarps + 1);  // + the warp that loads and issues
constexpr uint32_t kBwdTileBytes = kBwdBlock * kBwdDim * 2;  // [128 rows][64] 16-bit
constexpr uint32_t kBwdPanelBytes = kBwdBlock * 128;         // [128 query rows][64 keys] 16-bit
constexpr uint32_t kBwdTmemCols = 512;
constexpr uint32_t kBwdColS = 0, kBwdColDP = 128, kBwdColDV = 256, kBwdColDK = 320, kBwdColDQ = 384;
constexpr int kBwdMaxQBlocks = 16384 / kBwdBlock;

struct BwdSmem {
    alignas(1024) uint8_t k[kBwdTileBytes];
    alignas(1024) uint8_t v[kBwdTileBytes];
    alignas(1024) uint8_t q[2][kBwdTileBytes];
    alignas(1024) uint8_t dout[2][kBwdTileBytes];
    alignas(1024) uint8_t p[2][kBwdPanelBytes];   // two panels of 64 keys
    alignas(1024) uint8_t ds[2][kBwdPanelBytes];
    uint64_t bar_kv;        // TMA: K_j and V_j landed
    uint64_t bar_qdo[2];    // TMA: Q_i and dO_i landed in stage s
    uint64_t bar_sdp;       // tensor core: S and dP of the step are complete
    uint64_t bar_pds;       // 128 arrivals: P and dS of the step are in shared memory (and S, dP, dQ have been read)
    uint64_t bar_mma2;      // tensor core: dV, dK accumulated and dQ complete for the step
    uint32_t tmem_base;
    uint32_t abort_flag;
    uint32_t qblock_any[kBwdMaxQBlocks / 32];  // bit i: query block i keeps something in this CTA's keys
};

constexpr size_t bwd_smem_bytes() { return sizeof(BwdSmem) + 1024; }

struct BwdArgs {
    const uint32_t* mask_packed;  // [BH, N, ceil(N/32)]
    const float* lse;             // [BH, N], natural log; -inf for rows that keep nothing
    const float* delta;           // [BH, N]
    float* dq_accum;              // [BH, N, 64] fp32, zero on entry
    void* dk;                     // [BH, N, 64] 16-bit
    void* dv;
    int32_t BH;
    int32_t N;
    float scale;
};

// delta[row] = sum_d dout[row, d] * out[row, d]; dq_accum[row, :] = 0.  One warp per row of 64 values.
template <bool kBf16>
__global__ void __launch_bounds__(256)
bwd_prepare_kernel(const uint32_t* __restrict__ dout, const uint32_t* __restrict__ out, float* __restrict__ delta,
                   float* __restrict__ dq_accum, size_t rows) {
    const int lane = threadIdx.x & 31;
    const size_t warps = static_cast<size_t>(gridDim.x) * (blockDim.x >> 5);
    for (size_t row = static_cast<size_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
        const uint32_t a = dout[row * 32 + lane], b = out[row * 32 + lane];  // two 16-bit values each
        float a0, a1, b0, b1;
        if constexpr (kBf16) {
            a0 = __uint_as_float(a << 16), a1 = __uint_as_float(a & 0xFFFF0000u);
            b0 = __uint_as_float(b << 16), b1 = __uint_as_float(b & 0xFFFF0000u);
        } else {
            const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&a));
            const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&b));
            a0 = fa.x, a1 = fa.y, b0 = fb.x, b1 = fb.y;
        }
        float s = fmaf(a0, b0, a1 * b1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
        if (lane == 0) delta[row] = s;
        reinterpret_cast<float2*>(dq_accum)[row * 32 + lane] = make_float2(0.f, 0.f);
    }
}

// dq = round(dq_accum); n2 = number of pairs.
template <bool kBf16>
__global__ void __launch_bounds__(256)
bwd_finish_kernel(const float2* __restrict__ dq_accum, uint32_t* __restrict__ dq, size_t n2) {
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n2; i += stride) {
        const float2 x = dq_accum[i];
        dq[i] = kBf16 ? pack_bf16x2(x.x, x.y) : pack_f16x2(x.x, x.y);
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const BwdArgs args) {
    extern __shared__ uint8_t smem_raw[];
    BwdSmem& sm = *reinterpret_cast<BwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = args.N;
    const int nw = (N + 31) >> 5;
    const int nblk = (N + kBwdBlock - 1) / kBwdBlock;  // key blocks == query blocks
    const int j = static_cast<int>(blockIdx.x % nblk);  // this CTA's key block
    const int bh = static_cast<int>(blockIdx.x / nblk);
    constexpr uint32_t kFmt = kBf16 ? kFmtBF16 : kFmtF16;
    volatile uint32_t* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&sm.bar_kv, 1);
        mbar_init(&sm.bar_qdo[0], 1);
        mbar_init(&sm.bar_qdo[1], 1);
        mbar_init(&sm.bar_sdp, 1);
        mbar_init(&sm.bar_pds, 32 * kBwdComputeWarps);
        mbar_init(&sm.bar_mma2, 1);
        sm.abort_flag = 0u;
        for (int i = 0; i < kBwdMaxQBlocks / 32; ++i) sm.qblock_any[i] = 0u;
        mbar_init_fence();
    }
    __syncwarp();
    if (warp == kBwdComputeWarps) {
        tmem_alloc(&sm.tmem_base, kBwdTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = sm.tmem_base;

    // ---- which query blocks keep anything in keys 128j..128j+127: thread t looks at row t of every block ----
    const uint32_t* mask_bh = args.mask_packed + static_cast<size_t>(bh) * N * nw;
    if (warp < kBwdComputeWarps) {
        for (int i = warp >> 2; i < nblk; i += 2) {  // warps 0-3 take the even blocks, warps 4-7 the odd ones
            const int row = i * kBwdBlock + static_cast<int>(threadIdx.x & 127u);
            uint32_t any = 0u;
            if (row < N) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const int wi = 4 * j + w;
                    if (wi < nw) any |= ldg_u32(mask_bh + static_cast<size_t>(row) * nw + wi);
                }
            }
            const uint32_t some = __ballot_sync(0xFFFFFFFFu, any != 0u);
            if (lane == 0 && some != 0u) atomicOr(&sm.qblock_any[i >> 5], 1u << (i & 31));
        }
    }
    __syncthreads();

    const uint32_t a_bar_kv = smem_u32(&sm.bar_kv), a_bar_qdo = smem_u32(&sm.bar_qdo[0]), a_bar_sdp = smem_u32(&sm.bar_sdp),
                   a_bar_pds = smem_u32(&sm.bar_pds), a_bar_mma2 = smem_u32(&sm.bar_mma2);
    bool ok = true;  // false once a bounded wait has run out; the same in all lanes of a warp
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait_a(bar, parity, abort_flag));
    };
    // next query block >= i that keeps something, or nblk
    auto next_block = [&](int i) {
        while (i < nblk && !((sm.qblock_any[i >> 5] >> (i & 31)) & 1u)) ++i;
        return i;
    };

    uint32_t steps = 0;  // query blocks walked
    if (warp == kBwdComputeWarps) {
        // ===================================== loads and tensor-core issue =====================================
        const bool leader = lane == 0;
        constexpr uint32_t kHi = kSmemDescSw128Hi;
        constexpr uint32_t idesc_s = make_idesc(kFmt, kFmt, kMajorK, kMajorK, kBwdBlock, kBwdBlock, 0);    // [128 q][128 keys]
        constexpr uint32_t idesc_t = make_idesc(kFmt, kFmt, kMajorMN, kMajorMN, kBwdBlock, kBwdDim, 0);    // (P|dS)^T [128 keys][64]
        constexpr uint32_t idesc_q = make_idesc(kFmt, kFmt, kMajorK, kMajorMN, kBwdBlock, kBwdDim, 0);     // dS K [128 q][64]
        constexpr uint32_t kPanelLbo = (kBwdPanelBytes >> 4) << 16;  // second panel of 64 keys, for the transposed reads
        const uint32_t k_lo = smem_desc_sw128_lo(smem_u32(sm.k)), v_lo = smem_desc_sw128_lo(smem_u32(sm.v));
        const uint32_t p_t_lo = ((smem_u32(sm.p[0]) & 0x3FFFFu) >> 4) | kPanelLbo;
        const uint32_t ds_t_lo = ((smem_u32(sm.ds[0]) & 0x3FFFFu) >> 4) | kPanelLbo;
        const uint32_t ds_k_lo = smem_desc_sw128_lo(smem_u32(sm.ds[0]));
        if (leader) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            tma_prefetch_desc(&tmap_do);
        }
        __syncwarp();
        auto load_q_do = [&](uint32_t stage, int i) {
            if (leader && ok) {
                const uint32_t bar = a_bar_qdo + 8 * stage;
                mbar_arrive_expect_tx_a(bar, 2 * kBwdTileBytes);
                tma_load_3d_a(smem_u32(sm.q[stage]), &tmap_q, bar, 0, i * kBwdBlock, bh);
                tma_load_3d_a(smem_u32(sm.dout[stage]), &tmap_do, bar, 0, i * kBwdBlock, bh);
            }
            __syncwarp();
        };
        int i = next_block(0);
        if (i < nblk) {  // (a CTA whose keys nobody keeps loads nothing: it only writes zeros to dK_j, dV_j)
            if (leader) {
                mbar_arrive_expect_tx_a(a_bar_kv, 2 * kBwdTileBytes);
                tma_load_3d_a(smem_u32(sm.k), &tmap_k, a_bar_kv, 0, j * kBwdBlock, bh);
                tma_load_3d_a(smem_u32(sm.v), &tmap_v, a_bar_kv, 0, j * kBwdBlock, bh);
            }
            __syncwarp();
            load_q_do(0, i);
        }
        while (i < nblk && ok) {
            const uint32_t st = steps & 1u;
            const int i_next = next_block(i + 1);
            // the other stage was read by the second group of products of the step before
            if (i_next < nblk) {
                if (steps >= 1) wait(a_bar_mma2, (steps - 1) & 1u);
                load_q_do(st ^ 1u, i_next);
            }
            wait(a_bar_qdo + 8 * st, (steps >> 1) & 1u);
            if (steps == 0) wait(a_bar_kv, 0u);
            // S and dP of the step before have been read: its bar_pds phase was waited for below
            tc_fence_after_sync();
            const uint32_t q_lo = smem_desc_sw128_lo(smem_u32(sm.q[st])), do_lo = smem_desc_sw128_lo(smem_u32(sm.dout[st]));
            if (leader && ok) {
                // contraction over the head dimension: 16 elements = 32 bytes inside the swizzled 128-byte row
#pragma unroll
                for (int kk = 0; kk < kBwdDim / 16; ++kk) mma_ss_lh(tmem + kBwdColS, q_lo + 2 * kk, k_lo + 2 * kk, kHi, idesc_s, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < kBwdDim / 16; ++kk) mma_ss_lh(tmem + kBwdColDP, do_lo + 2 * kk, v_lo + 2 * kk, kHi, idesc_s, kk ? 1u : 0u);
                mma_commit_a(a_bar_sdp);
            }
            __syncwarp();
            wait(a_bar_pds, steps & 1u);  // P and dS are in shared memory; the dQ of the step before has been read
            tc_fence_after_sync();
            if (leader && ok) {
                const uint32_t acc0 = steps ? 1u : 0u;
                // contraction over the 128 query rows: 16 rows of 128 bytes = 2048 bytes per step, in both operands
#pragma unroll
                for (int kk = 0; kk < kBwdBlock / 16; ++kk) mma_ss_lh(tmem + kBwdColDV, p_t_lo + 128 * kk, do_lo + 128 * kk, kHi, idesc_t, kk ? 1u : acc0);
#pragma unroll
                for (int kk = 0; kk < kBwdBlock / 16; ++kk) mma_ss_lh(tmem + kBwdColDK, ds_t_lo + 128 * kk, q_lo + 128 * kk, kHi, idesc_t, kk ? 1u : acc0);
                // contraction over the 128 keys: dS is K-major, 64 keys per panel; K_j rows are keys
#pragma unroll
                for (int kk = 0; kk < kBwdBlock / 16; ++kk)
                    mma_ss_lh(tmem + kBwdColDQ, ds_k_lo + (kk >> 2) * (kBwdPanelBytes >> 4) + 2 * (kk & 3), k_lo + 128 * kk, kHi, idesc_q, kk ? 1u : 0u);
                mma_commit_a(a_bar_mma2);
            }
            __syncwarp();
            ++steps;
            i = i_next;
        }
    } else {
        // ================= two threads per query row (64 keys each): P, dS, dQ, and at the end dK, dV =================
        // Warps 0-3 take keys 0..63 of the block (panel 0), columns 0..31 of dQ and, at the end, dK; warps 4-7 keys
        // 64..127, columns 32..63 of dQ and dV.  A warp reaches the tensor-memory lanes 32 (warp % 4) .. + 31.
        const int t = static_cast<int>(threadIdx.x & 127u);
        const uint32_t half = threadIdx.x >> 7;
        const uint32_t tmem_lane = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16);
        const float scale_log2e = args.scale * 1.4426950408889634f;
        const uint32_t a_p = smem_u32(sm.p[half]) + static_cast<uint32_t>(t) * 128u;
        const uint32_t a_ds = smem_u32(sm.ds[half]) + static_cast<uint32_t>(t) * 128u;
        const uint32_t sw = static_cast<uint32_t>(t) & 7u;
        int prev_row = 0;
        // dQ of a finished step: tensor memory -> fp32 accumulator in global memory
        auto flush_dq = [&](uint32_t step, int row) {
            wait(a_bar_mma2, step & 1u);
            tc_fence_after_sync();
            if (!ok) return;
            float dq[32];
            tmem_ld32_f32(tmem_lane + kBwdColDQ + 32 * half, dq);
            tmem_wait_ld();
            if (row < N) {
                float4* dst = reinterpret_cast<float4*>(args.dq_accum + (static_cast<size_t>(bh) * N + row) * kBwdDim + 32 * half);
#pragma unroll
                for (int c = 0; c < 8; ++c) atomicAdd(dst + c, make_float4(dq[4 * c], dq[4 * c + 1], dq[4 * c + 2], dq[4 * c + 3]));
            }
        };
        int i = next_block(0);
        while (i < nblk && ok) {
            const int row = i * kBwdBlock + t;
            uint32_t mw[2] = {0u, 0u};
            float neg_lse_l2 = 0.f, delta = 0.f;
            if (row < N) {
                const float lse = args.lse[static_cast<size_t>(bh) * N + row];
                delta = args.delta[static_cast<size_t>(bh) * N + row];
                if (lse != -INFINITY) {  // a row that keeps nothing has P = 0 everywhere
                    neg_lse_l2 = -lse * 1.4426950408889634f;
#pragma unroll
                    for (int w = 0; w < 2; ++w) {
                        const int wi = 4 * j + 2 * static_cast<int>(half) + w;
                        if (wi < nw) mw[w] = ldg_u32(mask_bh + static_cast<size_t>(row) * nw + wi);
                    }
                }
            }
            // the products of the step before read P and dS from shared memory and wrote dQ: both must be over; the
            // atomics of its dQ run while the tensor core works on this step's S and dP
            if (steps >= 1) flush_dq(steps - 1, prev_row);
            wait(a_bar_sdp, steps & 1u);
            tc_fence_after_sync();
            if (!ok) break;
#pragma unroll
            for (int c = 0; c < 2; ++c) {  // 32 keys at a time
                float s[32], dp[32];
                tmem_ld32_f32(tmem_lane + kBwdColS + 64 * half + 32 * c, s);
                tmem_ld32_f32(tmem_lane + kBwdColDP + 64 * half + 32 * c, dp);
                tmem_wait_ld();
                const uint32_t bits = mw[c];
                uint32_t pw[16], dw[16];
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    const float p0 = ((bits >> e) & 1u) ? ex2_approx(fmaf(s[e], scale_log2e, neg_lse_l2)) : 0.f;
                    const float p1 = ((bits >> (e + 1)) & 1u) ? ex2_approx(fmaf(s[e + 1], scale_log2e, neg_lse_l2)) : 0.f;
                    const float d0 = p0 * (dp[e] - delta) * args.scale, d1 = p1 * (dp[e + 1] - delta) * args.scale;
                    pw[e >> 1] = kBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
                    dw[e >> 1] = kBf16 ? pack_bf16x2(d0, d1) : pack_f16x2(d0, d1);
                }
                // 32 keys = four 16-byte pieces of this thread's 128-byte row in its panel, pieces 4 c .. 4 c + 3, each
                // stored where the 128-byte swizzle puts it
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const uint32_t piece = ((static_cast<uint32_t>(4 * c + g)) ^ sw) * 16u;
                    sts_v4(a_p + piece, make_uint4(pw[4 * g], pw[4 * g + 1], pw[4 * g + 2], pw[4 * g + 3]));
                    sts_v4(a_ds + piece, make_uint4(dw[4 * g], dw[4 * g + 1], dw[4 * g + 2], dw[4 * g + 3]));
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive_a(a_bar_pds);
            prev_row = row;
            ++steps;
            i = next_block(i + 1);
        }
        if (steps >= 1 && ok) flush_dq(steps - 1, prev_row);
        // ---- dK_j (warps 0-3) and dV_j (warps 4-7): tensor-memory lane t is key 128 j + t ----
        const int key = j * kBwdBlock + t;
        if (ok) {
            uint32_t outw[kBwdDim / 2];
            if (steps >= 1) {
                float acc[kBwdDim];
                const uint32_t col = half ? kBwdColDV : kBwdColDK;
                tmem_ld32_f32(tmem_lane + col, &acc[0]);
                tmem_ld32_f32(tmem_lane + col + 32, &acc[32]);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < kBwdDim; e += 2) outw[e >> 1] = kBf16 ? pack_bf16x2(acc[e], acc[e + 1]) : pack_f16x2(acc[e], acc[e + 1]);
            } else {
#pragma unroll
                for (int e = 0; e < kBwdDim / 2; ++e) outw[e] = 0u;  // no query row keeps any of these keys
            }
            if (key < N) {
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint8_t*>(half ? args.dv : args.dk) +
                                                      (static_cast<size_t>(bh) * N + key) * kBwdDim * 2);
#pragma unroll
                for (int c = 0; c < kBwdDim / 8; ++c) dst[c] = make_uint4(outw[4 * c], outw[4 * c + 1], outw[4 * c + 2], outw[4 * c + 3]);
            }
        }
    }

    // ---- release tensor memory -------------------------------------------------------------------
    if (*abort_flag) {
        // a wait ran out: give the asynchronous units time to finish what was issued before the tensor memory and
        // the shared memory are given back (a bounded pause, nothing is waited for)
        const long long t0 = clock64();
        while (clock64() - t0 < 400000) __nanosleep(1000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == kBwdComputeWarps) tmem_dealloc(tmem, kBwdTmemCols);
}

}  // namespace sma
