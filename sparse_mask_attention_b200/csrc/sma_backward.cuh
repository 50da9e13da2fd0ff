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
//   attn_bwd_kernel     persistent CTAs, one per SM, that share out units of work = (batch*head, block of 128 keys)
//                       through a queue.  For a unit the CTA keeps K_j and V_j in shared memory, walks
//                       the blocks of 128 query rows that keep anything in its 128 keys, and per such block issues
//                       five tcgen05 products: S = Q K^T and dP = dO V^T into tensor memory; eight warps (two
//                       threads per query row, 64 keys each) turn them into P and dS, written as 16-bit tiles into
//                       shared memory; dV += P^T dO and dK += dS^T Q accumulate in tensor memory over the whole walk,
//                       dQ_i = dS K goes to tensor memory and from there, through a staging tile in shared memory and
//                       a TMA reduction (fp32 add), into the accumulator (each row of dQ receives one contribution
//                       per key block).  At the end dK_j, dV_j are rounded and stored.
//                       The walk is software-pipelined: P/dS, Q/dO and dQ exist twice, S and dP of block s+1 are
//                       issued as soon as the compute warps have read those of block s out of tensor memory, and the
//                       three products that consume P and dS of block s run under the arithmetic of block s+1.
//                       Ten warps: eight compute warps, one that issues the products, one that requests the tiles
//                       (TMA), takes the CTA's next unit from the queue and reads that unit's strip of the mask while
//                       the unit in work runs, so that the next unit's tiles are on their way before the boundary.
//   bwd_finish_kernel   dq = round(accumulator)
//
// P and dS are the A operands of products that contract over the query rows (P^T, dS^T: "MN-major" operands, read
// from shared memory transposed) and, for dQ, over the keys (K-major): one buffer serves both.  A buffer is two
// panels of [128 query rows][64 keys] 16-bit values, rows of 128 bytes with the 128-byte swizzle, the second panel
// 16 KB behind the first (the leading byte offset of the MN-major descriptor).
//
// dQ is summed in fp32 in the order in which the CTAs' reductions arrive: its last bits can differ from run to run,
// so it is reproducible to rounding, not bit for bit.  dK and dV are deterministic.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "sma_common.cuh"

namespace sma {

constexpr int kBwdBlock = 128;              // query rows per step, and keys per CTA
constexpr int kBwdDim = 64;                 // head dimension
constexpr int kBwdComputeWarps = 8;         // two threads per query row: 64 keys each
constexpr int kBwdThreads = 32 * (kBwdComputeWarps + 2);  // + the warp that issues the products + the warp that loads
constexpr uint32_t kBwdTileBytes = kBwdBlock * kBwdDim * 2;  // [128 rows][64] 16-bit
constexpr uint32_t kBwdPanelBytes = kBwdBlock * 128;         // [128 query rows][64 keys] 16-bit
constexpr uint32_t kBwdTmemCols = 512;
constexpr uint32_t kBwdColS = 0, kBwdColDP = 128, kBwdColDV = 256, kBwdColDK = 320, kBwdColDQ = 384;  // dQ: two buffers of 64
constexpr int kBwdMaxQBlocks = 16384 / kBwdBlock;

struct BwdSmem {
    alignas(1024) uint8_t k[kBwdTileBytes];
    alignas(1024) uint8_t v[kBwdTileBytes];
    alignas(1024) uint8_t q[2][kBwdTileBytes];
    alignas(1024) uint8_t dout[2][kBwdTileBytes];
    alignas(1024) uint8_t p[2][2][kBwdPanelBytes];   // [step % 2][panel of 64 keys]
    alignas(1024) uint8_t ds[2][2][kBwdPanelBytes];
    uint64_t bar_kv;        // TMA: K_j and V_j landed
    uint64_t bar_q[2];      // TMA: Q_i landed in stage s
    uint64_t bar_do[2];     // TMA: dO_i landed in stage s
    uint64_t bar_sdp;       // tensor core: S and dP of the step are complete
    uint64_t bar_sfree;     // all compute threads: S and dP of the step have been read out of tensor memory
    // The next two exist once per step parity.  A thread that waits for step g of one of them may already have done
    // everything that step g + 1 needs from it (the issuing warp has S and dP of step g + 1 out before it waits for
    // P and dS of step g; a compute thread arrives for step g before it waits for the products of step g - 1), so on
    // a single barrier phase g + 1 could complete before the waiter has looked, and a parity wait would then take
    // it for phase g - 1.  Step g + 2 always needs the waiter to have moved on.
    uint64_t bar_pds[2];    // all compute threads: P and dS of the step are in shared memory, its S and dP and the
                            // dQ of the step before last have been read out of tensor memory
    uint64_t bar_mma2[2];   // tensor core: dV, dK accumulated and dQ complete for the step
    uint64_t bar_half[2];   // the 128 compute threads of a half meet here (a bounded wait, unlike bar.sync)
    uint64_t bar_q_free;    // tensor core: the last product that reads the step's Q tile (dK) is complete
    uint64_t bar_do_free;   // tensor core: the last product that reads the step's dO tile (dV) is complete
    uint64_t bar_done;      // tensor core: every product of the unit is complete (one phase per unit)
    uint32_t tmem_base;
    uint32_t abort_flag;
    // Double-buffered by the parity of the CTA's unit count: while a unit is in work the loading warp names the one
    // after it and marks that unit's query blocks.
    uint32_t unit_id[2];                          // the unit (>= the number of units: none is left)
    uint32_t qblock_any[2][kBwdMaxQBlocks / 32];  // bit i: query block i keeps something in the keys of the unit
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
    // Work queue of the persistent CTAs (units = (key block, batch*head) pairs), or nullptr: a 32-bit word that
    // bwd_prepare_kernel, the kernel before this one in the stream, has set to zero.  A CTA's first unit is its own
    // index; every further one comes from the queue (without it: index + k * grid).
    uint32_t* unit_counter;
};

// delta[row] = sum_d dout[row, d] * out[row, d]; dq_accum[row, :] = 0.  One warp per row of 64 values.
template <bool kBf16>
__global__ void __launch_bounds__(256)
bwd_prepare_kernel(const uint32_t* __restrict__ dout, const uint32_t* __restrict__ out, float* __restrict__ delta,
                   float* __restrict__ dq_accum, size_t rows, uint32_t* __restrict__ unit_counter) {
    const int lane = threadIdx.x & 31;
    grid_launch_dependents();  // attn_bwd_kernel's CTAs may set themselves up as this grid's retire
    if (unit_counter != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *unit_counter = 0u;  // attn_bwd_kernel's work queue
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
    grid_dependency_wait();  // launched to overlap with attn_bwd_kernel's last CTAs: its reductions are complete from here on
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
                const __grid_constant__ CUtensorMap tmap_dq, const BwdArgs args) {
    extern __shared__ uint8_t smem_raw[];
    BwdSmem& sm = *reinterpret_cast<BwdSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~static_cast<uintptr_t>(1023u));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int N = args.N;
    const int nw = (N + 31) >> 5;
    const int nblk = (N + kBwdBlock - 1) / kBwdBlock;  // key blocks == query blocks
    // A unit of work = (key block j, batch*head bh); unit u = j * BH + bh, so that for causal-like masks, whose early
    // key blocks are kept by the most query blocks, the long units come first.  CTAs are persistent.
    const long long units = static_cast<long long>(args.BH) * nblk;
    int j = 0, bh = 0;                      // of the unit in work
    const uint32_t* mask_bh = nullptr;
    uint32_t g = 0;                         // steps (query blocks walked) over all units of this CTA: barrier phases
    uint32_t unit_no = 0;                   // units done by this CTA
    constexpr uint32_t kFmt = kBf16 ? kFmtBF16 : kFmtF16;
    volatile uint32_t* abort_flag = &sm.abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&sm.bar_kv, 1);
        mbar_init(&sm.bar_q[0], 1);
        mbar_init(&sm.bar_q[1], 1);
        mbar_init(&sm.bar_do[0], 1);
        mbar_init(&sm.bar_do[1], 1);
        mbar_init(&sm.bar_sdp, 1);
        mbar_init(&sm.bar_sfree, 32 * kBwdComputeWarps);
        mbar_init(&sm.bar_pds[0], 32 * kBwdComputeWarps);
        mbar_init(&sm.bar_pds[1], 32 * kBwdComputeWarps);
        mbar_init(&sm.bar_mma2[0], 1);
        mbar_init(&sm.bar_mma2[1], 1);
        mbar_init(&sm.bar_q_free, 1);
        mbar_init(&sm.bar_do_free, 1);
        mbar_init(&sm.bar_done, 1);
        mbar_init(&sm.bar_half[0], 128);
        mbar_init(&sm.bar_half[1], 128);
        sm.abort_flag = 0u;
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
    // Launched to overlap with bwd_prepare_kernel: barriers and tensor memory are set up while that grid drains; its
    // outputs (delta, the zeroed accumulator, the queue word) are there from here on.  bwd_finish_kernel in turn may
    // be scheduled as this grid's CTAs retire.
    grid_dependency_wait();
    grid_launch_dependents();

    const uint32_t a_bar_kv = smem_u32(&sm.bar_kv), a_bar_q = smem_u32(&sm.bar_q[0]), a_bar_do = smem_u32(&sm.bar_do[0]),
                   a_bar_sdp = smem_u32(&sm.bar_sdp), a_bar_pds = smem_u32(&sm.bar_pds[0]), a_bar_mma2 = smem_u32(&sm.bar_mma2[0]),
                   a_bar_sfree = smem_u32(&sm.bar_sfree), a_bar_q_free = smem_u32(&sm.bar_q_free),
                   a_bar_do_free = smem_u32(&sm.bar_do_free), a_bar_done = smem_u32(&sm.bar_done);
    bool ok = true;  // false once a bounded wait has run out; the same in all lanes of a warp
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait_a(bar, parity, abort_flag));
    };
    // next query block >= i that keeps something (by the flags in `slot`), or nblk
    auto next_block = [&](uint32_t slot, int i) {
        while (i < nblk && !((sm.qblock_any[slot][i >> 5] >> (i & 31)) & 1u)) ++i;
        return i;
    };

    auto begin_unit = [&](long long u) {
        j = static_cast<int>(u / args.BH);
        bh = static_cast<int>(u % args.BH);
        mask_bh = args.mask_packed + static_cast<size_t>(bh) * N * nw;
    };
    if (warp == kBwdComputeWarps) {
        // ========================================= tensor-core issue =========================================
        // all lanes run the control flow (operands stay in uniform registers); one elected lane issues
        const bool leader = elect_one();
        constexpr uint32_t kHi = kSmemDescSw128Hi;
        constexpr uint32_t idesc_s = make_idesc(kFmt, kFmt, kMajorK, kMajorK, kBwdBlock, kBwdBlock, 0);    // [128 q][128 keys]
        constexpr uint32_t idesc_t = make_idesc(kFmt, kFmt, kMajorMN, kMajorMN, kBwdBlock, kBwdDim, 0);    // (P|dS)^T [128 keys][64]
        constexpr uint32_t idesc_q = make_idesc(kFmt, kFmt, kMajorK, kMajorMN, kBwdBlock, kBwdDim, 0);     // dS K [128 q][64]
        constexpr uint32_t kPanelLbo = (kBwdPanelBytes >> 4) << 16;  // second panel of 64 keys, for the transposed reads
        const uint32_t k_lo = smem_desc_sw128_lo(smem_u32(sm.k)), v_lo = smem_desc_sw128_lo(smem_u32(sm.v));
        constexpr uint32_t kStageUnits = (2 * kBwdPanelBytes) >> 4;  // from one P/dS buffer to the other, in descriptor units
        const uint32_t p_t_lo0 = ((smem_u32(sm.p[0][0]) & 0x3FFFFu) >> 4) | kPanelLbo;
        const uint32_t ds_t_lo0 = ((smem_u32(sm.ds[0][0]) & 0x3FFFFu) >> 4) | kPanelLbo;
        const uint32_t ds_k_lo0 = smem_desc_sw128_lo(smem_u32(sm.ds[0][0]));
        // S = Q K^T and dP = dO V^T of the query block whose tiles arrive in stage `st`, each as soon as its tile is there
        // (contraction over the head dimension: 16 elements = 32 bytes inside the swizzled 128-byte row).  `step` is the
        // step the block belongs to; before S and dP are overwritten, those of the step before have left tensor memory.
        auto issue_s_dp = [&](uint32_t step, bool first) {
            const uint32_t st = step & 1u, ph = (step >> 1) & 1u;
            const uint32_t q_lo = smem_desc_sw128_lo(smem_u32(sm.q[st])), do_lo = smem_desc_sw128_lo(smem_u32(sm.dout[st]));
            wait(a_bar_q + 8 * st, ph);
            if (!first) wait(a_bar_sfree, (step - 1) & 1u);
            tc_fence_after_sync();
            if (leader && ok) {
#pragma unroll
                for (int kk = 0; kk < kBwdDim / 16; ++kk) mma_ss_lh(tmem + kBwdColS, q_lo + 2 * kk, k_lo + 2 * kk, kHi, idesc_s, kk ? 1u : 0u);
            }
            __syncwarp();
            wait(a_bar_do + 8 * st, ph);
            if (leader && ok) {
#pragma unroll
                for (int kk = 0; kk < kBwdDim / 16; ++kk) mma_ss_lh(tmem + kBwdColDP, do_lo + 2 * kk, v_lo + 2 * kk, kHi, idesc_s, kk ? 1u : 0u);
                mma_commit_a(a_bar_sdp);
            }
            __syncwarp();
        };
        for (;;) {
            // The unit before is over for every thread (its accumulators have left tensor memory); the loading warp has
            // named this unit and marked its query blocks during the unit before.
            __syncthreads();
            const uint32_t slot = unit_no & 1u;
            if (sm.unit_id[slot] >= units || *abort_flag) break;
            uint32_t s = 0;  // steps of this unit
            int i = next_block(slot, 0);
            if (i < nblk) {
                wait(a_bar_kv, unit_no & 1u);
                issue_s_dp(g, true);
            }
            // Step: as soon as the compute warps have turned S and dP of a block into P and dS, the tensor core gets S
            // and dP of the next block (which the compute warps then work on) and, behind them, the three products
            // that consume P and dS of this one.  P/dS, Q/dO and dQ exist twice, so the products of a block run under
            // the arithmetic of the next.
            while (i < nblk && ok) {
                const uint32_t st = g & 1u;
                const int i_next = next_block(slot, i + 1);
                // S and dP of the next block go to the tensor core as soon as this block's have left tensor memory,
                // while the compute warps are still busy with the arithmetic on them
                if (i_next < nblk) issue_s_dp(g + 1, false);
                wait(a_bar_pds + 8 * (g & 1u), (g >> 1) & 1u);
                tc_fence_after_sync();
                const uint32_t q_lo = smem_desc_sw128_lo(smem_u32(sm.q[st])), do_lo = smem_desc_sw128_lo(smem_u32(sm.dout[st]));
                const uint32_t p_t_lo = p_t_lo0 + st * kStageUnits, ds_t_lo = ds_t_lo0 + st * kStageUnits, ds_k_lo = ds_k_lo0 + st * kStageUnits;
                if (leader && ok) {
                    const uint32_t acc0 = s ? 1u : 0u;
                    // contraction over the 128 query rows: 16 rows of 128 bytes = 2048 bytes per step, in both operands.
                    // dK first: it is the last reader of the Q tile, which the next S needs before anything else.
#pragma unroll
                    for (int kk = 0; kk < kBwdBlock / 16; ++kk) mma_ss_lh(tmem + kBwdColDK, ds_t_lo + 128 * kk, q_lo + 128 * kk, kHi, idesc_t, kk ? 1u : acc0);
                    mma_commit_a(a_bar_q_free);
#pragma unroll
                    for (int kk = 0; kk < kBwdBlock / 16; ++kk) mma_ss_lh(tmem + kBwdColDV, p_t_lo + 128 * kk, do_lo + 128 * kk, kHi, idesc_t, kk ? 1u : acc0);
                    mma_commit_a(a_bar_do_free);
                    // contraction over the 128 keys: dS is K-major, 64 keys per panel; K_j rows are keys
#pragma unroll
                    for (int kk = 0; kk < kBwdBlock / 16; ++kk)
                        mma_ss_lh(tmem + kBwdColDQ + 64 * st, ds_k_lo + (kk >> 2) * (kBwdPanelBytes >> 4) + 2 * (kk & 3), k_lo + 128 * kk, kHi,
                                  idesc_q, kk ? 1u : 0u);
                    mma_commit_a(a_bar_mma2 + 8 * st);
                }
                __syncwarp();
                ++s;
                ++g;
                i = i_next;
            }
            // The loading warp, which runs ahead of this one, learns here that K_j, V_j and the Q/dO stages are free.
            // (It waits for every phase of this barrier in turn; a barrier that it skipped phases of would answer for
            // the wrong one.)
            if (leader && ok) {
                if (s >= 1) mma_commit_a(a_bar_done);
                else mbar_arrive_a(a_bar_done);
            }
            __syncwarp();
            ++unit_no;
        }
    } else if (warp == kBwdComputeWarps + 1) {
        // ================================ loads, and the choice of the next unit ================================
        const bool leader = elect_one();
        if (leader) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            tma_prefetch_desc(&tmap_do);
        }
        __syncwarp();
        auto load_q = [&](uint32_t stage, int i) {
            if (leader && ok) {
                mbar_arrive_expect_tx_a(a_bar_q + 8 * stage, kBwdTileBytes);
                tma_load_3d_a(smem_u32(sm.q[stage]), &tmap_q, a_bar_q + 8 * stage, 0, i * kBwdBlock, bh);
            }
            __syncwarp();
        };
        auto load_do = [&](uint32_t stage, int i) {
            if (leader && ok) {
                mbar_arrive_expect_tx_a(a_bar_do + 8 * stage, kBwdTileBytes);
                tma_load_3d_a(smem_u32(sm.dout[stage]), &tmap_do, a_bar_do + 8 * stage, 0, i * kBwdBlock, bh);
            }
            __syncwarp();
        };
        // Which query blocks keep anything in the 128 keys of a unit: this warp reads the unit's column strip of
        // the mask (plain loads: written by kernels that completed before bwd_prepare_kernel started),
        // four query blocks at a time, one lane per four rows of a block.  It does so for the unit AFTER the one in
        // work, between its loads, so that at a unit's end the next unit's tiles can be requested at once.
        const bool scan_vec = (nw & 3) == 0 && (reinterpret_cast<uintptr_t>(args.mask_packed) & 15u) == 0;
        const uint32_t* scan_strip = nullptr;
        int scan_words = 0, scan_blk = nblk;
        auto scan_begin = [&](long long us, uint32_t slot) {
            if (lane < kBwdMaxQBlocks / 32) sm.qblock_any[slot][lane] = 0u;
            __syncwarp();
            scan_blk = nblk;
            if (us < units) {
                const int jj = static_cast<int>(us / args.BH), bb = static_cast<int>(us % args.BH);
                scan_strip = args.mask_packed + static_cast<size_t>(bb) * N * nw + 4 * jj;
                scan_words = nw - 4 * jj < 4 ? nw - 4 * jj : 4;
                scan_blk = 0;
            }
        };
        // The loads of four query blocks are requested in one call and looked at in the next (a step later): the warp
        // does not stand waiting for them with tiles to request.
        uint4 pend[16];
        int pend_blk = -1;  // the first of the four blocks whose words are on their way, or none
        auto scan_step = [&](uint32_t slot) {
            if (pend_blk >= 0) {
                uint32_t bits = 0u;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    uint32_t any = 0u;
#pragma unroll
                    for (int r = 0; r < 4; ++r) any |= pend[4 * b + r].x | pend[4 * b + r].y | pend[4 * b + r].z | pend[4 * b + r].w;
                    if (__any_sync(0xFFFFFFFFu, any != 0u)) bits |= 1u << b;
                }
                if (lane == 0 && bits != 0u) sm.qblock_any[slot][pend_blk >> 5] |= bits << (pend_blk & 31);  // pend_blk % 4 == 0
                __syncwarp();
                pend_blk = -1;
            }
            if (scan_blk < nblk) {
#pragma unroll
                for (int b = 0; b < 4; ++b) {
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        uint4 x = make_uint4(0u, 0u, 0u, 0u);
                        const int row = (scan_blk + b) * kBwdBlock + lane + 32 * r;  // (past the last block: past N as well)
                        if (row < N) {
                            const uint32_t* mrow = scan_strip + static_cast<size_t>(row) * nw;
                            if (scan_vec) {
                                x = *reinterpret_cast<const uint4*>(mrow);
                            } else {
                                x.x = mrow[0];
                                if (scan_words > 1) x.y = mrow[1];
                                if (scan_words > 2) x.z = mrow[2];
                                if (scan_words > 3) x.w = mrow[3];
                            }
                        }
                        pend[4 * b + r] = x;
                    }
                }
                pend_blk = scan_blk;
                scan_blk += 4;
            }
        };
        auto scan_pending = [&]() { return pend_blk >= 0 || scan_blk < nblk; };
        // K_j, V_j and the first Q/dO tiles of unit u, whose flags are in `slot`; i = its first query block
        int i = nblk;
        long long u = blockIdx.x;  // < units: the grid has at most one CTA per unit
        auto load_unit = [&](uint32_t slot) {
            begin_unit(u);
            i = next_block(slot, 0);
            if (leader && ok) {
                mbar_arrive_expect_tx_a(a_bar_kv, 2 * kBwdTileBytes);
                tma_load_3d_a(smem_u32(sm.k), &tmap_k, a_bar_kv, 0, j * kBwdBlock, bh);
                tma_load_3d_a(smem_u32(sm.v), &tmap_v, a_bar_kv, 0, j * kBwdBlock, bh);
            }
            __syncwarp();
            if (i < nblk) {
#ifdef SMA_WAIT_TEST_BUILD
                // test build only: on request, the first Q tile of unit 0 is never asked for, nothing completes its
                // barrier, and the issuing warp's wait for it runs out
                const bool withheld = g_test_withhold_q_load != 0 && u == 0;
#else
                constexpr bool withheld = false;
#endif
                if (!withheld) load_q(g & 1u, i);
                load_do(g & 1u, i);
            }
        };
        scan_begin(u, 0u);
        while (scan_pending()) scan_step(0u);
        if (lane == 0) sm.unit_id[0] = static_cast<uint32_t>(u);
        __syncwarp();
        load_unit(0u);
        for (;;) {
            // The unit before is over for every thread (nobody reads its flags any more); the other warps find this
            // unit's number and flags, written during the unit before.
            __syncthreads();
            if (u >= units || *abort_flag) break;
            const uint32_t slot = unit_no & 1u;
            uint32_t s = 0;  // steps of this unit
            // the unit after this one: asked for now, looked at behind the first step's requests (the answer takes a while)
            long long next = u + gridDim.x;
            if (leader && args.unit_counter != nullptr) next = static_cast<long long>(gridDim.x) + atomicAdd(args.unit_counter, 1u);
            long long u_next = units;
            bool named = false;
            auto name_next = [&]() {
                if (leader) sm.unit_id[slot ^ 1u] = static_cast<uint32_t>(next < units ? next : units);
                __syncwarp();
                u_next = sm.unit_id[slot ^ 1u];
                scan_begin(u_next, slot ^ 1u);
                named = true;
            };
            // A stage's Q tile is free once the dK product of the step that used it is complete, its dO tile once dV is
            // (at a unit's first step: of the unit before, long complete).
            while (i < nblk && ok) {
                const uint32_t st = g & 1u;
                const int i_next = next_block(slot, i + 1);
                if (i_next < nblk) {
                    if (s >= 1) wait(a_bar_q_free, (g - 1) & 1u);
                    load_q(st ^ 1u, i_next);
                    if (s >= 1) wait(a_bar_do_free, (g - 1) & 1u);
                    load_do(st ^ 1u, i_next);
                }
                if (!named) name_next();
                if (scan_pending()) scan_step(slot ^ 1u);
                ++s;
                ++g;
                i = i_next;
            }
            if (!named) name_next();
            while (scan_pending()) scan_step(slot ^ 1u);
            // K_j, V_j and both Q/dO stages are free once the last step's products are complete (and the K/V copy has
            // landed, also in a unit whose keys nobody keeps): the next unit's tiles travel while the compute warps take
            // this unit's dQ, dK and dV out of tensor memory
            wait(a_bar_done, unit_no & 1u);
            wait(a_bar_kv, unit_no & 1u);
            u = u_next;
            ++unit_no;
            i = nblk;
            if (u < units) load_unit(slot ^ 1u);
        }
    } else {
        // ================= two threads per query row (64 keys each): P, dS, dQ, and at the end dK, dV =================
        // Warps 0-3 take keys 0..63 of the block (panel 0), columns 0..31 of dQ and, at the end, dK; warps 4-7 keys
        // 64..127, columns 32..63 of dQ and dV.  A warp reaches the tensor-memory lanes 32 (warp % 4) .. + 31.
        const int t = static_cast<int>(threadIdx.x & 127u);
        const uint32_t half = threadIdx.x >> 7;
        const uint32_t tmem_lane = tmem + (static_cast<uint32_t>(32 * (warp & 3)) << 16);
        const float scale_log2e = args.scale * 1.4426950408889634f;
        const uint32_t a_p0 = smem_u32(sm.p[0][half]) + static_cast<uint32_t>(t) * 128u;
        const uint32_t a_ds0 = smem_u32(sm.ds[0][half]) + static_cast<uint32_t>(t) * 128u;
        const uint32_t sw = static_cast<uint32_t>(t) & 7u;
        int prev_row0 = 0;
        // dQ of a finished step leaves through shared memory and one TMA reduction per half (fp32 add into the
        // accumulator in global memory).  Per-thread atomics (8 vector atomics per thread and step) filled the
        // load/store queue that the issuing warp's barrier and shared-memory accesses also go through, and held it up
        // for as long as they took.  The staging tile is the P panel of the finished step, free once its products are
        // complete: [128 rows][32 fp32 = 128 bytes], 128-byte swizzle, this half's columns.
        const bool reducer = (threadIdx.x & 127u) == 0;  // the thread of a half that issues its reductions
        const uint32_t a_bar_half = smem_u32(&sm.bar_half[half]);
        uint32_t half_phase = 0;
        // the 128 threads of the half meet (a bounded wait: a thread that gave up elsewhere holds nobody for ever)
        auto half_sync = [&]() {
            mbar_arrive_a(a_bar_half);
            wait(a_bar_half, half_phase & 1u);
            ++half_phase;
        };
        auto read_dq = [&](uint32_t step, float (&dq)[32]) {
            wait(a_bar_mma2 + 8 * (step & 1u), (step >> 1) & 1u);
            tc_fence_after_sync();
            if (!ok) return;
            tmem_ld32_f32(tmem_lane + kBwdColDQ + 64 * (step & 1u) + 32 * half, dq);
            tmem_wait_ld();
        };
        auto reduce_dq = [&](uint32_t step, const float (&dq)[32], int row0) {
            const uint32_t a_stage = smem_u32(sm.p[step & 1u][half]);
            const uint32_t a_row = a_stage + static_cast<uint32_t>(t) * 128u;
#pragma unroll
            for (int g = 0; g < 8; ++g)
                sts_v4(a_row + ((static_cast<uint32_t>(g) ^ sw) << 4),
                       make_uint4(__float_as_uint(dq[4 * g]), __float_as_uint(dq[4 * g + 1]), __float_as_uint(dq[4 * g + 2]),
                                  __float_as_uint(dq[4 * g + 3])));
            fence_proxy_async_smem();
            half_sync();
            if (reducer && ok) {
                tma_reduce_add_3d(&tmap_dq, a_stage, 32 * static_cast<int>(half), row0, bh);
                tma_store_commit();
            }
        };
        // before the half writes a P panel again: the reduction that used it as its staging tile has read it
        auto staging_free = [&]() {
            if (reducer) tma_store_wait_read();
            half_sync();
        };
        // this thread's inputs for a block of query rows: log-sum-exp and delta of its row, its two mask words.  Requested
        // one block ahead, so that the loads' latency lies under the block in work.
        struct RowIn {
            float lse, delta;
            uint32_t mw0, mw1;
        };
        auto load_row = [&](int blk) {
            RowIn r{0.f, 0.f, 0u, 0u};
            const int row = blk * kBwdBlock + t;
            if (blk < nblk && row < N) {
                r.lse = args.lse[static_cast<size_t>(bh) * N + row];
                r.delta = args.delta[static_cast<size_t>(bh) * N + row];
                const int wi = 4 * j + 2 * static_cast<int>(half);
                const uint32_t* mrow = mask_bh + static_cast<size_t>(row) * nw;
                if (wi < nw) r.mw0 = mrow[wi];
                if (wi + 1 < nw) r.mw1 = mrow[wi + 1];
            } else {
                r.lse = -INFINITY;  // rows past the end keep nothing
            }
            return r;
        };
        for (;;) {
            // The unit before is over for every thread; the loading warp has named this one and marked the query blocks
            // that keep anything in its keys.
            __syncthreads();
            const uint32_t slot = unit_no & 1u;
            const long long u = sm.unit_id[slot];
            if (u >= units || *abort_flag) break;
            begin_unit(u);
            uint32_t steps = 0;  // steps of this unit
            int i = next_block(slot, 0);
            RowIn in_next = load_row(i);
            while (i < nblk && ok) {
                const RowIn in = in_next;
                const int i_next = next_block(slot, i + 1);
                in_next = load_row(i_next);
                uint32_t mw[2] = {in.mw0, in.mw1};
                float neg_lse_l2 = 0.f;
                const float delta = in.delta;
                if (in.lse != -INFINITY) {
                    neg_lse_l2 = -in.lse * 1.4426950408889634f;
                } else {  // a row that keeps nothing has P = 0 everywhere
                    mw[0] = mw[1] = 0u;
                }
                wait(a_bar_sdp, g & 1u);
                tc_fence_after_sync();
                if (!ok) break;
                // this step's P/dS buffer was last read by the products of the step before last: complete, because this
                // thread waited for them before it arrived for the step before (below)
                const uint32_t a_p = a_p0 + (g & 1u) * 2 * kBwdPanelBytes, a_ds = a_ds0 + (g & 1u) * 2 * kBwdPanelBytes;
                if (g >= 2) staging_free();  // the dQ of the step before last (of this unit or the one before) went out through this P panel
#pragma unroll
                for (int c = 0; c < 2; ++c) {  // 32 keys at a time
                    float s[32], dp[32];
                    tmem_ld32_f32(tmem_lane + kBwdColS + 64 * half + 32 * c, s);
                    tmem_ld32_f32(tmem_lane + kBwdColDP + 64 * half + 32 * c, dp);
                    tmem_wait_ld();
                    if (c == 1) {  // this thread's part of S and dP is in registers: the tensor core may overwrite it
                        tc_fence_before_sync();
                        mbar_arrive_a(a_bar_sfree);
                    }
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
                mbar_arrive_a(a_bar_pds + 8 * (g & 1u));
                // dQ of the step before (its products ran under this step's arithmetic) leaves tensor memory behind the
                // arrival, which nothing then holds up: the products of this step write the other dQ buffer, and the ones
                // after them, issued behind this thread's next arrival, this one
                if (steps >= 1) {
                    float dq[32];
                    read_dq(g - 1, dq);
                    if (ok) reduce_dq(g - 1, dq, prev_row0);
                }
                prev_row0 = i * kBwdBlock;
                ++steps;
                ++g;
                i = i_next;
            }
            if (steps >= 1 && ok) {
                float dq[32];
                read_dq(g - 1, dq);
                if (ok) reduce_dq(g - 1, dq, prev_row0);
            }
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
            // (the next unit's products that overwrite dK and dV in tensor memory are issued behind the CTA-wide barrier
            // above, which this thread reaches after the loads have completed)
            tc_fence_before_sync();
            ++unit_no;
        }
        if (reducer) tma_store_wait_all();  // the reductions are complete before the CTA (and its shared memory) goes
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
