// Fused sparse-mask attention forward for sm_100a.
//
// Computes, per (batch, head):  out = softmax(keep ? scale * q k^T : -inf) v   with the keep mask given
// as packed bits, fp32 accumulation, fp16 or bf16 inputs/outputs, and optionally the row-wise
// log-sum-exp.  Same result contract as the reference kernels sparse_attn_wmma_full_fp16
// (csrc/sparse_attention.cu:82-412) and sparse_attention_fwd_kernel<...,bf16> (:418-543): rows with no
// kept column give zeros, masked columns contribute exactly nothing.
//
// Structure: one persistent CTA of 512 threads per SM runs two independent "streams".  A stream owns one work
// item at a time — 128 consecutive query rows of one (batch, head) — walks its keys in chunks of 512 (eight
// 64-key tiles, sixteen packed-mask words per row) and visits only the tiles that hold at least one kept bit
// for those rows.  Warp roles:
//   * loader warp (1 per stream): per chunk it brings the 128 x 16-word strip of packed-mask words into
//     shared memory (one TMA tile copy; plain loads for shapes a tensor map cannot describe), finds the
//     non-empty tiles in it (or copies them from a list computed ahead, kPlanned) and publishes a chunk
//     descriptor; then it issues the TMA loads (128-byte swizzle) of the item's Q tile and of the listed
//     K/V tile pairs into a three-stage ring, as the P V products release the stages.
//   * MMA warp (1 per stream): one thread walks the stream's tile sequence, across chunks and work items
//     without draining, and issues every tcgen05.mma of the stream:
//         S[128x64]  = Q K^T   (operands in shared memory)
//         O[128x64] += P V     (P from tensor memory, V MN-major from shared memory)
//     S runs one tile ahead of the softmax threads (two S/P buffers); Q and O are double-buffered, so the
//     first products of the next item run while the previous item is still being finished.
//   * softmax warps (4 per stream): thread r owns query row r (tensor-memory lane r).  Per tile it reads
//     its S row with tcgen05.ld, applies its two mask words from the strip, updates the running max / sum
//     and writes P (16-bit) with tcgen05.st over the columns its S row came from.  At the end of an item it
//     leaves 1/sum in shared memory for the epilogue warps and goes straight on to the next item.
//   * epilogue warps (4, shared by both streams): warp w owns rows 32w..32w+31 (its tensor-memory lane
//     quadrant) of whichever stream finishes an item: it reads O, normalises, rounds, stages the rows in
//     shared memory and stores them with one TMA store.
// Hand-offs are mbarriers (TMA transaction counts, tcgen05.commit, thread arrivals); every wait is bounded.
// Orderings that need no barrier of their own, because one thread issues all products of a stream and the
// tensor core runs them in issue order:
//   * S(j) may overwrite buffer j%2 once P V(j-2) has been issued: that product read the buffer's previous P.
//   * P(j) may overwrite S(j) in place: the softmax threads read S(j) before they write P(j).
#pragma once

#include <stddef.h>

#include "sma_common.cuh"

namespace sma {

constexpr int kBlockM = 128;       // query rows per work item (= tcgen05.mma M)
constexpr int kBlockN = 64;        // keys per tile (the tile-skip granule)
constexpr int kHeadDim = 64;       // D; one row = 128 bytes = one swizzle span
constexpr int kTmemCols = 512;
constexpr int kNumStreams = 2;
constexpr int kStages = 3;         // K/V ring depth
constexpr int kSlots = 2;          // chunks (mask strip + descriptor) in flight per stream
constexpr int kChunkTiles = 8;     // key tiles per chunk
constexpr int kChunkWords = 2 * kChunkTiles;       // packed-mask words per row and chunk
constexpr int kChunkKeys = kBlockN * kChunkTiles;  // 512
constexpr int kAttnThreads = 512;

// Tensor-memory layout of one stream (256 columns): two S/P buffers (64 columns each; P takes the first
// 32 of them, or all 64 as hi|lo halves for the bf16 split), then two O accumulators (64 each).
constexpr int kColsPerStream = 256;
constexpr int kSBuffers = 2;
constexpr int kColS = 0;
constexpr int kColO = 64 * kSBuffers;

constexpr int kMaxSeqLen = 16384;  // == SMA_MAX_SEQ_LEN
constexpr float kRescaleThreshold = 8.f;  // O is rescaled only when a row max grows by more than 2^8

constexpr uint32_t kQTileBytes = kBlockM * kHeadDim * 2;
constexpr uint32_t kKVTileBytes = kBlockN * kHeadDim * 2;
constexpr uint32_t kStripRowBytes = kChunkWords * 4;
constexpr uint32_t kStripBytes = kBlockM * kStripRowBytes;
constexpr uint32_t kStageRowsOut = 32;  // rows per TMA store of the epilogue (one warp's rows)

struct StreamTiles {
    alignas(1024) uint8_t q[2][kQTileBytes];
    alignas(1024) uint8_t k[kStages][kKVTileBytes];
    alignas(1024) uint8_t v[kStages][kKVTileBytes];
    alignas(128) uint8_t strip[kSlots][kStripBytes];  // [row][word] of the chunk, 64 bytes per row
};

// What the loader publishes per chunk.  meta = count | last << 8: `count` non-empty key tiles, ascending, in
// entry[]; entry = tile index | (group flags << 8), flag g set when rows 32g..32g+31 of the item keep something
// in that tile; `last` marks the final chunk of the work item.  item < 0 ends the stream.
struct ChunkDesc {
    int32_t item;
    uint32_t meta;
    uint16_t entry[kChunkTiles];
    uint32_t pad[2];
};
static_assert(sizeof(ChunkDesc) == 32, "descriptor addressing below assumes 32 bytes");

// A parity wait cannot tell a phase from the one two before it, nor wait for a phase while the one before it
// is still open.  Every barrier below is therefore indexed (by ring stage, buffer or slot) such that a waiter
// has always seen the previous phase of its barrier, and the next-but-one phase cannot open before every
// waiter of the current one has passed.
struct StreamCtrl {
    alignas(8) uint64_t bar_q[2];          // TMA: Q tile of item r landed in buffer r % 2
    uint64_t bar_q_free[2];                // tcgen05.commit: every S of item r is complete
    uint64_t bar_kv[kStages];              // TMA: K and V tile landed
    uint64_t bar_pv_done[kStages];         // tcgen05.commit: P V complete (the K/V stage is free again)
    uint64_t bar_s_full[kSBuffers];        // tcgen05.commit: S tile complete
    uint64_t bar_p_full[kSBuffers];        // 128 arrivals: P written over the S buffer (and O rescaled)
    uint64_t bar_list_full[kSlots];        // 1 arrival: chunk descriptor published
    uint64_t bar_strip_full[kSlots];       // TMA (or 1 arrival): the chunk's mask strip is in shared memory
    uint64_t bar_slot_free[kSlots];        // 129 arrivals: softmax threads and MMA warp left the chunk
    uint64_t bar_stat_full[2];             // 128 arrivals: row sums of item r published
    uint64_t bar_o_full[2];                // tcgen05.commit: every P V of item r is complete
    uint64_t bar_o_free[2];                // 4 arrivals: the epilogue warps have read O and the row sums
    ChunkDesc desc[kSlots];
    int32_t stat_item[2];                  // work item the row sums belong to (< 0: the stream has ended)
    float stat_inv_l[2][kBlockM];          // 1 / row sum (0 for a row that keeps nothing)
};

struct AttnSmem {
    StreamTiles tiles[kNumStreams];
    alignas(1024) uint8_t staging[4][kStageRowsOut * 128];  // one per epilogue warp
    StreamCtrl ctrl[kNumStreams];
    uint32_t tmem_base;
    uint32_t abort_flag;  // raised by the first bounded wait that runs out
};

constexpr size_t attn_smem_bytes() { return sizeof(AttnSmem) + 1024; }  // + slack to align the base to 1024

// Multiplies this thread's row of an O accumulator (64 fp32 columns at addr) by alpha.  Kept out of line: it runs
// only when a row maximum jumps, and the softmax loop is sensitive to the size of its body.
__device__ __noinline__ void rescale_o_row(uint32_t addr, float alpha) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t o[32];
        tmem_ld32(addr + half * 32, o);
        tmem_wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
        tmem_st32(addr + half * 32, o);
    }
}

struct AttnArgs {
    const uint32_t* mask_packed;
    const uint32_t* plan;   // tile lists computed ahead (sma_plan.cuh), or nullptr: the loader warps build them
    uint32_t plan_stride;   // words per work item in plan
    float* lse;
    int32_t BH;
    int32_t N;
    int32_t num_q_tiles;
    float scale_log2e;   // |scale| * log2(e)
    uint32_t negate_q;   // 1 if scale < 0: S is computed as (-Q) K^T
    int32_t save_lse;
    int32_t mask_tma;    // 1: the packed mask has a tensor map (rows are whole 16-byte vectors, aligned base)
};

// kBf16   : element type of q/k/v/out (false = fp16).  P takes the same 16-bit format: tcgen05.mma
//           kind::f16 raises an illegal-instruction fault when the A and B formats differ, so an
//           fp16 P cannot be multiplied with a bf16 V.
// kSplitP : bf16 only.  true = P = hi + lo, both bf16, two P*V products per tile (16 significant bits, so
//           the result meets the same tolerance as the fp16 path); false = P rounded once to bf16.
// kPlanned: the tile lists come from AttnArgs::plan instead of being built by the loader warps.
template <bool kBf16, bool kSplitP, bool kPlanned>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                const __grid_constant__ CUtensorMap tmap_m, const AttnArgs args) {
    static_assert(kBf16 || !kSplitP, "the hi+lo split exists for bf16 only");
    static_assert(kNumStreams * kColsPerStream <= kTmemCols, "tensor memory over-committed");
    static_assert(kSlots == 2 && kSBuffers == 2, "slot and buffer indices below are ordinal & 1");
    // register budgets: 512 threads start at 128 registers each; 256 * 200 + 256 * 56 = 512 * 128
    constexpr int kRegsSoftmax = 200;
    constexpr int kRegsOther = 56;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u));

    // Warpgroup 0 holds the MMA warps (warps 0, 1) and the loader warps (2, 3) of the two streams, warpgroups
    // 1 and 2 are the softmax warps of stream 0 and 1, warpgroup 3 the epilogue warps.  warp % 4 decides the
    // tensor-memory lane quadrant a warp may touch.  The index is broadcast from lane 0 so that the compiler
    // knows it (and every address derived from it) to be the same in all lanes of a warp and keeps such values
    // in uniform registers: tcgen05.mma, the TMA instructions and the barrier instructions take their operands
    // from there.
    const int warp = __shfl_sync(0xFFFFFFFFu, static_cast<int>(threadIdx.x >> 5), 0);
    const int wg = warp >> 2;
    const int wq = warp & 3;
    const int lane = threadIdx.x & 31;
    const int N = args.N;
    const int BH = args.BH;
    const int nw = (N + 31) >> 5;                             // packed words per mask row
    const int num_chunks = (N + kChunkKeys - 1) / kChunkKeys;
    const int total_items = BH * args.num_q_tiles;
    const int item_stride = kNumStreams * static_cast<int>(gridDim.x);

    // ---- set-up: barriers (one thread per stream), tensor memory (one warp) --------------------------
    if ((wg == 1 || wg == 2) && (threadIdx.x & 127) == 0) {
        StreamCtrl& ct = sm.ctrl[wg - 1];
        for (int s = 0; s < 2; ++s) {
            mbar_init(&ct.bar_q[s], 1);
            mbar_init(&ct.bar_q_free[s], 1);
            mbar_init(&ct.bar_s_full[s], 1);
            mbar_init(&ct.bar_p_full[s], 128);
            mbar_init(&ct.bar_list_full[s], 1);
            mbar_init(&ct.bar_strip_full[s], 1);
            mbar_init(&ct.bar_slot_free[s], 129);
            mbar_init(&ct.bar_stat_full[s], 128);
            mbar_init(&ct.bar_o_full[s], 1);
            mbar_init(&ct.bar_o_free[s], 4);
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&ct.bar_kv[s], 1);
            mbar_init(&ct.bar_pv_done[s], 1);
        }
        if (wg == 1) sm.abort_flag = 0u;
        mbar_init_fence();
    }
    __syncwarp();
    if (warp == 0) {
        tmem_alloc(&sm.tmem_base, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    // everything above overlaps with the tail of the previous kernel in the stream; nothing below may
    grid_launch_dependents();
    grid_dependency_wait();

    // Work items are dealt round-robin: item j belongs to CTA j % grid; the CTA's items go to its streams
    // in turn (stream s takes items blockIdx + s*grid, then every 2*grid further).  Item j is
    // (row block, batch*head) with the later row blocks first: for causal-like masks they hold most work.
    auto item_bh = [&](int item) { return item % BH; };
    auto item_row0 = [&](int item) { return (args.num_q_tiles - 1 - item / BH) * kBlockM; };
    bool ok = true;  // false once a bounded wait has run out; the same in all lanes of a warp
    volatile uint32_t* const abort_flag = &sm.abort_flag;
    // Bounded wait on an mbarrier phase.  After a failure nothing is waited for any more, and the warp's lanes
    // agree on the outcome (the .sync.aligned instructions that follow need a converged warp).
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (ok) ok = __all_sync(0xFFFFFFFFu, mbar_wait_a(bar, parity, abort_flag));
    };

    if (wg == 3) {
        // =========================================== epilogue warps ==========================================
        setmaxnreg_dec<kRegsOther>();
        const uint32_t a_stage = smem_u32(sm.staging[wq]);
        const uint32_t tmem_q = sm.tmem_base + (static_cast<uint32_t>(wq * 32) << 16);
        uint32_t e[kNumStreams] = {0u, 0u};       // items finished per stream
        bool done[kNumStreams] = {false, false};
        long long t_idle = clock64();
        bool staged = false;  // a TMA store of this warp may still be reading the staging tile
        while (ok && !(done[0] && done[1])) {
            bool progressed = false;
#pragma unroll
            for (int s = 0; s < kNumStreams; ++s) {
                if (done[s]) continue;
                const uint32_t ct_a = smem_u32(&sm.ctrl[s]);
                const uint32_t b = e[s] & 1u, par = (e[s] >> 1) & 1u;
                const uint32_t a_stat_full = ct_a + offsetof(StreamCtrl, bar_stat_full) + 8 * b;
                if (!__any_sync(0xFFFFFFFFu, mbar_try_wait_suspend_a(a_stat_full, par, 500))) continue;
                wait(a_stat_full, par);  // every lane takes the acquire itself
                progressed = true;
                const int item = static_cast<int>(lds_u32(ct_a + offsetof(StreamCtrl, stat_item) + 4 * b));
                if (item < 0) {
                    done[s] = true;
                    continue;
                }
                const float inv_l = lds_f32(ct_a + offsetof(StreamCtrl, stat_inv_l) + (b * kBlockM + wq * 32 + lane) * 4);
                wait(ct_a + offsetof(StreamCtrl, bar_o_full) + 8 * b, par);
                tc_fence_after_sync();
                // the previous store of this warp must have finished reading the staging tile
                if (staged && lane == 0) tma_store_wait_read();
                __syncwarp();
                const uint32_t o_addr = tmem_q + s * kColsPerStream + kColO + 64u * b;
                // row `lane` of the warp occupies 128 bytes; its 16-byte chunk j sits at chunk position j ^ (lane & 7)
                const uint32_t a_row = a_stage + lane * 128;
#pragma unroll
                for (int q16 = 0; q16 < 4; ++q16) {
                    uint32_t o[16];
                    tmem_ld16(o_addr + q16 * 16, o);
                    tmem_wait_ld();
                    uint32_t pk[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float x = __uint_as_float(o[2 * j]) * inv_l;
                        const float y = __uint_as_float(o[2 * j + 1]) * inv_l;
                        // inv_l == 0: the row keeps nothing (its accumulator may hold anything, even NaN)
                        pk[j] = inv_l == 0.f ? 0u : (kBf16 ? pack_bf16x2(x, y) : pack_f16x2(x, y));
                    }
                    sts_v4(a_row + (((2 * q16) ^ (lane & 7)) << 4), make_uint4(pk[0], pk[1], pk[2], pk[3]));
                    sts_v4(a_row + (((2 * q16 + 1) ^ (lane & 7)) << 4), make_uint4(pk[4], pk[5], pk[6], pk[7]));
                }
                tc_fence_before_sync();
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_a(ct_a + offsetof(StreamCtrl, bar_o_free) + 8 * b);
                    const int row0 = item_row0(item) + wq * static_cast<int>(kStageRowsOut);
                    if (row0 < N && ok) {
                        tma_store_3d(&tmap_o, sm.staging[wq], 0, row0, item_bh(item));
                        tma_store_commit();
                    }
                }
                staged = true;
                ++e[s];
            }
            if (progressed) {
                t_idle = clock64();
            } else {
                if (*abort_flag) ok = false;
                if (clock64() - t_idle > kWaitLimitCycles) {
                    *abort_flag = 1u;
                    atomicExch(&g_device_status, kDeviceTimeout);
                    ok = false;
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    } else {
        const int stream = wg == 0 ? (warp & 1) : (wg - 1);
        StreamTiles& tl = sm.tiles[stream];
        StreamCtrl& ct = sm.ctrl[stream];
        // 32-bit shared-memory addresses of the stream's barriers, descriptors and strips
        const uint32_t ct_a = smem_u32(&ct);
        const uint32_t a_bar_q = ct_a + offsetof(StreamCtrl, bar_q);
        const uint32_t a_bar_q_free = ct_a + offsetof(StreamCtrl, bar_q_free);
        const uint32_t a_bar_kv = ct_a + offsetof(StreamCtrl, bar_kv);
        const uint32_t a_bar_pv_done = ct_a + offsetof(StreamCtrl, bar_pv_done);
        const uint32_t a_bar_s_full = ct_a + offsetof(StreamCtrl, bar_s_full);
        const uint32_t a_bar_p_full = ct_a + offsetof(StreamCtrl, bar_p_full);
        const uint32_t a_bar_list_full = ct_a + offsetof(StreamCtrl, bar_list_full);
        const uint32_t a_bar_strip_full = ct_a + offsetof(StreamCtrl, bar_strip_full);
        const uint32_t a_bar_slot_free = ct_a + offsetof(StreamCtrl, bar_slot_free);
        const uint32_t a_bar_stat_full = ct_a + offsetof(StreamCtrl, bar_stat_full);
        const uint32_t a_bar_o_full = ct_a + offsetof(StreamCtrl, bar_o_full);
        const uint32_t a_bar_o_free = ct_a + offsetof(StreamCtrl, bar_o_free);
        const uint32_t a_desc0 = ct_a + offsetof(StreamCtrl, desc);
        const uint32_t a_strip0 = smem_u32(tl.strip[0]);
        const uint32_t tmem = sm.tmem_base + stream * kColsPerStream;
        const int first_item = blockIdx.x + stream * gridDim.x;

        if (wg != 0) {
            // =========================================== softmax warps ===========================================
            setmaxnreg_inc<kRegsSoftmax>();
            const int stid = threadIdx.x & 127;  // row inside the work item
            const uint32_t tmem_lane = tmem + (static_cast<uint32_t>(wq * 32) << 16);
            const float c = args.scale_log2e;

            uint32_t g = 0;                 // key tiles processed by this stream so far (drives the barrier phases)
            uint32_t sbuf = 0, sphase = 0;  // g % 2 and (g / 2) & 1
            uint32_t u = 0;                 // chunks consumed so far
            uint32_t r = 0;                 // work items started so far
            float sc[64] = {};              // scores of the tile in work
            for (;;) {
                const uint32_t ob = r & 1u;  // O accumulator (and row-sum buffer) of this item
                float m_run = -INFINITY;     // reference max of the unscaled scores (lags the true max by < 8/c)
                float l_run = 0.f;           // running sum of exp2(c * (s - m_run))
                int item = -1;
                bool last = false;
                // new reference max after a tile with maximum m_tile; returns the factor for what was accumulated before
                auto advance_max = [&](float m_tile, float& neg_mc_out) -> float {
                    // the reference max moves only when the tile max exceeds it by more than 2^8 (exp2 units)
                    const bool grow = fmaf(m_tile - m_run, c, -kRescaleThreshold) > 0.f;  // false for -inf - -inf
                    const float m_new = grow ? m_tile : m_run;
                    const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
                    neg_mc_out = -m_use * c;
                    // nothing kept so far: the sum is 0 and the accumulator row is 0 or not yet written, no factor needed
                    const float a = (grow && m_run != -INFINITY) ? ex2_approx(fmaf(m_run, c, neg_mc_out)) : 1.f;
                    m_run = m_new;
                    return a;
                };
                do {
                    const uint32_t slot = u & 1u, spar = (u >> 1) & 1u;
                    wait(a_bar_list_full + 8 * slot, spar);
                    if (!ok) break;
                    const uint32_t a_desc = a_desc0 + slot * 32u;
                    item = static_cast<int>(lds_u32(a_desc));
                    if (item < 0) break;
                    const uint32_t meta = lds_u32(a_desc + 4);
                    const int count = static_cast<int>(meta & 0xFFu);
                    last = (meta >> 8) & 1u;
                    const uint32_t a_entries = a_desc + 8;
                    if (count > 0) {
                        wait(a_bar_strip_full + 8 * slot, spar);
                        const uint32_t a_row = a_strip0 + slot * kStripBytes + stid * kStripRowBytes;
                        // entry of the tile in work; `has`: this warp's 32 rows keep something in it
                        uint32_t e_cur = lds_u16(a_entries);
                        wait(a_bar_s_full + 8 * sbuf, sphase);
                        tc_fence_after_sync();
                        if ((e_cur >> (8 + wq)) & 1u) {
                            tmem_ld32_f32(tmem_lane + kColS + 64u * sbuf, &sc[0]);
                            tmem_ld32_f32(tmem_lane + kColS + 64u * sbuf + 32, &sc[32]);
                        }
                        // The tile loop is one rolled body (mask + maximum, then exponentials + P) on one register
                        // set; two tiles per loop body let the compiler overlap the tail of one tile with the head of
                        // the next.  Longer bodies (the bf16 hi+lo one twice, any one three times) run slower: the
                        // loop lives at the edge of what instruction fetch sustains.
                        constexpr int kTileUnroll = kSplitP ? 1 : 2;
#pragma unroll kTileUnroll
                        for (int local = 0; local < count; ++local) {
                            const uint32_t s_col = kColS + 64u * sbuf;  // S of this tile; P goes over the same columns
                            if ((e_cur >> (8 + wq)) & 1u) {
                                const uint2 w = lds_v2(a_row + ((e_cur & (kChunkTiles - 1)) << 3));
                                tmem_wait_ld();  // scores of this tile (requested at the end of the previous step)
                                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                                for (int j = 0; j < 32; ++j) {
                                    const uint32_t wsel = j < 16 ? w.x : w.y;
                                    const int b = (2 * j) & 31;
                                    sc[2 * j] = (wsel & (1u << b)) ? sc[2 * j] : -INFINITY;
                                    sc[2 * j + 1] = (wsel & (2u << b)) ? sc[2 * j + 1] : -INFINITY;
                                    mx[j & 3] = max3(mx[j & 3], sc[2 * j], sc[2 * j + 1]);
                                }
                                float neg_mc;
                                const float alpha = advance_max(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), neg_mc);
                                // packed two-lane fp32 arithmetic (one instruction per pair of scores) for the scaling and the row sum
                                const uint64_t c2 = pack_f32x2(c, c), neg_mc2 = pack_f32x2(neg_mc, neg_mc);
                                uint64_t ls2[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
                                for (int half = 0; half < 2; ++half) {
                                    uint32_t pk[16];
                                    [[maybe_unused]] uint32_t pk_lo[16];
#pragma unroll
                                    for (int j = 0; j < 16; ++j) {
                                        const int e = half * 32 + 2 * j;
                                        float x0, x1;
                                        unpack_f32x2(fma_f32x2(pack_f32x2(sc[e], sc[e + 1]), c2, neg_mc2), x0, x1);
                                        const float p0 = ex2_approx(x0);
                                        const float p1 = ex2_approx(x1);
                                        ls2[j & 3] = add_f32x2(ls2[j & 3], pack_f32x2(p0, p1));
                                        if constexpr (kSplitP) {
                                            const uint32_t h = pack_bf16x2(p0, p1);
                                            const float r0 = p0 - __uint_as_float(h << 16);
                                            const float r1 = p1 - __uint_as_float(h & 0xFFFF0000u);
                                            pk[j] = h;
                                            pk_lo[j] = pack_bf16x2(r0, r1);
                                        } else {
                                            pk[j] = kBf16 ? pack_bf16x2(p0, p1) : pack_f16x2(p0, p1);
                                        }
                                    }
                                    tmem_st16(tmem_lane + s_col + half * 16, pk);
                                    if constexpr (kSplitP) tmem_st16(tmem_lane + s_col + 32 + half * 16, pk_lo);
                                }
                                float l_even, l_odd;
                                unpack_f32x2(add_f32x2(add_f32x2(ls2[0], ls2[1]), add_f32x2(ls2[2], ls2[3])), l_even, l_odd);
                                l_run = fmaf(l_run, alpha, l_even + l_odd);

                                // rescale the O accumulator when some row of this warp moved its reference max
                                if (__any_sync(0xFFFFFFFFu, alpha != 1.f)) {
                                    // every P V issued so far must have landed in O: the newest one is tile g-1 (alpha != 1
                                    // implies that an earlier tile of this item kept something, so g >= 1)
                                    wait(a_bar_pv_done + 8 * ((g - 1) % kStages), ((g - 1) / kStages) & 1);
                                    tc_fence_after_sync();
                                    rescale_o_row(tmem_lane + kColO + 64u * ob, alpha);
                                }
                            } else {
                                // none of this warp's rows keeps a key of the tile: P = 0, nothing else changes
                                uint32_t z[32];
#pragma unroll
                                for (int j = 0; j < 32; ++j) z[j] = 0u;
                                tmem_st32(tmem_lane + s_col, z);
                                if constexpr (kSplitP) tmem_st32(tmem_lane + s_col + 32, z);
                            }
                            tmem_wait_st();
                            tc_fence_before_sync();
                            mbar_arrive_a(a_bar_p_full + 8 * sbuf);

                            ++g;
                            sbuf ^= 1u;
                            sphase ^= sbuf ^ 1u;  // flips when sbuf wraps to 0
                            // scores of the next tile into the registers that have just been used up
                            if (local + 1 < count) {
                                e_cur = lds_u16(a_entries + 2 * (local + 1));
                                wait(a_bar_s_full + 8 * sbuf, sphase);
                                tc_fence_after_sync();
                                if ((e_cur >> (8 + wq)) & 1u) {
                                    tmem_ld32_f32(tmem_lane + kColS + 64u * sbuf, &sc[0]);
                                    tmem_ld32_f32(tmem_lane + kColS + 64u * sbuf + 32, &sc[32]);
                                }
                            }
                        }
                    }
                    mbar_arrive_a(a_bar_slot_free + 8 * slot);  // this thread is done with the chunk
                    ++u;
                } while (!last);
                if (!ok) break;

                // ---- end of the item (or of the stream): hand the row sums to the epilogue warps ----------------
                // the buffers were last used by item r-2: its epilogue must have read them
                if (r >= 2) wait(a_bar_o_free + 8 * ob, ((r >> 1) - 1) & 1u);
                if (item >= 0) {
                    sts_f32(ct_a + offsetof(StreamCtrl, stat_inv_l) + (ob * kBlockM + stid) * 4, l_run > 0.f ? 1.f / l_run : 0.f);
                    const int row = item_row0(item) + stid;
                    if (args.save_lse && row < N) {
                        const float kLn2 = 0.6931471805599453f;
                        args.lse[static_cast<size_t>(item_bh(item)) * N + row] =
                            l_run > 0.f ? (fmaf(m_run, c, lg2_approx(l_run)) * kLn2) : -INFINITY;
                    }
                }
                if (stid == 0) sts_u32(ct_a + offsetof(StreamCtrl, stat_item) + 4 * ob, static_cast<uint32_t>(item));
                mbar_arrive_a(a_bar_stat_full + 8 * ob);
                if (item < 0) break;
                ++r;
            }
        } else {
            setmaxnreg_dec<kRegsOther>();
            if (warp < kNumStreams) {
                // ================================= MMA warp of one stream =================================
                // All 32 lanes run the control flow and the address arithmetic (values the compiler can prove to be
                // warp-uniform stay in uniform registers, where tcgen05.mma wants its operands); lane 0 alone issues.
                constexpr uint32_t kInFmt = kBf16 ? kFmtBF16 : kFmtF16;
                const uint32_t idesc_s = make_idesc(kInFmt, kInFmt, kMajorK, kMajorK, kBlockM, kBlockN, args.negate_q);
                constexpr uint32_t idesc_pv = make_idesc(kInFmt, kInFmt, kMajorK, kMajorMN, kBlockM, kHeadDim, 0);
                const uint32_t q_lo0 = smem_desc_sw128_lo(smem_u32(tl.q[0]));
                const uint32_t k_lo0 = smem_desc_sw128_lo(smem_u32(tl.k[0]));
                const uint32_t v_lo0 = smem_desc_sw128_lo(smem_u32(tl.v[0]));
                constexpr uint32_t kStageStep = kKVTileBytes >> 4;  // descriptor address units are 16 bytes
                constexpr uint32_t kQStep = kQTileBytes >> 4;
                constexpr uint32_t kHi = kSmemDescSw128Hi;

                uint32_t j = 0;    // tiles whose S has been issued
                uint32_t jp = 0;   // tiles whose P V has been issued; at most one behind j between tiles
                // per tile in flight (tile ordinal % 4, four bits each): 1 = first tile of its item (P V overwrites O),
                // 2 = last tile of its item (commit bar_o_full behind its P V), 4 = O accumulator of the item
                uint32_t tinfo = 0;
                auto issue_pv = [&]() {  // P V of tile jp
                    const uint32_t stage = jp % kStages;
                    const uint32_t pbuf = jp & 1u;
                    const uint32_t info = (tinfo >> (4 * (jp & 3u))) & 0xFu;
                    wait(a_bar_p_full + 8 * pbuf, (jp >> 1) & 1u);
                    tc_fence_after_sync();
                    const uint32_t v_lo = v_lo0 + stage * kStageStep;
                    const uint32_t p_addr = tmem + kColS + 64u * pbuf;
                    const uint32_t o_addr = tmem + kColO + 64u * ((info >> 2) & 1u);
                    const uint32_t acc = (info & 1u) ^ 1u;
                    if (lane == 0 && ok) {
                        // 16 keys = 16 rows of 128 bytes = 2048 bytes of V; 16 P values = 8 tensor-memory columns
                        mma_ts_lh(o_addr, p_addr, v_lo, kHi, idesc_pv, acc);
                        if constexpr (kSplitP) mma_ts_lh(o_addr, p_addr + 32, v_lo, kHi, idesc_pv, 1u);
#pragma unroll
                        for (int kk = 1; kk < kBlockN / 16; ++kk) {
                            mma_ts_lh(o_addr, p_addr + 8 * kk, v_lo + 128 * kk, kHi, idesc_pv, 1u);
                            if constexpr (kSplitP) mma_ts_lh(o_addr, p_addr + 32 + 8 * kk, v_lo + 128 * kk, kHi, idesc_pv, 1u);
                        }
                        mma_commit_a(a_bar_pv_done + 8 * stage);
                        if (info & 2u) mma_commit_a(a_bar_o_full + 8 * ((info >> 2) & 1u));
                    }
                    __syncwarp();
                    ++jp;
                };
                uint32_t u = 0;  // chunks consumed
                uint32_t r = 0;  // work items started
                bool in_item = false;
                uint32_t item_tiles = 0;
                while (ok) {
                    const uint32_t slot = u & 1u, spar = (u >> 1) & 1u;
                    if (!__all_sync(0xFFFFFFFFu, mbar_test_wait_a(a_bar_list_full + 8 * slot, spar))) {
                        // The descriptor is not there yet.  Before blocking, issue what is pending, so that the end
                        // of the previous item does not wait for the next one to be found.
                        while (jp < j && ok) issue_pv();
                        wait(a_bar_list_full + 8 * slot, spar);
                        if (!ok) break;
                    }
                    const uint32_t a_desc = a_desc0 + slot * 32u;
                    const int item = static_cast<int>(__shfl_sync(0xFFFFFFFFu, lds_u32(a_desc), 0));
                    if (item < 0) break;
                    const uint32_t meta = __shfl_sync(0xFFFFFFFFu, lds_u32(a_desc + 4), 0);
                    const uint32_t count = meta & 0xFFu;
                    const bool last = (meta >> 8) & 1u;
                    const uint32_t ob = r & 1u, rpar = (r >> 1) & 1u;
                    if (!in_item) {
                        in_item = true;
                        item_tiles = 0;
                        // O accumulator r % 2 was last used by item r-2: its epilogue must have read it.  That epilogue
                        // may itself be waiting for a P V that is still pending here (when item r-1 had no tiles), so
                        // what is pending is issued before this warp blocks.
                        if (r >= 2 && !__all_sync(0xFFFFFFFFu, mbar_test_wait_a(a_bar_o_free + 8 * ob, rpar ^ 1u))) {
                            while (jp < j && ok) issue_pv();
                            wait(a_bar_o_free + 8 * ob, rpar ^ 1u);
                        }
                    }
                    for (uint32_t i = 0; i < count && ok; ++i) {
                        // S(j) goes to buffer j % 2, whose previous tenant P(j-2) was read by P V(j-2), issued before.
                        const uint32_t stage = j % kStages;
                        const uint32_t sb = j & 1u;
                        if (item_tiles == 0) wait(a_bar_q + 8 * ob, rpar);
                        wait(a_bar_kv + 8 * stage, (j / kStages) & 1u);
                        tc_fence_after_sync();
                        const uint32_t q_lo = q_lo0 + ob * kQStep;
                        const uint32_t k_lo = k_lo0 + stage * kStageStep;
                        const uint32_t s_addr = tmem + kColS + 64u * sb;
                        if (lane == 0 && ok) {
                            // 16 elements of the contraction = 32 bytes inside the swizzled 128-byte row
                            mma_ss_lh(s_addr, q_lo, k_lo, kHi, idesc_s, 0u);
#pragma unroll
                            for (int kk = 1; kk < kHeadDim / 16; ++kk) mma_ss_lh(s_addr, q_lo + 2 * kk, k_lo + 2 * kk, kHi, idesc_s, 1u);
                            mma_commit_a(a_bar_s_full + 8 * sb);
                        }
                        __syncwarp();
                        const uint32_t info = (item_tiles == 0 ? 1u : 0u) | ((last && i + 1 == count) ? 2u : 0u) | (ob << 2);
                        tinfo = (tinfo & ~(0xFu << (4 * (j & 3u)))) | (info << (4 * (j & 3u)));
                        ++j;
                        ++item_tiles;
                        if (j - jp > 1) issue_pv();  // P V of the tile before the one just issued
                    }
                    if (lane == 0) mbar_arrive_a(a_bar_slot_free + 8 * slot);
                    __syncwarp();
                    ++u;
                    if (last) {
                        // ---- end of the item: its Q tile and (behind the last P V) its O accumulator are complete ----
                        if (item_tiles == 0) {
                            // nothing was issued for this item; its Q tile was requested all the same and must have
                            // landed before the buffer is declared free
                            wait(a_bar_q + 8 * ob, rpar);
                        }
                        bool commit_o_now = true;
                        if (item_tiles > 0 && (tinfo >> (4 * ((j - 1) & 3u)) & 2u) == 0u) {
                            // the final chunk was empty: the item's last tile is the newest one
                            if (jp < j) {
                                tinfo |= 2u << (4 * ((j - 1) & 3u));  // its P V is still to come: commit behind it
                                commit_o_now = false;
                            }
                        } else if (item_tiles > 0) {
                            commit_o_now = false;  // marked when the tile was issued
                        }
                        if (lane == 0 && ok) {
                            mma_commit_a(a_bar_q_free + 8 * ob);
                            if (commit_o_now) mma_commit_a(a_bar_o_full + 8 * ob);
                        }
                        __syncwarp();
                        in_item = false;
                        ++r;
                    }
                }
                while (jp < j && ok) issue_pv();
            } else {
                // ================================ loader warp of one stream ================================
                if (lane == 0) {
                    tma_prefetch_desc(&tmap_q);
                    tma_prefetch_desc(&tmap_k);
                    tma_prefetch_desc(&tmap_v);
                    if (args.mask_tma) tma_prefetch_desc(&tmap_m);
                }
                const uint32_t tail_bits = (N & 31) ? ((1u << (N & 31)) - 1u) : 0xFFFFFFFFu;
                const uint32_t q_a0 = smem_u32(tl.q[0]), k_a0 = smem_u32(tl.k[0]), v_a0 = smem_u32(tl.v[0]);
                const bool mask_tma = args.mask_tma != 0;

                // The strip of chunk `c` of a work item: rows row0..row0+127, words 16c..16c+15 of each row, zeros
                // outside the mask.  With a tensor map it is one TMA tile copy that completes on bar_strip_full;
                // otherwise the warp copies it with plain loads (and the caller arrives on the barrier).
                auto strip_tma = [&](uint32_t slot, int item, int c) {
                    if (lane == 0 && ok) {
                        const uint32_t bar = a_bar_strip_full + 8 * slot;
                        mbar_arrive_expect_tx_a(bar, kStripBytes);
                        tma_load_3d_a(a_strip0 + slot * kStripBytes, &tmap_m, bar, c * kChunkWords, item_row0(item), item_bh(item));
                    }
                    __syncwarp();
                };
                auto strip_copy = [&](uint32_t slot, int item, int c) {
                    const int bh = item_bh(item), row0 = item_row0(item);
                    const uint32_t* base = args.mask_packed + static_cast<size_t>(bh) * N * nw;
                    const uint32_t a_strip = a_strip0 + slot * kStripBytes;
#pragma unroll 1
                    for (int it = 0; it < kBlockM * kChunkWords / 32; it += 8) {
                        uint32_t val[8];
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const int i = (it + k) * 32 + lane;
                            const int row = row0 + (i >> 4), w = c * kChunkWords + (i & 15);
                            val[k] = (row < N && w < nw) ? ldg_u32(base + static_cast<size_t>(row) * nw + w) : 0u;
                            if (w == nw - 1) val[k] &= tail_bits;
                        }
#pragma unroll
                        for (int k = 0; k < 8; ++k) sts_u32(a_strip + ((it + k) * 32 + lane) * 4, val[k]);
                    }
                    __syncwarp();
                };
                // Non-empty tiles of the chunk whose strip sits in `slot`, written into the slot's descriptor; returns
                // their number.  Lane l looks at rows l, 32+l, 64+l, 96+l.
                auto list_from_strip = [&](uint32_t slot, int c) -> uint32_t {
                    const uint32_t a_strip = a_strip0 + slot * kStripBytes;
                    uint32_t grp[4];
#pragma unroll
                    for (int gq = 0; gq < 4; ++gq) {
                        const uint32_t a_row = a_strip + (gq * 32 + lane) * kStripRowBytes;
                        uint32_t mine = 0;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint4 x = lds_v4(a_row + 16 * k);
                            if ((x.x | x.y) != 0u) mine |= 1u << (2 * k);
                            if ((x.z | x.w) != 0u) mine |= 2u << (2 * k);
                        }
                        grp[gq] = __reduce_or_sync(0xFFFFFFFFu, mine);
                    }
                    const uint32_t any = grp[0] | grp[1] | grp[2] | grp[3];
                    if (lane < kChunkTiles && ((any >> lane) & 1u)) {
                        const uint32_t pos = __popc(any & ((1u << lane) - 1u));
                        const uint32_t flags = ((grp[0] >> lane) & 1u) | (((grp[1] >> lane) & 1u) << 1) |
                                               (((grp[2] >> lane) & 1u) << 2) | (((grp[3] >> lane) & 1u) << 3);
                        sts_u16(a_desc0 + slot * 32u + 8 + 2 * pos, (c * kChunkTiles + lane) | (flags << 8));
                    }
                    return __popc(any);
                };

                uint32_t u = 0;  // chunks published
                uint32_t j = 0;  // tiles of this stream whose K/V loads have been issued
                uint32_t r = 0;  // work items started
                bool pre = false;  // the strip of chunk u has already been requested (early, from the K/V loop)
                auto wait_slot_free = [&](uint32_t un) {
                    if (un >= kSlots) wait(a_bar_slot_free + 8 * (un & 1u), ((un >> 1) - 1) & 1u);
                };
                // K/V loads of the tiles listed in `slot` (for item bh), each as soon as its ring stage is free.  While
                // waiting, the strip of the following chunk (item_n, c_n) is requested as soon as its slot is free.
                auto issue_kv = [&](uint32_t slot, uint32_t count, int bh, bool have_n, int item_n, int c_n) {
                    const uint32_t a_entries = a_desc0 + slot * 32u + 8;
                    for (uint32_t i = 0; i < count && ok; ++i) {
                        const int t = static_cast<int>(__shfl_sync(0xFFFFFFFFu, lds_u16(a_entries + 2 * i), 0) & 0xFFu);
                        const uint32_t stage = j % kStages;
                        if (!kPlanned && mask_tma && have_n && !pre) {
                            const uint32_t un = u + 1;
                            if (un < kSlots ||
                                __all_sync(0xFFFFFFFFu, mbar_test_wait_a(a_bar_slot_free + 8 * (un & 1u), ((un >> 1) - 1) & 1u))) {
                                wait_slot_free(un);  // returns at once; every lane takes the acquire itself
                                strip_tma(un & 1u, item_n, c_n);
                                pre = true;
                            }
                        }
                        // Tile ordinal j uses stage j % 3 of the K/V ring.  A stage is reloaded when P V of its previous
                        // tenant (tile j-3) has completed, which also covers that tile's S.
                        if (j >= kStages) wait(a_bar_pv_done + 8 * stage, ((j / kStages) - 1) & 1u);
                        // after a failed wait nothing more is loaded: the buffers may still be in use
                        if (lane == 0 && ok) {
                            const uint32_t bar = a_bar_kv + 8 * stage;
                            mbar_arrive_expect_tx_a(bar, 2 * kKVTileBytes);
                            tma_load_3d_a(k_a0 + stage * kKVTileBytes, &tmap_k, bar, 0, t * kBlockN, bh);
                            tma_load_3d_a(v_a0 + stage * kKVTileBytes, &tmap_v, bar, 0, t * kBlockN, bh);
                        }
                        __syncwarp();
                        ++j;
                    }
                };
                auto publish = [&](uint32_t slot, int item, uint32_t count, bool last) {
                    if (lane == 0) {
                        sts_u32(a_desc0 + slot * 32u, static_cast<uint32_t>(item));
                        sts_u32(a_desc0 + slot * 32u + 4, count | (last ? 0x100u : 0u));
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive_a(a_bar_list_full + 8 * slot);
                    __syncwarp();
                };

                for (int item = first_item; item < total_items && ok; item += item_stride, ++r) {
                    const int bh = item_bh(item);
                    const int item_next = item + item_stride;
                    // Q tile into buffer r % 2, last used by item r-2: all its S products must be complete
                    if (r >= 2) wait(a_bar_q_free + 8 * (r & 1u), ((r >> 1) - 1) & 1u);
                    if (lane == 0 && ok) {
                        const uint32_t bar = a_bar_q + 8 * (r & 1u);
                        mbar_arrive_expect_tx_a(bar, kQTileBytes);
                        tma_load_3d_a(q_a0 + (r & 1u) * kQTileBytes, &tmap_q, bar, 0, item_row0(item), bh);
                    }
                    __syncwarp();
                    if constexpr (kPlanned) {
                        // the item's list was computed ahead: count word, then 16-bit entries in ascending tile order;
                        // one chunk descriptor per chunk that holds tiles (one empty descriptor for an empty item)
                        const uint32_t* plan = args.plan + static_cast<size_t>(item) * args.plan_stride;
                        const uint16_t* entries = reinterpret_cast<const uint16_t*>(plan + 1);
                        const uint32_t total = __shfl_sync(0xFFFFFFFFu, ldg_u32(plan), 0);
                        uint32_t pos = 0;
                        do {
                            const uint32_t slot = u & 1u;
                            wait_slot_free(u);
                            const uint32_t mine =
                                (lane < kChunkTiles && pos + lane < total) ? ldg_u16(entries + pos + lane) : 0xFFFFu;
                            const int c = static_cast<int>((__shfl_sync(0xFFFFFFFFu, mine, 0) & 0xFFu) / kChunkTiles);
                            const bool in_chunk = mine != 0xFFFFu && static_cast<int>((mine & 0xFFu) / kChunkTiles) == c;
                            const uint32_t count = __popc(__ballot_sync(0xFFFFFFFFu, in_chunk));
                            if (in_chunk) sts_u16(a_desc0 + slot * 32u + 8 + 2 * lane, mine);
                            if (count > 0) {
                                if (mask_tma) {
                                    strip_tma(slot, item, c);
                                } else {
                                    strip_copy(slot, item, c);
                                    if (lane == 0) mbar_arrive_a(a_bar_strip_full + 8 * slot);
                                }
                            } else if (lane == 0) {
                                mbar_arrive_a(a_bar_strip_full + 8 * slot);  // no strip: keep the barrier's phase in step
                            }
                            __syncwarp();
                            pos += count;
                            publish(slot, item, count, pos >= total);
                            issue_kv(slot, count, bh, false, 0, 0);
                            ++u;
                        } while (pos < total && ok);
                    } else {
                        for (int c = 0; c < num_chunks && ok; ++c) {
                            const uint32_t slot = u & 1u;
                            if (!pre) {
                                wait_slot_free(u);
                                if (mask_tma) strip_tma(slot, item, c);
                            }
                            pre = false;
                            if (mask_tma) {
                                wait(a_bar_strip_full + 8 * slot, (u >> 1) & 1u);
                            } else {
                                strip_copy(slot, item, c);
                                if (lane == 0) mbar_arrive_a(a_bar_strip_full + 8 * slot);
                                __syncwarp();
                            }
                            const uint32_t count = list_from_strip(slot, c);
                            const bool last = c + 1 == num_chunks;
                            publish(slot, item, count, last);
                            const bool have_n = !last || item_next < total_items;
                            issue_kv(slot, count, bh, have_n, last ? item_next : item, last ? 0 : c + 1);
                            ++u;
                        }
                    }
                }
                // end of the stream: a descriptor without a work item
                if (ok) {
                    wait_slot_free(u);
                    publish(u & 1u, -1, 0u, true);
                }
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
    if (warp == 0) tmem_dealloc(sm.tmem_base, kTmemCols);
}

}  // namespace sma
