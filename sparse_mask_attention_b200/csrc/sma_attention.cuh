// Fused sparse-mask attention forward for sm_100a.
//
// Computes, per (batch, head):  out = softmax(keep ? scale * q k^T : -inf) v   with the keep mask given
// as packed bits, fp32 accumulation, fp16 or bf16 inputs/outputs, and optionally the row-wise
// log-sum-exp.  Same result contract as the reference kernels sparse_attn_wmma_full_fp16
// (csrc/sparse_attention.cu:82-412) and sparse_attention_fwd_kernel<...,bf16> (:418-543): rows with no
// kept column give zeros, masked columns contribute exactly nothing.
//
// Structure: one persistent CTA of 384 threads per SM runs two independent "streams".  A stream owns one work
// item at a time — 128 consecutive query rows of one (batch, head) — walks its keys in chunks of 512 (eight
// 64-key tiles, sixteen packed-mask words per row) and visits only the tiles that hold at least one kept bit
// for those rows.  Warp roles:
//   * loader warp (1 per stream): per chunk it brings the 128 x 16-word strip of packed-mask words into
//     shared memory (one TMA tile copy, requested from inside the K loop of the chunk before; plain loads for
//     shapes a tensor map cannot describe), finds the non-empty tiles in it (or takes them from a list or from
//     occupancy bits computed ahead, kLists) and publishes a chunk descriptor.  Tile by tile it then requests K
//     (TMA, 128-byte swizzle, three-stage ring of its own) as soon as the stage is free, and, once the product
//     P V of three tiles back has released the tile's S/P buffer and V stage, requests V and issues
//         S[128x64]  = Q K^T   (operands in shared memory)
//     for the tile whose K landed a tile ago.  All lanes run the control flow, one elected lane issues.
//   * P V warp (1 per stream): walks the chunk descriptors and issues, as the softmax threads publish P,
//         O[128x64] += P V     (P from tensor memory, V MN-major from shared memory).
//     S runs two tiles ahead of the softmax threads (three S/P buffers) and Q is double-buffered, so the
//     first S products of the next item run while the previous item is still being finished; the next item's
//     first P V waits until the softmax warps have copied the previous item's O out of tensor memory.
//   * softmax warps (4 per stream): thread r owns query row r (tensor-memory lane r).  Per tile it reads
//     its S row with tcgen05.ld, applies its two mask words from the strip, updates the running max / sum
//     and writes P (16-bit) with tcgen05.st over the columns its S row came from.  At the end of an item it
//     goes straight on to the first tile of the next item (whose S is ready) and finishes the previous item
//     behind that tile, when its last P V has long completed: each warp reads its 32 rows of O, normalises,
//     rounds, stages them in shared memory and stores them with one TMA store.  On dense single-chunk work the
//     two softmax warps that share a scheduler (one of each stream) take turns at the exponentials.
// Work items are dealt to the CTAs round-robin, or, when the call provides a counter, taken from a queue shared by
// all CTAs (AttnArgs::work_counter).
// Hand-offs are mbarriers (TMA transaction counts, tcgen05.commit, thread arrivals); every wait is bounded.
// Orderings that hold because the tensor core runs a CTA's products in issue order and a buffer's two products come
// from warps that hand it to one another through those barriers:
//   * S(j) is issued only after P V(j-3) has completed (its commit is what the loader waits for): that product read
//     the previous P of buffer j%3 and the previous V of the stage.
//   * P(j) may overwrite S(j) in place: the softmax threads read S(j) before they write P(j).
#pragma once

#include <stddef.h>

#include <type_traits>

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
constexpr int kAttnThreads = 384;

// Tensor-memory layout of one stream (256 columns): three S/P buffers (64 columns each; P takes the first
// 32 of them, or all 64 as hi|lo halves for the bf16 split), then the O accumulator (64).
constexpr int kColsPerStream = 256;
constexpr int kSBuffers = 3;
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
    uint64_t bar_k[kStages];               // TMA: K tile landed
    uint64_t bar_v[kStages];               // TMA: V tile landed
    uint64_t bar_pv_done[kStages];         // tcgen05.commit: P V complete (the K/V stage is free again)
    uint64_t bar_s_full[kSBuffers];        // tcgen05.commit: S tile complete
    uint64_t bar_p_full[kSBuffers];        // 128 arrivals: P written over the S buffer (and O rescaled)
    uint64_t bar_list_full[kSlots];        // 1 arrival: chunk descriptor published
    uint64_t bar_strip_full[kSlots];       // TMA (or 1 arrival): the chunk's mask strip is in shared memory
    uint64_t bar_slot_free[kSlots];        // 129 arrivals: softmax threads and MMA warp left the chunk
    uint64_t bar_o_full;                   // tcgen05.commit: every P V of item r is complete (one phase per item)
    uint64_t bar_o_free;                   // 4 arrivals: the softmax warps have read O of item r
    ChunkDesc desc[kSlots];
};

struct AttnSmem {
    StreamTiles tiles[kNumStreams];
    alignas(1024) uint8_t staging[kNumStreams][4][kStageRowsOut * 128];  // one per softmax warp
    StreamCtrl ctrl[kNumStreams];
    uint32_t tmem_base;
    uint32_t abort_flag;  // raised by the first bounded wait that runs out
    uint32_t next_item;   // how many of the CTA's work items its two streams have taken
    // Turn-taking of the two softmax warps that share a warp scheduler (quadrant q of stream 0 and of stream 1), see
    // the exponentials in the softmax loop.  bar_turn[q][s]: 1 arrival, "warp (s, q) may run its exponentials".
    alignas(8) uint64_t bar_turn[4][kNumStreams];
    uint32_t turn_alive[4][kNumStreams];  // 0 once warp (s, q) has left the softmax loop for good
    uint32_t first_count[kNumStreams];    // tiles in the first chunk a stream's loader published (~0u: not yet known)
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

// One warp's share of the end of a work item: its 32 rows of the O accumulator (tensor-memory lanes of the
// warp's quadrant, 64 fp32 columns at o_addr) times the row's 1/sum, rounded to 16 bit, staged in the warp's
// shared-memory tile (128-byte swizzle, as the tensor map of `out` expects) and stored with one TMA store of
// 32 rows.  inv_l == 0 marks a row that keeps nothing: it is written as zeros whatever the accumulator holds.
// Arrives on bar_o_free once O is in registers.  Kept out of line: it runs once per work item, and the tile
// loop around its call site is sensitive to the size of its body.
template <bool kBf16, bool kFourD>
__device__ __noinline__ void finish_rows(uint32_t o_addr, float inv_l, uint32_t a_stage, uint32_t a_bar_o_free,
                                         const CUtensorMap* tmap_o, int row0, int h, int b, bool store) {
    const int lane = threadIdx.x & 31;
    // the previous store of this warp must have finished reading the staging tile
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
    // row `lane` of the warp occupies 128 bytes; its 16-byte chunk j sits at chunk position j ^ (lane & 7)
    const uint32_t a_row = a_stage + lane * 128;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        uint32_t o[32];
        tmem_ld32(o_addr + half * 32, o);
        tmem_wait_ld();
        if (half == 1) {
            // O is in registers (or already staged): the stream may overwrite it
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_a(a_bar_o_free);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float x = __uint_as_float(o[8 * q + 2 * j]) * inv_l;
                const float y = __uint_as_float(o[8 * q + 2 * j + 1]) * inv_l;
                pk[j] = inv_l == 0.f ? 0u : (kBf16 ? pack_bf16x2(x, y) : pack_f16x2(x, y));
            }
            sts_v4(a_row + (((4 * half + q) ^ (lane & 7)) << 4), make_uint4(pk[0], pk[1], pk[2], pk[3]));
        }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && store) {
        // (h, b) = (head, batch entry), or (batch*head, unused) with three-dimensional tensor maps
        if constexpr (kFourD)
            tma_store_4d(tmap_o, reinterpret_cast<const void*>(__cvta_shared_to_generic(a_stage)), 0, row0, h, b);
        else
            tma_store_3d(tmap_o, reinterpret_cast<const void*>(__cvta_shared_to_generic(a_stage)), 0, row0, h);
        tma_store_commit();
    }
}

struct AttnArgs {
    const uint32_t* mask_packed;
    const uint32_t* plan;   // tile lists computed ahead (sma_plan.cuh), or nullptr: the loader warps build them
    uint32_t plan_stride;   // words per work item in plan
    // Where the mask keeps anything, as written by the packing kernel next to the packed words (sma_pack.cuh): one
    // 16-bit word per 32 consecutive packed words, bit b = words 2b, 2b+1 of them hold a set bit.  When given (N a
    // multiple of 64, kListsFromBits kernel) the loader warps derive the tile lists from it.
    const uint16_t* tile_bits;
    // Work queue shared by all CTAs of the launch, or nullptr.  A 32-bit word that the kernel before this one in the
    // stream (packing or tile-list kernel of the same library call) has set to zero.  With it, a stream's first
    // work item is fixed (item = CTA + stream * grid) and every further one is taken from the queue, so CTAs whose
    // items hold fewer tiles, or whose SM runs faster, take more of them; without it item j belongs to CTA j % grid.
    uint32_t* work_counter;
    float* lse;
    int32_t BH;
    int32_t H;           // heads per batch entry (kFourD kernels)
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
// kLists  : where the loader warps take the tile lists from.  kListsFromStrips: they scan every chunk's mask strip.
//           kListsFromPlan: AttnArgs::plan.  kListsFromBits: AttnArgs::tile_bits.  In the last two, strips of chunks
//           without a tile are not loaded at all.  (One instantiation each: the kernel is sensitive to its code size.)
// kFourD  : the tensor maps of q, k, v, out are four-dimensional (64, N, H, B) and tiles are named (row, head, batch
//           entry), for layouts in which batch*head is not one dimension.  false: three-dimensional (64, N, B*H), tiles
//           named (row, batch*head), which every layout whose batch stride is H head strides admits (the dense one
//           among them).  An instantiation of its own: as a run-time switch in the loader warps the second form cost
//           the dense layout 1-6 % of the launch.
constexpr int kListsFromStrips = 0, kListsFromPlan = 1, kListsFromBits = 2;
template <bool kBf16, bool kSplitP, int kLists, bool kFourD>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                const __grid_constant__ CUtensorMap tmap_m, const AttnArgs args) {
    static_assert(kBf16 || !kSplitP, "the hi+lo split exists for bf16 only");
    static_assert(kNumStreams * kColsPerStream <= kTmemCols, "tensor memory over-committed");
    static_assert(kSlots == 2, "slot indices below are ordinal & 1");
    // register budgets: 384 threads start at 168 registers each; 256 * 216 + 128 * 72 = 384 * 168
    constexpr int kRegsSoftmax = 216;
    constexpr int kRegsOther = 72;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u));

    // Warpgroup 0 holds the P V warps (warps 0, 1) and the loader warps (2, 3) of the two streams, warpgroups
    // 1 and 2 are the softmax warps of stream 0 and 1.  warp % 4 decides the
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

    // ---- set-up: barriers (one thread per stream), tensor memory (one warp) --------------------------
    if ((wg == 1 || wg == 2) && (threadIdx.x & 127) == 0) {
        StreamCtrl& ct = sm.ctrl[wg - 1];
        for (int s = 0; s < 2; ++s) {
            mbar_init(&ct.bar_q[s], 1);
            mbar_init(&ct.bar_q_free[s], 1);
            mbar_init(&ct.bar_list_full[s], 1);
            mbar_init(&ct.bar_strip_full[s], 1);
            mbar_init(&ct.bar_slot_free[s], 129);
        }
        mbar_init(&ct.bar_o_full, 1);
        mbar_init(&ct.bar_o_free, 4);
        for (int s = 0; s < kSBuffers; ++s) {
            mbar_init(&ct.bar_s_full[s], 1);
            mbar_init(&ct.bar_p_full[s], 128);
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&ct.bar_k[s], 1);
            mbar_init(&ct.bar_v[s], 1);
            mbar_init(&ct.bar_pv_done[s], 1);
        }
        if (wg == 1) {
            sm.abort_flag = 0u;
            sm.next_item = 0u;
            sm.first_count[0] = sm.first_count[1] = ~0u;
            for (int q = 0; q < 4; ++q) {
                for (int st = 0; st < kNumStreams; ++st) {
                    mbar_init(&sm.bar_turn[q][st], 1);
                    sm.turn_alive[q][st] = 1u;
                }
                mbar_arrive_a(smem_u32(&sm.bar_turn[q][0]));  // stream 0 begins
            }
        }
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

    // Work items are dealt round-robin to the CTAs: item j belongs to CTA j % grid.  Inside the CTA the two
    // streams take its items one at a time as they become free (a counter in shared memory), so that a stream
    // which the warp schedulers favour, or whose items hold fewer tiles, does more of them.  Item j is
    // (row block, batch*head) with the later row blocks first: for causal-like masks they hold most work.
    auto item_bh = [&](int item) { return item % BH; };
    auto item_row0 = [&](int item) { return (args.num_q_tiles - 1 - item / BH) * kBlockM; };
    // q, k, v and out may have any batch, head and row strides; the packed mask, the log-sum-exp and the side-bands
    // are dense.  (head, batch entry) of a batch*head index for the four-dimensional maps, (batch*head, 0) otherwise.
    auto split_bh = [&](int bh, int& h, int& b) {
        b = kFourD ? bh / args.H : 0;
        h = bh - b * args.H;
    };
    bool ok = true;  // false once a bounded wait has run out; the same in all lanes of a warp
    volatile uint32_t* const abort_flag = &sm.abort_flag;
    // Bounded wait on an mbarrier phase.  After a failure nothing is waited for any more.  The lanes of a warp
    // test the barrier with one instruction and so take the fast path together; on the polling path they agree
    // on the outcome before they go on (the .sync.aligned instructions that follow need a converged warp).
    auto wait = [&](uint32_t bar, uint32_t parity) {
        if (ok && !mbar_try_wait_a(bar, parity)) ok = __all_sync(0xFFFFFFFFu, mbar_wait_poll(bar, parity, abort_flag));
    };

    {
        const int stream = wg == 0 ? (warp & 1) : (wg - 1);
        StreamTiles& tl = sm.tiles[stream];
        StreamCtrl& ct = sm.ctrl[stream];
        // 32-bit shared-memory addresses of the stream's barriers, descriptors and strips
        const uint32_t ct_a = smem_u32(&ct);
        const uint32_t a_bar_q = ct_a + offsetof(StreamCtrl, bar_q);
        const uint32_t a_bar_q_free = ct_a + offsetof(StreamCtrl, bar_q_free);
        const uint32_t a_bar_k = ct_a + offsetof(StreamCtrl, bar_k);
        const uint32_t a_bar_v = ct_a + offsetof(StreamCtrl, bar_v);
        const uint32_t a_bar_pv_done = ct_a + offsetof(StreamCtrl, bar_pv_done);
        const uint32_t a_bar_s_full = ct_a + offsetof(StreamCtrl, bar_s_full);
        const uint32_t a_bar_p_full = ct_a + offsetof(StreamCtrl, bar_p_full);
        const uint32_t a_bar_list_full = ct_a + offsetof(StreamCtrl, bar_list_full);
        const uint32_t a_bar_strip_full = ct_a + offsetof(StreamCtrl, bar_strip_full);
        const uint32_t a_bar_slot_free = ct_a + offsetof(StreamCtrl, bar_slot_free);
        const uint32_t a_bar_o_full = ct_a + offsetof(StreamCtrl, bar_o_full);
        const uint32_t a_bar_o_free = ct_a + offsetof(StreamCtrl, bar_o_free);
        const uint32_t a_desc0 = ct_a + offsetof(StreamCtrl, desc);
        const uint32_t a_strip0 = smem_u32(tl.strip[0]);
        const uint32_t tmem = sm.tmem_base + stream * kColsPerStream;

        if (wg != 0) {
            // =========================================== softmax warps ===========================================
            setmaxnreg_inc<kRegsSoftmax>();
            const int stid = threadIdx.x & 127;  // row inside the work item
            const uint32_t tmem_lane = tmem + (static_cast<uint32_t>(wq * 32) << 16);
            const float c = args.scale_log2e;

            // Turn-taking with the other stream's warp on this warp's scheduler (same lane quadrant), kTurns.  The
            // scheduler favours the warp with the lower index whenever both are ready, so on a dense mask stream 0 ran a
            // fifth faster than stream 1, took the same number of work items and then sat idle at the end of the kernel;
            // and the two warps tend to run their exponentials (special-function pipe) at the same time and their masking
            // (ALU pipe) at the same time.  Taking turns at the exponentials keeps the two streams in step and puts one
            // warp's masking and waiting under the other's exponentials: 8 % at the dense headline workload.  Where the
            // work items differ in length (block-sparse, causal masks) it costs 4-16 % instead, so the CTA decides once,
            // when both loaders have published their first chunk: turns are taken if work items are a single chunk
            // (N <= 512: few items per stream, where an uneven finish weighs most) and both first chunks are full of
            // tiles.  The loop exists in both forms (it is too sensitive to the size of its body to carry the other
            // form's code).
            // One turn exists per pair of warps: it sits, as a completed phase, on the barrier of the warp whose turn it
            // is; a warp takes its turn only while the other one is still in the loop and hands a turn it holds back
            // when it leaves, so nobody waits for a warp that is gone.
            auto softmax_role = [&](auto turns_tag) {
            constexpr bool kTurns = decltype(turns_tag)::value;
            uint32_t g = 0;                 // key tiles processed by this stream so far (drives the barrier phases)
            uint32_t sbuf = 0, sphase = 0;  // g % 3 and (g / 3) & 1
            uint32_t u = 0;                 // chunks consumed so far
            uint32_t r = 0;                 // work items started so far
            float sc[64] = {};              // scores of the tile in work
            // The end of an item (reading O, normalising, storing) is put off until the first tile of the next item
            // is done: by then the item's last P V has long completed, and the next item's S is waiting anyway.
            bool fin_on = false;   // an item is waiting to be finished
            float fin_inv_l = 0.f; // 1 / row sum of this thread's row of it (0: the row keeps nothing)
            int fin_item = 0;
            uint32_t fin_r = 0;    // its ordinal (phase of bar_o_full)
            const uint32_t a_stage = smem_u32(sm.staging[stream][wq]);
            const uint32_t a_my_turn = smem_u32(&sm.bar_turn[wq][stream]);
            const uint32_t a_other_turn = smem_u32(&sm.bar_turn[wq][stream ^ 1]);
            volatile uint32_t* const other_alive = &sm.turn_alive[wq][stream ^ 1];
            uint32_t turns = 0;  // turns taken so far (phase of bar_turn[wq][stream])
            // hands a turn this warp holds but does not need right now to the other warp
            auto pass_turn_on = [&]() {
                if constexpr (kTurns) {
                    if (*other_alive && __all_sync(0xFFFFFFFFu, mbar_test_wait_a(a_my_turn, turns & 1u))) {
                        ++turns;
                        if (lane == 0) mbar_arrive_a(a_other_turn);
                    }
                }
            };
            // A wait of a softmax warp for its own stream's progress.  That progress needs all four softmax warps of
            // the stream, and another one of them may be waiting for a turn that the other stream's warp holds while
            // it waits, in the same way, for a turn held here.  A warp therefore never sits on a turn while it waits:
            // whatever turn it holds, or is handed while it polls, goes straight back.
            auto swait = [&](uint32_t bar, uint32_t parity) {
                if constexpr (!kTurns) {
                    wait(bar, parity);
                    return;
                }
                if (!ok || mbar_try_wait_a(bar, parity)) return;
                const long long t0 = clock64();
                for (;;) {
                    pass_turn_on();
                    if (__all_sync(0xFFFFFFFFu, mbar_try_wait_suspend_a(bar, parity, 1000))) return;
                    const bool out_of_time = clock64() - t0 > kWaitLimitCycles;
                    if (__any_sync(0xFFFFFFFFu, *abort_flag != 0u || out_of_time)) {
                        if (out_of_time) {
                            *abort_flag = 1u;
                            atomicExch(&g_device_status, kDeviceTimeout);
                        }
                        ok = false;
                        return;
                    }
                }
            };
            auto finish_pending = [&]() {
                swait(a_bar_o_full, fin_r & 1u);
                tc_fence_after_sync();
                const int row0 = item_row0(fin_item) + wq * static_cast<int>(kStageRowsOut);
                int fin_h, fin_b;
                split_bh(item_bh(fin_item), fin_h, fin_b);
                finish_rows<kBf16, kFourD>(tmem_lane + kColO, fin_inv_l, a_stage, a_bar_o_free, &tmap_o, row0, fin_h, fin_b,
                                           row0 < N && ok);
                fin_on = false;
            };
            for (;;) {
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
                    swait(a_bar_list_full + 8 * slot, spar);
                    if (!ok) break;
                    const uint32_t a_desc = a_desc0 + slot * 32u;
                    item = static_cast<int>(lds_u32(a_desc));
                    if (item < 0) break;
                    const uint32_t meta = lds_u32(a_desc + 4);
                    const int count = static_cast<int>(meta & 0xFFu);
                    last = (meta >> 8) & 1u;
                    const uint32_t a_entries = a_desc + 8;
                    if (count > 0) {
                        swait(a_bar_strip_full + 8 * slot, spar);
                        const uint32_t a_row = a_strip0 + slot * kStripBytes + stid * kStripRowBytes;
                        // entry of the tile in work; `has`: this warp's 32 rows keep something in it
                        uint32_t e_cur = lds_u16(a_entries);
                        swait(a_bar_s_full + 8 * sbuf, sphase);
                        tc_fence_after_sync();
                        if ((e_cur >> (8 + wq)) & 1u) {
                            tmem_ld32_f32(tmem_lane + kColS + 64u * sbuf, &sc[0]);
                            tmem_ld32_f32(tmem_lane + kColS + 64u * sbuf + 32, &sc[32]);
                        }
                        // The tile loop is one rolled body (mask + maximum, then exponentials + P) on one register
                        // set, one tile per pass: the loop lives at the edge of what instruction fetch sustains, and
                        // every unrolled form that was tried ran slower.  A warp issues in order, so an instruction
                        // whose result the next one needs at once (a barrier test, the wait for a tensor-memory load or
                        // store) costs its whole latency, and with the two warps of a scheduler taking turns a warp's own
                        // chain is what a pass costs.  The loop therefore keeps such pairs apart: the barriers of the
                        // next tile's S and of this warp's turn are tested at the top and looked at after the masking,
                        // the next tile's scores are requested right after the exponentials, and the wait for the P
                        // stores with the arrival on bar_p_full moves to the top of the next pass.
                        uint32_t pub_bar = 0;  // bar_p_full of the tile whose P has been stored but not yet published
#pragma unroll 1
                        for (int local = 0; local < count; ++local) {
                            const uint32_t s_col = kColS + 64u * sbuf;  // S of this tile; P goes over the same columns
                            const uint32_t my_bar = a_bar_p_full + 8 * sbuf;
                            uint32_t nbuf = sbuf + 1, nphase = sphase;  // S/P buffer and phase of the tile after this one
                            if (nbuf == kSBuffers) {
                                nbuf = 0;
                                nphase ^= 1u;
                            }
                            const bool have_next = local + 1 < count;
                            const uint32_t e_next = have_next ? lds_u16(a_entries + 2 * (local + 1)) : 0u;
                            const uint32_t next_bar = a_bar_s_full + 8 * nbuf;
                            // scores of the next tile into the score registers (S runs two tiles ahead: normally complete)
                            auto request_next = [&](bool next_ready) {
                                if (have_next) {
                                    if (!next_ready) swait(next_bar, nphase);
                                    tc_fence_after_sync();
                                    if ((e_next >> (8 + wq)) & 1u) {
                                        tmem_ld32_f32(tmem_lane + kColS + 64u * nbuf, &sc[0]);
                                        tmem_ld32_f32(tmem_lane + kColS + 64u * nbuf + 32, &sc[32]);
                                    }
                                }
                            };
                            if ((e_cur >> (8 + wq)) & 1u) {
                                // (rows are 64 bytes apart, so the lanes of this load meet on two pairs of banks; with the
                                // strip in the 64-byte swizzle they spread over eight, and the launch took as long or longer)
                                const uint2 w = lds_v2(a_row + ((e_cur & (kChunkTiles - 1)) << 3));
                                const bool next_ready = have_next && mbar_test_wait_a(next_bar, nphase);
                                [[maybe_unused]] bool turn_ready = false;
                                if constexpr (kTurns) turn_ready = mbar_test_wait_a(a_my_turn, turns & 1u);
                                tmem_wait_ld();  // scores of this tile (requested during the previous pass)
                                if (pub_bar) {   // the previous tile's P stores have long landed
                                    tmem_wait_st();
                                    tc_fence_before_sync();
                                    mbar_arrive_a(pub_bar);
                                }
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
                                if constexpr (kTurns) {
                                    if (*other_alive) {
                                        if (!turn_ready) wait(a_my_turn, turns & 1u);
                                        ++turns;
                                    }
                                }
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
                                    if constexpr (kTurns) {
                                        // the other warp's turn, once half of this warp's exponentials are through: its
                                        // first ones then run under the rest of these, and the hand-over costs nothing
                                        // (handing over at the start, so that both run together, lost 12 %; at the end 1 %)
                                        if (half == 0) {
                                            __syncwarp();
                                            if (lane == 0) mbar_arrive_a(a_other_turn);
                                        }
                                    }
                                }
                                request_next(next_ready);
                                float l_even, l_odd;
                                unpack_f32x2(add_f32x2(add_f32x2(ls2[0], ls2[1]), add_f32x2(ls2[2], ls2[3])), l_even, l_odd);
                                l_run = fmaf(l_run, alpha, l_even + l_odd);

                                // rescale the O accumulator when some row of this warp moved its reference max
                                if (__any_sync(0xFFFFFFFFu, alpha != 1.f)) {
                                    // every P V issued so far must have landed in O: the newest one is tile g-1 (alpha != 1
                                    // implies that an earlier tile of this item kept something, so g >= 1), whose P was
                                    // published at the top of this pass or when its chunk ended
                                    swait(a_bar_pv_done + 8 * ((g - 1) % kStages), ((g - 1) / kStages) & 1);
                                    tc_fence_after_sync();
                                    rescale_o_row(tmem_lane + kColO, alpha);
                                }
                            } else {
                                // none of this warp's rows keeps a key of the tile: P = 0, nothing else changes; a turn at
                                // the exponentials that this warp holds goes straight back
                                if (pub_bar) {
                                    tmem_wait_st();
                                    tc_fence_before_sync();
                                    mbar_arrive_a(pub_bar);
                                }
                                pass_turn_on();
                                uint32_t z[32];
#pragma unroll
                                for (int j = 0; j < 32; ++j) z[j] = 0u;
                                tmem_st32(tmem_lane + s_col, z);
                                if constexpr (kSplitP) tmem_st32(tmem_lane + s_col + 32, z);
                                request_next(false);
                            }
                            pub_bar = my_bar;
                            if (fin_on) finish_pending();  // the previous item, behind this item's first tile

                            ++g;
                            sbuf = nbuf;
                            sphase = nphase;
                            e_cur = e_next;
                        }
                        // the chunk's last tile is published here
                        tmem_wait_st();
                        tc_fence_before_sync();
                        mbar_arrive_a(pub_bar);
                    }
                    mbar_arrive_a(a_bar_slot_free + 8 * slot);  // this thread is done with the chunk
                    ++u;
                } while (!last);
                if (!ok) break;

                // ---- end of the item (or of the stream) ---------------------------------------------------------
                if (fin_on) finish_pending();  // an item without tiles in between, or the end of the stream
                if (item < 0) break;
                {
                    const int row = item_row0(item) + stid;
                    if (args.save_lse && row < N) {
                        const float kLn2 = 0.6931471805599453f;
                        args.lse[static_cast<size_t>(item_bh(item)) * N + row] =
                            l_run > 0.f ? (fmaf(m_run, c, lg2_approx(l_run)) * kLn2) : -INFINITY;
                    }
                }
                fin_on = true;
                fin_inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
                fin_item = item;
                fin_r = r;
                ++r;
            }
            // leaving for good: a turn this warp holds goes back to the other one
            __syncwarp();
            if (lane == 0) {
                if constexpr (kTurns) {
                    sm.turn_alive[wq][stream] = 0u;
                    __threadfence_block();
                    if (mbar_test_wait_a(a_my_turn, turns & 1u)) mbar_arrive_a(a_other_turn);
                }
                tma_store_wait_all();
            }
            };
            bool take_turns = false;
            {
                volatile uint32_t* const fc = sm.first_count;
                const long long t0 = clock64();
                while ((fc[0] == ~0u || fc[1] == ~0u) && *abort_flag == 0u && clock64() - t0 < kWaitLimitCycles) __nanosleep(64);
                take_turns = __all_sync(0xFFFFFFFFu, num_chunks == 1 && fc[0] == kChunkTiles && fc[1] == kChunkTiles);
            }
            if (take_turns)
                softmax_role(std::true_type{});
            else
                softmax_role(std::false_type{});
        } else {
            setmaxnreg_dec<kRegsOther>();
            const bool leader = elect_one();  // the lane that issues this warp's single-thread instructions
            const int leader_lane = __ffs(__ballot_sync(0xFFFFFFFFu, leader)) - 1;
            // shared by the two helper warps of a stream: tcgen05.mma operand descriptors
            constexpr uint32_t kInFmt = kBf16 ? kFmtBF16 : kFmtF16;
            constexpr uint32_t kStageStep = kKVTileBytes >> 4;  // descriptor address units are 16 bytes
            constexpr uint32_t kQStep = kQTileBytes >> 4;
            constexpr uint32_t kHi = kSmemDescSw128Hi;
            static_assert(kStages == kSBuffers, "tile j uses K/V stage j % 3 and S/P buffer j % 3: one counter serves both");
            if (warp < kNumStreams) {
                // ================================= P V warp of one stream =================================
                // All 32 lanes run the control flow and the address arithmetic (values the compiler can prove to be
                // warp-uniform stay in uniform registers, where tcgen05.mma wants its operands); an elected lane issues.
                // The warp walks the chunk descriptors and issues O (+)= P V tile by tile, as the softmax threads
                // publish P.  (S = Q K^T is issued by the loader warp: one thread issuing both took longer per tile
                // than the softmax threads need, and every tcgen05.mma costs its issuer some 60-80 cycles.)
                constexpr uint32_t idesc_pv = make_idesc(kInFmt, kInFmt, kMajorK, kMajorMN, kBlockM, kHeadDim, 0);
                const uint32_t v_lo0 = smem_desc_sw128_lo(smem_u32(tl.v[0]));
                const uint32_t o_addr = tmem + kColO;
                uint32_t pb = 0, pphase = 0;   // (tiles done) % 3 and (tiles done / 3) & 1
                uint32_t u = 0;  // chunks consumed
                uint32_t r = 0;  // work items started
                uint32_t item_tiles = 0;  // tiles issued for the item in work
                while (ok) {
                    const uint32_t slot = u & 1u, spar = (u >> 1) & 1u;
                    wait(a_bar_list_full + 8 * slot, spar);
                    if (!ok) break;
                    const uint32_t a_desc = a_desc0 + slot * 32u;
                    const int item = static_cast<int>(__shfl_sync(0xFFFFFFFFu, lds_u32(a_desc), 0));
                    if (item < 0) break;
                    const uint32_t meta = __shfl_sync(0xFFFFFFFFu, lds_u32(a_desc + 4), 0);
                    const uint32_t count = meta & 0xFFu;
                    const bool last = (meta >> 8) & 1u;
                    for (uint32_t i = 0; i < count && ok; ++i) {
                        wait(a_bar_p_full + 8 * pb, pphase);
                        // the item's first product overwrites O: the epilogue must have read the previous item's
                        if (item_tiles == 0 && r >= 1) wait(a_bar_o_free, (r - 1) & 1u);
                        wait(a_bar_v + 8 * pb, pphase);  // V landed (requested when P V of tile j-3 completed)
                        tc_fence_after_sync();
                        const uint32_t v_lo = v_lo0 + pb * kStageStep;
                        const uint32_t p_addr = tmem + kColS + 64u * pb;
                        const uint32_t acc = item_tiles == 0 ? 0u : 1u;
                        if (leader && ok) {
                            // 16 keys = 16 rows of 128 bytes = 2048 bytes of V; 16 P values = 8 tensor-memory columns
                            mma_ts_lh(o_addr, p_addr, v_lo, kHi, idesc_pv, acc);
                            if constexpr (kSplitP) mma_ts_lh(o_addr, p_addr + 32, v_lo, kHi, idesc_pv, 1u);
#pragma unroll
                            for (int kk = 1; kk < kBlockN / 16; ++kk) {
                                mma_ts_lh(o_addr, p_addr + 8 * kk, v_lo + 128 * kk, kHi, idesc_pv, 1u);
                                if constexpr (kSplitP) mma_ts_lh(o_addr, p_addr + 32 + 8 * kk, v_lo + 128 * kk, kHi, idesc_pv, 1u);
                            }
                            mma_commit_a(a_bar_pv_done + 8 * pb);
                            if (last && i + 1 == count) mma_commit_a(a_bar_o_full);
                        }
                        __syncwarp();
                        ++item_tiles;
                        if (++pb == kSBuffers) {
                            pb = 0;
                            pphase ^= 1u;
                        }
                    }
                    if (leader) mbar_arrive_a(a_bar_slot_free + 8 * slot);
                    __syncwarp();
                    ++u;
                    if (last) {
                        // ---- end of the item.  bar_o_full has one phase per item; when the item's last tile was not
                        // in its final chunk (or the item has no tile at all) the commit comes here.  It may only move
                        // on once the epilogue has passed the previous item's phase.
                        if (count == 0) {
                            if (item_tiles == 0 && r >= 1) wait(a_bar_o_free, (r - 1) & 1u);
                            if (leader && ok) mma_commit_a(a_bar_o_full);
                            __syncwarp();
                        }
                        item_tiles = 0;
                        ++r;
                    }
                }
            } else {
                // ======================== loader warp of one stream (also issues S = Q K^T) ========================
                if (leader) {
                    tma_prefetch_desc(&tmap_q);
                    tma_prefetch_desc(&tmap_k);
                    tma_prefetch_desc(&tmap_v);
                    if (args.mask_tma) tma_prefetch_desc(&tmap_m);
                }
                const uint32_t tail_bits = (N & 31) ? ((1u << (N & 31)) - 1u) : 0xFFFFFFFFu;
                const uint32_t q_a0 = smem_u32(tl.q[0]), k_a0 = smem_u32(tl.k[0]), v_a0 = smem_u32(tl.v[0]);
                const bool mask_tma = args.mask_tma != 0;
                const uint32_t idesc_s = make_idesc(kInFmt, kInFmt, kMajorK, kMajorK, kBlockM, kBlockN, args.negate_q);
                const uint32_t q_lo0 = smem_desc_sw128_lo(q_a0);
                const uint32_t k_lo0 = smem_desc_sw128_lo(k_a0);

                // The strip of chunk `c` of a work item: rows row0..row0+127, words 16c..16c+15 of each row, zeros
                // outside the mask.  With a tensor map it is one TMA tile copy that completes on bar_strip_full;
                // otherwise the warp copies it with plain loads (and the caller arrives on the barrier).
                auto strip_tma = [&](uint32_t slot, int item, int c) {
                    if (leader && ok) {
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
                // their number.  The strip is read as 16 runs of 512 consecutive bytes (eight rows), lane l taking the
                // l-th 16-byte piece of a run: row 8 i + l / 4, key tiles 2 (l % 4) and 2 (l % 4) + 1.  (Consecutive
                // lanes on consecutive pieces: a lane per row, 64 bytes apart, put four lanes on every bank.)
                auto list_from_strip = [&](uint32_t slot, int c) -> uint32_t {
                    const uint4* strip = reinterpret_cast<const uint4*>(tl.strip[slot]);
                    uint32_t grp[4];
#pragma unroll
                    for (int g = 0; g < 4; ++g) {  // one group of 32 rows = four runs
                        uint4 x[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k) x[k] = strip[(4 * g + k) * 32 + lane];
                        const uint32_t lo = x[0].x | x[0].y | x[1].x | x[1].y | x[2].x | x[2].y | x[3].x | x[3].y;
                        const uint32_t hi = x[0].z | x[0].w | x[1].z | x[1].w | x[2].z | x[2].w | x[3].z | x[3].w;
                        const uint32_t mine = ((lo != 0u ? 1u : 0u) | (hi != 0u ? 2u : 0u)) << (2 * (lane & 3));
                        grp[g] = __reduce_or_sync(0xFFFFFFFFu, mine);
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
                uint32_t j = 0;  // tiles of this stream whose K load has been issued
                uint32_t ls = 0, lph = 0;  // j % 3 and (j / 3) & 1
                uint32_t js = 0;           // tiles whose V load and S product have been issued (js == j or j - 1)
                uint32_t ss = 0, sph = 0;  // js % 3 and (js / 3) & 1
                uint32_t r = 0;  // work items started
                bool pre = false;  // the strip of chunk u has already been requested (early, from the K loop)
                // The K and V tiles of a key tile travel separately, because they are needed at different times.  S(j)
                // should be complete two tiles before the softmax threads get to tile j, so K(j) is requested as soon as
                // its ring stage is free, which is when S(j-3) has completed.  V(j) is needed only after the softmax
                // threads have finished tile j; its stage and the S/P buffer j % 3 become free together, when P V(j-3)
                // completes, and at that moment this warp requests V(j) and issues S(j), whose K tile landed a tile
                // ago.  Loads therefore never sit on the path from "P(j-3) published" to "S(j) complete".
                // What the V load and the S product of the tile whose K was requested last need to know:
                bool pend = false;        // such a tile exists (then js == j - 1)
                bool pend_first = false;  // first tile of its item: the item's Q tile must have landed
                bool pend_last = false;   // last tile of its item: behind it the Q buffer is free again
                uint32_t pend_r = 0;      // ordinal of its item
                int pend_t = 0, pend_h = 0, pend_b = 0;  // its key tile, head and batch entry
                int cur_h = 0, cur_b = 0;                // head and batch entry of the item whose tiles are being requested
                bool pend_first_of_item = false;  // the next tile to be loaded is the first of its item
                auto issue_s = [&]() {  // V load and S product of the pending tile (S/P buffer and ring stage ss)
                    // buffer and stage are free when P V of their previous tenant (tile js-3) has completed: that product
                    // read P(js-3) and V(js-3)
                    if (js >= kStages) wait(a_bar_pv_done + 8 * ss, sph ^ 1u);
                    // after a failed wait nothing more is loaded or issued: the buffers may still be in use
                    if (leader && ok) {
                        const uint32_t bar = a_bar_v + 8 * ss;
                        mbar_arrive_expect_tx_a(bar, kKVTileBytes);
                        if constexpr (kFourD)
                            tma_load_4d_a(v_a0 + ss * kKVTileBytes, &tmap_v, bar, 0, pend_t * kBlockN, pend_h, pend_b);
                        else
                            tma_load_3d_a(v_a0 + ss * kKVTileBytes, &tmap_v, bar, 0, pend_t * kBlockN, pend_h);
                    }
                    __syncwarp();
                    const uint32_t qb = pend_r & 1u;
                    if (pend_first) wait(a_bar_q + 8 * qb, (pend_r >> 1) & 1u);
                    wait(a_bar_k + 8 * ss, sph);
                    tc_fence_after_sync();
                    const uint32_t q_lo = q_lo0 + qb * kQStep;
                    const uint32_t k_lo = k_lo0 + ss * kStageStep;
                    const uint32_t s_addr = tmem + kColS + 64u * ss;
                    if (leader && ok) {
                        // 16 elements of the contraction = 32 bytes inside the swizzled 128-byte row
                        mma_ss_lh(s_addr, q_lo, k_lo, kHi, idesc_s, 0u);
#pragma unroll
                        for (int kk = 1; kk < kHeadDim / 16; ++kk) mma_ss_lh(s_addr, q_lo + 2 * kk, k_lo + 2 * kk, kHi, idesc_s, 1u);
                        mma_commit_a(a_bar_s_full + 8 * ss);
                        if (pend_last) mma_commit_a(a_bar_q_free + 8 * qb);
                    }
                    __syncwarp();
                    ++js;
                    if (++ss == kSBuffers) {
                        ss = 0;
                        sph ^= 1u;
                    }
                    pend = false;
                };
                // the same, if nothing it needs is still outstanding (never blocks)
                auto try_issue_s = [&]() {
                    if (pend && __all_sync(0xFFFFFFFFu, mbar_test_wait_a(a_bar_k + 8 * ss, sph) &&
                                                            (js < kStages || mbar_test_wait_a(a_bar_pv_done + 8 * ss, sph ^ 1u))))
                        issue_s();
                };
                // Waits until the consumers have left the chunk that used the slot of chunk `un`.  They cannot leave a
                // chunk whose last S product is still pending here, so that one is issued before this warp blocks.
                auto wait_slot_free = [&](uint32_t un) {
                    if (un < kSlots) return;
                    const uint32_t bar = a_bar_slot_free + 8 * (un & 1u), par = ((un >> 1) - 1) & 1u;
                    if (pend && !__all_sync(0xFFFFFFFFu, mbar_test_wait_a(bar, par))) issue_s();
                    wait(bar, par);
                };
                // K loads of the tiles listed in `slot` (of the item in work: cur_h, cur_b), each as soon as its ring stage is free, and behind
                // each the V load and the S product of the tile before.  While waiting, the strip of the following chunk
                // (item_n, c_n) is requested as soon as its slot is free.
                auto issue_kv = [&](uint32_t slot, uint32_t count, bool last, bool have_n, int item_n, int c_n) {
                    const uint32_t a_entries = a_desc0 + slot * 32u + 8;
                    for (uint32_t i = 0; i < count && ok; ++i) {
                        const int t = static_cast<int>(__shfl_sync(0xFFFFFFFFu, lds_u16(a_entries + 2 * i), 0) & 0xFFu);
                        if (kLists == kListsFromStrips && mask_tma && have_n && !pre) {
                            const uint32_t un = u + 1;
                            if (un < kSlots ||
                                __all_sync(0xFFFFFFFFu, mbar_test_wait_a(a_bar_slot_free + 8 * (un & 1u), ((un >> 1) - 1) & 1u))) {
                                strip_tma(un & 1u, item_n, c_n);
                                pre = true;
                            }
                        }
                        // Tile ordinal j uses stage j % 3 of the K ring, free when S(j-3) has completed (issued two steps ago)
                        if (j >= kStages) wait(a_bar_s_full + 8 * ls, lph ^ 1u);
                        if (leader && ok) {
                            const uint32_t bar = a_bar_k + 8 * ls;
                            mbar_arrive_expect_tx_a(bar, kKVTileBytes);
                            if constexpr (kFourD)
                                tma_load_4d_a(k_a0 + ls * kKVTileBytes, &tmap_k, bar, 0, t * kBlockN, cur_h, cur_b);
                            else
                                tma_load_3d_a(k_a0 + ls * kKVTileBytes, &tmap_k, bar, 0, t * kBlockN, cur_h);
                        }
                        __syncwarp();
                        if (pend) issue_s();
                        pend = true;
                        pend_first = i == 0 && pend_first_of_item;
                        pend_last = last && i + 1 == count;
                        pend_r = r;
                        pend_t = t;
                        pend_h = cur_h;
                        pend_b = cur_b;
                        if (i == 0) pend_first_of_item = false;
                        ++j;
                        if (++ls == kStages) {
                            ls = 0;
                            lph ^= 1u;
                        }
                    }
                };
                auto publish = [&](uint32_t slot, int item, uint32_t count, bool last) {
                    if (leader) {
                        sts_u32(a_desc0 + slot * 32u, static_cast<uint32_t>(item));
                        sts_u32(a_desc0 + slot * 32u + 4, count | (last ? 0x100u : 0u));
                        if (u == 0) sm.first_count[stream] = item >= 0 ? count : 0u;  // the softmax warps' cue
                    }
                    __syncwarp();
                    if (leader) mbar_arrive_a(a_bar_list_full + 8 * slot);
                    __syncwarp();
                };
                // next work item of this CTA for this stream, or -1 when all have been taken
                auto take_item = [&]() -> int {
                    uint32_t k = 0;
                    long long it;
                    if (args.work_counter != nullptr) {
                        if (leader) k = atomicAdd(args.work_counter, 1u);
                        k = __shfl_sync(0xFFFFFFFFu, k, leader_lane);
                        it = 2ll * gridDim.x + k;
                    } else {
                        if (leader) k = atomicAdd(&sm.next_item, 1u);
                        k = __shfl_sync(0xFFFFFFFFu, k, leader_lane);
                        it = static_cast<long long>(blockIdx.x) + static_cast<long long>(k) * gridDim.x;
                    }
                    return it < total_items ? static_cast<int>(it) : -1;
                };
                // with a work queue the first item of a stream is fixed, so that nothing waits for an atomic's round
                // trip through global memory at the start; later items are taken one item ahead
                auto first_item = [&]() -> int {
                    if (args.work_counter == nullptr) return take_item();
                    const long long it = static_cast<long long>(blockIdx.x) + static_cast<long long>(stream) * gridDim.x;
                    return it < total_items ? static_cast<int>(it) : -1;
                };
                // Side-band bits of chunks c0..c0+3 of a work item, as this lane sees them: lane l looks at rows l, 32+l,
                // 64+l, 96+l of the item; raw[g] byte cc = tile bits of chunk c0+cc in row 32g+l.  Only issues the loads.
                auto load_bits = [&](int item, int c0, uint32_t (&raw)[4]) {
                    const int bh = item_bh(item), row0 = item_row0(item);
                    const size_t row_words0 = (static_cast<size_t>(bh) * N + row0) * nw;
#pragma unroll
                    for (int g = 0; g < 4; ++g) raw[g] = 0u;
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        const int c = c0 + cc;
                        const int need = min(kChunkWords, nw - c * kChunkWords);  // words of the chunk in a row
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if (c < num_chunks && row0 + 32 * g + lane < N) {
                                const size_t widx = row_words0 + static_cast<size_t>(32 * g + lane) * nw + c * kChunkWords;
                                const uint32_t in_block = static_cast<uint32_t>(widx) & 31u;
                                uint32_t v = ldg_u16(args.tile_bits + (widx >> 5));
                                // the chunk's words may run into the next block of 32
                                if (in_block + need > 32u) v |= static_cast<uint32_t>(ldg_u16(args.tile_bits + (widx >> 5) + 1)) << 16;
                                raw[g] |= ((v >> (in_block >> 1)) & ((1u << ((need + 1) >> 1)) - 1u)) << (8 * cc);
                            }
                        }
                    }
                };
                // The same bits when every row has a whole number of chunks (N a multiple of 512): a row's bits are then
                // one byte per chunk, the item's 128 rows are contiguous, and lane l takes rows 4l..4l+3.  Returns byte
                // cc = tile bits of chunk c0+cc OR-ed over those four rows.  Covers one or two chunks per row and multiples
                // of four (aligned 32-bit loads); other lengths use load_bits.
                const bool row_bytes = (nw % kChunkWords) == 0 && (num_chunks <= 2 || (num_chunks & 3) == 0);
                auto lane_bits = [&](int item, int c0) -> uint32_t {
                    const uint8_t* base = reinterpret_cast<const uint8_t*>(args.tile_bits) +
                                          (static_cast<size_t>(item_bh(item)) * N + item_row0(item) + 4 * lane) * num_chunks + c0;
                    if (num_chunks == 1) {
                        uint32_t x = ldg_u32(reinterpret_cast<const uint32_t*>(base));
                        x |= x >> 16;
                        return (x | (x >> 8)) & 0xFFu;
                    }
                    if (num_chunks == 2) {
                        const uint32_t x = ldg_u32(reinterpret_cast<const uint32_t*>(base)) | ldg_u32(reinterpret_cast<const uint32_t*>(base + 4));
                        return (x | (x >> 16)) & 0xFFFFu;
                    }
                    return ldg_u32(reinterpret_cast<const uint32_t*>(base)) | ldg_u32(reinterpret_cast<const uint32_t*>(base + num_chunks)) |
                           ldg_u32(reinterpret_cast<const uint32_t*>(base + 2 * num_chunks)) |
                           ldg_u32(reinterpret_cast<const uint32_t*>(base + 3 * num_chunks));
                };
                constexpr bool from_bits = kLists == kListsFromBits;
                int item_next = first_item();
                uint32_t mine_next = 0u;  // lane_bits of the first four chunks of item_next, requested an item ahead
                if (from_bits && row_bytes && item_next >= 0) mine_next = lane_bits(item_next, 0);
                while (item_next >= 0 && ok) {
                    const int item = item_next;
                    item_next = take_item();  // taken one item ahead: its first mask strip is requested early
                    const int bh = item_bh(item);
                    split_bh(bh, cur_h, cur_b);
                    // Q tile into buffer r % 2, last used by item r-2: all its S products must be complete
                    if (r >= 2) wait(a_bar_q_free + 8 * (r & 1u), ((r >> 1) - 1) & 1u);
#ifdef SMA_WAIT_TEST_BUILD
                    // test build only: on request, the Q tile of work item 0 (whichever stream of CTA 0 takes it) is never
                    // asked for, nothing completes its barrier, and this warp's wait for it runs out
                    const bool withheld = g_test_withhold_q_load != 0 && item == 0;
#else
                    constexpr bool withheld = false;
#endif
                    if (leader && ok && !withheld) {
                        const uint32_t bar = a_bar_q + 8 * (r & 1u);
                        mbar_arrive_expect_tx_a(bar, kQTileBytes);
                        if constexpr (kFourD)
                            tma_load_4d_a(q_a0 + (r & 1u) * kQTileBytes, &tmap_q, bar, 0, item_row0(item), cur_h, cur_b);
                        else
                            tma_load_3d_a(q_a0 + (r & 1u) * kQTileBytes, &tmap_q, bar, 0, item_row0(item), cur_h);
                    }
                    __syncwarp();
                    pend_first_of_item = true;
                    bool item_has_tiles = false, last_marked = false;
                    if constexpr (from_bits) {
                        // The packing kernel left one bit per (mask row, 64-key tile); OR-ed over the rows of each of the
                        // item's four row groups they are its tile lists.  Chunks without a tile are passed over; when the
                        // item's final chunk is one of those, an empty descriptor closes the item.
                        uint32_t mine = mine_next;
                        if (row_bytes && item_next >= 0) mine_next = lane_bits(item_next, 0);
                        for (int c0 = 0; c0 < num_chunks && ok; c0 += 4) {
                            uint32_t raw[4];  // per row group: byte cc = tile bits of chunk c0 + cc
                            if (row_bytes) {
                                if (c0 > 0) mine = lane_bits(item, c0);
                                // rows 32g..32g+31 sit in lanes 8g..8g+7
                                const uint32_t red = __reduce_or_sync(0xFFu << (lane & 24), mine);
#pragma unroll
                                for (int g = 0; g < 4; ++g) raw[g] = __shfl_sync(0xFFFFFFFFu, red, 8 * g);
                            } else {
                                load_bits(item, c0, raw);
                                try_issue_s();
#pragma unroll
                                for (int g = 0; g < 4; ++g) raw[g] = __reduce_or_sync(0xFFFFFFFFu, raw[g]);
                            }
#pragma unroll 1
                            for (int cc = 0; cc < 4 && c0 + cc < num_chunks && ok; ++cc) {
                                const int c = c0 + cc;
                                const uint32_t g0 = (raw[0] >> (8 * cc)) & 0xFFu, g1 = (raw[1] >> (8 * cc)) & 0xFFu,
                                               g2 = (raw[2] >> (8 * cc)) & 0xFFu, g3 = (raw[3] >> (8 * cc)) & 0xFFu;
                                const uint32_t any = g0 | g1 | g2 | g3;
                                if (any == 0u) continue;
                                const uint32_t slot = u & 1u;
                                wait_slot_free(u);
                                if (mask_tma) strip_tma(slot, item, c);
                                if (lane < kChunkTiles && ((any >> lane) & 1u)) {
                                    const uint32_t pos = __popc(any & ((1u << lane) - 1u));
                                    const uint32_t flags = ((g0 >> lane) & 1u) | (((g1 >> lane) & 1u) << 1) |
                                                           (((g2 >> lane) & 1u) << 2) | (((g3 >> lane) & 1u) << 3);
                                    sts_u16(a_desc0 + slot * 32u + 8 + 2 * pos, (c * kChunkTiles + lane) | (flags << 8));
                                }
                                if (!mask_tma) {
                                    strip_copy(slot, item, c);
                                    if (leader) mbar_arrive_a(a_bar_strip_full + 8 * slot);
                                }
                                __syncwarp();
                                const bool last = c + 1 == num_chunks;
                                publish(slot, item, __popc(any), last);
                                // (requesting the next descriptor's strip from inside the K loop, as the strip-scanning
                                // loader does, was measured here too and gained nothing)
                                issue_kv(slot, __popc(any), last, false, 0, 0);
                                item_has_tiles = true;
                                last_marked = last;
                                ++u;
                            }
                        }
                        if (ok && !last_marked) {
                            const uint32_t slot = u & 1u;
                            wait_slot_free(u);
                            if (leader) mbar_arrive_a(a_bar_strip_full + 8 * slot);  // no strip: keep the barrier's phase in step
                            __syncwarp();
                            publish(slot, item, 0u, true);
                            ++u;
                        }
                    } else if constexpr (kLists == kListsFromPlan) {
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
                                    if (leader) mbar_arrive_a(a_bar_strip_full + 8 * slot);
                                }
                            } else if (leader) {
                                mbar_arrive_a(a_bar_strip_full + 8 * slot);  // no strip: keep the barrier's phase in step
                            }
                            __syncwarp();
                            pos += count;
                            const bool last = pos >= total;
                            publish(slot, item, count, last);
                            issue_kv(slot, count, last, false, 0, 0);
                            item_has_tiles |= count > 0;
                            last_marked = last && count > 0;
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
                            try_issue_s();
                            if (mask_tma) {
                                wait(a_bar_strip_full + 8 * slot, (u >> 1) & 1u);
                            } else {
                                strip_copy(slot, item, c);
                                if (leader) mbar_arrive_a(a_bar_strip_full + 8 * slot);
                                __syncwarp();
                            }
                            const uint32_t count = list_from_strip(slot, c);
                            const bool last = c + 1 == num_chunks;
                            publish(slot, item, count, last);
                            const bool have_n = !last || item_next >= 0;
                            issue_kv(slot, count, last, have_n, last ? item_next : item, last ? 0 : c + 1);
                            item_has_tiles |= count > 0;
                            last_marked = last && count > 0;
                            ++u;
                        }
                    }
                    // ---- end of the item on the S side: behind its last S product its Q buffer is free again.  When that
                    // tile could not be marked (the final chunk was empty) the commit comes here, behind everything issued.
                    if (!last_marked) {
                        if (pend) issue_s();
                        // an item without tiles never waited for its Q tile, which must have landed before the buffer
                        // is declared free
                        if (!item_has_tiles) wait(a_bar_q + 8 * (r & 1u), (r >> 1) & 1u);
                        if (leader && ok) mma_commit_a(a_bar_q_free + 8 * (r & 1u));
                        __syncwarp();
                    }
                    ++r;
                }
                if (pend && ok) issue_s();
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
