/*
 * sma.h — C ABI of libsma_b200.so: bit-packing of boolean attention masks and the fused
 * sparse-mask attention forward pass for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers and sizes, launches asynchronously on the stream it
 * is given (a cudaStream_t passed as void*; NULL = the legacy default stream), never synchronises,
 * never allocates device memory and never throws or exits: it returns SMA_OK or a negative
 * sma_status code.  The device that owns the pointers must be current when the call is made.
 *
 * The entry points replace the launch interface of the reference project
 * (csrc/sparse_attention.h in xgbj/sparse-mask-attention); each declaration cites the reference
 * symbol it stands in for.
 */
#ifndef SMA_B200_H_
#define SMA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMA_ABI_VERSION 4

typedef enum sma_status {
    SMA_OK                 = 0,
    SMA_ERR_NULL_POINTER   = -1,  /* a required pointer is NULL                                   */
    SMA_ERR_BAD_SHAPE      = -2,  /* B, H or N < 1, or B*H*N*N does not fit the index range        */
    SMA_ERR_BAD_HEAD_DIM   = -3,  /* D != 64 (the only head size the reference kernels support)    */
    SMA_ERR_BAD_DTYPE      = -4,  /* dtype is neither SMA_DTYPE_F16 nor SMA_DTYPE_BF16             */
    SMA_ERR_MISALIGNED     = -5,  /* q/k/v/out not 16-byte aligned, mask_packed/lse not 4-byte     */
    SMA_ERR_BAD_SCALE      = -6,  /* scale is zero, NaN or infinite                                */
    SMA_ERR_SEQ_TOO_LONG   = -7,  /* N above SMA_MAX_SEQ_LEN                                       */
    SMA_ERR_CUDA           = -8,  /* a CUDA runtime/driver call failed; see sma_last_cuda_error()  */
    SMA_ERR_WRONG_ARCH     = -9,  /* current device is not compute capability 10.x                 */
    SMA_ERR_DEVICE_TIMEOUT = -10, /* a kernel gave up on a bounded wait (reported by sma_device_status) */
    SMA_ERR_BAD_VARIANT    = -11, /* unknown value in sma_attention_params.variant                 */
    SMA_ERR_WORKSPACE_TOO_SMALL = -12, /* workspace smaller than sma_attention_workspace_bytes()  */
    SMA_ERR_STATIC_WORKSPACE_EXCEEDED = -13, /* shape needs more than SMA_STATIC_WORKSPACE_BYTES   */
    SMA_ERR_BAD_STRIDE     = -14  /* a stride is not a positive multiple of 8 elements, or strides where none are taken */
} sma_status;

typedef enum sma_dtype {
    SMA_DTYPE_F16  = 0,  /* IEEE binary16 */
    SMA_DTYPE_BF16 = 1   /* bfloat16      */
} sma_dtype;

/* Largest sequence length sma_attention_fwd accepts (the kernel keeps one occupancy bit per
 * 64-key tile in shared memory). */
#define SMA_MAX_SEQ_LEN 16384

/* Kernel variants (sma_attention_params.variant).
 * The probabilities P are rounded to the 16-bit type of q/k/v before the P*V product (the tensor
 * core needs both operands in one format).  fp16 keeps 11 significant bits.  For bf16 the default
 * splits P into hi + lo (two bf16 numbers, two products per tile), which keeps 16 bits and meets the
 * same tolerance as fp16; SMA_VARIANT_BF16_SINGLE_P rounds P once to bf16 (8 bits): faster, but a
 * few outputs per million can miss |err| <= 2e-3 + 1e-2*|ref| when a row keeps only 2-3 columns. */
#define SMA_VARIANT_DEFAULT        0
#define SMA_VARIANT_BF16_SINGLE_P  1

/*
 * Argument block of the attention forward pass.
 * Replaces: struct SparseAttentionParams, csrc/sparse_attention.h:12-38 (the reference declares
 * stride fields that it never sets nor reads; tensors are dense row-major here as there).
 *
 *   q, k, v, out : [B, H, N, D] row-major, D == 64, element type given by dtype
 *   mask_packed  : [B, H, N, ceil(N/32)] uint32; bit j of word w of a row = keep(col 32*w + j)
 *   lse          : [B, H, N] float32 or NULL; written only if save_lse != 0:
 *                  log(sum_j exp(scale * q.k_j)) over kept j, -inf for a row with no kept column
 *   out rows with no kept column are written as zeros.
 */
typedef struct sma_attention_params {
    const void*     q;
    const void*     k;
    const void*     v;
    const uint32_t* mask_packed;
    void*           out;
    float*          lse;
    int32_t         B;
    int32_t         H;
    int32_t         N;
    int32_t         D;
    float           scale;     /* softmax scale, normally 1/sqrt(D); may be negative, not 0 */
    int32_t         dtype;     /* sma_dtype                                                  */
    int32_t         save_lse;  /* reference: SparseAttentionParams::is_training              */
    int32_t         variant;   /* SMA_VARIANT_*                                              */
    /*
     * Strides of q, k, v and out in ELEMENTS: {batch, head, row}; the 64 values of a row are always contiguous.
     * All three zero (what a zero-initialised struct gives) = the dense [B, H, N, 64] layout.  Otherwise every stride
     * must be positive and a multiple of 8 elements (16 bytes): a packed projection [B, N, 3, H, 64] viewed as
     * q[b, h, n, :] is {3*N*H*64, 64, 3*H*64}, no copy needed.  Reference: SparseAttentionParams::stride_qb ...
     * stride_on (csrc/sparse_attention.h:29-33), which its kernels never read (its binding copies to the dense layout
     * first, csrc/binding.cpp:28-33).  mask_packed and lse are always dense.  The forward entry points honour the
     * strides; sma_attention_bwd takes dense tensors only (SMA_ERR_BAD_STRIDE otherwise).
     */
    int64_t         q_strides[3];
    int64_t         k_strides[3];
    int64_t         v_strides[3];
    int64_t         out_strides[3];
} sma_attention_params;

/* Returns SMA_ABI_VERSION of the loaded library. */
int sma_abi_version(void);

/* Human-readable text for a status code (static storage). */
const char* sma_strerror(int status);

/* cudaError_t value of the last failing CUDA call seen by this thread (0 if none). */
int sma_last_cuda_error(void);

/*
 * Pack a boolean mask into bits.
 * Replaces: pack_mask_bits(), csrc/sparse_attention.h:67-72 (kernel csrc/sparse_attention.cu:549-568,
 * launcher :603-610) and the allocation-free part of pack_mask() in csrc/binding.cpp:49-66.
 *
 *   mask   : [B, H, N, N] bytes, any non-zero byte = keep
 *   packed : [B, H, N, ceil(N/32)] uint32, every word is written; bit j of word w = mask[.., 32*w+j],
 *            bits for columns >= N are zero.
 */
int sma_pack_mask(const uint8_t* mask, uint32_t* packed, int32_t B, int32_t H, int32_t N, void* stream);

/*
 * Fused masked attention forward: out = softmax(keep ? scale*q.k^T : -inf) * v.
 * Replaces: sparse_attention_fwd_fp16() and sparse_attention_fwd_bf16(),
 * csrc/sparse_attention.h:45-54 (launchers csrc/sparse_attention.cu:574-601) and the marshalling in
 * forward(), csrc/binding.cpp:9-47.
 */
int sma_attention_fwd(const sma_attention_params* params, void* stream);

/*
 * Mask packing and the forward pass behind one call: packs `mask` into params->mask_packed (the caller's buffer,
 * [B, H, N, ceil(N/32)] uint32, every word written) and runs sma_attention_fwd on it, both on `stream`, in that
 * order.  Same results as the two calls made one after the other; what it saves is one trip through the caller's
 * foreign-function layer per step, which for a headline-sized batch costs as much host time as the kernels run.
 * Replaces: the pair pack_mask() + forward() that the reference's Python layer issues for every call of
 * sparse_attention() (python/sparse_attention.py:139-146, 64 and 170-171; csrc/binding.cpp:9-66).
 * tile_bits: NULL, or a device buffer of sma_tile_bits_bytes(B, H, N) bytes; with it the two kernels work as
 * sma_pack_mask_tiles and sma_attention_fwd_tiles do (below).  A buffer given for a shape that has no side-band
 * (sma_tile_bits_bytes() == 0, or a mask that is not 32-byte aligned) is ignored.
 * work_counter: NULL, or 4 bytes of device memory (4-byte aligned, contents do not matter) that belong to this
 * call until its kernels have run.  With it the attention kernel's CTAs take their work items (blocks of 128 query
 * rows) from one queue instead of a fixed share each, which evens out masks whose row blocks keep different
 * numbers of key tiles (block-sparse, causal): the packing kernel zeroes the word, the attention kernel counts in
 * it.  Results do not depend on it.
 */
int sma_sparse_attention_fwd(const sma_attention_params* params, const uint8_t* mask, void* tile_bits,
                             void* work_counter, void* stream);

/*
 * Packing that also tells the attention kernel where the mask keeps anything.
 * The attention kernel visits only the 64-key tiles in which some query row of a 128-row block keeps a key; with
 * sma_attention_fwd its loader warps find them by reading the packed words again, one warp per block.  The packing
 * kernel already holds every packed word in a register, so here each of its warps also writes one 16-bit word of
 * occupancy for the 32 packed words it produces: bit b = packed words 2b and 2b+1 of the 32 (the 64 keys of one tile
 * in one mask row) hold a set bit.  tile_bits[i] covers packed words 32i..32i+31 of the flat [B, H, N, N/32] array;
 * the buffer has sma_tile_bits_bytes(B, H, N) bytes, 1/64 of the packed mask.  sma_attention_fwd_tiles derives its
 * tile lists from it (a few hundred bytes per block of query rows instead of the block's packed rows), loads the
 * packed words only of chunks of 512 keys that hold a tile, and so also serves long, sparse sequences without the
 * tile-list kernel and workspace of sma_attention_fwd_planned.
 * Exists for N a multiple of 64 (sma_tile_bits_bytes() returns 0 otherwise: SMA_ERR_BAD_SHAPE), a mask that is
 * 32-byte aligned and a tile_bits buffer that is 16-byte aligned (SMA_ERR_MISALIGNED otherwise).  `tile_bits` must describe `params->mask_packed` as it is when the
 * attention kernel runs: a caller who edits the packed words afterwards uses sma_attention_fwd.
 * Results are those of sma_pack_mask and sma_attention_fwd, bit for bit.
 * No counterpart in the reference, whose kernel tests every tile of every row block for emptiness itself
 * (csrc/sparse_attention.cu:236-252); the packed words are the reference's (csrc/sparse_attention.cu:549-568).
 */
size_t sma_tile_bits_bytes(int32_t B, int32_t H, int32_t N);
int sma_pack_mask_tiles(const uint8_t* mask, uint32_t* packed, void* tile_bits, int32_t B, int32_t H, int32_t N,
                        void* stream);
int sma_attention_fwd_tiles(const sma_attention_params* params, const void* tile_bits, void* stream);

/*
 * The same forward pass for long, sparse sequences, with a workspace.
 * sma_attention_fwd finds the non-empty 64-key tiles of each block of 128 query rows inside the attention
 * kernel, one warp reading that block's packed-mask rows; beyond a thousand keys or so, and when most tiles are
 * empty, that search costs more than the attention itself.  Here a small kernel computes all tile lists first,
 * with the whole GPU, into `workspace` (device memory, 16-byte aligned, at least
 * sma_attention_workspace_bytes(B, H, N) bytes, owned by the caller and free again when the call's work on the
 * stream has finished).  The workspace's last 16 bytes hold the word through which the attention kernel's CTAs
 * share out the work items (see work_counter of sma_sparse_attention_fwd).  Results are identical to
 * sma_attention_fwd.
 * Replaces: the tile skip of the reference kernels, which test every tile of every row block in the kernel
 * (csrc/sparse_attention.cu:243-252, 485-487).
 */
size_t sma_attention_workspace_bytes(int32_t B, int32_t H, int32_t N);  /* 0 for a shape that is rejected */
int sma_attention_fwd_planned(const sma_attention_params* params, void* workspace, size_t workspace_bytes,
                              void* stream);

/*
 * Backward pass: dq, dk, dv (same shape, layout and dtype as q, k, v) from dout, the upstream gradient of out.
 * `params` is the forward call's (q, k, v, mask_packed, B, H, N, D = 64, scale, dtype) with out and lse holding
 * what the forward pass wrote with save_lse = 1; the attention probabilities are recomputed from lse, and key
 * blocks in which a block of query rows keeps nothing are skipped as in the forward pass.
 * `workspace`: sma_attention_bwd_workspace_bytes(B, H, N) bytes of device memory, 16-byte aligned (the row sums
 * dout . out and an fp32 accumulator for dq; contents on entry do not matter).  dq is summed by fp32 atomics over
 * the key blocks, so its last bits can differ from run to run; dk and dv are deterministic.
 * Replaces: sparse_attention_bwd_bf16(params, dout, dq, dk, dv, stream), csrc/sparse_attention.h:57-64, which the
 * reference declares but never defines, and sparse_attn_cuda.backward(dout, q, k, v, out, lse, mask_packed, dq, dk,
 * dv, scale), which its autograd function calls (python/sparse_attention.py:90-94) but its extension does not
 * export; the gradient it computes is the one of the PyTorch branch there (python/sparse_attention.py:96-111).
 */
size_t sma_attention_bwd_workspace_bytes(int32_t B, int32_t H, int32_t N);
int sma_attention_bwd(const sma_attention_params* params, const void* dout, void* dq, void* dk, void* dv,
                      void* workspace, size_t workspace_bytes, void* stream);

/*
 * sma_attention_fwd_planned without a workspace argument, for callers that must not allocate device memory and
 * have none to spare: code that runs after a service has frozen its memory budget, inside a latency-critical
 * loop where cudaMalloc's device-wide synchronisation is not acceptable, or behind a plug-in interface that
 * hands the library tensors but no allocator.  This entry point has no counterpart in the reference project.
 *
 * The tile lists go into an array of SMA_STATIC_WORKSPACE_BYTES that is part of the library image: every GPU on
 * which the library is used holds that much memory from then until the process exits, whether or not this
 * function is ever called.  The call allocates nothing (no cudaMalloc, no cudaFree, no allocating library
 * routine); inputs and outputs are the caller's, as for the other entry points.
 *
 *   - Shapes whose tile lists need more than SMA_STATIC_WORKSPACE_BYTES (sma_attention_workspace_bytes(B, H, N)
 *     minus the 16 bytes of its work-queue word tells how much) are refused with
 *     SMA_ERR_STATIC_WORKSPACE_EXCEEDED; nothing is launched.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current).  Make that first call outside any stream capture.
 *   - All calls on a device share the one array, and each call overwrites what the previous one left there.  Two
 *     calls whose kernels can run at the same time on one device (different streams, or different host threads
 *     without ordering between their streams) race on it and give wrong results: keep such calls on one stream,
 *     or order them with events.
 * Results are identical to sma_attention_fwd.
 */
#define SMA_STATIC_WORKSPACE_BYTES (1u << 20)
int sma_attention_fwd_static_workspace(const sma_attention_params* params, void* stream);

/*
 * Reads (and clears) the device-side status word of the current device.  Kernels of this library
 * bound every wait they perform; a wait that runs out stores SMA_ERR_DEVICE_TIMEOUT there and the
 * kernel returns after releasing what it holds.  This call synchronises the device.
 * Returns SMA_OK, SMA_ERR_DEVICE_TIMEOUT, or SMA_ERR_CUDA.
 */
int sma_device_status(void);

#ifdef __cplusplus
}
#endif
#endif /* SMA_B200_H_ */
