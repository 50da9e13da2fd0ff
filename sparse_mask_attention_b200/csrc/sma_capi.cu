// Host side of libsma_b200.so: the extern "C" entry points declared in include/sma.h.
// Validates arguments, builds the TMA tensor maps and launches the sm_100a kernels on the caller's
// stream.  The whole library is this one translation unit.
#include "../../include/sma.h"

#include <cmath>
#include <cstring>
#include <mutex>
#include <utility>

#include "sma_attention.cuh"
#include "sma_common.cuh"
#include "sma_pack.cuh"
#include "sma_plan.cuh"
#include "sma_backward.cuh"

namespace {

thread_local int tls_cuda_error = 0;

inline bool cuda_ok(cudaError_t e) {
    if (e == cudaSuccess) return true;
    tls_cuda_error = static_cast<int>(e);
    (void)cudaGetLastError();  // clear the sticky-free error so later calls start clean
    return false;
}

constexpr int kMaxDevices = 64;

struct DeviceInfo {
    bool checked = false;
    bool is_sm100 = false;
    int sm_count = 0;
    bool attn_attr_set[18] = {};
    bool bwd_attr_set[2] = {};
};
DeviceInfo g_dev[kMaxDevices];
std::mutex g_dev_mutex;

// Looks up (once per device) whether the current device can run sm_100a code.
int current_device_info(DeviceInfo** out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return SMA_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return SMA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.checked) {
        int major = 0;
        if (!cuda_ok(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev))) return SMA_ERR_CUDA;
        if (!cuda_ok(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev))) return SMA_ERR_CUDA;
        d.is_sm100 = (major == 10);
        d.checked = true;
    }
    *out = &d;
    return d.is_sm100 ? SMA_OK : SMA_ERR_WRONG_ARCH;
}

// cuTensorMapEncodeTiled, fetched through the runtime so that the library has no link-time
// dependency on libcuda.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Makes the device's primary context current to the calling host thread.  Runtime calls do that by themselves, the
// driver call that encodes a tensor map does not: in a thread that has made no context-binding runtime call yet (a
// framework's worker thread entering the library for the first time) it fails with CUDA_ERROR_INVALID_CONTEXT.
bool bind_primary_context() {
    int dev = 0;
    return cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess;
}

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Tensor maps are pure functions of (base address, shape, element type, box), and encoding one costs the host
// about a microsecond; a step of a training or serving loop passes the same few tensors again and again.  Each
// host thread therefore keeps the maps it encoded last in a small direct-mapped table.
struct TensorMapKey {
    const void* base;
    int32_t bh;
    int32_t n;
    int32_t kind;  // box rows for q/k/v/out maps (fp16), + 1000 for bf16, -1 for the packed-mask map
    int64_t stride[3] = {0, 0, 0};  // element strides {batch, head, row} of the strided maps, zero otherwise
    int32_t heads = 0;              // heads per batch entry of the strided maps
    bool operator==(const TensorMapKey& o) const {
        return base == o.base && bh == o.bh && n == o.n && kind == o.kind && stride[0] == o.stride[0] &&
               stride[1] == o.stride[1] && stride[2] == o.stride[2] && heads == o.heads;
    }
};
struct TensorMapSlot {
    TensorMapKey key = {nullptr, 0, 0, 0, {0, 0, 0}, 0};
    CUtensorMap map;
};
constexpr int kTensorMapSlots = 64;
thread_local TensorMapSlot tls_tensor_maps[kTensorMapSlots];

TensorMapSlot& tensor_map_slot(const TensorMapKey& key) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(key.base);
    const size_t h = (a >> 8) * 0x9E3779B97F4A7C15ull + static_cast<size_t>(key.kind) * 0x632BE5ABull +
                     static_cast<size_t>(key.n) * 31u + static_cast<size_t>(key.bh);
    return tls_tensor_maps[(h >> 20) % kTensorMapSlots];
}

// Element strides {batch, head, row} of one of q/k/v/out: the caller's, or those of the dense [B, H, N, 64] layout
// when all three are zero.  false: not positive multiples of 8 elements.
bool resolve_strides(const int64_t (&given)[3], int H, int N, int64_t (&out)[3]) {
    if (given[0] == 0 && given[1] == 0 && given[2] == 0) {
        out[0] = static_cast<int64_t>(H) * N * 64;
        out[1] = static_cast<int64_t>(N) * 64;
        out[2] = 64;
        return true;
    }
    for (int i = 0; i < 3; ++i) {
        if (given[i] <= 0 || (given[i] & 7) != 0 || given[i] >= (1ll << 38)) return false;
        out[i] = given[i];
    }
    return true;
}

// Tensor map over a 16-bit tensor addressed as [B][H][N][64] with element strides {batch, head, row}; one box =
// box_rows x 64 elements of one (batch, head), written to shared memory with the 128-byte swizzle.  Rows past N
// read as zeros.  four_d: dimensions (64, N, H, B); otherwise (64, N, B*H), for layouts whose batch stride is H head
// strides.
int make_strided_tensor_map(CUtensorMap* map, const void* base, int B, int H, int N, const int64_t (&stride)[3],
                            int box_rows, bool bf16, bool four_d) {
    TensorMapKey key = {base, B * H, N, (four_d ? 4000 : 2000) + box_rows + (bf16 ? 1000 : 0), {stride[0], stride[1], stride[2]}, H};
    TensorMapSlot& slot = tensor_map_slot(key);
    if (slot.key == key) {
        *map = slot.map;
        return SMA_OK;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return SMA_ERR_CUDA;
    const cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(four_d ? H : B * H),
                                static_cast<cuuint64_t>(B)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(stride[2]) * 2, static_cast<cuuint64_t>(stride[1]) * 2,
                                   static_cast<cuuint64_t>(stride[0]) * 2};
    const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
    const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
    auto encode_once = [&]() {
        return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, four_d ? 4 : 3,
                      const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    CUresult r = encode_once();
    if (r == CUDA_ERROR_INVALID_CONTEXT && bind_primary_context()) r = encode_once();
    if (r != CUDA_SUCCESS) {
        tls_cuda_error = static_cast<int>(cudaErrorInvalidValue);
        return SMA_ERR_CUDA;
    }
    slot.key = key;
    slot.map = *map;
    return SMA_OK;
}

// Tensor map over a [BH, N, 64] row-major 16-bit tensor; one box = box_rows x 64 elements of one
// (batch, head), written to shared memory with the 128-byte swizzle.  Rows past N read as zeros.
// (The backward pass, which takes dense tensors only.)
int make_qkv_tensor_map(CUtensorMap* map, const void* base, int BH, int N, int box_rows, bool bf16) {
    const TensorMapKey key = {base, BH, N, box_rows + (bf16 ? 1000 : 0)};
    TensorMapSlot& slot = tensor_map_slot(key);
    if (slot.key == key) {
        *map = slot.map;
        return SMA_OK;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return SMA_ERR_CUDA;
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(BH)};
    const cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(N) * 128};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    auto encode_once = [&]() {
        return encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                      const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    CUresult r = encode_once();
    if (r == CUDA_ERROR_INVALID_CONTEXT && bind_primary_context()) r = encode_once();
    if (r != CUDA_SUCCESS) {
        tls_cuda_error = static_cast<int>(cudaErrorInvalidValue);
        return SMA_ERR_CUDA;
    }
    slot.key = key;
    slot.map = *map;
    return SMA_OK;
}

// Tensor map over the backward pass's fp32 dQ accumulator [BH, N, 64]; one box = 128 rows x 32 columns (128 bytes),
// 128-byte swizzle: the tile one half of the backward kernel's compute warps adds to it per step.
int make_dq_accum_tensor_map(CUtensorMap* map, const float* base, int BH, int N) {
    const TensorMapKey key = {base, BH, N, 5000};
    TensorMapSlot& slot = tensor_map_slot(key);
    if (slot.key == key) {
        *map = slot.map;
        return SMA_OK;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return SMA_ERR_CUDA;
    const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(BH)};
    const cuuint64_t strides[2] = {256, static_cast<cuuint64_t>(N) * 256};
    const cuuint32_t box[3] = {32, 128, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    auto encode_once = [&]() {
        return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, elem_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    CUresult r = encode_once();
    if (r == CUDA_ERROR_INVALID_CONTEXT && bind_primary_context()) r = encode_once();
    if (r != CUDA_SUCCESS) {
        tls_cuda_error = static_cast<int>(cudaErrorInvalidValue);
        return SMA_ERR_CUDA;
    }
    slot.key = key;
    slot.map = *map;
    return SMA_OK;
}

// Whether the packed mask [BH, N, nw] can be described by a tensor map: 16-byte aligned base and row pitch.
bool mask_has_tensor_map(const uint32_t* base, int N) {
    const int nw = (N + 31) / 32;
    return (reinterpret_cast<uintptr_t>(base) & 15u) == 0 && (nw % 4) == 0;
}

// Tensor map over the packed mask [BH, N, nw] (32-bit words); one box = the 16 words x 128 rows a work item
// needs for one chunk of 512 keys, dense in shared memory (64 bytes per row).  Words past nw and rows past N
// read as zeros.
int make_mask_tensor_map(CUtensorMap* map, const uint32_t* base, int BH, int N) {
    const TensorMapKey key = {base, BH, N, -1};
    TensorMapSlot& slot = tensor_map_slot(key);
    if (slot.key == key) {
        *map = slot.map;
        return SMA_OK;
    }
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) return SMA_ERR_CUDA;
    const cuuint64_t nw = static_cast<cuuint64_t>((N + 31) / 32);
    const cuuint64_t dims[3] = {nw, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(BH)};
    const cuuint64_t strides[2] = {nw * 4, static_cast<cuuint64_t>(N) * nw * 4};
    const cuuint32_t box[3] = {sma::kChunkWords, sma::kBlockM, 1};
    const cuuint32_t elem_strides[3] = {1, 1, 1};
    auto encode_once = [&]() {
        return encode(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<uint32_t*>(base), dims, strides, box, elem_strides,
                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    };
    CUresult r = encode_once();
    if (r == CUDA_ERROR_INVALID_CONTEXT && bind_primary_context()) r = encode_once();
    if (r != CUDA_SUCCESS) {
        tls_cuda_error = static_cast<int>(cudaErrorInvalidValue);
        return SMA_ERR_CUDA;
    }
    slot.key = key;
    slot.map = *map;
    return SMA_OK;
}

// Launch with programmatic stream serialisation: the grid may be scheduled while the previous kernel of the
// stream is draining; the kernels call griddepcontrol.wait before they touch global memory, so only their
// set-up (barriers, tensor memory, descriptor prefetch) and the launch latency overlap with the predecessor.
template <typename... KArgs, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(KArgs...), unsigned blocks, unsigned threads, size_t smem,
                              cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

// An ordinary launch whose outcome is the launch call's own return value.  (The error state that cudaGetLastError
// reads is per host thread and shared with everything else that thread runs: another library's harmless failed
// query, left there, would be reported as this library's launch failure.)
template <typename... KArgs, typename... Args>
cudaError_t launch_plain(void (*kernel)(KArgs...), unsigned blocks, unsigned threads, size_t smem, cudaStream_t stream,
                         Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks);
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cfg.attrs = nullptr;
    cfg.numAttrs = 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}

template <bool kBf16, bool kSplitP, int kLists, bool kFourD>
int launch_attention(DeviceInfo* dev, int slot, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                     const CUtensorMap& to, const CUtensorMap& tm, const sma::AttnArgs& args, cudaStream_t stream) {
    auto kernel = sma::attn_fwd_kernel<kBf16, kSplitP, kLists, kFourD>;
    constexpr size_t smem = sma::attn_smem_bytes();
    // One CTA per SM: the kernel allocates all 512 tensor-memory columns, and more than half of the
    // SM's shared memory keeps a second CTA from becoming resident next to it.
    static_assert(smem > 116 * 1024 && smem <= 227 * 1024, "shared memory must pin occupancy to one CTA per SM");
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!dev->attn_attr_set[slot]) {
            if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              static_cast<int>(smem))))
                return SMA_ERR_CUDA;
            dev->attn_attr_set[slot] = true;
        }
    }
    const long long items = static_cast<long long>(args.BH) * args.num_q_tiles;
    const unsigned blocks = static_cast<unsigned>(items < dev->sm_count ? items : dev->sm_count);
    return cuda_ok(launch_overlapped(kernel, blocks, sma::kAttnThreads, smem, stream, tq, tk, tv, to, tm, args))
               ? SMA_OK
               : SMA_ERR_CUDA;
}

// fmt: 0 fp16, 1 bf16 with P = hi + lo, 2 bf16 with P rounded once
template <int kLists>
int launch_attention_fmt(int fmt, bool four_d, DeviceInfo* dev, int slot, const CUtensorMap& tq, const CUtensorMap& tk,
                         const CUtensorMap& tv, const CUtensorMap& to, const CUtensorMap& tm, const sma::AttnArgs& args,
                         cudaStream_t stream) {
    if (fmt == 0)
        return four_d ? launch_attention<false, false, kLists, true>(dev, slot, tq, tk, tv, to, tm, args, stream)
                      : launch_attention<false, false, kLists, false>(dev, slot, tq, tk, tv, to, tm, args, stream);
    if (fmt == 1)
        return four_d ? launch_attention<true, true, kLists, true>(dev, slot, tq, tk, tv, to, tm, args, stream)
                      : launch_attention<true, true, kLists, false>(dev, slot, tq, tk, tv, to, tm, args, stream);
    return four_d ? launch_attention<true, false, kLists, true>(dev, slot, tq, tk, tv, to, tm, args, stream)
                  : launch_attention<true, false, kLists, false>(dev, slot, tq, tk, tv, to, tm, args, stream);
}

}  // namespace

template <bool kBf16>
static int launch_backward(DeviceInfo* dev, const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                           const CUtensorMap& tdo, const CUtensorMap& tdq, const sma::BwdArgs& args, const void* dout, const void* out, void* dq,
                           cudaStream_t stream) {
    const size_t rows = static_cast<size_t>(args.BH) * args.N;
    {
        const size_t warps_per_block = 8;
        size_t blocks = (rows + warps_per_block - 1) / warps_per_block;
        const size_t cap = static_cast<size_t>(dev->sm_count) * 8;
        if (blocks > cap) blocks = cap;
        if (!cuda_ok(launch_plain(sma::bwd_prepare_kernel<kBf16>, static_cast<unsigned>(blocks), 256, 0, stream,
                                  static_cast<const uint32_t*>(dout), static_cast<const uint32_t*>(out),
                                  const_cast<float*>(args.delta), args.dq_accum, rows, args.unit_counter)))
            return SMA_ERR_CUDA;
    }
    auto kernel = sma::attn_bwd_kernel<kBf16>;
    constexpr size_t smem = sma::bwd_smem_bytes();
    static_assert(smem > 116 * 1024 && smem <= 227 * 1024, "shared memory must pin occupancy to one CTA per SM");
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!dev->bwd_attr_set[kBf16 ? 1 : 0]) {
            if (!cuda_ok(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))))
                return SMA_ERR_CUDA;
            dev->bwd_attr_set[kBf16 ? 1 : 0] = true;
        }
    }
    // persistent CTAs, one per SM, that share out the (key block, batch*head) units through a queue
    const long long units = static_cast<long long>(args.BH) * ((args.N + sma::kBwdBlock - 1) / sma::kBwdBlock);
    const unsigned blocks = static_cast<unsigned>(units < dev->sm_count ? units : dev->sm_count);
    if (!cuda_ok(launch_overlapped(kernel, blocks, sma::kBwdThreads, smem, stream, tq, tk, tv, tdo, tdq, args))) return SMA_ERR_CUDA;
    {
        const size_t n2 = rows * sma::kBwdDim / 2;
        size_t blocks2 = (n2 + 255) / 256;
        const size_t cap = static_cast<size_t>(dev->sm_count) * 16;
        if (blocks2 > cap) blocks2 = cap;
        if (!cuda_ok(launch_overlapped(sma::bwd_finish_kernel<kBf16>, static_cast<unsigned>(blocks2), 256, 0, stream,
                                  reinterpret_cast<const float2*>(args.dq_accum), static_cast<uint32_t*>(dq), n2)))
            return SMA_ERR_CUDA;
    }
    return SMA_OK;
}

extern "C" {

int sma_abi_version(void) { return SMA_ABI_VERSION; }

const char* sma_strerror(int status) {
    switch (status) {
        case SMA_OK: return "ok";
        case SMA_ERR_NULL_POINTER: return "a required pointer is NULL";
        case SMA_ERR_BAD_SHAPE: return "B, H and N must be >= 1 and B*H*N*N must fit the index range";
        case SMA_ERR_BAD_HEAD_DIM: return "head dimension must be 64";
        case SMA_ERR_BAD_DTYPE: return "dtype must be fp16 or bf16";
        case SMA_ERR_MISALIGNED: return "q/k/v/out must be 16-byte aligned, mask_packed and lse 4-byte aligned";
        case SMA_ERR_BAD_SCALE: return "scale must be finite and non-zero";
        case SMA_ERR_SEQ_TOO_LONG: return "sequence length above SMA_MAX_SEQ_LEN";
        case SMA_ERR_CUDA: return "a CUDA call failed (see sma_last_cuda_error)";
        case SMA_ERR_WRONG_ARCH: return "the current device is not an sm_100 (B200-class) GPU";
        case SMA_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
        case SMA_ERR_WORKSPACE_TOO_SMALL: return "the workspace is smaller than sma_attention_workspace_bytes() asks for";
        case SMA_ERR_STATIC_WORKSPACE_EXCEEDED:
            return "B*H*N is too large for the built-in workspace of sma_attention_fwd_static_workspace "
                   "(SMA_STATIC_WORKSPACE_BYTES); use sma_attention_fwd or sma_attention_fwd_planned";
        case SMA_ERR_BAD_VARIANT: return "unknown kernel variant";
        case SMA_ERR_BAD_STRIDE:
            return "strides of q/k/v/out must be positive multiples of 8 elements (or all zero for the dense layout); "
                   "the backward pass takes dense tensors only";
        default: return "unknown status";
    }
}

int sma_last_cuda_error(void) { return tls_cuda_error; }

// Bytes of the occupancy side-band for B x H x N, or 0 when the shape has none (N not a multiple of 64).
static size_t tile_bits_bytes(int32_t B, int32_t H, int32_t N) {
    if (B < 1 || H < 1 || N < 1 || N > SMA_MAX_SEQ_LEN || N % 64 != 0) return 0;
    return static_cast<size_t>(1ull * B * H * N * (N / 32) / 32 * sizeof(uint16_t));
}

// Shared body of the packing entry points; tile_bits == nullptr: packed words only.
static int pack_mask(const uint8_t* mask, uint32_t* packed, uint16_t* tile_bits, uint32_t* work_counter, int32_t B,
                     int32_t H, int32_t N, void* stream_v) {
    if (!mask || !packed) return SMA_ERR_NULL_POINTER;
    if (B < 1 || H < 1 || N < 1) return SMA_ERR_BAD_SHAPE;
    const unsigned long long rows = 1ull * B * H * N;
    if (rows > (1ull << 40) / static_cast<unsigned long long>(N)) return SMA_ERR_BAD_SHAPE;
    if (reinterpret_cast<uintptr_t>(packed) & 3u) return SMA_ERR_MISALIGNED;
    const bool flat = (N % 32 == 0) && ((reinterpret_cast<uintptr_t>(mask) & 31u) == 0);
    if (tile_bits) {
        if (tile_bits_bytes(B, H, N) == 0) return SMA_ERR_BAD_SHAPE;
        if (!flat || (reinterpret_cast<uintptr_t>(tile_bits) & 15u)) return SMA_ERR_MISALIGNED;
    }
    DeviceInfo* dev = nullptr;
    if (int st = current_device_info(&dev)) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    if (flat) {
        const size_t n_words = static_cast<size_t>(rows) * (N / 32);
        const size_t per_block = static_cast<size_t>(sma::kPackThreads) * sma::pack_unroll(tile_bits != nullptr);
        size_t blocks = (n_words + per_block - 1) / per_block;
        // One block per 256 words up to the grid limit (the kernel strides over the rest): blocks that finish
        // hand their SM to the next one, so SMs that become free early (the tail of a kernel running before this
        // one) take more of the work.  A grid capped at the resident blocks was 3 % slower alone and 2 % per step.
        if (blocks > 0x7FFFFFFFu) blocks = 0x7FFFFFFFu;
        const cudaError_t e =
            tile_bits ? launch_overlapped(sma::pack_flat_kernel<true>, static_cast<unsigned>(blocks), sma::kPackThreads, 0,
                                          stream, mask, packed, tile_bits, n_words, work_counter)
                      : launch_overlapped(sma::pack_flat_kernel<false>, static_cast<unsigned>(blocks), sma::kPackThreads, 0,
                                          stream, mask, packed, static_cast<uint16_t*>(nullptr), n_words, work_counter);
        if (!cuda_ok(e)) return SMA_ERR_CUDA;
    } else {
        const size_t warps_per_block = sma::kPackThreads / 32;
        size_t blocks = (static_cast<size_t>(rows) + warps_per_block - 1) / warps_per_block;
        const size_t cap = static_cast<size_t>(dev->sm_count) * 8 * 4;
        if (blocks > cap) blocks = cap;
        if (!cuda_ok(launch_overlapped(sma::pack_rows_kernel, static_cast<unsigned>(blocks), sma::kPackThreads, 0, stream,
                                       mask, packed, static_cast<size_t>(rows), N, work_counter)))
            return SMA_ERR_CUDA;
    }
    return SMA_OK;
}

int sma_pack_mask(const uint8_t* mask, uint32_t* packed, int32_t B, int32_t H, int32_t N, void* stream_v) {
    return pack_mask(mask, packed, nullptr, nullptr, B, H, N, stream_v);
}

size_t sma_tile_bits_bytes(int32_t B, int32_t H, int32_t N) { return tile_bits_bytes(B, H, N); }

int sma_pack_mask_tiles(const uint8_t* mask, uint32_t* packed, void* tile_bits, int32_t B, int32_t H, int32_t N,
                        void* stream_v) {
    if (!tile_bits) return SMA_ERR_NULL_POINTER;
    return pack_mask(mask, packed, static_cast<uint16_t*>(tile_bits), nullptr, B, H, N, stream_v);
}

// Shared body of the attention entry points.  plan == nullptr and tile_bits == nullptr: the kernel's loader warps
// find the non-empty tiles themselves by reading the packed mask.  plan: a workspace of at least
// attention_workspace_bytes() bytes that the tile-list kernel fills first.  tile_bits: the occupancy side-band that
// sma_pack_mask_tiles wrote for this mask_packed.
static int attention_forward(const sma_attention_params* p, uint32_t* plan, const uint16_t* tile_bits,
                             uint32_t* work_counter, void* stream_v) {
    if (!p) return SMA_ERR_NULL_POINTER;
    if (!p->q || !p->k || !p->v || !p->mask_packed || !p->out) return SMA_ERR_NULL_POINTER;
    if (p->save_lse && !p->lse) return SMA_ERR_NULL_POINTER;
    if (p->B < 1 || p->H < 1 || p->N < 1) return SMA_ERR_BAD_SHAPE;
    if (p->D != sma::kHeadDim) return SMA_ERR_BAD_HEAD_DIM;
    if (p->dtype != SMA_DTYPE_F16 && p->dtype != SMA_DTYPE_BF16) return SMA_ERR_BAD_DTYPE;
    if (p->N > SMA_MAX_SEQ_LEN) return SMA_ERR_SEQ_TOO_LONG;
    if (!std::isfinite(p->scale) || p->scale == 0.f) return SMA_ERR_BAD_SCALE;
    const long long BH = 1ll * p->B * p->H;
    const int num_q_tiles = (p->N + sma::kBlockM - 1) / sma::kBlockM;
    if (BH * num_q_tiles > 0x7FFFFFFFll || BH > 0x7FFFFFFFll) return SMA_ERR_BAD_SHAPE;
    const uintptr_t align16 = reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) |
                              reinterpret_cast<uintptr_t>(p->v) | reinterpret_cast<uintptr_t>(p->out);
    if (align16 & 15u) return SMA_ERR_MISALIGNED;
    if ((reinterpret_cast<uintptr_t>(p->mask_packed) & 3u) || (reinterpret_cast<uintptr_t>(p->lse) & 3u))
        return SMA_ERR_MISALIGNED;
    if (tile_bits) {
        if (tile_bits_bytes(p->B, p->H, p->N) == 0) return SMA_ERR_BAD_SHAPE;
        if (reinterpret_cast<uintptr_t>(tile_bits) & 15u) return SMA_ERR_MISALIGNED;
    }

    const bool bf16 = p->dtype == SMA_DTYPE_BF16;
    bool split_p = bf16;
    switch (p->variant) {
        case SMA_VARIANT_DEFAULT: break;
        case SMA_VARIANT_BF16_SINGLE_P:
            if (!bf16) return SMA_ERR_BAD_VARIANT;
            split_p = false;
            break;
        default: return SMA_ERR_BAD_VARIANT;
    }

    int64_t sq[3], sk[3], sv[3], so[3];
    if (!resolve_strides(p->q_strides, p->H, p->N, sq) || !resolve_strides(p->k_strides, p->H, p->N, sk) ||
        !resolve_strides(p->v_strides, p->H, p->N, sv) || !resolve_strides(p->out_strides, p->H, p->N, so))
        return SMA_ERR_BAD_STRIDE;
    DeviceInfo* dev = nullptr;
    if (int st = current_device_info(&dev)) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    // three-dimensional maps (cheaper for the kernel's loader warps) when batch*head is one dimension of all four
    const auto linear = [&](const int64_t (&st)[3]) { return st[0] == static_cast<int64_t>(p->H) * st[1]; };
    const bool four_d = !(linear(sq) && linear(sk) && linear(sv) && linear(so));
    CUtensorMap tq, tk, tv, to, tm;
    if (int st = make_strided_tensor_map(&tq, p->q, p->B, p->H, p->N, sq, sma::kBlockM, bf16, four_d)) return st;
    if (int st = make_strided_tensor_map(&to, p->out, p->B, p->H, p->N, so, sma::kStageRowsOut, bf16, four_d)) return st;
    if (int st = make_strided_tensor_map(&tk, p->k, p->B, p->H, p->N, sk, sma::kBlockN, bf16, four_d)) return st;
    if (int st = make_strided_tensor_map(&tv, p->v, p->B, p->H, p->N, sv, sma::kBlockN, bf16, four_d)) return st;
    const bool mask_tma = mask_has_tensor_map(p->mask_packed, p->N);
    if (mask_tma) {
        if (int st = make_mask_tensor_map(&tm, p->mask_packed, static_cast<int>(BH), p->N)) return st;
    } else {
        tm = tq;  // never used by the kernel: the loader warps copy the mask words with plain loads
    }

    sma::AttnArgs args;
    args.mask_packed = p->mask_packed;
    args.plan = plan;
    args.tile_bits = tile_bits;
    args.work_counter = work_counter;
    args.plan_stride = sma::plan_stride_words(p->N);
    args.lse = p->lse;
    args.BH = static_cast<int32_t>(BH);
    args.H = p->H;
    args.N = p->N;
    args.num_q_tiles = num_q_tiles;
    args.scale_log2e = std::fabs(p->scale) * 1.4426950408889634f;
    args.negate_q = p->scale < 0.f ? 1u : 0u;
    args.save_lse = p->save_lse ? 1 : 0;
    args.mask_tma = mask_tma ? 1 : 0;

    if (plan) {
        const unsigned items = static_cast<unsigned>(BH * num_q_tiles);
        if (!cuda_ok(launch_plain(sma::build_tile_lists_kernel, items, sma::kPlanRows, 0, stream, p->mask_packed, plan,
                                  static_cast<int>(BH), p->N, num_q_tiles, args.plan_stride, work_counter)))
            return SMA_ERR_CUDA;
    }
    // one instantiation per (element type, P format, source of the tile lists, rank of the tensor maps)
    const int lists = plan ? sma::kListsFromPlan : tile_bits ? sma::kListsFromBits : sma::kListsFromStrips;
    const int fmt = !bf16 ? 0 : split_p ? 1 : 2;
    const int slot = ((lists * 3) + fmt) * 2 + (four_d ? 1 : 0);
    if (lists == sma::kListsFromPlan)
        return launch_attention_fmt<sma::kListsFromPlan>(fmt, four_d, dev, slot, tq, tk, tv, to, tm, args, stream);
    if (lists == sma::kListsFromBits)
        return launch_attention_fmt<sma::kListsFromBits>(fmt, four_d, dev, slot, tq, tk, tv, to, tm, args, stream);
    return launch_attention_fmt<sma::kListsFromStrips>(fmt, four_d, dev, slot, tq, tk, tv, to, tm, args, stream);
}

static size_t plan_lists_bytes(long long items, int32_t N) {
    return static_cast<size_t>(items) * sma::plan_stride_words(N) * sizeof(uint32_t);
}

// The work-queue word at the end of a tile-list workspace (zeroed by the tile-list kernel of the same call).
static uint32_t* plan_work_counter(uint32_t* workspace, const sma_attention_params* p) {
    const long long items = 1ll * p->B * p->H * ((p->N + sma::kBlockM - 1) / sma::kBlockM);
    return workspace + plan_lists_bytes(items, p->N) / sizeof(uint32_t);
}

// Bytes of workspace for B x H x N, or 0 for a shape the attention entry points reject.
static size_t attention_workspace_bytes(int32_t B, int32_t H, int32_t N) {
    if (B < 1 || H < 1 || N < 1 || N > SMA_MAX_SEQ_LEN) return 0;
    const long long items = 1ll * B * H * ((N + sma::kBlockM - 1) / sma::kBlockM);
    if (items > 0x7FFFFFFFll) return 0;
    return plan_lists_bytes(items, N) + 16;  // the tile lists, then the attention kernel's work-queue word
}

int sma_attention_fwd(const sma_attention_params* p, void* stream_v) {
    return attention_forward(p, nullptr, nullptr, nullptr, stream_v);
}

int sma_attention_fwd_tiles(const sma_attention_params* p, const void* tile_bits, void* stream_v) {
    if (!tile_bits) return SMA_ERR_NULL_POINTER;
    return attention_forward(p, nullptr, static_cast<const uint16_t*>(tile_bits), nullptr, stream_v);
}

int sma_sparse_attention_fwd(const sma_attention_params* p, const uint8_t* mask, void* tile_bits, void* work_counter,
                             void* stream_v) {
    if (!p || !mask) return SMA_ERR_NULL_POINTER;
    if (!p->mask_packed) return SMA_ERR_NULL_POINTER;
    // the side-band exists for N % 64 == 0 and a 32-byte aligned mask; the caller who passes a buffer for another
    // shape gets the plain pair of kernels
    uint16_t* bits = static_cast<uint16_t*>(tile_bits);
    if (bits && (tile_bits_bytes(p->B, p->H, p->N) == 0 || (reinterpret_cast<uintptr_t>(mask) & 31u))) bits = nullptr;
    if (reinterpret_cast<uintptr_t>(work_counter) & 3u) return SMA_ERR_MISALIGNED;
    uint32_t* counter = static_cast<uint32_t*>(work_counter);
    if (int st = pack_mask(mask, const_cast<uint32_t*>(p->mask_packed), bits, counter, p->B, p->H, p->N, stream_v)) return st;
    return attention_forward(p, nullptr, bits, counter, stream_v);
}

size_t sma_attention_workspace_bytes(int32_t B, int32_t H, int32_t N) { return attention_workspace_bytes(B, H, N); }

int sma_attention_fwd_planned(const sma_attention_params* p, void* workspace, size_t workspace_bytes, void* stream_v) {
    if (!p || !workspace) return SMA_ERR_NULL_POINTER;
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return SMA_ERR_MISALIGNED;
    const size_t need = attention_workspace_bytes(p->B, p->H, p->N);
    if (need != 0 && workspace_bytes < need) return SMA_ERR_WORKSPACE_TOO_SMALL;
    if (need == 0) return attention_forward(p, nullptr, nullptr, nullptr, stream_v);  // the shape checks in there report why
    uint32_t* plan = static_cast<uint32_t*>(workspace);
    return attention_forward(p, plan, nullptr, plan_work_counter(plan, p), stream_v);
}

// ---- backward pass -------------------------------------------------------------------------------------------
// Workspace: delta [BH, N] fp32 (rounded up to 256 bytes), then the dQ accumulator [BH, N, 64] fp32, then 256 bytes
// whose first word is the backward kernel's work queue.
static size_t bwd_delta_bytes(long long BH, int N) { return (static_cast<size_t>(BH) * N * sizeof(float) + 255u) & ~size_t(255); }

size_t sma_attention_bwd_workspace_bytes(int32_t B, int32_t H, int32_t N) {
    if (B < 1 || H < 1 || N < 1 || N > SMA_MAX_SEQ_LEN) return 0;
    const long long BH = 1ll * B * H;
    if (BH * ((N + sma::kBwdBlock - 1) / sma::kBwdBlock) > 0x7FFFFFFFll) return 0;
    return bwd_delta_bytes(BH, N) + static_cast<size_t>(BH) * N * sma::kBwdDim * sizeof(float) + 256;
}

int sma_attention_bwd(const sma_attention_params* p, const void* dout, void* dq, void* dk, void* dv, void* workspace,
                      size_t workspace_bytes, void* stream_v) {
    if (!p || !dout || !dq || !dk || !dv || !workspace) return SMA_ERR_NULL_POINTER;
    if (!p->q || !p->k || !p->v || !p->mask_packed || !p->out || !p->lse) return SMA_ERR_NULL_POINTER;
    if (p->B < 1 || p->H < 1 || p->N < 1) return SMA_ERR_BAD_SHAPE;
    if (p->D != sma::kBwdDim) return SMA_ERR_BAD_HEAD_DIM;
    if (p->dtype != SMA_DTYPE_F16 && p->dtype != SMA_DTYPE_BF16) return SMA_ERR_BAD_DTYPE;
    if (p->N > SMA_MAX_SEQ_LEN) return SMA_ERR_SEQ_TOO_LONG;
    if (!std::isfinite(p->scale) || p->scale == 0.f) return SMA_ERR_BAD_SCALE;
    for (const int64_t* st : {p->q_strides, p->k_strides, p->v_strides, p->out_strides}) {
        const bool zero = st[0] == 0 && st[1] == 0 && st[2] == 0;
        const bool dense = st[0] == static_cast<int64_t>(p->H) * p->N * 64 && st[1] == static_cast<int64_t>(p->N) * 64 && st[2] == 64;
        if (!zero && !dense) return SMA_ERR_BAD_STRIDE;
    }
    const size_t need = sma_attention_bwd_workspace_bytes(p->B, p->H, p->N);
    if (need == 0) return SMA_ERR_BAD_SHAPE;
    if (workspace_bytes < need) return SMA_ERR_WORKSPACE_TOO_SMALL;
    const uintptr_t align16 = reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->k) |
                              reinterpret_cast<uintptr_t>(p->v) | reinterpret_cast<uintptr_t>(p->out) |
                              reinterpret_cast<uintptr_t>(dout) | reinterpret_cast<uintptr_t>(dq) |
                              reinterpret_cast<uintptr_t>(dk) | reinterpret_cast<uintptr_t>(dv) |
                              reinterpret_cast<uintptr_t>(workspace);
    if (align16 & 15u) return SMA_ERR_MISALIGNED;
    if ((reinterpret_cast<uintptr_t>(p->mask_packed) & 3u) || (reinterpret_cast<uintptr_t>(p->lse) & 3u)) return SMA_ERR_MISALIGNED;
    const long long BH = 1ll * p->B * p->H;
    const bool bf16 = p->dtype == SMA_DTYPE_BF16;
    DeviceInfo* dev = nullptr;
    if (int st = current_device_info(&dev)) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);

    CUtensorMap tq, tk, tv, tdo;
    if (int st = make_qkv_tensor_map(&tq, p->q, static_cast<int>(BH), p->N, sma::kBwdBlock, bf16)) return st;
    if (int st = make_qkv_tensor_map(&tk, p->k, static_cast<int>(BH), p->N, sma::kBwdBlock, bf16)) return st;
    if (int st = make_qkv_tensor_map(&tv, p->v, static_cast<int>(BH), p->N, sma::kBwdBlock, bf16)) return st;
    if (int st = make_qkv_tensor_map(&tdo, dout, static_cast<int>(BH), p->N, sma::kBwdBlock, bf16)) return st;

    sma::BwdArgs args;
    args.mask_packed = p->mask_packed;
    args.lse = p->lse;
    args.delta = static_cast<float*>(workspace);
    args.dq_accum = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + bwd_delta_bytes(BH, p->N));
    args.unit_counter = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(args.dq_accum) +
                                                   static_cast<size_t>(BH) * p->N * sma::kBwdDim * sizeof(float));
    args.dk = dk;
    args.dv = dv;
    args.BH = static_cast<int32_t>(BH);
    args.N = p->N;
    args.scale = p->scale;
    CUtensorMap tdq;
    if (int st = make_dq_accum_tensor_map(&tdq, args.dq_accum, static_cast<int>(BH), p->N)) return st;
    return bf16 ? launch_backward<true>(dev, tq, tk, tv, tdo, tdq, args, dout, p->out, dq, stream)
                : launch_backward<false>(dev, tq, tk, tv, tdo, tdq, args, dout, p->out, dq, stream);
}

// ---- the entry point that allocates nothing -----------------------------------------------------------------
// Built-in workspace of sma_attention_fwd_static_workspace.  It lives in the library's device image: every GPU
// that loads the library carries these SMA_STATIC_WORKSPACE_BYTES from the first CUDA call to process exit.
// In host code the name below only identifies the symbol; the address a kernel can use comes from
// cudaGetSymbolAddress on the device in question.
// (plus the 16 bytes of the attention kernel's work-queue word that every tile-list workspace ends with)
static __device__ __align__(256) uint32_t g_static_workspace[(SMA_STATIC_WORKSPACE_BYTES + 16) / sizeof(uint32_t)];

namespace {
uint32_t* g_static_workspace_addr[kMaxDevices] = {};  // per device, resolved by the first call made on it

// Device address of g_static_workspace on the current device (looked up once per device).
int static_workspace_of_current_device(uint32_t** out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev))) return SMA_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return SMA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (!g_static_workspace_addr[dev]) {
        void* ptr = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&ptr, g_static_workspace)) || !ptr) return SMA_ERR_CUDA;
        g_static_workspace_addr[dev] = static_cast<uint32_t*>(ptr);
    }
    *out = g_static_workspace_addr[dev];
    return SMA_OK;
}
}  // namespace

int sma_attention_fwd_static_workspace(const sma_attention_params* p, void* stream_v) {
    if (!p) return SMA_ERR_NULL_POINTER;
    const size_t need = attention_workspace_bytes(p->B, p->H, p->N);
    if (need > SMA_STATIC_WORKSPACE_BYTES + 16) return SMA_ERR_STATIC_WORKSPACE_EXCEEDED;
    // the device is looked at before the array's address: on a GPU for which the library holds no code the
    // caller should hear SMA_ERR_WRONG_ARCH, like from the other entry points, not a failed symbol look-up
    DeviceInfo* dev = nullptr;
    if (int st = current_device_info(&dev)) return st;
    uint32_t* workspace = nullptr;
    if (int st = static_workspace_of_current_device(&workspace)) return st;
    // Nothing in the workspace has to start at zero: the tile-list kernel writes every word the attention kernel
    // reads (the count of each work item and that many entries), so the previous call's leftovers are never seen.
    if (need == 0) return attention_forward(p, nullptr, nullptr, nullptr, stream_v);  // the shape checks in there report why
    return attention_forward(p, workspace, nullptr, plan_work_counter(workspace, p), stream_v);
}

#ifdef SMA_WAIT_TEST_BUILD
// Test build only (not declared in include/sma.h): while on, every attention launch, forward or backward, leaves one
// Q tile unrequested.
int sma_test_withhold_q_load(int on) {
    const int value = on ? 1 : 0;
    return cuda_ok(cudaMemcpyToSymbol(sma::g_test_withhold_q_load, &value, sizeof(int))) ? SMA_OK : SMA_ERR_CUDA;
}
#endif

int sma_device_status(void) {
    if (!cuda_ok(cudaDeviceSynchronize())) return SMA_ERR_CUDA;
    int status = 0;
    if (!cuda_ok(cudaMemcpyFromSymbol(&status, sma::g_device_status, sizeof(int)))) return SMA_ERR_CUDA;
    if (status != 0) {
        const int zero = 0;
        if (!cuda_ok(cudaMemcpyToSymbol(sma::g_device_status, &zero, sizeof(int)))) return SMA_ERR_CUDA;
    }
    return status == 0 ? SMA_OK : SMA_ERR_DEVICE_TIMEOUT;
}

}  // extern "C"
