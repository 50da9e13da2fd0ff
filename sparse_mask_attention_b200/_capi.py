"""ctypes binding of libsma_b200.so — the C ABI declared in include/sma.h.

There is no fallback: if the shared library is missing or does not export every symbol of the header,
importing this module raises, and every call checks the returned status and raises ``SmaError``.
"""
from __future__ import annotations

import ctypes
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG_DIR, "libsma_b200.so")

SMA_ABI_VERSION = 4
SMA_DTYPE_F16 = 0
SMA_DTYPE_BF16 = 1
SMA_VARIANT_DEFAULT = 0
SMA_VARIANT_BF16_SINGLE_P = 1
SMA_MAX_SEQ_LEN = 16384

SMA_OK = 0
SMA_ERR_NULL_POINTER = -1
SMA_ERR_BAD_SHAPE = -2
SMA_ERR_BAD_HEAD_DIM = -3
SMA_ERR_BAD_DTYPE = -4
SMA_ERR_MISALIGNED = -5
SMA_ERR_BAD_SCALE = -6
SMA_ERR_SEQ_TOO_LONG = -7
SMA_ERR_CUDA = -8
SMA_ERR_WRONG_ARCH = -9
SMA_ERR_DEVICE_TIMEOUT = -10
SMA_ERR_BAD_VARIANT = -11
SMA_ERR_WORKSPACE_TOO_SMALL = -12
SMA_ERR_STATIC_WORKSPACE_EXCEEDED = -13
SMA_ERR_BAD_STRIDE = -14
SMA_STATIC_WORKSPACE_BYTES = 1 << 20

# every symbol include/sma.h declares
EXPORTED_SYMBOLS = (
    "sma_abi_version",
    "sma_strerror",
    "sma_last_cuda_error",
    "sma_pack_mask",
    "sma_attention_fwd",
    "sma_sparse_attention_fwd",
    "sma_tile_bits_bytes",
    "sma_pack_mask_tiles",
    "sma_attention_fwd_tiles",
    "sma_attention_workspace_bytes",
    "sma_attention_fwd_planned",
    "sma_attention_fwd_static_workspace",
    "sma_attention_bwd_workspace_bytes",
    "sma_attention_bwd",
    "sma_device_status",
)


class SmaError(RuntimeError):
    """A call into libsma_b200.so returned a non-zero status."""

    def __init__(self, status: int, message: str):
        super().__init__("libsma_b200: %s (status %d)" % (message, status))
        self.status = status


class AttentionParams(ctypes.Structure):
    """Mirror of ``struct sma_attention_params`` in include/sma.h."""

    _fields_ = [
        ("q", ctypes.c_void_p),
        ("k", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("mask_packed", ctypes.c_void_p),
        ("out", ctypes.c_void_p),
        ("lse", ctypes.c_void_p),
        ("B", ctypes.c_int32),
        ("H", ctypes.c_int32),
        ("N", ctypes.c_int32),
        ("D", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("dtype", ctypes.c_int32),
        ("save_lse", ctypes.c_int32),
        ("variant", ctypes.c_int32),
        # element strides {batch, head, row} of q, k, v, out; all zero = the dense [B, H, N, 64] layout
        ("q_strides", ctypes.c_int64 * 3),
        ("k_strides", ctypes.c_int64 * 3),
        ("v_strides", ctypes.c_int64 * 3),
        ("out_strides", ctypes.c_int64 * 3),
    ]


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            "%s is missing: build it with `python sparse_mask_attention_b200/build.py` "
            "(there is no CPU or PyTorch fallback for the CUDA path)" % LIB_PATH
        )
    lib = ctypes.CDLL(LIB_PATH)
    missing = [s for s in EXPORTED_SYMBOLS if not hasattr(lib, s)]
    if missing:
        raise ImportError("%s does not export %s" % (LIB_PATH, ", ".join(missing)))
    lib.sma_abi_version.restype = ctypes.c_int
    lib.sma_abi_version.argtypes = []
    lib.sma_strerror.restype = ctypes.c_char_p
    lib.sma_strerror.argtypes = [ctypes.c_int]
    lib.sma_last_cuda_error.restype = ctypes.c_int
    lib.sma_last_cuda_error.argtypes = []
    lib.sma_pack_mask.restype = ctypes.c_int
    lib.sma_pack_mask.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                  ctypes.c_void_p]
    lib.sma_attention_fwd.restype = ctypes.c_int
    lib.sma_attention_fwd.argtypes = [ctypes.POINTER(AttentionParams), ctypes.c_void_p]
    lib.sma_sparse_attention_fwd.restype = ctypes.c_int
    lib.sma_sparse_attention_fwd.argtypes = [ctypes.POINTER(AttentionParams), ctypes.c_void_p, ctypes.c_void_p,
                                             ctypes.c_void_p, ctypes.c_void_p]
    lib.sma_tile_bits_bytes.restype = ctypes.c_size_t
    lib.sma_tile_bits_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.sma_pack_mask_tiles.restype = ctypes.c_int
    lib.sma_pack_mask_tiles.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.sma_attention_fwd_tiles.restype = ctypes.c_int
    lib.sma_attention_fwd_tiles.argtypes = [ctypes.POINTER(AttentionParams), ctypes.c_void_p, ctypes.c_void_p]
    lib.sma_attention_workspace_bytes.restype = ctypes.c_size_t
    lib.sma_attention_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.sma_attention_fwd_planned.restype = ctypes.c_int
    lib.sma_attention_fwd_planned.argtypes = [ctypes.POINTER(AttentionParams), ctypes.c_void_p, ctypes.c_size_t,
                                              ctypes.c_void_p]
    lib.sma_attention_fwd_static_workspace.restype = ctypes.c_int
    lib.sma_attention_fwd_static_workspace.argtypes = [ctypes.POINTER(AttentionParams), ctypes.c_void_p]
    lib.sma_attention_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.sma_attention_bwd_workspace_bytes.argtypes = [ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    lib.sma_attention_bwd.restype = ctypes.c_int
    lib.sma_attention_bwd.argtypes = [ctypes.POINTER(AttentionParams)] + [ctypes.c_void_p] * 5 + [ctypes.c_size_t,
                                                                                                 ctypes.c_void_p]
    lib.sma_device_status.restype = ctypes.c_int
    lib.sma_device_status.argtypes = []
    if lib.sma_abi_version() != SMA_ABI_VERSION:
        raise ImportError("%s has ABI version %d, expected %d" % (LIB_PATH, lib.sma_abi_version(), SMA_ABI_VERSION))
    return lib


lib = _load()


def strerror(status: int) -> str:
    return lib.sma_strerror(status).decode()


def check(status: int) -> None:
    if status != SMA_OK:
        msg = strerror(status)
        if status == SMA_ERR_CUDA:
            msg += " [cudaError %d]" % lib.sma_last_cuda_error()
        raise SmaError(status, msg)


def pack_mask(mask_ptr: int, packed_ptr: int, B: int, H: int, N: int, stream: int) -> None:
    check(lib.sma_pack_mask(mask_ptr, packed_ptr, B, H, N, stream))


def attention_fwd(params: AttentionParams, stream: int) -> None:
    check(lib.sma_attention_fwd(ctypes.byref(params), stream))


def sparse_attention_fwd(params: AttentionParams, mask_ptr: int, tile_bits_ptr, work_counter_ptr, stream: int) -> None:
    """pack_mask into params.mask_packed, then the forward pass, behind one call into the library.

    tile_bits_ptr: None, or a device buffer of tile_bits_bytes(B, H, N) bytes for the occupancy side-band.
    work_counter_ptr: None, or 4 bytes of device memory for the attention kernel's work queue."""
    check(lib.sma_sparse_attention_fwd(ctypes.byref(params), mask_ptr, tile_bits_ptr, work_counter_ptr, stream))


def tile_bits_bytes(B: int, H: int, N: int) -> int:
    """Bytes of the occupancy side-band of a B x H x N mask; 0 when the shape has none (N % 64 != 0)."""
    return int(lib.sma_tile_bits_bytes(B, H, N))


def pack_mask_tiles(mask_ptr: int, packed_ptr: int, tile_bits_ptr: int, B: int, H: int, N: int, stream: int) -> None:
    check(lib.sma_pack_mask_tiles(mask_ptr, packed_ptr, tile_bits_ptr, B, H, N, stream))


def attention_fwd_tiles(params: AttentionParams, tile_bits_ptr: int, stream: int) -> None:
    check(lib.sma_attention_fwd_tiles(ctypes.byref(params), tile_bits_ptr, stream))


def attention_workspace_bytes(B: int, H: int, N: int) -> int:
    return int(lib.sma_attention_workspace_bytes(B, H, N))


def attention_fwd_planned(params: AttentionParams, workspace_ptr: int, workspace_bytes: int, stream: int) -> None:
    check(lib.sma_attention_fwd_planned(ctypes.byref(params), workspace_ptr, workspace_bytes, stream))


def attention_bwd_workspace_bytes(B: int, H: int, N: int) -> int:
    return int(lib.sma_attention_bwd_workspace_bytes(B, H, N))


def attention_bwd(params: AttentionParams, dout_ptr: int, dq_ptr: int, dk_ptr: int, dv_ptr: int, workspace_ptr: int,
                  workspace_bytes: int, stream: int) -> None:
    check(lib.sma_attention_bwd(ctypes.byref(params), dout_ptr, dq_ptr, dk_ptr, dv_ptr, workspace_ptr, workspace_bytes,
                                stream))


def attention_fwd_static_workspace(params: AttentionParams, stream: int) -> None:
    """The forward pass with the tile lists in the library's built-in workspace (allocates nothing; calls on one
    device must not overlap; at most SMA_STATIC_WORKSPACE_BYTES of tile lists)."""
    check(lib.sma_attention_fwd_static_workspace(ctypes.byref(params), stream))


def device_status() -> None:
    """Synchronises the current device and raises if a kernel reported a bounded-wait timeout."""
    check(lib.sma_device_status())
