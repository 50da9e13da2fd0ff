"""Stand-in for the reference's compiled extension module ``sparse_attn_cuda``.

Exposes the two functions the reference binds in csrc/binding.cpp:68-71 — ``forward`` (:9-47) and
``pack_mask`` (:49-66) — with the same positional signatures, on top of the C ABI of libsma_b200.so.
Differences from the reference binding, all on the safe side:

* launches under a device guard for the tensors' device (the reference uses the current device's
  stream whatever device the tensors live on);
* validates what the reference leaves unchecked (D == 64, matching shapes/devices/dtypes, mask
  shape, contiguity of the outputs) and raises ``RuntimeError`` like ``TORCH_CHECK`` does;
* ``lse`` may be ``None`` when ``is_training`` is false (the reference's Python wrapper passes None);
* ``pack_mask`` allocates with ``torch.empty``: the kernel writes every word.
"""
from __future__ import annotations

import ctypes

import torch

from . import _capi

_DTYPES = {torch.float16: _capi.SMA_DTYPE_F16, torch.bfloat16: _capi.SMA_DTYPE_BF16}

# Kernel variant used by forward(); tests switch it to exercise the alternatives.
variant = _capi.SMA_VARIANT_DEFAULT

# Sequences longer than this take sma_attention_fwd_planned: the tile lists are computed by a kernel of their own
# into a workspace allocated here, instead of by one warp per 128 query rows inside the attention kernel.  Up to
# 32 key tiles per row block the search inside the kernel is hidden behind the arithmetic (measured on B200: equal
# at N = 2048, 71 -> 55 us at N = 4096 block-sparse, 110 -> 60 us at N = 16384 banded).
PLAN_ABOVE_SEQ_LEN = 2048


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream_of(device: torch.device) -> int:
    """Handle of torch's current stream on ``device`` (the fast accessor when this torch has it)."""
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


class _device_guard:
    """Makes ``device`` current for the launch; does nothing when it already is (the common case)."""

    __slots__ = ("index", "prev")

    def __init__(self, device: torch.device) -> None:
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = -1

    def __enter__(self) -> None:
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc) -> None:
        if self.prev >= 0:
            torch.cuda.set_device(self.prev)


def pack_mask(mask: torch.Tensor) -> torch.Tensor:
    """bool [B, H, N, N] on a CUDA device -> int32 [B, H, N, ceil(N/32)], LSB-first bits, zero tail."""
    _require(isinstance(mask, torch.Tensor), "mask must be a tensor")
    _require(mask.is_cuda, "mask must be CUDA tensor")
    _require(mask.dim() == 4, "mask must be 4D [B, H, N, N]")
    _require(mask.dtype in (torch.bool, torch.uint8), "mask must be bool")
    B, H, N, N2 = mask.shape
    _require(N == N2, "mask must be square in its last two dimensions")
    _require(B >= 1 and H >= 1 and N >= 1, "mask dimensions must be >= 1")
    mask = mask.contiguous()
    n_words = (N + 31) // 32
    packed = torch.empty((B, H, N, n_words), dtype=torch.int32, device=mask.device)
    with _device_guard(mask.device):
        _capi.pack_mask(mask.data_ptr(), packed.data_ptr(), B, H, N, _stream_of(mask.device))
    return packed


def _strided_ok(t: torch.Tensor) -> bool:
    """Whether the library can address ``t`` ([B, H, N, 64]) in place: rows contiguous, every other stride a positive
    multiple of 8 elements (16 bytes), base 16-byte aligned."""
    if t.is_contiguous():
        return True
    s = t.stride()
    return s[3] == 1 and s[0] > 0 and s[1] > 0 and s[2] > 0 and (s[0] | s[1] | s[2]) % 8 == 0 and t.data_ptr() % 16 == 0


def _params_for(q, k, v, out, lse, scale, is_training, dense: bool = False):
    """Checks q/k/v/out/lse against one another (one pass) and fills the argument block; returns it with the q, k, v
    it points to (the caller keeps them alive until the launch has been issued).  ``dense``: copy anything that is
    not in the dense layout (the backward pass takes no strides)."""
    _require(q.is_cuda, "q must be CUDA tensor")
    _require(q.dim() == 4, "q must be 4D")
    dtype = _DTYPES.get(q.dtype)
    _require(dtype is not None, "Unsupported dtype, need BF16 or FP16")
    B, H, N, D = q.shape
    _require(D == 64, "head dimension must be 64")
    sig = (q.shape, q.dtype, q.device)
    if (k.shape, k.dtype, k.device) != sig or (v.shape, v.dtype, v.device) != sig or (out.shape, out.dtype, out.device) != sig:
        for name, t in (("k", k), ("v", v), ("out", out)):
            _require(t.shape == q.shape, "%s must have the shape of q" % name)
            _require(t.dtype == q.dtype, "%s must have the dtype of q" % name)
            _require(t.device == q.device, "%s must be on the device of q" % name)
    save_lse = bool(is_training)
    if save_lse:
        _require(lse is not None, "lse is required when is_training is true")
        _require(lse.device == q.device and lse.dtype == torch.float32, "lse must be float32 on the device of q")
        _require(tuple(lse.shape) == (B, H, N) and lse.is_contiguous(), "lse must be contiguous [B, H, N]")
    # The library reads q, k, v and writes out through their own strides as long as rows are contiguous and every
    # other stride is a multiple of 16 bytes (a view into a packed projection, a transposed [B, N, H, 64] tensor ...);
    # only other layouts are copied to the dense one, which is what the reference's binding always does
    # (csrc/binding.cpp:28-33).
    if dense:
        q, k, v, out = q.contiguous(), k.contiguous(), v.contiguous(), out.contiguous()  # out is an input there
    else:
        q, k, v = (t if _strided_ok(t) else t.contiguous() for t in (q, k, v))
        _require(_strided_ok(out), "out must have contiguous rows and strides that are multiples of 8 elements")
    params = _capi.AttentionParams()
    params.q, params.k, params.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    params.out = out.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("out_strides", out)):
        if not t.is_contiguous():
            setattr(params, name, (ctypes.c_int64 * 3)(t.stride(0), t.stride(1), t.stride(2)))
    params.lse = lse.data_ptr() if save_lse else None
    params.B, params.H, params.N, params.D = B, H, N, D
    params.scale = float(scale)
    params.dtype = dtype
    params.save_lse = int(save_lse)
    params.variant = int(variant)
    return params, (q, k, v, out)


def forward(q, k, v, mask_packed, out, lse, scale, is_training) -> None:
    """Fused masked attention forward; writes ``out`` (and ``lse`` when ``is_training``) in place."""
    params, keep = _params_for(q, k, v, out, lse, scale, is_training)
    B, H, N = params.B, params.H, params.N
    _require(mask_packed.device == q.device, "mask_packed must be on the device of q")
    _require(mask_packed.dtype == torch.int32, "mask_packed must be int32")
    _require(tuple(mask_packed.shape) == (B, H, N, (N + 31) // 32), "mask_packed must be [B, H, N, ceil(N/32)]")
    mask_packed = mask_packed.contiguous()
    params.mask_packed = mask_packed.data_ptr()
    with _device_guard(q.device):
        if N > PLAN_ABOVE_SEQ_LEN:
            nbytes = _capi.attention_workspace_bytes(B, H, N)
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=q.device)  # stream-ordered: safe to drop on return
            _capi.attention_fwd_planned(params, workspace.data_ptr(), nbytes, _stream_of(q.device))
        else:
            _capi.attention_fwd(params, _stream_of(q.device))


def backward(dout, q, k, v, out, lse, mask_packed, dq, dk, dv, scale) -> None:
    """Gradients of the fused attention: writes ``dq``, ``dk``, ``dv`` in place.  The argument list is the one the
    reference's autograd function passes to ``sparse_attn_cuda.backward`` (python/sparse_attention.py:90-94), a
    function its extension never got; the gradient is that of its PyTorch branch (python/sparse_attention.py:96-111)."""
    params, keep = _params_for(q, k, v, out, lse, scale, True, dense=True)
    B, H, N = params.B, params.H, params.N
    for name, t in (("dout", dout), ("dq", dq), ("dk", dk), ("dv", dv)):
        _require(t.shape == q.shape and t.dtype == q.dtype and t.device == q.device, "%s must match q" % name)
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        _require(t.is_contiguous(), "%s must be contiguous" % name)
    _require(mask_packed.device == q.device, "mask_packed must be on the device of q")
    _require(mask_packed.dtype in (torch.int32, torch.uint32), "mask_packed must be int32")
    _require(tuple(mask_packed.shape) == (B, H, N, (N + 31) // 32), "mask_packed must be [B, H, N, ceil(N/32)]")
    dout = dout.contiguous()
    mask_packed = mask_packed.contiguous()
    params.mask_packed = mask_packed.data_ptr()
    with _device_guard(q.device):
        nbytes = _capi.attention_bwd_workspace_bytes(B, H, N)
        workspace = torch.empty(nbytes, dtype=torch.uint8, device=q.device)  # stream-ordered: safe to drop on return
        _capi.attention_bwd(params, dout.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), workspace.data_ptr(),
                            nbytes, _stream_of(q.device))


def pack_and_forward(q, k, v, mask, out, lse, scale, is_training) -> torch.Tensor:
    """``pack_mask(mask)`` followed by ``forward(...)`` with one call into the library (one trip through ctypes
    instead of two); returns the packed mask.  Not part of the reference extension's interface: the Python layer
    above uses it where the reference calls the two functions back to back (python/sparse_attention.py:139-146)."""
    params, keep = _params_for(q, k, v, out, lse, scale, is_training)
    B, H, N = params.B, params.H, params.N
    _require(mask.device == q.device, "mask must be on the device of q")
    _require(mask.dtype in (torch.bool, torch.uint8), "mask must be bool")
    _require(tuple(mask.shape) == (B, H, N, N), "mask must be [B, H, N, N]")
    mask = mask.contiguous()
    packed = torch.empty((B, H, N, (N + 31) // 32), dtype=torch.int32, device=q.device)
    params.mask_packed = packed.data_ptr()
    with _device_guard(q.device):
        if N > PLAN_ABOVE_SEQ_LEN and N % 64 == 0 and mask.data_ptr() % 32 == 0:
            # long sequences: the packing kernel leaves a bit per (mask row, 64-key tile) beside the packed words and
            # the attention kernel takes its tile lists from them -- as fast as the tile-list kernel with its
            # workspace (below), with two launches instead of three and one call into the library.  Up to
            # PLAN_ABOVE_SEQ_LEN the attention kernel's own scan of the packed mask is faster than either.
            tile_bits = torch.empty(_capi.tile_bits_bytes(B, H, N) // 2 + 2, dtype=torch.int16, device=q.device)
            counter = tile_bits.data_ptr() + tile_bits.numel() * 2 - 4  # the attention kernel's work queue
            _capi.sparse_attention_fwd(params, mask.data_ptr(), tile_bits.data_ptr(), counter, _stream_of(q.device))
        elif N > PLAN_ABOVE_SEQ_LEN:
            stream = _stream_of(q.device)
            _capi.pack_mask(mask.data_ptr(), packed.data_ptr(), B, H, N, stream)
            nbytes = _capi.attention_workspace_bytes(B, H, N)
            workspace = torch.empty(nbytes, dtype=torch.uint8, device=q.device)
            _capi.attention_fwd_planned(params, workspace.data_ptr(), nbytes, stream)
        else:
            counter = torch.empty(1, dtype=torch.int32, device=q.device)  # the attention kernel's work queue
            _capi.sparse_attention_fwd(params, mask.data_ptr(), None, counter.data_ptr(), _stream_of(q.device))
    return packed
