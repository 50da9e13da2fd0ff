"""Python API of sparse-mask attention on B200 — same surface as the reference's
python/sparse_attention.py: ``sparse_attention`` (:120-154), ``sparse_attention_func`` (:157-177),
``SparseAttentionFunction`` (:49-113), ``pack_mask`` (:184-201), ``sparse_attention_ref`` (:24-42) and
``generate_random_sparse_mask`` (:204-211).

The compute path is the CUDA library only.  Where the reference silently falls back to PyTorch when
its extension is absent or the tensors are on the CPU, this module raises: the library must be built
and the tensors must be on a CUDA device.
"""
from __future__ import annotations

import math

import torch
from torch.autograd import Function

from . import sparse_attn_cuda

HAS_CUDA_EXT = True  # importing sparse_attn_cuda above raises if the library is missing


def sparse_attention_ref(q, k, v, mask):
    """Dense masked-softmax attention in plain PyTorch (any device), for checking results.

    mask: bool [B, H, N, N], True = keep.  Rows without a kept column give zeros.
    Never used by sparse_attention()/sparse_attention_func().
    """
    d = q.shape[-1]
    logits = (q @ k.transpose(-1, -2)) * (1.0 / math.sqrt(d))
    logits = logits.masked_fill(mask.logical_not(), float("-inf"))
    weights = torch.nan_to_num(torch.softmax(logits, dim=-1), nan=0.0)
    return weights @ v


class SparseAttentionFunction(Function):
    """autograd wrapper: CUDA forward and CUDA backward (no dense [N, N] tensor in either direction)."""

    @staticmethod
    def forward(ctx, q, k, v, mask_packed, mask_bool, scale, seq_len):
        B, H, N, D = q.shape
        out = torch.empty_like(q, memory_format=torch.contiguous_format)
        lse = torch.empty(B, H, N, device=q.device, dtype=torch.float32)
        sparse_attn_cuda.forward(q, k, v, mask_packed, out, lse, scale, True)
        ctx.save_for_backward(q, k, v, out, lse, mask_packed, mask_bool)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        # The reference's autograd function hands exactly these arguments to sparse_attn_cuda.backward
        # (python/sparse_attention.py:80-94); the gradient is the one its PyTorch branch defines (:96-111).
        q, k, v, out, lse, mask_packed, mask_bool = ctx.saved_tensors
        dq = torch.empty_like(q, memory_format=torch.contiguous_format)
        dk = torch.empty_like(k, memory_format=torch.contiguous_format)
        dv = torch.empty_like(v, memory_format=torch.contiguous_format)
        sparse_attn_cuda.backward(dout, q, k, v, out, lse, mask_packed, dq, dk, dv, ctx.scale)
        return dq, dk, dv, None, None, None, None


def _check_inputs(q, k, v, mask):
    assert q.shape == k.shape == v.shape, "q/k/v must have the same shape"
    assert q.device == k.device == v.device == mask.device, "all tensors must be on the same device"
    assert mask.dtype == torch.bool, "mask must be a bool tensor"
    if not q.is_cuda:
        raise RuntimeError("sparse_attention needs CUDA tensors: there is no CPU path "
                           "(use sparse_attention_ref for a PyTorch check on the CPU)")


def sparse_attention(q, k, v, mask):
    """Masked attention ``softmax(mask ? q k^T / sqrt(D) : -inf) v``.

    q, k, v: [B, H, N, 64], fp16 / bf16 / fp32 (fp32 is computed in bf16 and returned as fp32, as in the
    reference); mask: bool [B, H, N, N], True = keep.  Returns [B, H, N, 64] in the input dtype.
    """
    _check_inputs(q, k, v, mask)
    B, H, N, D = q.shape
    scale = 1.0 / math.sqrt(D)
    orig_dtype = q.dtype
    if orig_dtype == torch.float32:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    mask_packed = pack_mask(mask)
    out = SparseAttentionFunction.apply(q, k, v, mask_packed, mask, scale, N)
    if orig_dtype == torch.float32:
        out = out.float()
    return out


def sparse_attention_func(q, k, v, mask):
    """Inference-only variant of sparse_attention: no autograd graph, no log-sum-exp output."""
    _check_inputs(q, k, v, mask)
    scale = 1.0 / math.sqrt(q.shape[-1])
    orig_dtype = q.dtype
    if orig_dtype == torch.float32:
        q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    # (nothing below is seen by autograd: the output is allocated here and written by the library)
    out = torch.empty_like(q, memory_format=torch.contiguous_format)
    sparse_attn_cuda.pack_and_forward(q, k, v, mask, out, None, scale, False)
    if orig_dtype == torch.float32:
        out = out.float()
    return out


_host_streams = {}  # device index -> the two side streams of sparse_attention_host


def sparse_attention_host(q, k, v, mask, out=None, device=None, chunks: int = 4, sync: bool = True):
    """`sparse_attention_func` for tensors that live in HOST memory: copies q, k, v, mask to the GPU, runs
    pack_mask + the fused forward there and copies the result back, pipelined over `chunks` slices of the batch
    on two streams so that the copy of one slice to the device, the kernels of another and the copy back of a
    third overlap (PCIe carries both directions at once).  Not part of the reference's API, which takes CUDA
    tensors only (python/sparse_attention.py:132-134).

    q, k, v: [B, H, N, 64] fp16 / bf16 / fp32 on the CPU, mask bool [B, H, N, N] on the CPU; pinned memory makes the
    copies asynchronous.  `out`: optional CPU tensor like q (pinned for an asynchronous copy back).  With
    `sync=False` the call returns once everything is queued behind the device's current stream, and `out` is valid
    after that stream has been synchronised.
    """
    assert q.shape == k.shape == v.shape, "q/k/v must have the same shape"
    assert mask.dtype == torch.bool, "mask must be a bool tensor"
    if q.is_cuda or k.is_cuda or v.is_cuda or mask.is_cuda:
        raise RuntimeError("sparse_attention_host takes CPU tensors; use sparse_attention_func for CUDA tensors")
    if not torch.cuda.is_available():
        raise RuntimeError("sparse_attention_host needs a CUDA device: there is no CPU path")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    B = q.shape[0]
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    assert out.shape == q.shape and out.dtype == q.dtype and not out.is_cuda, "out must be a CPU tensor like q"
    q, k, v, mask = (t.contiguous() for t in (q, k, v, mask))
    n_chunks = max(1, min(int(chunks), B))
    bounds = [(B * c) // n_chunks for c in range(n_chunks + 1)]
    with torch.cuda.device(dev):
        side = _host_streams.get(dev.index)
        if side is None:
            side = _host_streams[dev.index] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
        current = torch.cuda.current_stream(dev)
        for s in side:
            s.wait_stream(current)
        for c in range(n_chunks):
            b0, b1 = bounds[c], bounds[c + 1]
            if b0 == b1:
                continue
            with torch.cuda.stream(side[c % 2]):
                dq, dk, dv, dm = (t[b0:b1].to(dev, non_blocking=True) for t in (q, k, v, mask))
                o = sparse_attention_func(dq, dk, dv, dm)
                out[b0:b1].copy_(o, non_blocking=True)
        for s in side:
            current.wait_stream(s)
        if sync:
            current.synchronize()
    return out


def pack_mask(mask: torch.Tensor) -> torch.Tensor:
    """bool [B, H, N, N] -> int32 [B, H, N, ceil(N/32)]; bit j of word w is mask[..., 32*w + j]."""
    return sparse_attn_cuda.pack_mask(mask)


def generate_random_sparse_mask(B, H, N, sparsity=0.75, device="cuda"):
    """i.i.d. mask with P(keep) = 1 - sparsity."""
    return torch.rand(B, H, N, N, device=device) > sparsity
