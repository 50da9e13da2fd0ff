"""CPU oracle for the mask-packing + masked-attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy (and in torch-on-CPU for the timed baseline), what the reference
project computes for this path; it exists to check the CUDA library and to provide the CPU baseline
that bench.py reports.  Nothing in the product package imports it.

Pinned: tests/test_oracle_golden.py checks every function here against vectors produced by the
reference's own Python code (tests/golden/make_golden.py imports the reference and writes them).

Reference code followed (paths inside xgbj/sparse-mask-attention):
  pack_mask_*      python/sparse_attention.py:184-201 (CPU branch), csrc/sparse_attention.cu:549-568
  attention_*      python/sparse_attention.py:24-42 (sparse_attention_ref), duplicate run.py:158-165
  lse              python/sparse_attention.py:72-74 (torch.logsumexp over the masked, scaled scores)
  attention_bwd_np python/sparse_attention.py:96-111 (the autograd function's PyTorch gradient)
"""
from __future__ import annotations

import math

import numpy as np


# --------------------------------------------------------------------------------------------
# mask packing (bit-exact)
# --------------------------------------------------------------------------------------------
def pack_mask_np(mask: np.ndarray) -> np.ndarray:
    """bool [B,H,N,N] -> int32 [B,H,N,ceil(N/32)]: bit j of word w = mask[..., 32*w + j]; tail bits 0.

    Follows python/sparse_attention.py:194-201: ``packed[..., w] |= mask[..., col].int() << bit``.
    """
    mask = np.asarray(mask)
    B, H, N, N2 = mask.shape
    assert N == N2
    nw = (N + 31) // 32
    padded = np.zeros((B, H, N, nw * 32), dtype=np.uint8)
    padded[..., :N] = mask != 0
    as_bytes = np.packbits(padded, axis=-1, bitorder="little")        # [B,H,N,nw*4], LSB-first
    words = as_bytes.reshape(B, H, N, nw, 4).astype(np.uint32)
    packed = words[..., 0] | (words[..., 1] << 8) | (words[..., 2] << 16) | (words[..., 3] << 24)
    return packed.astype(np.uint32).view(np.int32)


def pack_mask_loops(mask) -> list:
    """Same packing as nested Python loops over single elements (tiny inputs only); returns nested
    lists of unsigned ints.  Mirrors csrc/sparse_attention.cu:561-567."""
    mask = np.asarray(mask)
    B, H, N, _ = mask.shape
    nw = (N + 31) // 32
    out = [[[[0] * nw for _ in range(N)] for _ in range(H)] for _ in range(B)]
    for b in range(B):
        for h in range(H):
            for r in range(N):
                for w in range(nw):
                    word = 0
                    for bit in range(32):
                        col = 32 * w + bit
                        if col < N and mask[b, h, r, col]:
                            word |= 1 << bit
                    out[b][h][r][w] = word
    return out


def unpack_mask_np(packed: np.ndarray, N: int) -> np.ndarray:
    """Inverse of pack_mask_np (reader semantics of csrc/utils.cuh:47-56)."""
    words = np.asarray(packed).view(np.uint32)
    cols = np.arange(N)
    return ((words[..., cols // 32] >> (cols % 32).astype(np.uint32)) & 1).astype(bool)


# --------------------------------------------------------------------------------------------
# masked attention
# --------------------------------------------------------------------------------------------
def attention_np(q, k, v, mask, scale=None, dtype=np.float32):
    """out [B,H,N,D], lse [B,H,N] for ``softmax(mask ? scale*q k^T : -inf) v`` computed in ``dtype``.

    Rows with no kept column: out = 0 (python/sparse_attention.py:38-39 nan_to_num), lse = -inf.
    """
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    mask = np.asarray(mask).astype(bool)
    D = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    scores = np.matmul(q, np.swapaxes(k, -1, -2)) * dtype(scale)
    scores = np.where(mask, scores, dtype(-np.inf))
    row_max = scores.max(axis=-1, keepdims=True)
    safe_max = np.where(np.isfinite(row_max), row_max, dtype(0))
    e = np.exp(scores - safe_max)                    # masked entries: exp(-inf) = 0
    denom = e.sum(axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        attn = np.where(denom > 0, e / denom, dtype(0))
        lse = np.where(denom[..., 0] > 0, safe_max[..., 0] + np.log(denom[..., 0]), dtype(-np.inf))
    out = np.matmul(attn, v)
    return out.astype(dtype), lse.astype(dtype)


def attention_bwd_np(q, k, v, mask, dout, scale=None, dtype=np.float64):
    """dq, dk, dv of ``out = softmax(mask ? scale*q k^T : -inf) v`` for the upstream gradient ``dout``.

    Restates the PyTorch fallback of the reference's autograd function (python/sparse_attention.py:96-111):
    attn with rows that keep nothing set to 0, dv = attn^T dout, dattn = dout v^T (0 where masked),
    ds = scale * attn * (dattn - rowsum(dattn * attn)), dq = ds k, dk = ds^T q.
    """
    q = np.asarray(q, dtype=dtype)
    k = np.asarray(k, dtype=dtype)
    v = np.asarray(v, dtype=dtype)
    dout = np.asarray(dout, dtype=dtype)
    mask = np.asarray(mask).astype(bool)
    D = q.shape[-1]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    scores = np.matmul(q, np.swapaxes(k, -1, -2)) * dtype(scale)
    scores = np.where(mask, scores, dtype(-np.inf))
    row_max = scores.max(axis=-1, keepdims=True)
    safe_max = np.where(np.isfinite(row_max), row_max, dtype(0))
    e = np.exp(scores - safe_max)
    denom = e.sum(axis=-1, keepdims=True)
    with np.errstate(divide="ignore", invalid="ignore"):
        attn = np.where(denom > 0, e / denom, dtype(0))
    dv = np.matmul(np.swapaxes(attn, -1, -2), dout)
    dattn = np.where(mask, np.matmul(dout, np.swapaxes(v, -1, -2)), dtype(0))
    ds = attn * (dattn - (dattn * attn).sum(axis=-1, keepdims=True)) * dtype(scale)
    dq = np.matmul(ds, k)
    dk = np.matmul(np.swapaxes(ds, -1, -2), q)
    return dq.astype(dtype), dk.astype(dtype), dv.astype(dtype)


def attention_torch_cpu(q, k, v, mask):
    """The reference's sparse_attention_ref restated with torch CPU ops (multi-threaded); this is what
    the reference itself runs when its tensors are on the CPU (python/sparse_attention.py:148-149)."""
    import torch

    d = q.shape[-1]
    s = torch.matmul(q, k.transpose(-2, -1)) * (1.0 / math.sqrt(d))
    s = s.masked_fill(~mask, float("-inf"))
    a = torch.nan_to_num(torch.softmax(s, dim=-1), nan=0.0)
    return torch.matmul(a, v)


def pack_mask_torch_cpu(mask):
    """Reference CPU packing loop (python/sparse_attention.py:194-201) restated with torch ops."""
    import torch

    B, H, N, _ = mask.shape
    nw = (N + 31) // 32
    packed = torch.zeros(B, H, N, nw, dtype=torch.int32)
    for w in range(nw):
        lo, hi = 32 * w, min(32 * w + 32, N)
        for bit, col in enumerate(range(lo, hi)):
            packed[..., w] |= mask[..., col].to(torch.int32) << bit
    return packed


# --------------------------------------------------------------------------------------------
# tolerance used everywhere: |out - ref| <= atol + rtol * |ref|
# --------------------------------------------------------------------------------------------
ATOL = 2e-3
RTOL = 1e-2


def compare(out, ref, atol=ATOL, rtol=RTOL):
    """Returns dict(ok, max_abs, max_rel, worst_excess, n_bad) for the element-wise tolerance check."""
    out = np.asarray(out, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    err = np.abs(out - ref)
    bound = atol + rtol * np.abs(ref)
    bad = ~(err <= bound)  # NaN counts as bad
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.where(np.abs(ref) > 1e-3, err / np.abs(ref), 0.0)
    return dict(ok=not bad.any(), max_abs=float(np.nanmax(err)) if err.size else 0.0,
                max_rel=float(np.nanmax(rel)) if rel.size else 0.0,
                worst_excess=float(np.nanmax(err - bound)) if err.size else 0.0, n_bad=int(bad.sum()))
