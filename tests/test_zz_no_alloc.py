"""sma_attention_fwd_static_workspace: the forward pass for callers that may not allocate device memory (a
service past its start-up phase with a fixed memory budget, a latency-critical loop that cannot afford the
device-wide synchronisation of cudaMalloc, a plug-in host that passes tensors but no allocator).  Its tile lists
live in an array inside the library image instead of a caller's workspace.

This file sorts last on purpose: if the entry point is broken, a run that stops at the first failure has already
run every other test.  It needs nothing from the other tests and passes in a fresh process as well.
"""
import pytest
import torch

import gpu_util as gu
from sparse_mask_attention_b200 import _capi, sparse_attn_cuda, workloads

pytestmark = pytest.mark.gpu


def _inputs(B, H, N, kind, keep, dtype, seed):
    cfg = workloads.Config("no_alloc", B, H, N, dtype, kind, keep, seed=seed)
    return workloads.make_inputs(cfg)


def _case(B, H, N, kind, keep, dtype, seed):
    q, k, v, mask = (t.cuda() for t in _inputs(B, H, N, kind, keep, dtype, seed))
    return q, k, v, sparse_attn_cuda.pack_mask(mask)


def _call(entry, q, k, v, packed):
    B, H, N, D = q.shape
    out = torch.full_like(q, 5.0)
    lse = torch.full((B, H, N), 9.0, dtype=torch.float32, device=q.device)
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed = q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr()
    p.out, p.lse = out.data_ptr(), lse.data_ptr()
    p.B, p.H, p.N, p.D, p.scale = B, H, N, D, D ** -0.5
    p.dtype = _capi.SMA_DTYPE_F16 if q.dtype == torch.float16 else _capi.SMA_DTYPE_BF16
    p.save_lse, p.variant = 1, _capi.SMA_VARIANT_DEFAULT
    entry(p, None)
    torch.cuda.synchronize()
    _capi.device_status()
    return out, lse


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    # a long block-sparse problem first, a short dense-ish one second: the second call finds the first call's tile
    # lists still in the shared array and must not be affected by them
    cases = [_case(1, 2, 2048, "block", 0.1, torch.float16, 21), _case(2, 3, 320, "iid", 0.3, torch.bfloat16, 22)]
    want = [_call(_capi.attention_fwd, *c) for c in cases]
    free_before, _ = torch.cuda.mem_get_info()
    got = [_call(_capi.attention_fwd_static_workspace, *c) for c in cases]
    free_after, _ = torch.cuda.mem_get_info()
    for (o_want, l_want), (o_got, l_got) in zip(want, got):
        # same kernels on the same tile lists: the tests' tolerance (2e-3 + 1e-2*|ref|) holds with room to spare,
        # the results are in fact bitwise equal
        assert torch.equal(o_got, o_want) and torch.equal(l_got, l_want)
    # and once more in the opposite order
    again = [_call(_capi.attention_fwd_static_workspace, *c) for c in reversed(cases)]
    assert torch.equal(again[0][0], want[1][0]) and torch.equal(again[1][0], want[0][0])
    # the outputs above are torch's; the entry point itself took nothing from the device
    assert free_after >= free_before - (2 << 20)
    # and the results are right, not merely equal to one another: the fp32 oracle on the same inputs
    for (B, H, N, kind, keep, dtype, seed), (o_got, l_got) in zip(
            [(1, 2, 2048, "block", 0.1, torch.float16, 21), (2, 3, 320, "iid", 0.3, torch.bfloat16, 22)], got):
        q, k, v, mask = _inputs(B, H, N, kind, keep, dtype, seed)
        ref, ref_lse = gu.oracle_for(q, k, v, mask)
        gu.assert_close(gu.to_np32(o_got), ref, "static workspace N=%d" % N)
        gu.assert_lse_close(l_got.cpu().numpy(), ref_lse, "static workspace N=%d" % N)


def test_calls_queued_without_synchronising_each_see_their_own_tile_lists():
    # Four calls of different shapes and masks queued on one stream, nothing waited for in between.  They all
    # use the same built-in array, and each attention kernel becomes resident while the tile-list kernel before
    # it is still running: it must read that kernel's lists, never a stale copy of the previous call's.
    specs = [(2, 4, 512, "block", 0.2, torch.float16, 41), (1, 3, 1024, "causal_iid", 0.5, torch.bfloat16, 42),
             (3, 2, 384, "iid", 0.1, torch.float16, 43), (2, 4, 512, "block", 0.6, torch.float16, 44)]
    cases = [_case(*s) for s in specs]
    want = [_call(_capi.attention_fwd, *c) for c in cases]
    outs = []
    torch.cuda.synchronize()
    for q, k, v, packed in cases:
        B, H, N, D = q.shape
        out = torch.full_like(q, 5.0)
        lse = torch.full((B, H, N), 9.0, dtype=torch.float32, device=q.device)
        p = _capi.AttentionParams()
        p.q, p.k, p.v, p.mask_packed = q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr()
        p.out, p.lse = out.data_ptr(), lse.data_ptr()
        p.B, p.H, p.N, p.D, p.scale = B, H, N, D, D ** -0.5
        p.dtype = _capi.SMA_DTYPE_F16 if q.dtype == torch.float16 else _capi.SMA_DTYPE_BF16
        p.save_lse, p.variant = 1, _capi.SMA_VARIANT_DEFAULT
        _capi.attention_fwd_static_workspace(p, None)
        outs.append((out, lse))
    torch.cuda.synchronize()
    _capi.device_status()
    for (o_want, l_want), (o_got, l_got) in zip(want, outs):
        assert torch.equal(o_got, o_want) and torch.equal(l_got, l_want)


def test_shapes_beyond_the_built_in_workspace_are_refused():
    q, k, v, packed = _case(1, 1, 64, "iid", 0.5, torch.float16, 23)
    out = torch.full_like(q, 5.0)
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr(), out.data_ptr(), None
    p.D, p.scale, p.dtype, p.save_lse, p.variant = 64, 0.125, _capi.SMA_DTYPE_F16, 0, 0
    # 64 x 64 heads of 16384 keys need 64*64*128 items x 528 bytes of tile lists, far beyond 1 MiB
    p.B, p.H, p.N = 64, 64, 16384
    assert _capi.attention_workspace_bytes(64, 64, 16384) > _capi.SMA_STATIC_WORKSPACE_BYTES
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_fwd_static_workspace(p, None)
    assert e.value.status == _capi.SMA_ERR_STATIC_WORKSPACE_EXCEEDED and "built-in workspace" in str(e.value)
    torch.cuda.synchronize()
    assert (out == 5.0).all(), "nothing may be launched for a refused shape"
    # the largest headline-like batch that still fits: 1 MiB / 32 bytes per item at N = 512 (a workspace also holds
    # the 16 bytes of the attention kernel's work-queue word, which the built-in array has on top of its 1 MiB)
    assert _capi.attention_workspace_bytes(128, 64, 512) == _capi.SMA_STATIC_WORKSPACE_BYTES + 16
