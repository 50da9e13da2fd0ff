"""sma_attention_fwd_planned (tile lists computed ahead into a caller's workspace) against sma_attention_fwd
(tile lists found inside the attention kernel): same inputs, bitwise the same outputs; workspace checks."""
import numpy as np
import pytest
import torch

import gpu_util as gu
from sparse_mask_attention_b200 import _capi, sparse_attn_cuda, workloads

pytestmark = pytest.mark.gpu


def _params(q, k, v, packed, out, lse):
    B, H, N, D = q.shape
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr(), out.data_ptr()
    p.lse = lse.data_ptr()
    p.B, p.H, p.N, p.D, p.scale = B, H, N, D, D ** -0.5
    p.dtype = _capi.SMA_DTYPE_F16 if q.dtype == torch.float16 else _capi.SMA_DTYPE_BF16
    p.save_lse, p.variant = 1, 0
    return p


@pytest.mark.parametrize("N,kind,dtype", [(64, "iid", torch.float16), (100, "iid", torch.float16),
                                          (512, "block", torch.float16), (1024, "causal_iid", torch.bfloat16),
                                          (2112, "block", torch.float16), (4096, "block", torch.float16)])
def test_planned_equals_unplanned_bitwise(N, kind, dtype):
    cfg = workloads.Config("planned", 2, 3, N, dtype, kind, 0.2, seed=N)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    packed = sparse_attn_cuda.pack_mask(mask)
    B, H = 2, 3
    outs = []
    for planned in (False, True):
        out = torch.full_like(q, 3.0)
        lse = torch.full((B, H, N), 7.0, dtype=torch.float32, device="cuda")
        p = _params(q, k, v, packed, out, lse)
        if planned:
            nbytes = _capi.attention_workspace_bytes(B, H, N)
            assert nbytes > 0 and nbytes % 16 == 0
            ws = torch.full((nbytes + 32,), 0xAB, dtype=torch.uint8, device="cuda")
            _capi.attention_fwd_planned(p, ws.data_ptr(), nbytes, None)
            torch.cuda.synchronize()
            assert (ws[nbytes:] == 0xAB).all(), "write past the workspace"
        else:
            _capi.attention_fwd(p, None)
        torch.cuda.synchronize()
        _capi.device_status()
        outs.append((out, lse))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    # and both agree with the fp32 oracle on these inputs, not only with each other
    ref, ref_lse = gu.oracle_for(q, k, v, mask)
    gu.assert_close(gu.to_np32(outs[1][0]), ref, "planned N=%d %s" % (N, kind))
    gu.assert_lse_close(outs[1][1].cpu().numpy(), ref_lse, "planned N=%d %s" % (N, kind))


@pytest.mark.parametrize("planned", [False, True])
def test_many_row_blocks_that_keep_nothing(planned):
    # 960 work items (128-row blocks) on 296 streams, three quarters of them without a single kept key, scattered:
    # every stream meets runs of empty items between non-empty ones, which is where a tile-list slot could be
    # recycled while a consumer still has to read it
    B, H, N = 10, 12, 1024
    cfg = workloads.Config("empty_blocks", B, H, N, torch.float16, "iid", 0.3, seed=77)
    q, k, v, mask = workloads.make_inputs(cfg)
    g = torch.Generator().manual_seed(78)
    dead = torch.rand(B, H, N // 128, generator=g) < 0.75
    mask &= ~dead.repeat_interleave(128, dim=-1)[..., None]
    qd, kd, vd, md = (t.cuda() for t in (q, k, v, mask))
    packed = sparse_attn_cuda.pack_mask(md)
    out = torch.full_like(qd, 3.0)
    lse = torch.full((B, H, N), 7.0, dtype=torch.float32, device="cuda")
    p = _params(qd, kd, vd, packed, out, lse)
    if planned:
        nbytes = _capi.attention_workspace_bytes(B, H, N)
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        _capi.attention_fwd_planned(p, ws.data_ptr(), nbytes, None)
    else:
        _capi.attention_fwd(p, None)
    torch.cuda.synchronize()
    _capi.device_status()
    ref, ref_lse = gu.oracle_for(q, k, v, mask)
    gu.assert_close(gu.to_np32(out), ref, "empty row blocks")
    gu.assert_lse_close(lse.cpu().numpy(), ref_lse, "empty row blocks")
    empty = ~mask.numpy().any(axis=-1)
    assert empty.mean() > 0.7 and not gu.to_np32(out)[empty].any()


def test_pack_then_forward_into_reused_buffers_without_synchronising():
    # three different masks packed into ONE packed buffer and attended into ONE output buffer, all queued on the
    # stream before anything is waited for: each forward must see its own pack's words although the attention
    # kernel becomes resident while the pack kernel before it is still writing them
    B, H, N = 4, 6, 512
    cases = []
    for seed, kind, keep in ((31, "iid", 0.25), (32, "block", 0.3), (33, "causal_iid", 0.5)):
        cfg = workloads.Config("reuse", B, H, N, torch.float16, kind, keep, seed=seed)
        cases.append(tuple(t.cuda() for t in workloads.make_inputs(cfg)))
    want = []
    for q, k, v, mask in cases:
        out = torch.empty_like(q)
        sparse_attn_cuda.forward(q, k, v, sparse_attn_cuda.pack_mask(mask), out, None, 0.125, False)
        torch.cuda.synchronize()
        want.append(out)
    packed = torch.empty(B, H, N, N // 32, dtype=torch.int32, device="cuda")
    out = torch.empty_like(cases[0][0])
    got = []
    torch.cuda.synchronize()
    for q, k, v, mask in cases:
        _capi.pack_mask(mask.data_ptr(), packed.data_ptr(), B, H, N, None)
        lse = torch.empty(B, H, N, dtype=torch.float32, device="cuda")
        p = _params(q, k, v, packed, out, lse)
        p.save_lse = 0
        _capi.attention_fwd(p, None)
        got.append(out.clone())  # a copy kernel on the same stream, still nothing synchronised
    torch.cuda.synchronize()
    _capi.device_status()
    for w, g_ in zip(want, got):
        assert torch.equal(w, g_)


def test_workspace_size_and_errors():
    assert _capi.attention_workspace_bytes(16, 12, 512) == 16 * 12 * 4 * 8 * 4 + 16  # 768 items x 8 words + work queue
    assert _capi.attention_workspace_bytes(0, 1, 64) == 0 and _capi.attention_workspace_bytes(1, 1, 16385) == 0
    cfg = workloads.Config("planned", 1, 1, 256, torch.float16, "iid", 0.25, seed=1)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    packed = sparse_attn_cuda.pack_mask(mask)
    out, lse = torch.empty_like(q), torch.empty(1, 1, 256, device="cuda")
    p = _params(q, k, v, packed, out, lse)
    nbytes = _capi.attention_workspace_bytes(1, 1, 256)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_fwd_planned(p, ws.data_ptr(), nbytes - 1, None)
    assert e.value.status == _capi.SMA_ERR_WORKSPACE_TOO_SMALL
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_fwd_planned(p, None, nbytes, None)
    assert e.value.status == _capi.SMA_ERR_NULL_POINTER
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_fwd_planned(p, ws.data_ptr() + 4, nbytes, None)
    assert e.value.status == _capi.SMA_ERR_MISALIGNED
