"""q, k, v and out with their own batch / head / row strides (reference: the stride fields of SparseAttentionParams,
csrc/sparse_attention.h:29-33, which its kernels never read): the forward pass addresses them in place through 4-D
tensor maps.  Results must be bitwise those of the dense layout, whatever the strides."""
import ctypes

import pytest
import torch

import gpu_util as gu
from sparse_mask_attention_b200 import _capi, sparse_attn_cuda, workloads
from sparse_mask_attention_b200.sparse_attention import sparse_attention, sparse_attention_func

pytestmark = pytest.mark.gpu


def _views(kind, q, k, v):
    """q, k, v [B, H, N, 64] re-laid out in memory as `kind`, returned as [B, H, N, 64] views."""
    B, H, N, D = q.shape
    if kind == "packed_b_n_3_h_d":  # one projection output [B, N, 3, H, 64]
        qkv = torch.stack([t.permute(0, 2, 1, 3) for t in (q, k, v)], dim=2).contiguous()
        return tuple(qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    if kind == "b_n_h_d":  # [B, N, H, 64] tensors, transposed views
        return tuple(t.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3) for t in (q, k, v))
    if kind == "padded_rows":  # rows 96 elements apart
        out = []
        for t in (q, k, v):
            buf = torch.zeros(B, H, N, 96, dtype=t.dtype, device=t.device)
            buf[..., :64] = t
            out.append(buf[..., :64])
        return tuple(out)
    if kind == "h_b_n_d":  # batch and head swapped in memory
        return tuple(t.permute(1, 0, 2, 3).contiguous().permute(1, 0, 2, 3) for t in (q, k, v))
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["packed_b_n_3_h_d", "b_n_h_d", "padded_rows", "h_b_n_d"])
@pytest.mark.parametrize("N,dtype,mask_kind", [(512, torch.float16, "iid"), (200, torch.bfloat16, "iid"),
                                               (1024, torch.float16, "causal_iid"), (2112, torch.float16, "block")])
def test_strided_inputs_give_the_dense_result(kind, N, dtype, mask_kind):
    B, H = 3, 4
    cfg = workloads.Config("strided", B, H, N, dtype, mask_kind, 0.3, seed=N)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    qs, ks, vs = _views(kind, q, k, v)
    assert not qs.is_contiguous() and torch.equal(qs, q)
    packed = sparse_attn_cuda.pack_mask(mask)
    dense = torch.empty_like(q)
    lse_d = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
    sparse_attn_cuda.forward(q, k, v, packed, dense, lse_d, 0.125, True)
    # strided inputs, dense output
    out1 = torch.empty_like(q)
    lse1 = torch.empty_like(lse_d)
    sparse_attn_cuda.forward(qs, ks, vs, packed, out1, lse1, 0.125, True)
    # strided inputs and a strided output ([B, N, H, 64] in memory)
    out2 = torch.full((B, N, H, 64), 7.0, dtype=dtype, device="cuda").permute(0, 2, 1, 3)
    sparse_attn_cuda.forward(qs, ks, vs, packed, out2, None, 0.125, False)
    torch.cuda.synchronize()
    _capi.device_status()
    assert torch.equal(out1, dense) and torch.equal(lse1, lse_d)
    assert torch.equal(out2, dense)
    # the Python layer takes the same tensors without copying them
    assert torch.equal(sparse_attention_func(qs, ks, vs, mask), dense)
    if N <= 1024:
        ref, _ = gu.oracle_for(q.cpu(), k.cpu(), v.cpu(), mask.cpu())
        gu.assert_close(gu.to_np32(out1), ref, "strided %s N=%d" % (kind, N))


def test_layouts_the_library_cannot_address_are_copied():
    cfg = workloads.Config("odd", 2, 2, 128, torch.float16, "iid", 0.3, seed=3)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    # rows 68 elements apart: not a multiple of 16 bytes, so the Python layer falls back to a dense copy
    buf = torch.zeros(2, 2, 128, 68, dtype=torch.float16, device="cuda")
    buf[..., :64] = q
    assert torch.equal(sparse_attention_func(buf[..., :64], k, v, mask), sparse_attention_func(q, k, v, mask))
    # through the C ABI such strides are refused
    packed = sparse_attn_cuda.pack_mask(mask)
    out = torch.empty_like(q)
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr(), out.data_ptr(), None
    p.B, p.H, p.N, p.D, p.scale, p.dtype, p.save_lse, p.variant = 2, 2, 128, 64, 0.125, _capi.SMA_DTYPE_F16, 0, 0
    p.q_strides = (ctypes.c_int64 * 3)(2 * 128 * 68, 128 * 68, 68)
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_fwd(p, None)
    assert e.value.status == _capi.SMA_ERR_BAD_STRIDE


def test_autograd_through_strided_inputs():
    cfg = workloads.Config("strided_bwd", 2, 4, 256, torch.float16, "iid", 0.25, seed=8)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    qkv = torch.stack([t.permute(0, 2, 1, 3) for t in (q, k, v)], dim=2).contiguous().requires_grad_(True)  # [B, N, 3, H, 64]
    qs, ks, vs = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    out = sparse_attention(qs, ks, vs, mask)
    g = torch.Generator(device="cuda").manual_seed(1)
    dout = torch.randn(out.shape, generator=g, device="cuda").half()
    out.backward(dout)
    qd, kd, vd = (t.clone().requires_grad_(True) for t in (q, k, v))
    sparse_attention(qd, kd, vd, mask).backward(dout)
    torch.cuda.synchronize()
    _capi.device_status()
    grads = qkv.grad.permute(2, 0, 3, 1, 4)  # [3, B, H, N, 64]
    for got, want in zip(grads, (qd.grad, kd.grad, vd.grad)):
        # dK and dV are deterministic; dQ is summed in an order that may differ between the two runs
        assert (got.float() - want.float()).abs().max().item() <= 2e-3 * max(1.0, want.float().abs().max().item())
