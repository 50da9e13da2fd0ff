"""sma_attention_bwd (dq, dk, dv on the tensor cores) against the fp64 gradient oracle, which is itself pinned to the
reference's own autograd function by tests/golden/backward_golden.npz (see test_oracle_golden.py).

Tolerance.  The kernel rounds P and dS to 16 bits before the products that contract over 128 rows or keys at a
time, accumulates in fp32 and rounds the results to the 16-bit output type.  Per element that is a relative error
of some 2^-11 (fp16) or 2^-8 (bf16) on terms that add up like a random walk, so the bound is stated against the
size of the whole gradient tensor:  |err| <= atol_rel * max|ref| + rtol * |ref|  with (atol_rel, rtol) = (4e-3, 1e-2)
for fp16 and (2e-2, 4e-2) for bf16."""
import os

import numpy as np
import pytest
import torch

import gpu_util as gu
from oracle import sma_oracle as orc
from sparse_mask_attention_b200 import _capi, sparse_attn_cuda, workloads
from sparse_mask_attention_b200.sparse_attention import SparseAttentionFunction, sparse_attention

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "backward_golden.npz")
TOL = {torch.float16: (4e-3, 1e-2), torch.bfloat16: (2e-2, 4e-2)}


def assert_grad_close(got, ref, dtype, what):
    atol_rel, rtol = TOL[dtype]
    got = got.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all(), "%s: non-finite values" % what
    bound = atol_rel * max(np.abs(ref).max(), 1e-6) + rtol * np.abs(ref)
    err = np.abs(got - ref)
    bad = err > bound
    assert not bad.any(), "%s: %d of %d outside tolerance (max err %.3e, max|ref| %.3e)" % (
        what, int(bad.sum()), bad.size, float(err.max()), float(np.abs(ref).max()))


def run_backward(q, k, v, mask, dout, scale=None):
    """forward + backward through the library; returns out, dq, dk, dv (device tensors)."""
    B, H, N, D = q.shape
    scale = D ** -0.5 if scale is None else scale
    qd, kd, vd, md, dod = (t.cuda() for t in (q, k, v, mask, dout))
    packed = sparse_attn_cuda.pack_mask(md)
    out = torch.empty_like(qd)
    lse = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
    sparse_attn_cuda.forward(qd, kd, vd, packed, out, lse, scale, True)
    dq, dk, dv = (torch.full_like(qd, float("nan")) for _ in range(3))
    sparse_attn_cuda.backward(dod, qd, kd, vd, out, lse, packed, dq, dk, dv, scale)
    torch.cuda.synchronize()
    _capi.device_status()
    return out, dq, dk, dv


def check_against_oracle(q, k, v, mask, dout, dtype, what, scale=None):
    out, dq, dk, dv = run_backward(q, k, v, mask, dout, scale)
    rq, rk, rv = orc.attention_bwd_np(gu.to_np32(q), gu.to_np32(k), gu.to_np32(v), mask.numpy(), gu.to_np32(dout), scale=scale)
    assert_grad_close(dv, rv, dtype, what + " dv")
    assert_grad_close(dk, rk, dtype, what + " dk")
    assert_grad_close(dq, rq, dtype, what + " dq")


def test_golden_cases_of_the_reference_autograd_function():
    g = np.load(GOLDEN)
    for name in g["names"]:
        q, k, v, dout = (torch.from_numpy(g["%s_%s" % (name, x)]) for x in ("q", "k", "v", "dout"))
        mask = torch.from_numpy(g[name + "_mask"])
        out, dq, dk, dv = run_backward(q, k, v, mask, dout)
        for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            assert_grad_close(got, g["%s_%s" % (name, key)].astype(np.float64), torch.float16, "%s %s" % (name, key))


@pytest.mark.parametrize("N,kind,keep,dtype", [
    (128, "iid", 0.25, torch.float16), (128, "iid", 0.25, torch.bfloat16), (100, "iid", 0.3, torch.float16),
    (130, "iid", 0.1, torch.bfloat16), (256, "causal_iid", 0.5, torch.float16), (512, "iid", 0.25, torch.float16),
    (512, "block", 0.25, torch.float16), (1024, "causal_iid", 0.5, torch.bfloat16), (1024, "block", 0.05, torch.float16),
    (40, "iid", 0.5, torch.float16), (2112, "block", 0.1, torch.float16)])
def test_backward_matches_the_gradient_oracle(N, kind, keep, dtype):
    B, H = 2, 3
    cfg = workloads.Config("bwd", B, H, N, dtype, kind, keep, seed=N + 1)
    q, k, v, mask = workloads.make_inputs(cfg)
    g = torch.Generator().manual_seed(N + 2)
    dout = torch.randn(B, H, N, 64, generator=g).to(dtype)
    check_against_oracle(q, k, v, mask, dout, dtype, "N=%d %s" % (N, kind))


def test_rows_and_key_blocks_that_keep_nothing():
    B, H, N = 1, 2, 384
    g = torch.Generator().manual_seed(3)
    q, k, v, dout = (torch.randn(B, H, N, 64, generator=g).half() for _ in range(4))
    mask = torch.rand(B, H, N, N, generator=g) < 0.2
    mask[:, :, 5, :] = False          # a query row that keeps nothing: lse = -inf, no gradient through it
    mask[:, :, 128:256, :] = False    # a whole block of query rows
    mask[:, :, :, 256:384] = False    # a whole block of keys: dk = dv = 0 there
    out, dq, dk, dv = run_backward(q, k, v, mask, dout)
    assert (dq[:, :, 5] == 0).all() and (dq[:, :, 128:256] == 0).all()
    assert (dk[:, :, 256:] == 0).all() and (dv[:, :, 256:] == 0).all()
    check_against_oracle(q, k, v, mask, dout, torch.float16, "empty rows and blocks")


def test_negative_and_unusual_scale():
    B, H, N = 1, 2, 256
    g = torch.Generator().manual_seed(4)
    q, k, v, dout = (torch.randn(B, H, N, 64, generator=g).half() for _ in range(4))
    mask = torch.rand(B, H, N, N, generator=g) < 0.3
    check_against_oracle(q, k, v, mask, dout, torch.float16, "scale -0.05", scale=-0.05)


def test_autograd_function_uses_the_kernels():
    cfg = workloads.Config("autograd", 2, 4, 256, torch.float16, "iid", 0.25, seed=9)
    q, k, v, mask = workloads.make_inputs(cfg)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    md = mask.cuda()
    out = sparse_attention(qd, kd, vd, md)
    g = torch.Generator().manual_seed(10)
    dout = torch.randn(out.shape, generator=g).half()
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    _capi.device_status()
    rq, rk, rv = orc.attention_bwd_np(gu.to_np32(q), gu.to_np32(k), gu.to_np32(v), mask.numpy(), gu.to_np32(dout))
    assert_grad_close(qd.grad, rq, torch.float16, "autograd dq")
    assert_grad_close(kd.grad, rk, torch.float16, "autograd dk")
    assert_grad_close(vd.grad, rv, torch.float16, "autograd dv")


def test_workspace_and_argument_checks():
    assert _capi.attention_bwd_workspace_bytes(2, 3, 128) == 2 * 3 * 128 * 4 + 2 * 3 * 128 * 64 * 4 + 256
    assert _capi.attention_bwd_workspace_bytes(0, 3, 128) == 0
    cfg = workloads.Config("chk", 1, 1, 128, torch.float16, "iid", 0.25, seed=1)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    packed = sparse_attn_cuda.pack_mask(mask)
    out = torch.empty_like(q)
    lse = torch.empty((1, 1, 128), dtype=torch.float32, device="cuda")
    sparse_attn_cuda.forward(q, k, v, packed, out, lse, 0.125, True)
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out, p.lse = (q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr(),
                                                  out.data_ptr(), lse.data_ptr())
    p.B, p.H, p.N, p.D, p.scale, p.dtype, p.save_lse, p.variant = 1, 1, 128, 64, 0.125, _capi.SMA_DTYPE_F16, 1, 0
    d = torch.empty_like(q)
    need = _capi.attention_bwd_workspace_bytes(1, 1, 128)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_bwd(p, q.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), ws.data_ptr(), need - 1, None)
    assert e.value.status == _capi.SMA_ERR_WORKSPACE_TOO_SMALL
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_bwd(p, None, d.data_ptr(), d.data_ptr(), d.data_ptr(), ws.data_ptr(), need, None)
    assert e.value.status == _capi.SMA_ERR_NULL_POINTER
    p.lse = None
    with pytest.raises(_capi.SmaError) as e:
        _capi.attention_bwd(p, q.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(), ws.data_ptr(), need, None)
    assert e.value.status == _capi.SMA_ERR_NULL_POINTER
