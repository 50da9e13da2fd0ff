"""The drop-in claim, tested with the reference's own Python layer: its unmodified python/sparse_attention.py
(a build output under oracle/_ref/, written by `make -C oracle ref_python` where the reference checkout is present)
is imported with this repository's root on sys.path, so that its ``import sparse_attn_cuda``
(python/sparse_attention.py:12-17) picks up the B200 library's stand-in.  Its public entry points then run the
CUDA path of this repository and are compared with the fp32 oracle."""
import importlib.util
import os
import sys

import numpy as np
import pytest
import torch

import gpu_util as gu
from sparse_mask_attention_b200 import workloads

pytestmark = pytest.mark.gpu

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_PY = os.path.join(REPO, "oracle", "_ref", "ref_python", "sparse_attention.py")


@pytest.fixture(scope="module")
def ref_module():
    if not os.path.exists(REF_PY):
        pytest.skip("the reference's python/sparse_attention.py has not been placed under oracle/_ref/ref_python")
    assert REPO in sys.path
    spec = importlib.util.spec_from_file_location("reference_sparse_attention", REF_PY)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.HAS_CUDA_EXT, "the reference's `import sparse_attn_cuda` did not resolve"
    import sparse_attn_cuda
    from sparse_mask_attention_b200 import sparse_attn_cuda as ours

    assert sparse_attn_cuda.forward is ours.forward and sparse_attn_cuda.pack_mask is ours.pack_mask
    return mod


def test_reference_sparse_attention_on_config1(ref_module):
    q, k, v, mask = workloads.make_inputs(workloads.CONFIGS[1])  # fp32 inputs: computed in bf16, returned as fp32
    out = ref_module.sparse_attention(q.cuda(), k.cuda(), v.cuda(), mask.cuda())
    assert out.dtype == torch.float32
    ref, _ = gu.oracle_for(q.bfloat16(), k.bfloat16(), v.bfloat16(), mask)
    gu.assert_close(out.cpu().numpy(), ref, "reference sparse_attention(), config 1")


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_reference_entry_points_on_a_headline_shard(ref_module, dtype):
    cfg = workloads.Config("shard", 2, 12, 512, dtype, "iid", 0.25, seed=5)
    q, k, v, mask = workloads.make_inputs(cfg)
    qd, kd, vd, md = (t.cuda() for t in (q, k, v, mask))
    ref, _ = gu.oracle_for(q, k, v, mask)
    # the autograd entry point (is_training=True, allocates lse) and the inference one (passes lse=None,
    # python/sparse_attention.py:170-171)
    out_a = ref_module.sparse_attention(qd, kd, vd, md)
    out_b = ref_module.sparse_attention_func(qd, kd, vd, md)
    torch.cuda.synchronize()
    gu.assert_close(gu.to_np32(out_a), ref, "reference sparse_attention()")
    gu.assert_close(gu.to_np32(out_b), ref, "reference sparse_attention_func()")
    assert torch.equal(out_a, out_b)
    # and its pack_mask wrapper
    packed = ref_module.pack_mask(md)
    from oracle import sma_oracle as orc

    assert np.array_equal(packed.cpu().numpy(), orc.pack_mask_np(mask.numpy()))


def test_reference_autograd_function_backward(ref_module):
    """The reference's own SparseAttentionFunction.backward calls sparse_attn_cuda.backward(dout, q, k, v, out, lse,
    mask_packed, dq, dk, dv, scale) (python/sparse_attention.py:90-94), which its extension never exported; with
    the stand-in on the path the call resolves and the gradients match the fp64 oracle of its PyTorch branch."""
    from oracle import sma_oracle as orc

    cfg = workloads.Config("ref_bwd", 2, 4, 256, torch.bfloat16, "iid", 0.25, seed=13)
    q, k, v, mask = workloads.make_inputs(cfg)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = ref_module.sparse_attention(qd, kd, vd, mask.cuda())
    g = torch.Generator().manual_seed(14)
    dout = torch.randn(out.shape, generator=g).bfloat16()
    out.backward(dout.cuda())
    torch.cuda.synchronize()
    rq, rk, rv = orc.attention_bwd_np(gu.to_np32(q), gu.to_np32(k), gu.to_np32(v), mask.numpy(), gu.to_np32(dout))
    for got, ref, name in ((qd.grad, rq, "dq"), (kd.grad, rk, "dk"), (vd.grad, rv, "dv")):
        got = got.float().cpu().numpy().astype(np.float64)
        bound = 2e-2 * np.abs(ref).max() + 4e-2 * np.abs(ref)  # the bf16 bound of tests/test_backward_gpu.py
        assert (np.abs(got - ref) <= bound).all(), name
