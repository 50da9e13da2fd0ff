"""The attention kernels' waits (forward and backward) are bounded: a wait that nothing will ever satisfy gives up, the
kernel winds down (no instruction issued behind the failed wait, tensor memory released), the library reports
SMA_ERR_DEVICE_TIMEOUT, and the next launch on the same context is correct.

The wait is made to run out without any fault: the test build of the library (libsma_b200_waittest.so, same
sources compiled with -DSMA_WAIT_TEST_BUILD) has a wait limit of some ten milliseconds and a switch that leaves the
first Q tile of one work item unrequested, so the barrier that the tile's arrival would complete stays where it is.
The product library has neither the switch nor the short limit."""
import ctypes
import os
import time

import pytest
import torch

import gpu_util as gu
from sparse_mask_attention_b200 import _capi, build, sparse_attn_cuda, workloads

pytestmark = pytest.mark.gpu


def _load_test_build():
    if not os.path.exists(build.WAIT_TEST_LIB_PATH):
        pytest.skip("libsma_b200_waittest.so has not been built (python sparse_mask_attention_b200/build.py)")
    lib = ctypes.CDLL(build.WAIT_TEST_LIB_PATH)
    lib.sma_attention_fwd.restype = ctypes.c_int
    lib.sma_attention_fwd.argtypes = [ctypes.POINTER(_capi.AttentionParams), ctypes.c_void_p]
    lib.sma_device_status.restype = ctypes.c_int
    lib.sma_test_withhold_q_load.restype = ctypes.c_int
    lib.sma_test_withhold_q_load.argtypes = [ctypes.c_int]
    lib.sma_attention_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.sma_attention_bwd_workspace_bytes.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.sma_attention_bwd.restype = ctypes.c_int
    lib.sma_attention_bwd.argtypes = ([ctypes.POINTER(_capi.AttentionParams)] + [ctypes.c_void_p] * 5
                                      + [ctypes.c_size_t, ctypes.c_void_p])
    return lib


def test_the_product_library_has_no_test_switch():
    assert not hasattr(_capi.lib, "sma_test_withhold_q_load")


@pytest.mark.parametrize("kind,N", [("iid", 512), ("causal_iid", 1024)])
def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_correct(kind, N):
    lib = _load_test_build()
    B, H = 4, 6
    cfg = workloads.Config("wait_limit", B, H, N, torch.float16, kind, 0.3, seed=11)
    q, k, v, mask = workloads.make_inputs(cfg)
    qd, kd, vd, md = (t.cuda() for t in (q, k, v, mask))
    packed = sparse_attn_cuda.pack_mask(md)
    out = torch.zeros_like(qd)
    lse = torch.zeros((B, H, N), dtype=torch.float32, device="cuda")
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out, p.lse = (qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), packed.data_ptr(),
                                                  out.data_ptr(), lse.data_ptr())
    p.B, p.H, p.N, p.D, p.scale, p.dtype, p.save_lse, p.variant = B, H, N, 64, 0.125, _capi.SMA_DTYPE_F16, 1, 0
    torch.cuda.synchronize()
    assert lib.sma_device_status() == _capi.SMA_OK

    # a launch in which one load is never requested: the wait for it gives up within the test build's limit
    assert lib.sma_test_withhold_q_load(1) == _capi.SMA_OK
    t0 = time.perf_counter()
    assert lib.sma_attention_fwd(ctypes.byref(p), None) == _capi.SMA_OK  # the launch itself succeeds
    status = lib.sma_device_status()  # synchronises
    elapsed = time.perf_counter() - t0
    assert status == _capi.SMA_ERR_DEVICE_TIMEOUT
    assert elapsed < 2.0, "the kernel took %.2f s to give up" % elapsed
    assert lib.sma_device_status() == _capi.SMA_OK, "reading the status clears it"

    # the context is intact: the same library, switch off, now computes everything
    assert lib.sma_test_withhold_q_load(0) == _capi.SMA_OK
    out.zero_()
    lse.zero_()
    assert lib.sma_attention_fwd(ctypes.byref(p), None) == _capi.SMA_OK
    assert lib.sma_device_status() == _capi.SMA_OK
    ref, ref_lse = gu.oracle_for(q, k, v, mask)
    gu.assert_close(gu.to_np32(out), ref, "launch after a wait that ran out")
    gu.assert_lse_close(lse.cpu().numpy(), ref_lse, "launch after a wait that ran out")
    # and so does the product library
    out2 = torch.empty_like(qd)
    lse2 = torch.empty_like(lse)
    sparse_attn_cuda.forward(qd, kd, vd, packed, out2, lse2, 0.125, True)
    torch.cuda.synchronize()
    _capi.device_status()
    assert torch.equal(out2, out) and torch.equal(lse2, lse)


@pytest.mark.parametrize("kind,N", [("iid", 512), ("causal_iid", 384)])
def test_the_backward_kernel_gives_up_too_and_the_next_call_is_correct(kind, N):
    lib = _load_test_build()
    B, H = 2, 3
    cfg = workloads.Config("wait_limit_bwd", B, H, N, torch.float16, kind, 0.3, seed=12)
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    packed = sparse_attn_cuda.pack_mask(mask)
    out = torch.empty_like(q)
    lse = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
    sparse_attn_cuda.forward(q, k, v, packed, out, lse, 0.125, True)
    dout = torch.randn_like(q)
    want = [torch.empty_like(q) for _ in range(3)]
    sparse_attn_cuda.backward(dout, q, k, v, out, lse, packed, *want, 0.125)  # the product library
    torch.cuda.synchronize()
    _capi.device_status()

    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out, p.lse = (q.data_ptr(), k.data_ptr(), v.data_ptr(), packed.data_ptr(),
                                                  out.data_ptr(), lse.data_ptr())
    p.B, p.H, p.N, p.D, p.scale, p.dtype, p.save_lse, p.variant = B, H, N, 64, 0.125, _capi.SMA_DTYPE_F16, 1, 0
    nbytes = lib.sma_attention_bwd_workspace_bytes(B, H, N)
    workspace = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    got = [torch.zeros_like(q) for _ in range(3)]

    def call():
        return lib.sma_attention_bwd(ctypes.byref(p), dout.data_ptr(), got[0].data_ptr(), got[1].data_ptr(),
                                     got[2].data_ptr(), workspace.data_ptr(), nbytes, None)

    assert lib.sma_device_status() == _capi.SMA_OK
    # the first Q tile of one unit of work is never requested: the wait for it gives up within the test build's limit
    assert lib.sma_test_withhold_q_load(1) == _capi.SMA_OK
    t0 = time.perf_counter()
    assert call() == _capi.SMA_OK  # the launches themselves succeed
    status = lib.sma_device_status()  # synchronises
    elapsed = time.perf_counter() - t0
    assert status == _capi.SMA_ERR_DEVICE_TIMEOUT
    assert elapsed < 2.0, "the kernel took %.2f s to give up" % elapsed
    assert lib.sma_device_status() == _capi.SMA_OK, "reading the status clears it"

    # the context is intact: the same library, switch off, computes the gradients of the product library
    assert lib.sma_test_withhold_q_load(0) == _capi.SMA_OK
    assert call() == _capi.SMA_OK
    assert lib.sma_device_status() == _capi.SMA_OK
    assert torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])  # dk, dv: deterministic
    # dq is summed in the order in which the reductions arrive: equal to rounding
    scale_ref = want[0].float().abs().max().item()
    assert (got[0].float() - want[0].float()).abs().max().item() <= 2e-3 * scale_ref + 1e-6
