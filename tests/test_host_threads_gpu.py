"""Entering the library for the first time from a host thread that has made no CUDA call of its own (a framework's
worker thread: PyTorch's autograd engine runs backward passes on one).  The runtime binds the device's primary
context to such a thread by itself, the driver call that encodes tensor maps does not; the library has to."""
import threading

import pytest
import torch

import gpu_util as gu
from sparse_mask_attention_b200 import _capi, sparse_attn_cuda, workloads

pytestmark = pytest.mark.gpu


def test_first_call_from_a_fresh_thread():
    cfg = workloads.Config("thread", 2, 3, 256, torch.float16, "iid", 0.25, seed=31)
    q, k, v, mask = workloads.make_inputs(cfg)
    qd, kd, vd, md = (t.cuda() for t in (q, k, v, mask))
    packed = sparse_attn_cuda.pack_mask(md)  # main thread: the library is initialised, the device is known
    out = torch.zeros_like(qd)
    lse = torch.zeros((2, 3, 256), dtype=torch.float32, device="cuda")
    p = _capi.AttentionParams()
    p.q, p.k, p.v, p.mask_packed, p.out, p.lse = (qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), packed.data_ptr(),
                                                  out.data_ptr(), lse.data_ptr())
    p.B, p.H, p.N, p.D, p.scale, p.dtype, p.save_lse, p.variant = 2, 3, 256, 64, 0.125, _capi.SMA_DTYPE_F16, 1, 0
    torch.cuda.synchronize()
    failure = []

    def worker():  # nothing but the library call: no torch op that would bind the context first
        try:
            _capi.attention_fwd(p, None)
        except Exception as e:  # noqa: BLE001
            failure.append(e)

    t = threading.Thread(target=worker)
    t.start()
    t.join()
    assert not failure, failure
    torch.cuda.synchronize()
    _capi.device_status()
    ref, ref_lse = gu.oracle_for(q, k, v, mask)
    gu.assert_close(gu.to_np32(out), ref, "forward issued from a fresh thread")
    gu.assert_lse_close(lse.cpu().numpy(), ref_lse, "forward issued from a fresh thread")
