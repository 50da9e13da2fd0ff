"""The attention kernel's work queue (sma_sparse_attention_fwd with a work_counter, the tile-list workspace's last
word): CTAs take their work items from one counter instead of a fixed share each.  Which CTA computes an item must
not show in the results: outputs are compared bit for bit with the fixed assignment, on masks whose row blocks hold
very different numbers of tiles, with the counter holding garbage on entry and shared by calls queued back to back."""
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


@pytest.mark.parametrize("B,H,N,kind,keep,dtype", [
    (16, 12, 512, "block", 0.25, torch.float16), (16, 12, 512, "iid", 0.25, torch.float16),
    (8, 16, 1024, "causal_iid", 0.5, torch.bfloat16), (3, 5, 200, "iid", 0.2, torch.float16),
    (1, 2, 128, "iid", 0.5, torch.float16), (2, 12, 2112, "block", 0.1, torch.float16)])
def test_queue_and_fixed_assignment_agree_bitwise(B, H, N, kind, keep, dtype):
    cfg = workloads.Config("queue", B, H, N, dtype, kind, keep, seed=N + B)
    q, k, v, mask = workloads.make_inputs(cfg)
    qd, kd, vd, md = (t.cuda() for t in (q, k, v, mask))
    nw = (N + 31) // 32
    results = []
    for use_queue in (False, True):
        out = torch.full_like(qd, 3.0)
        lse = torch.full((B, H, N), 7.0, dtype=torch.float32, device="cuda")
        packed = torch.empty((B, H, N, nw), dtype=torch.int32, device="cuda")
        counter = torch.full((3,), -559038737, dtype=torch.int32, device="cuda")  # garbage on entry; guards either side
        p = _params(qd, kd, vd, packed, out, lse)
        for _ in range(3 if use_queue else 1):  # queued calls share the word: each packing kernel zeroes it again
            _capi.sparse_attention_fwd(p, md.data_ptr(), None, counter[1:].data_ptr() if use_queue else None, None)
        torch.cuda.synchronize()
        _capi.device_status()
        if use_queue:
            items = B * H * ((N + 127) // 128)
            assert counter[0].item() == -559038737 and counter[2].item() == -559038737
            assert 0 <= counter[1].item() <= items + 2 * 148, "every stream asks once more than it gets"
        results.append((out, lse, packed))
    for a, b in zip(*results):
        assert torch.equal(a, b)
    if N <= 1024:
        ref, ref_lse = gu.oracle_for(q, k, v, mask)
        gu.assert_close(gu.to_np32(results[1][0]), ref, "work queue %s N=%d" % (kind, N))
        gu.assert_lse_close(results[1][1].cpu().numpy(), ref_lse, "work queue %s N=%d" % (kind, N))


@pytest.mark.parametrize("cfg", [workloads.CONFIGS[3],
                                 workloads.Config("long", 1, 6, 2112, torch.float16, "block", 0.1, seed=4),
                                 workloads.Config("long_bf16", 1, 4, 4096, torch.bfloat16, "causal_iid", 0.5, seed=5)])
def test_python_layer_results_unchanged(cfg):
    q, k, v, mask = (t.cuda() for t in workloads.make_inputs(cfg))
    from sparse_mask_attention_b200.sparse_attention import sparse_attention_func

    out = sparse_attention_func(q, k, v, mask)  # takes the queue (and, beyond 2048 keys, the occupancy side-band)
    packed = sparse_attn_cuda.pack_mask(mask)
    out2 = torch.empty_like(q)
    sparse_attn_cuda.forward(q, k, v, packed, out2, None, 0.125, False)  # fixed assignment (tile-list kernel when long)
    torch.cuda.synchronize()
    _capi.device_status()
    assert torch.equal(out, out2)
