"""pack_mask + the fused forward captured into a CUDA graph and replayed: the library's entry points only launch
(no allocation, no synchronisation, no host-side state that a replay would miss), their kernels are launched with
programmatic stream serialisation, which a capture keeps as programmatic edges, and the work-queue word that the
Python layer allocates per call comes from the graph's own memory pool.  A replay costs the host a few
microseconds instead of the Python layer's 25."""
import pytest
import torch

from sparse_mask_attention_b200 import _capi, workloads
from sparse_mask_attention_b200.sparse_attention import sparse_attention_func

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg", [workloads.Config("graph", 4, 12, 512, torch.float16, "iid", 0.25, seed=1),
                                 workloads.Config("graph_long", 1, 4, 2560, torch.bfloat16, "block", 0.1, seed=2)])
def test_replay_computes_on_the_current_contents_of_the_captured_buffers(cfg):
    first = [t.cuda() for t in workloads.make_inputs(cfg)]
    second = [t.cuda() for t in workloads.make_inputs(workloads.Config("graph2", cfg.B, cfg.H, cfg.N, cfg.dtype, cfg.mask_kind,
                                                                      cfg.keep_prob, seed=cfg.seed + 10))]
    q, k, v, mask = (t.clone() for t in first)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture (first-call set-up of the library and of torch)
        for _ in range(3):
            sparse_attention_func(q, k, v, mask)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = sparse_attention_func(q, k, v, mask)
    want_first = sparse_attention_func(*first)
    want_second = sparse_attention_func(*second)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want_first)
    for dst, src in zip((q, k, v, mask), second):
        dst.copy_(src)
    for _ in range(3):  # replays back to back: each packing kernel zeroes the work queue of its own replay
        graph.replay()
    torch.cuda.synchronize()
    _capi.device_status()
    assert torch.equal(out, want_second)
