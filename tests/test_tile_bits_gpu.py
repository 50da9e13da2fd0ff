"""The occupancy side-band: sma_pack_mask_tiles writes, beside the packed words, one bit per (mask row, 64-key
tile); sma_attention_fwd_tiles takes its tile lists from those bits.  Checked here: the packed words are those of
sma_pack_mask, the bits are what their definition says, and the attention results equal those of sma_attention_fwd
bit for bit (and the oracle's within tolerance) on shapes and masks that exercise every branch of the list
builder: chunks without a tile, an empty final chunk, row blocks that keep nothing, rows of 16-bit words that
straddle two blocks of 32 packed words."""
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


def _pack_tiles(mask):
    B, H, N, _ = mask.shape
    nbytes = _capi.tile_bits_bytes(B, H, N)
    assert nbytes == B * H * N * (N // 32) // 32 * 2
    packed = torch.full((B, H, N, N // 32), -1, dtype=torch.int32, device="cuda")
    bits = torch.full((nbytes // 2 + 8,), 0x5A5A, dtype=torch.int16, device="cuda")
    _capi.pack_mask_tiles(mask.data_ptr(), packed.data_ptr(), bits.data_ptr(), B, H, N, None)
    torch.cuda.synchronize()
    assert (bits[nbytes // 2:] == 0x5A5A).all(), "write past the side-band"
    return packed, bits[:nbytes // 2]


def _expected_bits(packed):
    w = packed.cpu().numpy().view(np.uint32).reshape(-1, 16, 2)  # blocks of 32 words as 16 pairs
    nz = (w != 0).any(axis=2)
    return (nz.astype(np.uint32) << np.arange(16, dtype=np.uint32)).sum(axis=1).astype(np.uint16)


def _masks(kind, B, H, N, seed):
    g = torch.Generator().manual_seed(seed)
    if kind == "iid":
        return torch.rand(B, H, N, N, generator=g) < 0.1
    if kind == "very_sparse":  # most tiles, many chunks and some row blocks keep nothing
        return torch.rand(B, H, N, N, generator=g) < 2.0 / N
    if kind == "causal":
        return torch.ones(N, N, dtype=torch.bool).tril().expand(B, H, N, N).clone()
    if kind == "front_half":  # the final chunks of every row block keep nothing
        m = torch.zeros(B, H, N, N, dtype=torch.bool)
        m[..., : max(64, N // 2 - 64)] = torch.rand(B, H, N, max(64, N // 2 - 64), generator=g) < 0.3
        return m
    if kind == "back_only":  # only the final tile keeps anything
        m = torch.zeros(B, H, N, N, dtype=torch.bool)
        m[..., N - 64:] = torch.rand(B, H, N, 64, generator=g) < 0.3
        return m
    if kind == "empty":
        return torch.zeros(B, H, N, N, dtype=torch.bool)
    if kind == "dead_blocks":
        m = torch.rand(B, H, N, N, generator=g) < 0.2
        dead = torch.rand(B, H, (N + 127) // 128, generator=g) < 0.6
        return m & ~dead.repeat_interleave(128, dim=-1)[..., :N, None]
    raise ValueError(kind)


CASES = [(64, "iid"), (128, "very_sparse"), (192, "iid"), (192, "very_sparse"), (320, "causal"), (448, "dead_blocks"),
         (512, "iid"), (512, "very_sparse"), (512, "causal"), (512, "empty"), (512, "dead_blocks"), (1024, "dead_blocks"), (576, "front_half"), (576, "back_only"),
         (1024, "very_sparse"), (1280, "front_half"), (1536, "causal"), (2048, "dead_blocks"), (2112, "back_only"),
         (2560, "very_sparse")]


@pytest.mark.parametrize("N,kind", CASES)
def test_side_band_bits_and_attention(N, kind):
    B, H = 2, 3
    dtype = torch.float16 if (N // 64) % 2 == 0 else torch.bfloat16
    g = torch.Generator().manual_seed(N)
    q, k, v = (torch.randn(B, H, N, 64, generator=g).to(dtype) for _ in range(3))
    mask = _masks(kind, B, H, N, N + 1)
    qd, kd, vd, md = (t.cuda() for t in (q, k, v, mask))
    packed, bits = _pack_tiles(md)
    assert torch.equal(packed, sparse_attn_cuda.pack_mask(md)), "packed words differ from sma_pack_mask"
    np.testing.assert_array_equal(bits.cpu().numpy().view(np.uint16), _expected_bits(packed))

    outs = []
    for tiles in (False, True):
        out = torch.full_like(qd, 3.0)
        lse = torch.full((B, H, N), 7.0, dtype=torch.float32, device="cuda")
        p = _params(qd, kd, vd, packed, out, lse)
        if tiles:
            _capi.attention_fwd_tiles(p, bits.data_ptr(), None)
        else:
            _capi.attention_fwd(p, None)
        torch.cuda.synchronize()
        _capi.device_status()
        outs.append((out, lse))
    assert torch.equal(outs[0][0], outs[1][0]), "out differs between the two ways of finding tiles"
    assert torch.equal(outs[0][1], outs[1][1]), "lse differs between the two ways of finding tiles"
    ref, ref_lse = gu.oracle_for(q, k, v, mask)
    gu.assert_close(gu.to_np32(outs[1][0]), ref, "tiles N=%d %s" % (N, kind))
    gu.assert_lse_close(outs[1][1].cpu().numpy(), ref_lse, "tiles N=%d %s" % (N, kind))


def test_headline_shape_through_the_combined_call():
    B, H, N = 16, 12, 512
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(B, H, N, 64, generator=g).half().cuda() for _ in range(3))
    mask = (torch.rand(B, H, N, N, generator=g) < 0.3).cuda()
    outs = []
    for with_bits in (False, True):
        out = torch.empty_like(q)
        lse = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
        packed = torch.empty((B, H, N, N // 32), dtype=torch.int32, device="cuda")
        p = _params(q, k, v, packed, out, lse)
        bits = torch.empty(_capi.tile_bits_bytes(B, H, N) // 2, dtype=torch.int16, device="cuda") if with_bits else None
        for _ in range(3):  # queued without synchronising: each call's attention kernel must see its own bits
            _capi.sparse_attention_fwd(p, mask.data_ptr(), bits.data_ptr() if with_bits else None, None, None)
        torch.cuda.synchronize()
        _capi.device_status()
        outs.append((out, lse, packed))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_shapes_without_a_side_band_are_refused():
    assert _capi.tile_bits_bytes(2, 3, 100) == 0
    assert _capi.tile_bits_bytes(2, 3, 96) == 0
    assert _capi.tile_bits_bytes(0, 3, 128) == 0
    B, H, N = 1, 2, 96
    mask = torch.ones(B, H, N, N, dtype=torch.bool, device="cuda")
    packed = torch.empty((B, H, N, 3), dtype=torch.int32, device="cuda")
    bits = torch.empty(64, dtype=torch.int16, device="cuda")
    with pytest.raises(_capi.SmaError) as e:
        _capi.pack_mask_tiles(mask.data_ptr(), packed.data_ptr(), bits.data_ptr(), B, H, N, None)
    assert e.value.status == _capi.SMA_ERR_BAD_SHAPE
    # a mask that does not start on a 32-byte boundary takes the row path, which writes no side-band
    N = 128
    buf = torch.ones(B * H * N * N + 32, dtype=torch.bool, device="cuda")
    packed = torch.empty((B, H, N, 4), dtype=torch.int32, device="cuda")
    with pytest.raises(_capi.SmaError) as e:
        _capi.pack_mask_tiles(buf.data_ptr() + 16, packed.data_ptr(), bits.data_ptr(), B, H, N, None)
    assert e.value.status == _capi.SMA_ERR_MISALIGNED
    # the combined call ignores the buffer there and still gives the right answer
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn(B, H, N, 64, generator=g).half() for _ in range(3))
    mask = torch.rand(B, H, N, N, generator=g) < 0.2
    buf[16:16 + mask.numel()] = mask.flatten().cuda()
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    out = torch.empty_like(qd)
    lse = torch.empty((B, H, N), dtype=torch.float32, device="cuda")
    p = _params(qd, kd, vd, packed, out, lse)
    big_bits = torch.empty(_capi.tile_bits_bytes(B, H, N) // 2, dtype=torch.int16, device="cuda")
    _capi.sparse_attention_fwd(p, buf.data_ptr() + 16, big_bits.data_ptr(), None, None)
    torch.cuda.synchronize()
    _capi.device_status()
    ref, _ = gu.oracle_for(q, k, v, mask)
    gu.assert_close(gu.to_np32(out), ref, "combined call, unaligned mask")
