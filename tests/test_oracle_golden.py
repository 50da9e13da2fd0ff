"""The oracle (numpy and C restatements) against vectors written by the reference's own Python code."""
import hashlib
import os

import numpy as np
import torch

from oracle import c_oracle
from oracle import sma_oracle as orc
from sparse_mask_attention_b200 import workloads


def _n_pack_cases(g):
    return len([k for k in g.files if k.startswith("mask_")])


def test_pack_numpy_matches_reference_vectors(pack_golden):
    for i in range(_n_pack_cases(pack_golden)):
        mask, want = pack_golden["mask_%d" % i], pack_golden["packed_%d" % i]
        got = orc.pack_mask_np(mask)
        assert got.dtype == np.int32 and got.shape == want.shape
        assert np.array_equal(got, want), "case %d" % i


def test_pack_c_matches_reference_vectors(pack_golden):
    for i in range(_n_pack_cases(pack_golden)):
        mask, want = pack_golden["mask_%d" % i], pack_golden["packed_%d" % i]
        assert np.array_equal(c_oracle.pack_mask_c(mask), want), "case %d" % i


def test_pack_loops_and_torch_restatements_agree(pack_golden):
    for i in range(_n_pack_cases(pack_golden)):
        mask, want = pack_golden["mask_%d" % i], pack_golden["packed_%d" % i]
        if mask.shape[2] <= 40:
            loops = np.array(orc.pack_mask_loops(mask), dtype=np.uint32).view(np.int32)
            assert np.array_equal(loops, want)
        assert np.array_equal(orc.pack_mask_torch_cpu(torch.from_numpy(mask)).numpy(), want)


def test_pack_tail_bits_zero_and_roundtrip(pack_golden):
    for i in range(_n_pack_cases(pack_golden)):
        mask = pack_golden["mask_%d" % i]
        N = mask.shape[2]
        packed = orc.pack_mask_np(mask)
        assert np.array_equal(orc.unpack_mask_np(packed, N), mask)
        if N % 32:
            last = packed.view(np.uint32)[..., -1]
            assert not (last >> np.uint32(N % 32)).any()


def test_attention_edge_cases_match_reference(edge_golden):
    for name in edge_golden["names"]:
        q, k, v = (edge_golden["%s_%s" % (name, t)].astype(np.float32) for t in "qkv")
        mask, want, want_lse = edge_golden[name + "_mask"], edge_golden[name + "_out"], edge_golden[name + "_lse"]
        for out, lse in (orc.attention_np(q, k, v, mask, dtype=np.float64), c_oracle.attention_c(q, k, v, mask)):
            assert np.abs(out - want).max() < 2e-6, name
            finite = np.isfinite(want_lse)
            assert np.array_equal(np.isneginf(lse), np.isneginf(want_lse)), name
            if finite.any():
                assert np.abs(lse[finite] - want_lse[finite]).max() < 2e-5, name
        out_t = orc.attention_torch_cpu(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v),
                                        torch.from_numpy(mask)).numpy()
        assert np.abs(out_t - want).max() < 2e-6, name


def test_fully_masked_rows_are_zero(edge_golden):
    out, lse = orc.attention_np(*(edge_golden["n8_row0_empty_" + t].astype(np.float32) for t in "qkv"),
                                edge_golden["n8_row0_empty_mask"])
    assert not out[0, 0, 0].any() and np.isneginf(lse[0, 0, 0]) and not np.isnan(out).any()
    out, lse = c_oracle.attention_c(*(edge_golden["n72_all_false_" + t].astype(np.float32) for t in "qkv"),
                                    edge_golden["n72_all_false_mask"])
    assert not out.any() and np.isneginf(lse).all()


def test_config1_inputs_reproduce_and_oracle_matches_reference(config1_golden):
    q, k, v, mask = workloads.make_inputs(workloads.CONFIGS[1])
    for name, t in (("q", q), ("k", k), ("v", v), ("mask", mask)):
        digest = hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()
        assert digest == str(config1_golden["sha_" + name]), "seeded %s differs from the golden run" % name
    assert np.array_equal(orc.pack_mask_np(mask.numpy()), config1_golden["packed"])
    out64, lse64 = orc.attention_np(q.numpy(), k.numpy(), v.numpy(), mask.numpy(), dtype=np.float64)
    assert np.abs(out64 - config1_golden["out_ref"]).max() < 2e-6
    assert np.abs(lse64 - config1_golden["lse"]).max() < 2e-5
    out_c, _ = c_oracle.attention_c(q.numpy(), k.numpy(), v.numpy(), mask.numpy())
    assert np.abs(out_c - config1_golden["out_ref"]).max() < 2e-6
    # the reference's public entry point rounds fp32 inputs to bf16 first: same oracle on rounded inputs
    qb, kb, vb = (t.bfloat16().float().numpy() for t in (q, k, v))
    out_b, _ = orc.attention_np(qb, kb, vb, mask.numpy(), dtype=np.float64)
    out_b = torch.from_numpy(out_b).bfloat16().float().numpy()
    assert np.abs(out_b - config1_golden["out_api"]).max() < 2e-2  # one bf16 ulp at |x| <= 4


def test_compare_helper_flags_nan_and_excess():
    ref = np.array([0.0, 1.0, -2.0])
    assert orc.compare(ref + 1e-3, ref)["ok"]
    assert not orc.compare(ref + np.array([0, 0.02, 0]), ref)["ok"]
    assert not orc.compare(np.array([np.nan, 1.0, -2.0]), ref)["ok"]


def test_gradient_oracle_matches_the_reference_autograd_function():
    """attention_bwd_np against dq, dk, dv that the reference's SparseAttentionFunction.backward produced on CPU
    (tests/golden/make_golden.py backward): fp32 arithmetic there, fp64 here."""
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "backward_golden.npz"))
    assert len(g["names"]) >= 6
    for name in g["names"]:
        dq, dk, dv = orc.attention_bwd_np(g[name + "_q"], g[name + "_k"], g[name + "_v"], g[name + "_mask"],
                                          g[name + "_dout"], 0.125)
        for got, key in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
            ref = g["%s_%s" % (name, key)]
            assert np.abs(got - ref).max() <= 1e-5 * max(1.0, np.abs(ref).max()), "%s %s" % (name, key)
    # rows that keep nothing pass no gradient
    dq, _, _ = orc.attention_bwd_np(g["n8_row0_empty_q"], g["n8_row0_empty_k"], g["n8_row0_empty_v"],
                                    g["n8_row0_empty_mask"], g["n8_row0_empty_dout"], 0.125)
    assert (dq[:, :, 0] == 0).all()
