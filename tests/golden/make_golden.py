"""Writes the golden vectors under tests/golden/ by running the REFERENCE project's own Python code.

Usage (only where the reference checkout exists):  python tests/golden/make_golden.py [reference_root]

It imports ``python/sparse_attention.py`` from the reference checkout (default: the directory named by
$SMA_REFERENCE_ROOT, else a directory "reference" inside or beside the repository), which on a
machine without the reference's CUDA extension runs its pure-PyTorch branches:
  * pack_mask()             -> the CPU packing loop (python/sparse_attention.py:194-201)
  * sparse_attention_ref()  -> the fp32 masked-softmax oracle (:24-42)
  * sparse_attention()      -> the public entry point on CPU tensors (:120-154), incl. fp32->bf16 casting
  * SparseAttentionFunction.forward fallback (:66-74) -> the log-sum-exp values
  * SparseAttentionFunction.backward fallback (:96-111) -> dq, dk, dv ("backward" as second argument writes only
    backward_golden.npz)
Inputs come from the CPU generator with fixed seeds, so they are stored only for the small cases; the
larger case stores checksums of its inputs and the reference outputs.
"""
from __future__ import annotations

import hashlib
import importlib.util
import io
import contextlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))


def load_reference(root: str):
    path = os.path.join(root, "python", "sparse_attention.py")
    spec = importlib.util.spec_from_file_location("reference_sparse_attention", path)
    mod = importlib.util.module_from_spec(spec)
    with contextlib.redirect_stdout(io.StringIO()):  # it prints a warning when its extension is absent
        spec.loader.exec_module(mod)
    assert not mod.HAS_CUDA_EXT
    return mod


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


def lse_of(ref, q, k, v, mask, scale):
    s = torch.matmul(q.float(), k.float().transpose(-2, -1)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    return torch.logsumexp(s, dim=-1)


def write_backward(ref):
    """Gradients from the reference's own autograd function on CPU tensors (its PyTorch branches), fp32 inputs that are
    exactly representable in fp16 so that a 16-bit kernel sees the same numbers."""
    out = {}
    names = []
    g = torch.Generator().manual_seed(21)
    cases = []
    for name, (B, H, N, kind) in {"n8_row0_empty": (1, 1, 8, "row0"), "n64_iid": (1, 2, 64, 0.3), "n100_iid": (1, 2, 100, 0.25),
                                  "n128_iid": (2, 2, 128, 0.25), "n200_sparse": (1, 1, 200, 0.03),
                                  "n256_causal": (1, 2, 256, "causal"), "n72_all_false": (1, 1, 72, 0.0)}.items():
        q, k, v, dout = [torch.randn(B, H, N, 64, generator=g).half().float() for _ in range(4)]
        if kind == "row0":
            m = torch.ones(B, H, N, N, dtype=torch.bool); m[:, :, 0, :] = False
        elif kind == "causal":
            m = torch.ones(N, N, dtype=torch.bool).tril().expand(B, H, N, N).clone()
        else:
            m = torch.rand(B, H, N, N, generator=g) < kind
        cases.append((name, q, k, v, dout, m))
    for name, q, k, v, dout, m in cases:
        qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
        y = ref.SparseAttentionFunction.apply(qr, kr, vr, ref.pack_mask(m), m, 0.125, q.shape[2])
        y.backward(dout)
        for key, t in (("q", q), ("k", k), ("v", v), ("dout", dout), ("dq", qr.grad), ("dk", kr.grad), ("dv", vr.grad)):
            out[name + "_" + key] = t.numpy().astype(np.float16 if key in ("q", "k", "v", "dout") else np.float32)
        out[name + "_mask"] = m.numpy()
        names.append(name)
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "backward_golden.npz"), **out)
    print("backward_golden.npz", os.path.getsize(os.path.join(HERE, "backward_golden.npz")), "bytes")


def main():
    args = [a for a in sys.argv[1:] if a != "backward"]
    root = args[0] if args else os.environ.get("SMA_REFERENCE_ROOT", "")
    if not root:
        candidates = (os.path.join(REPO, "reference"), os.path.join(os.path.dirname(REPO), "reference"))
        root = next((p for p in candidates if os.path.isdir(p)), "")
    ref = load_reference(root)
    if "backward" in sys.argv[1:]:
        write_backward(ref)
        return
    sys.path.insert(0, REPO)
    from sparse_mask_attention_b200 import workloads

    # ---- packing vectors: (B, H, N) incl. N not a multiple of 32, N < 32, N = 8 (reference's own edge) ----
    pack = {}
    for i, (B, H, N, keep) in enumerate([(1, 1, 8, 0.5), (1, 2, 40, 0.25), (2, 1, 100, 0.25), (1, 1, 64, 0.25),
                                         (2, 2, 128, 0.25), (1, 1, 33, 1.0), (1, 1, 31, 0.0), (1, 1, 96, 0.05)]):
        g = torch.Generator().manual_seed(100 + i)
        mask = torch.rand(B, H, N, N, generator=g) < keep
        packed = ref.pack_mask(mask)
        pack["mask_%d" % i] = mask.numpy()
        pack["packed_%d" % i] = packed.numpy()
    np.savez_compressed(os.path.join(HERE, "pack_golden.npz"), **pack)

    # ---- attention edge cases: fp16-representable inputs stored exactly, fp32 reference outputs ----
    edge = {}
    cases = []
    g = torch.Generator().manual_seed(7)

    def qkv(B, H, N):
        return [torch.randn(B, H, N, 64, generator=g).half() for _ in range(3)]

    # run.py:387-396: B=H=1, N=8, first row fully masked
    q, k, v = qkv(1, 1, 8)
    m = torch.ones(1, 1, 8, 8, dtype=torch.bool); m[:, :, 0, :] = False
    cases.append(("n8_row0_empty", q, k, v, m))
    for name, (B, H, N, keep) in {"n40_iid": (1, 2, 40, 0.25), "n100_iid": (1, 2, 100, 0.25),
                                  "n64_iid": (2, 2, 64, 0.25), "n130_iid": (1, 1, 130, 0.1)}.items():
        q, k, v = qkv(B, H, N)
        m = torch.rand(B, H, N, N, generator=g) < keep
        cases.append((name, q, k, v, m))
    q, k, v = qkv(1, 1, 72)
    cases.append(("n72_all_true", q, k, v, torch.ones(1, 1, 72, 72, dtype=torch.bool)))
    q, k, v = qkv(1, 1, 72)
    cases.append(("n72_all_false", q, k, v, torch.zeros(1, 1, 72, 72, dtype=torch.bool)))
    q, k, v = qkv(1, 2, 96)
    m = torch.zeros(1, 2, 96, 96, dtype=torch.bool)
    cols = torch.randint(0, 96, (1, 2, 96), generator=g)
    m.scatter_(3, cols.unsqueeze(-1), True)
    cases.append(("n96_one_per_row", q, k, v, m))
    names = []
    for name, q, k, v, m in cases:
        out = ref.sparse_attention_ref(q.float(), k.float(), v.float(), m)
        lse = lse_of(ref, q, k, v, m, 1.0 / 8.0)
        edge[name + "_q"], edge[name + "_k"], edge[name + "_v"] = q.numpy(), k.numpy(), v.numpy()
        edge[name + "_mask"], edge[name + "_out"], edge[name + "_lse"] = m.numpy(), out.numpy(), lse.numpy()
        names.append(name)
    edge["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "attention_edge_golden.npz"), **edge)

    # ---- configuration 1 (B2 H4 N128 D64 fp32, seed 0, keep 0.25, diagonal kept) --------------------
    cfg = workloads.CONFIGS[1]
    torch.manual_seed(0)
    q = torch.randn(cfg.B, cfg.H, cfg.N, 64)
    k = torch.randn(cfg.B, cfg.H, cfg.N, 64)
    v = torch.randn(cfg.B, cfg.H, cfg.N, 64)
    mask = torch.rand(cfg.B, cfg.H, cfg.N, cfg.N) > 0.75
    idx = torch.arange(cfg.N)
    mask[..., idx, idx] = True
    wq, wk, wv, wmask = workloads.make_inputs(cfg)
    assert torch.equal(q, wq) and torch.equal(k, wk) and torch.equal(v, wv) and torch.equal(mask, wmask)
    out_ref = ref.sparse_attention_ref(q, k, v, mask)              # fp32 oracle
    with contextlib.redirect_stdout(io.StringIO()):
        out_api = ref.sparse_attention(q, k, v, mask)              # public entry point: bf16 inputs, fp32 result
    cfg1 = dict(sha_q=np.array(sha(q)), sha_k=np.array(sha(k)), sha_v=np.array(sha(v)), sha_mask=np.array(sha(mask)),
                out_ref=out_ref.numpy(), out_api=out_api.numpy(),
                lse=lse_of(ref, q, k, v, mask, 1.0 / 8.0).numpy(), packed=ref.pack_mask(mask).numpy())
    np.savez_compressed(os.path.join(HERE, "config1_golden.npz"), **cfg1)
    for f in ("pack_golden.npz", "attention_edge_golden.npz", "config1_golden.npz"):
        print(f, os.path.getsize(os.path.join(HERE, f)), "bytes")
    write_backward(ref)


if __name__ == "__main__":
    main()
