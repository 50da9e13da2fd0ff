"""Import-path shim: the reference's Python layer does ``import sparse_attn_cuda`` (python/sparse_attention.py:12-17)
for its compiled extension.  With the repository root on ``sys.path`` that import resolves to this module, which
re-exports the two functions the reference binds (csrc/binding.cpp:68-71) from the B200 library's stand-in."""
from sparse_mask_attention_b200.sparse_attn_cuda import forward, pack_mask  # noqa: F401
