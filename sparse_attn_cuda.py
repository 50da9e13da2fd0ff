"""Import-path shim: the reference's Python layer does ``import sparse_attn_cuda`` (python/sparse_attention.py:12-17)
for its compiled extension.  With the repository root on ``sys.path`` that import resolves to this module, which
re-exports the two functions the reference binds (csrc/binding.cpp:68-71) from the B200 library's stand-in, and the
``backward`` that the reference's autograd function calls (python/sparse_attention.py:90-94) but its own extension
does not have."""
from sparse_mask_attention_b200.sparse_attn_cuda import backward, forward, pack_mask  # noqa: F401
