"""The C-ABI library on a machine without a GPU: it loads, exports every symbol include/sma.h declares,
and rejects bad arguments before touching CUDA.  No kernel is launched here."""
import ctypes
import os
import re

import pytest

from sparse_mask_attention_b200 import _capi

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(REPO, "include", "sma.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(sma_[a-z_0-9]+)\s*\(", text)))


def test_header_and_binding_list_the_same_symbols():
    assert declared_functions() == sorted(_capi.EXPORTED_SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_capi.LIB_PATH)
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert lib.sma_abi_version() == _capi.SMA_ABI_VERSION


def test_status_codes_and_messages_match_the_header():
    text = open(os.path.join(REPO, "include", "sma.h")).read()
    for name, value in re.findall(r"(SMA_(?:OK|ERR_[A-Z_]+))\s*=\s*(-?\d+)", text):
        assert getattr(_capi, name) == int(value), name
        msg = _capi.strerror(int(value))
        assert msg and msg != "unknown status"
    assert _capi.strerror(-12345) == "unknown status"
    for name, value in re.findall(r"#define\s+(SMA_[A-Z_0-9]+)\s+(\d+)\s", text):
        if hasattr(_capi, name):
            assert getattr(_capi, name) == int(value), name


def test_params_struct_layout_matches_the_header():
    # 6 pointers, 4 int32, float, 3 int32, then 4 x 3 int64 strides on an LP64 machine: 176 bytes
    assert ctypes.sizeof(_capi.AttentionParams) == 6 * 8 + 8 * 4 + 12 * 8
    assert _capi.AttentionParams.B.offset == 48 and _capi.AttentionParams.scale.offset == 64
    assert _capi.AttentionParams.variant.offset == 76
    assert _capi.AttentionParams.q_strides.offset == 80 and _capi.AttentionParams.out_strides.offset == 152


def _params(**kw):
    p = _capi.AttentionParams()
    p.q = p.k = p.v = p.mask_packed = p.out = 0x1000
    p.lse = None
    p.B, p.H, p.N, p.D = 1, 1, 64, 64
    p.scale, p.dtype, p.save_lse, p.variant = 0.125, _capi.SMA_DTYPE_F16, 0, 0
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,status", [
    (dict(q=None), _capi.SMA_ERR_NULL_POINTER),
    (dict(out=None), _capi.SMA_ERR_NULL_POINTER),
    (dict(save_lse=1), _capi.SMA_ERR_NULL_POINTER),           # lse required when save_lse is set
    (dict(B=0), _capi.SMA_ERR_BAD_SHAPE),
    (dict(N=-5), _capi.SMA_ERR_BAD_SHAPE),
    (dict(D=128), _capi.SMA_ERR_BAD_HEAD_DIM),
    (dict(dtype=7), _capi.SMA_ERR_BAD_DTYPE),
    (dict(N=_capi.SMA_MAX_SEQ_LEN + 1), _capi.SMA_ERR_SEQ_TOO_LONG),
    (dict(scale=0.0), _capi.SMA_ERR_BAD_SCALE),
    (dict(scale=float("nan")), _capi.SMA_ERR_BAD_SCALE),
    (dict(scale=float("inf")), _capi.SMA_ERR_BAD_SCALE),
    (dict(k=0x1008), _capi.SMA_ERR_MISALIGNED),
    (dict(q_strides=(ctypes.c_int64 * 3)(4096, 64, 100)), _capi.SMA_ERR_BAD_STRIDE),     # not a multiple of 8 elements
    (dict(v_strides=(ctypes.c_int64 * 3)(4096, 0, 64)), _capi.SMA_ERR_BAD_STRIDE),       # zero among non-zero strides
    (dict(out_strides=(ctypes.c_int64 * 3)(-4096, 64, 64)), _capi.SMA_ERR_BAD_STRIDE),
    (dict(mask_packed=0x1002), _capi.SMA_ERR_MISALIGNED),
    (dict(variant=99), _capi.SMA_ERR_BAD_VARIANT),
    (dict(variant=_capi.SMA_VARIANT_BF16_SINGLE_P), _capi.SMA_ERR_BAD_VARIANT),  # fp16 has no such variant
])
def test_attention_argument_validation_needs_no_gpu(kw, status):
    assert _capi.lib.sma_attention_fwd(ctypes.byref(_params(**kw)), None) == status


def test_attention_null_params():
    assert _capi.lib.sma_attention_fwd(None, None) == _capi.SMA_ERR_NULL_POINTER


@pytest.mark.parametrize("args,status", [
    ((None, 0x1000, 1, 1, 8), _capi.SMA_ERR_NULL_POINTER),
    ((0x1000, None, 1, 1, 8), _capi.SMA_ERR_NULL_POINTER),
    ((0x1000, 0x1000, 0, 1, 8), _capi.SMA_ERR_BAD_SHAPE),
    ((0x1000, 0x1000, 1, 1, 0), _capi.SMA_ERR_BAD_SHAPE),
    ((0x1000, 0x1002, 1, 1, 8), _capi.SMA_ERR_MISALIGNED),
    ((0x1000, 0x1000, 2 ** 20, 2 ** 10, 2 ** 20), _capi.SMA_ERR_BAD_SHAPE),  # index range
])
def test_pack_argument_validation_needs_no_gpu(args, status):
    assert _capi.lib.sma_pack_mask(*args, None) == status


def test_check_raises_with_status():
    with pytest.raises(_capi.SmaError) as e:
        _capi.check(_capi.SMA_ERR_BAD_HEAD_DIM)
    assert e.value.status == _capi.SMA_ERR_BAD_HEAD_DIM and "64" in str(e.value)
