"""The C-ABI library without a GPU: it loads, exports every symbol the header declares,
and rejects bad arguments before touching CUDA (no compute calls here)."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in os.listdir(inc):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(b200attn_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol(lib):
    from modern_llm_v1_b200 import _lib

    declared = _declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(_lib.SYMBOLS), "ctypes binding and header disagree"


def test_version_and_strerror(lib):
    assert lib.b200attn_version() >= 1
    for code in range(0, 10):
        assert lib.b200attn_strerror(code).decode() not in ("", "unknown status")
    assert lib.b200attn_strerror(12345).decode() == "unknown status"


def test_argument_validation_happens_before_any_cuda_call(lib):
    from modern_llm_v1_b200 import _lib

    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf)
    p16 = (p + 255) & ~255
    f = lib.b200attn_fwd
    assert f(None, p16, p16, p16, p16, 1, 128, 1, 1, 64, 0, 0.0, None) == _lib.ERR_INVALID_ARG
    assert f(p16, p16, p16, p16, p16, 0, 128, 1, 1, 64, 0, 0.0, None) == _lib.ERR_INVALID_ARG
    assert f(p16, p16, p16, p16, p16, 1, 128, 6, 4, 64, 0, 0.0, None) == _lib.ERR_INVALID_ARG  # Hq % Hkv
    assert f(p16, p16, p16, p16, p16, 1, 128, 1, 1, 64, 7, 0.0, None) == _lib.ERR_INVALID_ARG  # layout
    assert f(p16, p16, p16, p16, p16, 1, 128, 1, 1, 32, 0, 0.0, None) == _lib.ERR_UNSUPPORTED  # head dim
    assert f(p16 + 2, p16, p16, p16, p16, 1, 128, 1, 1, 64, 0, 0.0, None) == _lib.ERR_ALIGNMENT
    b = lib.b200attn_bwd
    args = [p16] * 9 + [1, 128, 1, 1, 64, 0, 0.0]
    assert b(*args, None, 0, None) == _lib.ERR_WORKSPACE
    assert b(*args, p16, 16, None) == _lib.ERR_WORKSPACE  # too small
    bm = lib.b200attn_bwd_mode
    assert bm(*args, 9, p16, 4096, None) == _lib.ERR_INVALID_ARG  # no such mode
    assert bm(*([p16] * 9 + [1, 128, 1, 1, 128, 0, 0.0]), _lib.BWD_ONE_PASS, p16, 4096, None) == _lib.ERR_UNSUPPORTED
    assert bm(*args, _lib.BWD_ONE_PASS, p16, 2 * 128 * 4, None) == _lib.ERR_WORKSPACE  # holds the vectors only
    d = lib.b200attn_decode
    assert d(p16, p16, p16, p16, None, 1, 128, 4, 3, 64, 0.0, 0, p16, 4096, None) == _lib.ERR_INVALID_ARG
    assert d(p16, p16, p16, p16, None, 1, 128, 4, 2, 64, 0.0, 0, None, 0, None) == _lib.ERR_WORKSPACE


def test_workspace_sizes(lib):
    from modern_llm_v1_b200 import _lib

    # two-pass: two FP32 vectors of B*Hq*ceil(T/128)*128; one-pass (D = 64): + an FP32 dq accumulator of that many rows
    w = lib.b200attn_bwd_workspace_bytes_mode
    assert w(32, 512, 6, 2, 64, _lib.BWD_TWO_PASS) == 2 * 32 * 6 * 512 * 4
    assert w(1, 77, 2, 1, 64, _lib.BWD_TWO_PASS) == 2 * 1 * 2 * 128 * 4
    assert w(32, 512, 6, 2, 64, _lib.BWD_ONE_PASS) == 2 * 32 * 6 * 512 * 4 + 32 * 6 * 512 * 64 * 4
    assert w(1, 77, 2, 1, 64, _lib.BWD_ONE_PASS) == 2 * 1 * 2 * 128 * 4 + 2 * 128 * 64 * 4
    assert w(4, 8192, 16, 4, 128, _lib.BWD_AUTO) == 2 * 4 * 16 * 8192 * 4  # D = 128 has no one-pass kernel
    assert w(1, 77, 2, 1, 64, 7) == 0
    if not os.environ.get("B200ATTN_BWD"):
        assert lib.b200attn_bwd_workspace_bytes(32, 512, 6, 2, 64) == w(32, 512, 6, 2, 64, _lib.BWD_TWO_PASS)
    assert lib.b200attn_bwd_workspace_bytes(0, 77, 2, 1, 64) == 0
    s = lib.b200attn_decode_default_splits(64, 4096, 16, 4, 64)
    assert 1 <= s <= 32
    assert lib.b200attn_decode_workspace_bytes(64, 4096, 16, 4, 64, 0) == 64 * 16 * s * (64 + 2) * 4
    assert lib.b200attn_decode_workspace_bytes(2, 100, 4, 2, 64, 9) == 2 * 4 * 1 * 66 * 4  # one tile -> one split
    assert lib.b200attn_decode_default_splits(1, 128, 6, 4, 64) == 0


def test_check_maps_status_to_reference_exception_types(lib):
    from modern_llm_v1_b200 import _lib

    _lib.check(0, "x")
    for code in (_lib.ERR_INVALID_ARG, _lib.ERR_UNSUPPORTED, _lib.ERR_ALIGNMENT, _lib.ERR_WORKSPACE):
        with pytest.raises(ValueError):
            _lib.check(code, "x")
    for code in (_lib.ERR_CUDA, _lib.ERR_TENSOR_MAP, _lib.ERR_DEVICE_WAIT, _lib.ERR_NO_DEVICE, 101):
        with pytest.raises(RuntimeError):
            _lib.check(code, "x")
