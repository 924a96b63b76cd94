"""ctypes binding of libb200attn.so (the C ABI declared in include/b200attn.h).

There is no fallback: if the library is missing or a call fails, an exception is
raised.  Exceptions follow the reference's convention (llm/src/model/flash_attn.cu:386-407,
llm/src/core/cuda_check.h:12-27): ValueError for bad arguments (std::invalid_argument
there), RuntimeError for CUDA / device failures (std::runtime_error there).
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libb200attn.so")

OK = 0
ERR_INVALID_ARG = 1
ERR_UNSUPPORTED = 2
ERR_ALIGNMENT = 3
ERR_WORKSPACE = 4
ERR_CUDA = 5
ERR_TENSOR_MAP = 6
ERR_DEVICE_WAIT = 7
ERR_NO_DEVICE = 8
ERR_TOO_LARGE = 9
BWD_STATIC_MAX_ROWS = 524288

LAYOUT_BHTD = 0
LAYOUT_BTHD = 1
LAYOUTS = {"BHTD": LAYOUT_BHTD, "BTHD": LAYOUT_BTHD}
DTYPE_BF16 = 0
DTYPE_F32 = 1
BWD_AUTO = 0
BWD_TWO_PASS = 1
BWD_ONE_PASS = 2
BWD_MODES = {"auto": BWD_AUTO, "two_pass": BWD_TWO_PASS, "one_pass": BWD_ONE_PASS}

# every symbol include/b200attn.h declares
SYMBOLS = (
    "b200attn_fwd",
    "b200attn_bwd",
    "b200attn_bwd_workspace_bytes",
    "b200attn_bwd_mode",
    "b200attn_bwd_workspace_bytes_mode",
    "b200attn_bwd_static",
    "b200attn_set_bwd_profile_events",
    "b200attn_set_bwd_profile_events4",
    "b200attn_decode",
    "b200attn_decode_workspace_bytes",
    "b200attn_decode_default_splits",
    "b200attn_decode_cached",
    "b200attn_fwd_kvcache",
    "b200attn_fwd_kvcache_at",
    "b200attn_kv_append",
    "b200attn_kv_append_at",
    "b200attn_item_deal",
    "b200attn_decode_ragged",
    "b200attn_rope_table",
    "b200attn_rope_norm_fwd",
    "b200attn_rope_norm_bwd",
    "b200attn_rope_norm_bwd_workspace_bytes",
    "b200attn_rope_norm_fwd_qk",
    "b200attn_rope_norm_bwd_qk",
    "b200attn_last_device_status",
    "b200attn_strerror",
    "b200attn_version",
)

_lib = None


def load() -> ctypes.CDLL:
    """Loads the library; raises RuntimeError if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m modern_llm_v1_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    L = ctypes.CDLL(LIB_PATH)
    vp, i, f, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    L.b200attn_fwd.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, f, vp]
    L.b200attn_fwd.restype = i
    L.b200attn_bwd.argtypes = [vp] * 9 + [i, i, i, i, i, i, f, vp, sz, vp]
    L.b200attn_bwd.restype = i
    L.b200attn_bwd_static.argtypes = [vp] * 9 + [i, i, i, i, i, i, f, vp]
    L.b200attn_bwd_static.restype = i
    L.b200attn_bwd_workspace_bytes.argtypes = [i, i, i, i, i]
    L.b200attn_bwd_workspace_bytes.restype = sz
    L.b200attn_bwd_mode.argtypes = [vp] * 9 + [i, i, i, i, i, i, f, i, vp, sz, vp]
    L.b200attn_bwd_mode.restype = i
    L.b200attn_bwd_workspace_bytes_mode.argtypes = [i, i, i, i, i, i]
    L.b200attn_bwd_workspace_bytes_mode.restype = sz
    L.b200attn_set_bwd_profile_events.argtypes = [vp, vp, vp]
    L.b200attn_set_bwd_profile_events.restype = i
    L.b200attn_set_bwd_profile_events4.argtypes = [vp, vp, vp, vp]
    L.b200attn_set_bwd_profile_events4.restype = i
    L.b200attn_decode.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, f, i, vp, sz, vp]
    L.b200attn_decode.restype = i
    L.b200attn_decode_workspace_bytes.argtypes = [i, i, i, i, i, i]
    L.b200attn_decode_workspace_bytes.restype = sz
    L.b200attn_decode_default_splits.argtypes = [i, i, i, i, i]
    L.b200attn_decode_default_splits.restype = i
    L.b200attn_decode_cached.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, f, i, vp, sz, vp]
    L.b200attn_decode_cached.restype = i
    L.b200attn_fwd_kvcache.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, vp]
    L.b200attn_fwd_kvcache.restype = i
    L.b200attn_fwd_kvcache_at.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, f, vp]
    L.b200attn_fwd_kvcache_at.restype = i
    L.b200attn_kv_append.argtypes = [vp, vp, vp, i, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, i, f, vp]
    L.b200attn_kv_append.restype = i
    L.b200attn_kv_append_at.argtypes = [vp, vp, vp, i, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, f, vp]
    L.b200attn_kv_append_at.restype = i
    L.b200attn_decode_ragged.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, f, i, vp, sz, vp]
    L.b200attn_decode_ragged.restype = i
    L.b200attn_item_deal.argtypes = [i, i, i, i, i, vp, vp]
    L.b200attn_item_deal.restype = i
    L.b200attn_rope_table.argtypes = [i, i, f, vp, vp]
    L.b200attn_rope_table.restype = i
    L.b200attn_rope_norm_fwd.argtypes = [vp, i, i, vp, i, vp, vp, vp, vp, i, i, i, i, f, vp]
    L.b200attn_rope_norm_fwd.restype = i
    L.b200attn_rope_norm_bwd.argtypes = [vp, i, vp, i, i, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, sz, vp]
    L.b200attn_rope_norm_bwd.restype = i
    L.b200attn_rope_norm_fwd_qk.argtypes = [vp, vp, i, i, vp, vp, i, vp, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp]
    L.b200attn_rope_norm_fwd_qk.restype = i
    L.b200attn_rope_norm_bwd_qk.argtypes = [vp, vp, i, vp, vp, i, i, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i, i, i, i, i,
                                            vp, sz, vp]
    L.b200attn_rope_norm_bwd_qk.restype = i
    L.b200attn_rope_norm_bwd_workspace_bytes.argtypes = [i]
    L.b200attn_rope_norm_bwd_workspace_bytes.restype = sz
    L.b200attn_last_device_status.argtypes = [vp]
    L.b200attn_last_device_status.restype = i
    L.b200attn_strerror.argtypes = [i]
    L.b200attn_strerror.restype = ctypes.c_char_p
    L.b200attn_version.restype = i
    _lib = L
    return L


def strerror(status: int) -> str:
    return load().b200attn_strerror(int(status)).decode()


def check(status: int, where: str) -> None:
    """Turns a non-zero status into the reference's exception types."""
    if status == OK:
        return
    msg = f"{where}: {strerror(status)} (status {status})"
    if status in (ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_WORKSPACE, ERR_TOO_LARGE):
        raise ValueError(msg)
    raise RuntimeError(msg)
