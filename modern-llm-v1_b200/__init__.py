"""B200-native causal grouped-query attention behind the flash-attention entry
points of AlsoTheZv3n/modern-llm-v1 (llm/src/model/flash_attn.h).

The compute lives in libb200attn.so (hand-written CUDA for sm_100a, C ABI in
include/b200attn.h); this package is the thin host side: a ctypes binding, the
reference-shaped operator functions over torch CUDA tensors, seeded input
builders for the benchmark shapes and the (batch, KV-head) shard arithmetic for
multi-GPU runs.
"""
from . import _lib  # noqa: F401
from .flash_attn import (  # noqa: F401
    device_status,
    flash_attn_backward,
    flash_attn_backward_gqa,
    flash_attn_decode,
    flash_attn_forward,
    flash_attn_forward_gqa,
)
from .kv_cache import KVCache  # noqa: F401
from .rope_norm import (  # noqa: F401
    make_rope_cache,
    rope_qknorm_backward,
    rope_qknorm_backward_qk,
    rope_qknorm_forward,
    rope_qknorm_forward_qk,
)

__all__ = [
    "flash_attn_forward",
    "flash_attn_backward",
    "flash_attn_forward_gqa",
    "flash_attn_backward_gqa",
    "flash_attn_decode",
    "device_status",
    "KVCache",
    "make_rope_cache",
    "rope_qknorm_forward",
    "rope_qknorm_backward",
    "rope_qknorm_forward_qk",
    "rope_qknorm_backward_qk",
]
