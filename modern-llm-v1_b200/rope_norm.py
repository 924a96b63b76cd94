"""Host-side mirror of the fused RoPE + QK-Norm operator (csrc/rope_norm.cuh).

The reference prepares q and k for attention with split_heads -> rope_apply_inplace ->
rmsnorm_forward (llm/src/model/modern_gpt.cu:351-370) and undoes it in the backward with
rmsnorm_backward -> rope_apply_backward_inplace -> merge_heads (llm/src/model/modern_gpt.cu:527-552).
The two functions here do each chain in one pass; argument names follow the reference's operators
(llm/src/model/rope.h, llm/src/model/rmsnorm.h): caller allocates every tensor, outputs are
overwritten, except ``d_gamma``, which is accumulated into as in the reference
(llm/src/model/rmsnorm.h:17).  Bad dtype / device / shape raise ValueError, CUDA failures
RuntimeError.  There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from . import _lib
from .flash_attn import _check_tensors, _stream_ptr, _workspace


def make_rope_cache(T_max: int, d_h: int, base: float = 10000.0, device="cuda"):
    """cos, sin tables [T_max, d_h / 2] FP32 with the values of the reference's make_rope_cache
    (llm/src/model/rope.cu:112-128), computed by the library on the host and copied to `device`."""
    if d_h % 2 != 0:
        raise ValueError("d_h must be even")
    cos = np.empty((T_max, d_h // 2), dtype=np.float32)
    sin = np.empty_like(cos)
    lib = _lib.load()
    _lib.check(lib.b200attn_rope_table(T_max, d_h, ctypes.c_float(base), cos.ctypes.data, sin.ctypes.data),
               "make_rope_cache")
    return torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device)


def _x_dtype(fn, x):
    if x.dtype == torch.bfloat16:
        return _lib.DTYPE_BF16
    if x.dtype == torch.float32:
        return _lib.DTYPE_F32
    raise ValueError(f"{fn}: x must be BF16 or FP32")


def _common(fn, first, x, cos, sin, gamma, rstd, B, T, H, D, x_layout, y_layout):
    f32 = torch.float32
    # every dtype first, then every device, like the reference's operators
    _check_tensors(fn, first + [(cos, "cos", f32), (sin, "sin", f32), (gamma, "gamma", f32), (rstd, "rstd", f32)])
    for name, lay in (("x_layout", x_layout), ("y_layout", y_layout)):
        if lay not in _lib.LAYOUTS:
            raise ValueError(f"{fn}: {name} must be BHTD or BTHD")
    if D % 2 != 0:
        raise ValueError(f"{fn}: d_h must be even")
    if x.numel() != B * T * H * D:
        raise ValueError(f"{fn}: x numel mismatch")
    if cos.numel() < T * (D // 2) or sin.numel() < T * (D // 2) or cos.shape[-1] != D // 2:
        raise ValueError(f"{fn}: cos/sin tables must be [>= T, d_h / 2]")
    if gamma.numel() != D:
        raise ValueError(f"{fn}: gamma must have d_h elements")
    if rstd.numel() != B * H * T:
        raise ValueError(f"{fn}: rstd must have B * H * T elements")


def rope_qknorm_forward(x, cos, sin, gamma, eps, y, rstd, B, T, H, D, x_layout="BTHD", y_layout="BHTD"):
    """y = RMSNorm(RoPE(x)) * gamma per head row, rstd = 1 / rms (FP32 [B, H, T]).  x: B*T*H rows of D
    elements, BF16 or FP32, in x_layout (BTHD = the projection output where it lies); y: BF16 in y_layout,
    ready for flash_attn_forward_gqa."""
    fn = "rope_qknorm_forward"
    xd = _x_dtype(fn, x)
    _common(fn, [(x, "x", x.dtype), (y, "y", torch.bfloat16)], x, cos, sin, gamma, rstd, B, T, H, D, x_layout, y_layout)
    if y.numel() != x.numel():
        raise ValueError(f"{fn}: y numel mismatch")
    lib = _lib.load()
    _lib.check(lib.b200attn_rope_norm_fwd(x.data_ptr(), xd, _lib.LAYOUTS[x_layout], y.data_ptr(), _lib.LAYOUTS[y_layout],
                                          rstd.data_ptr(), gamma.data_ptr(), cos.data_ptr(), sin.data_ptr(), B, T, H, D,
                                          ctypes.c_float(eps), _stream_ptr()), fn)


def rope_qknorm_backward(d_y, x, cos, sin, gamma, rstd, d_x, d_gamma, B, T, H, D, x_layout="BTHD", y_layout="BHTD"):
    """d_x (x's type and layout, overwritten) and d_gamma (FP32 [D], accumulated into) from d_y (BF16 in
    y_layout), the forward's input x and its rstd."""
    fn = "rope_qknorm_backward"
    xd = _x_dtype(fn, x)
    _common(fn, [(d_y, "d_y", torch.bfloat16), (x, "x", x.dtype), (d_x, "d_x", x.dtype),
                 (d_gamma, "d_gamma", torch.float32)], x, cos, sin, gamma, rstd, B, T, H, D, x_layout, y_layout)
    if d_y.numel() != x.numel() or d_x.numel() != x.numel() or d_gamma.numel() != D:
        raise ValueError(f"{fn}: shape mismatch (d_y/d_x/d_gamma)")
    lib = _lib.load()
    nbytes = int(lib.b200attn_rope_norm_bwd_workspace_bytes(D))
    ws = _workspace("rope_norm_bwd", nbytes, x.device)
    _lib.check(lib.b200attn_rope_norm_bwd(d_y.data_ptr(), _lib.LAYOUTS[y_layout], x.data_ptr(), xd,
                                          _lib.LAYOUTS[x_layout], rstd.data_ptr(), gamma.data_ptr(), cos.data_ptr(),
                                          sin.data_ptr(), d_x.data_ptr(), d_gamma.data_ptr(), B, T, H, D, ws.data_ptr(),
                                          ws.numel(), _stream_ptr()), fn)


def rope_qknorm_forward_qk(xq, xk, cos, sin, gamma_q, gamma_k, eps, yq, yk, rstd_q, rstd_k, B, T, Hq, Hkv, D,
                           x_layout="BTHD", y_layout="BHTD"):
    """rope_qknorm_forward for q (Hq heads) and k (Hkv heads) in one launch; bit-identical to two calls."""
    fn = "rope_qknorm_forward"
    xd = _x_dtype(fn, xq)
    if xk.dtype != xq.dtype:
        raise ValueError(f"{fn}: xq and xk must have the same dtype")
    bf = torch.bfloat16
    _common(fn, [(xq, "xq", xq.dtype), (xk, "xk", xq.dtype), (yq, "yq", bf), (yk, "yk", bf),
                 (gamma_k, "gamma_k", torch.float32), (rstd_k, "rstd_k", torch.float32)],
            xq, cos, sin, gamma_q, rstd_q, B, T, Hq, D, x_layout, y_layout)
    if xk.numel() != B * T * Hkv * D or yq.numel() != xq.numel() or yk.numel() != xk.numel():
        raise ValueError(f"{fn}: shape mismatch (xk/yq/yk)")
    if gamma_k.numel() != D or rstd_k.numel() != B * Hkv * T:
        raise ValueError(f"{fn}: shape mismatch (gamma_k/rstd_k)")
    lib = _lib.load()
    _lib.check(lib.b200attn_rope_norm_fwd_qk(xq.data_ptr(), xk.data_ptr(), xd, _lib.LAYOUTS[x_layout], yq.data_ptr(),
                                             yk.data_ptr(), _lib.LAYOUTS[y_layout], rstd_q.data_ptr(), rstd_k.data_ptr(),
                                             gamma_q.data_ptr(), gamma_k.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                             B, T, Hq, Hkv, D, ctypes.c_float(eps), _stream_ptr()), fn)


def rope_qknorm_backward_qk(d_yq, d_yk, xq, xk, cos, sin, gamma_q, gamma_k, rstd_q, rstd_k, d_xq, d_xk, d_gamma_q,
                            d_gamma_k, B, T, Hq, Hkv, D, x_layout="BTHD", y_layout="BHTD"):
    """rope_qknorm_backward for q and k in one launch; bit-identical to two calls."""
    fn = "rope_qknorm_backward"
    xd = _x_dtype(fn, xq)
    if xk.dtype != xq.dtype:
        raise ValueError(f"{fn}: xq and xk must have the same dtype")
    bf, f32 = torch.bfloat16, torch.float32
    _common(fn, [(d_yq, "d_yq", bf), (d_yk, "d_yk", bf), (xq, "xq", xq.dtype), (xk, "xk", xq.dtype),
                 (d_xq, "d_xq", xq.dtype), (d_xk, "d_xk", xq.dtype), (d_gamma_q, "d_gamma_q", f32),
                 (d_gamma_k, "d_gamma_k", f32), (gamma_k, "gamma_k", f32), (rstd_k, "rstd_k", f32)],
            xq, cos, sin, gamma_q, rstd_q, B, T, Hq, D, x_layout, y_layout)
    nq, nk = B * T * Hq * D, B * T * Hkv * D
    if xk.numel() != nk or d_yq.numel() != nq or d_yk.numel() != nk or d_xq.numel() != nq or d_xk.numel() != nk:
        raise ValueError(f"{fn}: shape mismatch (xk/d_y/d_x)")
    if gamma_k.numel() != D or rstd_k.numel() != B * Hkv * T or d_gamma_q.numel() != D or d_gamma_k.numel() != D:
        raise ValueError(f"{fn}: shape mismatch (gamma_k/rstd_k/d_gamma)")
    lib = _lib.load()
    nbytes = int(lib.b200attn_rope_norm_bwd_workspace_bytes(D))
    ws = _workspace("rope_norm_bwd", nbytes, xq.device)
    _lib.check(lib.b200attn_rope_norm_bwd_qk(d_yq.data_ptr(), d_yk.data_ptr(), _lib.LAYOUTS[y_layout], xq.data_ptr(),
                                             xk.data_ptr(), xd, _lib.LAYOUTS[x_layout], rstd_q.data_ptr(),
                                             rstd_k.data_ptr(), gamma_q.data_ptr(), gamma_k.data_ptr(), cos.data_ptr(),
                                             sin.data_ptr(), d_xq.data_ptr(), d_xk.data_ptr(), d_gamma_q.data_ptr(),
                                             d_gamma_k.data_ptr(), B, T, Hq, Hkv, D, ws.data_ptr(), ws.numel(),
                                             _stream_ptr()), fn)
