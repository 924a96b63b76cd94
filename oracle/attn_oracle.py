"""CPU oracle for causal grouped-query attention (numpy + the C restatement).

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels and
the timed CPU baseline of the benchmark.  Product code never imports it.

Two implementations of the same math live here:

* ``*_c``  : ctypes bindings of ``attn_oracle.c`` (OpenMP, double accumulation),
  which cites the reference lines it restates;
* ``*_np`` : a short vectorised numpy restatement (float64) used to cross-check
  the C code on small cases.

Both follow AlsoTheZv3n/modern-llm-v1: forward of ``attn_host``
(llm/tests/test_attention.cu:21-75), logsumexp of
llm/src/model/flash_attn.cu:124-130, backward of llm/src/model/flash_attn.cu:137-146,
GQA head mapping and group sum of llm/src/model/attention.cu:393-429.

Parity pin: the fixtures under tests/golden/ were produced by the reference's
own host functions compiled from its tree (see tests/golden/make_golden.py).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_attn.so")


class _Strides(ctypes.Structure):
    _fields_ = [("sb", ctypes.c_longlong), ("sh", ctypes.c_longlong), ("st", ctypes.c_longlong)]


def build(force: bool = False) -> str:
    """Compiles attn_oracle.c into liboracle_attn.so (gcc, OpenMP)."""
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "liboracle_attn.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        fp = ctypes.POINTER(ctypes.c_float)
        sp = ctypes.POINTER(_Strides)
        i = ctypes.c_int
        L.oracle_num_threads.restype = i
        L.oracle_set_num_threads.argtypes = [i]
        L.oracle_round_bf16.argtypes = [fp, ctypes.c_longlong]
        L.oracle_f32_to_bf16.argtypes = [fp, ctypes.POINTER(ctypes.c_uint16), ctypes.c_longlong]
        L.oracle_bf16_to_f32.argtypes = [ctypes.POINTER(ctypes.c_uint16), fp, ctypes.c_longlong]
        L.oracle_rope_inplace.argtypes = [fp, ctypes.c_longlong, i, i, ctypes.c_float, i]
        L.oracle_rmsnorm_rows.argtypes = [fp, ctypes.c_longlong, i, ctypes.c_float]
        L.oracle_rope_norm_fwd.argtypes = [fp, fp, fp, fp, ctypes.c_longlong, i, i, ctypes.c_float, ctypes.c_float]
        L.oracle_rope_norm_fwd_at.argtypes = [fp, fp, fp, fp, ctypes.c_longlong, i, i, ctypes.c_float, ctypes.c_float, i]
        L.oracle_rope_norm_bwd.argtypes = [fp, fp, fp, fp, fp, fp, ctypes.c_longlong, i, i, ctypes.c_float]
        L.oracle_attn_fwd.argtypes = [fp, fp, fp, fp, fp, i, i, i, i, i, ctypes.c_float, sp, sp, sp]
        L.oracle_attn_fwd_bwd.argtypes = [fp] * 9 + [i, i, i, i, i, ctypes.c_float, sp, sp, sp]
        L.oracle_decode.argtypes = [fp, fp, fp, fp, fp, i, i, i, i, i, ctypes.c_float, sp]
        _lib = L
    return _lib


def _fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float)) if a is not None else None


def _c32(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a


def _strides(shape_bhtd_layout: str, H: int, T: int, D: int) -> _Strides:
    if shape_bhtd_layout == "BHTD":
        return _Strides(H * T * D, T * D, D)
    if shape_bhtd_layout == "BTHD":
        return _Strides(T * H * D, D, H * D)
    raise ValueError(shape_bhtd_layout)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


# --------------------------------------------------------------------------
# element-wise helpers (pinned against the reference's dtype/rope/rmsnorm)
# --------------------------------------------------------------------------
def round_bf16(x: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even BF16 -> float32 (llm/src/core/dtype.h:34-49)."""
    y = _c32(x).copy()
    lib().oracle_round_bf16(_fp(y), y.size)
    return y


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = _c32(x)
    y = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_f32_to_bf16(_fp(x), y.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), x.size)
    return y


def from_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    y = np.empty(x.shape, dtype=np.float32)
    lib().oracle_bf16_to_f32(x.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), _fp(y), x.size)
    return y


def rope(x: np.ndarray, base: float = 10000.0, pos0: int = 0) -> np.ndarray:
    """RoPE over x[..., T, D] (interleaved pairs), token t at position pos0+t."""
    y = _c32(x).copy()
    T, D = y.shape[-2], y.shape[-1]
    lib().oracle_rope_inplace(_fp(y), y.size // (T * D), T, D, base, pos0)
    return y


def rmsnorm(x: np.ndarray, eps: float = 1e-5) -> np.ndarray:
    """RMSNorm over the last axis with gamma = 1."""
    y = _c32(x).copy()
    D = y.shape[-1]
    lib().oracle_rmsnorm_rows(_fp(y), y.size // D, D, eps)
    return y


def rope_norm_fwd(x: np.ndarray, gamma: np.ndarray, base: float = 10000.0, eps: float = 1e-5):
    """Fused RoPE + RMSNorm over x[..., T, D]: returns (y, rstd[..., T]).  The chain rope_apply_inplace ->
    rmsnorm_forward of llm/src/model/modern_gpt.cu:358-370."""
    x = _c32(x)
    g = _c32(gamma)
    T, D = x.shape[-2], x.shape[-1]
    y = np.empty_like(x)
    rstd = np.empty(x.shape[:-1], dtype=np.float32)
    lib().oracle_rope_norm_fwd(_fp(x), _fp(g), _fp(y), _fp(rstd), x.size // (T * D), T, D, base, eps)
    return y, rstd


def kv_append(xq, xk, xv, gamma_q, gamma_k, kcache, vcache, pos0, base: float = 10000.0, eps: float = 1e-5):
    """What a cached ModernGPT block does to its n_new newest tokens before attention
    (llm/src/model/modern_gpt.cu:351-370, with RoPE at the true positions pos0 + t): xq [B, n_new, Hq, D],
    xk / xv [B, n_new, Hkv, D] -> returns q [B, Hq, n_new, D] and writes rows pos0 .. of kcache / vcache
    [B, Hkv, L_cap, D] (FP32 arrays, updated in place; k rotated and normalised, v as it is)."""
    n_new = xq.shape[1]

    def prep(x, g):
        xt = _c32(np.swapaxes(_c32(x), 1, 2))  # [B, H, n_new, D]
        y = np.empty_like(xt)
        rstd = np.empty(xt.shape[:-1], dtype=np.float32)
        D = xt.shape[-1]
        lib().oracle_rope_norm_fwd_at(_fp(xt), _fp(_c32(g)), _fp(y), _fp(rstd), xt.size // (n_new * D), n_new, D, base,
                                      eps, int(pos0))
        return y

    q = prep(xq, gamma_q)
    kcache[:, :, pos0:pos0 + n_new, :] = prep(xk, gamma_k)
    vcache[:, :, pos0:pos0 + n_new, :] = np.swapaxes(_c32(xv), 1, 2)
    return q


def rope_norm_bwd(dy: np.ndarray, x: np.ndarray, gamma: np.ndarray, rstd: np.ndarray, base: float = 10000.0):
    """Backward of rope_norm_fwd: returns (dx, d_gamma) with d_gamma summed over all rows
    (rmsnorm_backward -> rope_apply_backward_inplace, llm/src/model/modern_gpt.cu:527-544)."""
    dy, x, g, rstd = _c32(dy), _c32(x), _c32(gamma), _c32(rstd)
    T, D = x.shape[-2], x.shape[-1]
    dx = np.empty_like(x)
    dg = np.zeros(D, dtype=np.float32)
    lib().oracle_rope_norm_bwd(_fp(dy), _fp(x), _fp(g), _fp(rstd), _fp(dx), _fp(dg), x.size // (T * D), T, D, base)
    return dx, dg


# --------------------------------------------------------------------------
# attention, C implementation.  q: [B,Hq,T,D] ("BHTD") or [B,T,Hq,D] ("BTHD")
# --------------------------------------------------------------------------
def _dims(q, k, layout):
    if layout == "BHTD":
        B, Hq, T, D = q.shape
        Hkv = k.shape[1]
    else:
        B, T, Hq, D = q.shape
        Hkv = k.shape[2]
    if Hq % Hkv:
        raise ValueError("Hq must be a multiple of Hkv")
    return B, T, Hq, Hkv, D


def attn_fwd_c(q, k, v, scale=None, layout="BHTD"):
    q, k, v = _c32(q), _c32(k), _c32(v)
    B, T, Hq, Hkv, D = _dims(q, k, layout)
    scale = np.float32(1.0 / np.sqrt(np.float32(D))) if scale is None else np.float32(scale)
    o = np.zeros_like(q)
    lse = np.zeros((B, Hq, T), dtype=np.float32)
    sq, skv = _strides(layout, Hq, T, D), _strides(layout, Hkv, T, D)
    lib().oracle_attn_fwd(_fp(q), _fp(k), _fp(v), _fp(o), _fp(lse), B, T, Hq, Hkv, D, scale,
                          ctypes.byref(sq), ctypes.byref(skv), ctypes.byref(sq))
    return o, lse


def attn_fwd_bwd_c(q, k, v, dout, scale=None, layout="BHTD"):
    q, k, v, dout = _c32(q), _c32(k), _c32(v), _c32(dout)
    B, T, Hq, Hkv, D = _dims(q, k, layout)
    scale = np.float32(1.0 / np.sqrt(np.float32(D))) if scale is None else np.float32(scale)
    o = np.zeros_like(q)
    lse = np.zeros((B, Hq, T), dtype=np.float32)
    dq = np.zeros_like(q)
    dk = np.zeros_like(k)
    dv = np.zeros_like(v)
    sq, skv = _strides(layout, Hq, T, D), _strides(layout, Hkv, T, D)
    lib().oracle_attn_fwd_bwd(_fp(q), _fp(k), _fp(v), _fp(dout), _fp(o), _fp(lse), _fp(dq), _fp(dk), _fp(dv),
                              B, T, Hq, Hkv, D, scale, ctypes.byref(sq), ctypes.byref(skv), ctypes.byref(sq))
    return o, lse, dq, dk, dv


def decode_c(q, kc, vc, scale=None):
    """q [B,Hq,D]; kc, vc [B,Hkv,L,D].  Returns o [B,Hq,D], lse [B,Hq]."""
    q, kc, vc = _c32(q), _c32(kc), _c32(vc)
    B, Hq, D = q.shape
    Hkv, L = kc.shape[1], kc.shape[2]
    scale = np.float32(1.0 / np.sqrt(np.float32(D))) if scale is None else np.float32(scale)
    o = np.zeros_like(q)
    lse = np.zeros((B, Hq), dtype=np.float32)
    skv = _strides("BHTD", Hkv, L, D)
    lib().oracle_decode(_fp(q), _fp(kc), _fp(vc), _fp(o), _fp(lse), B, L, Hq, Hkv, D, scale, ctypes.byref(skv))
    return o, lse


# --------------------------------------------------------------------------
# attention, numpy float64 restatement (small cases; BHTD only)
# --------------------------------------------------------------------------
def attn_fwd_bwd_np(q, k, v, dout=None, scale=None):
    q64, k64, v64 = (np.asarray(a, dtype=np.float64) for a in (q, k, v))
    B, Hq, T, D = q64.shape
    Hkv = k64.shape[1]
    g = Hq // Hkv
    scale = 1.0 / np.sqrt(np.float32(D)) if scale is None else scale
    scale = float(np.float32(scale))
    kk = np.repeat(k64, g, axis=1)  # repeat_kv_heads: consecutive q heads share a kv head
    vv = np.repeat(v64, g, axis=1)
    s = np.einsum("bhid,bhjd->bhij", q64, kk) * scale
    mask = np.tril(np.ones((T, T), dtype=bool))
    s = np.where(mask, s, -np.inf)
    m = s.max(axis=-1, keepdims=True)
    e = np.exp(s - m)
    l = e.sum(axis=-1, keepdims=True)
    p = e / l
    o = np.einsum("bhij,bhjd->bhid", p, vv)
    lse = (m + np.log(l))[..., 0]
    if dout is None:
        return o, lse
    do64 = np.asarray(dout, dtype=np.float64)
    dp = np.einsum("bhid,bhjd->bhij", do64, vv)
    dd = (p * dp).sum(axis=-1, keepdims=True)
    ds = p * (dp - dd)
    dq = scale * np.einsum("bhij,bhjd->bhid", ds, kk)
    dkf = scale * np.einsum("bhij,bhid->bhjd", ds, q64)
    dvf = np.einsum("bhij,bhid->bhjd", p, do64)
    dk = dkf.reshape(B, Hkv, g, T, D).sum(axis=2)  # accumulate_kv_grads
    dv = dvf.reshape(B, Hkv, g, T, D).sum(axis=2)
    return o, lse, dq, dk, dv


# --------------------------------------------------------------------------
# error metrics used by every parity test
# --------------------------------------------------------------------------
def max_abs(a, b) -> float:
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64)))) if np.size(a) else 0.0


def rel_l2(a, b) -> float:
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    den = np.sqrt((b * b).sum())
    return float(np.sqrt(((a - b) ** 2).sum()) / den) if den > 0 else 0.0
