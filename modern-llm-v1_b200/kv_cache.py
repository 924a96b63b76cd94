"""Per-layer KV cache for token-by-token sampling (csrc/kv_cache.cuh, csrc/attn_decode.cuh).

The reference's sampler keeps no cache: every generated token re-runs the model over the whole
T-token window (llm/apps/infer_modern_gpt.cu:13,253-255), and the cache is listed as future work
(TODO.md, "KV cache for inference").  This class is the attention side of that cache for a
ModernGPT block (llm/src/model/modern_gpt.cu:351-378): per layer a BF16 K and V buffer
[B, Hkv, L_cap, D]; `append` does split_heads + RoPE at the true positions + QK-Norm for the newest
tokens and stores their k and v, `attend` runs attention for them (causal forward over the prompt,
or the split-KV decode kernel for one token), `advance` moves the length once every layer is done.
The B sequences advance in lock step until `set_lengths` gives each its own length (a batch of
prompts of different lengths); from then on `append` and `attend` take one token per sequence at the
sequence's own position.  Like the reference's operators, the caller allocates every
input and output; bad arguments raise ValueError, CUDA failures RuntimeError; there is no CPU or
PyTorch fallback.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from .flash_attn import _check_tensors, _stream_ptr, _workspace
from .rope_norm import _x_dtype, make_rope_cache


class KVCache:
    def __init__(self, n_layers: int, B: int, Hq: int, Hkv: int, D: int, L_cap: int, device="cuda",
                 rope_base: float = 10000.0, eps: float = 1e-5):
        if min(n_layers, B, Hq, Hkv, D, L_cap) <= 0 or Hq % Hkv != 0:
            raise ValueError("KVCache: sizes must be positive and Hq a multiple of Hkv")
        if D not in (64, 128):
            raise ValueError("KVCache: d_h must be 64 or 128")
        _lib.load()  # fail now, not at the first token, when the CUDA library is missing
        self.n_layers, self.B, self.Hq, self.Hkv, self.D, self.L_cap = n_layers, B, Hq, Hkv, D, L_cap
        self.eps = float(eps)
        self.device = torch.device(device)
        self.k = torch.zeros((n_layers, B, Hkv, L_cap, D), dtype=torch.bfloat16, device=self.device)
        self.v = torch.zeros_like(self.k)
        self.cos, self.sin = make_rope_cache(L_cap, D, rope_base, device=self.device)
        self.length = 0  # tokens held by every layer (the longest sequence's, once lengths differ)
        self.lengths = None  # per-sequence lengths [B] int32 on the device, once set_lengths was called
        self._lens_next = None  # lengths + 1: what the decode kernel reads while the newest token is being attended
        self._lengths_host = None

    def reset(self) -> None:
        """Forgets every token (the buffers keep their bytes; rows >= length are never read)."""
        self.length = 0
        self.lengths = self._lens_next = self._lengths_host = None

    def set_lengths(self, lengths) -> None:
        """Gives every sequence its own length (e.g. after a padded prompt batch went through `append` /
        `attend` / `advance` with the longest prompt's length): rows at and beyond a sequence's length are
        treated as not yet written."""
        host = [int(x) for x in lengths]
        if len(host) != self.B or min(host) < 0 or max(host) > self.L_cap:
            raise ValueError("KVCache.set_lengths: need B lengths in [0, L_cap]")
        self._lengths_host = host
        self.length = max(host)
        self.lengths = torch.tensor(host, dtype=torch.int32, device=self.device)
        self._lens_next = self.lengths + 1

    def _layer(self, fn: str, layer: int) -> None:
        if not 0 <= layer < self.n_layers:
            raise ValueError(f"{fn}: layer {layer} out of range")

    def append(self, layer: int, xq, xk, xv, gamma_q, gamma_k, q_out) -> None:
        """xq [B, n_new, Hq, D], xk / xv [B, n_new, Hkv, D] (the projection outputs, FP32 or BF16, all the
        same type) are the n_new tokens after the `length` cached ones.  Writes q_out [B, Hq, n_new, D] BF16
        (rotated, normalised, times gamma_q) and the tokens' rows of this layer's K (same chain with gamma_k)
        and V (converted to BF16)."""
        fn = "KVCache.append"
        self._layer(fn, layer)
        xd = _x_dtype(fn, xq)
        f32 = torch.float32
        _check_tensors(fn, [(xq, "xq", xq.dtype), (xk, "xk", xq.dtype), (xv, "xv", xq.dtype),
                            (q_out, "q_out", torch.bfloat16), (gamma_q, "gamma_q", f32), (gamma_k, "gamma_k", f32)])
        B, Hq, Hkv, D = self.B, self.Hq, self.Hkv, self.D
        if xq.dim() != 4 or xq.shape[0] != B or xq.shape[2] != Hq or xq.shape[3] != D:
            raise ValueError(f"{fn}: xq must be [B, n_new, Hq, D]")
        n_new = int(xq.shape[1])
        if n_new <= 0:
            raise ValueError(f"{fn}: no tokens")
        if tuple(xk.shape) != (B, n_new, Hkv, D) or tuple(xv.shape) != (B, n_new, Hkv, D):
            raise ValueError(f"{fn}: xk and xv must be [B, n_new, Hkv, D]")
        if q_out.numel() != xq.numel():
            raise ValueError(f"{fn}: q_out numel mismatch")
        if gamma_q.numel() != D or gamma_k.numel() != D:
            raise ValueError(f"{fn}: gamma_q and gamma_k must have d_h elements")
        if self.length + n_new > self.L_cap:
            raise ValueError(f"{fn}: {self.length} + {n_new} tokens exceed the capacity {self.L_cap}")
        lib = _lib.load()
        if self.lengths is not None:
            if n_new != 1:
                raise ValueError(f"{fn}: one token per sequence once the lengths differ")
            with torch.cuda.device(self.device):
                rc = lib.b200attn_kv_append_at(xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), xd, q_out.data_ptr(),
                                               self.k[layer].data_ptr(), self.v[layer].data_ptr(), gamma_q.data_ptr(),
                                               gamma_k.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                                               self.lengths.data_ptr(), B, 1, self.L_cap, Hq, Hkv, D,
                                               ctypes.c_float(self.eps), _stream_ptr())
            _lib.check(rc, fn)
            return
        with torch.cuda.device(self.device):
            rc = lib.b200attn_kv_append(xq.data_ptr(), xk.data_ptr(), xv.data_ptr(), xd, q_out.data_ptr(),
                                        self.k[layer].data_ptr(), self.v[layer].data_ptr(), gamma_q.data_ptr(),
                                        gamma_k.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(), B, n_new,
                                        self.length, self.L_cap, Hq, Hkv, D, ctypes.c_float(self.eps), _stream_ptr())
        _lib.check(rc, fn)

    def attend(self, layer: int, q, ctx, lse, n_new: int = 1, softmax_scale=None) -> None:
        """Attention of the n_new appended tokens over the length + n_new cached ones.  q, ctx: [B, Hq, n_new, D]
        BF16; lse: [B, Hq, n_new] FP32 (may be None for n_new == 1).  n_new == 1 is the split-KV decode kernel;
        n_new > 1 is the causal forward of the new tokens over the cache: a whole prompt into an empty cache, or a
        further chunk of it behind the tokens already cached (chunked prefill; lock-step sequences only)."""
        fn = "KVCache.attend"
        self._layer(fn, layer)
        bf = torch.bfloat16
        items = [(q, "q", bf), (ctx, "ctx", bf)]
        if lse is not None:
            items.append((lse, "lse", torch.float32))
        _check_tensors(fn, items)
        B, Hq, Hkv, D = self.B, self.Hq, self.Hkv, self.D
        if n_new <= 0 or self.length + n_new > self.L_cap:
            raise ValueError(f"{fn}: n_new out of range")
        if q.numel() != B * Hq * n_new * D or ctx.numel() != q.numel():
            raise ValueError(f"{fn}: q and ctx must be [B, Hq, n_new, D]")
        if lse is not None and lse.numel() != B * Hq * n_new:
            raise ValueError(f"{fn}: lse must be [B, Hq, n_new]")
        lib = _lib.load()
        scale = float(softmax_scale or 0.0)
        kc, vc = self.k[layer], self.v[layer]
        with torch.cuda.device(self.device):
            if n_new == 1:
                L = self.length + 1
                nbytes = int(lib.b200attn_decode_workspace_bytes(B, L, Hq, Hkv, D, 0))
                ws = _workspace("decode", nbytes, self.device)
                rc = lib.b200attn_decode_ragged(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(),
                                                lse.data_ptr() if lse is not None else None,
                                                self._lens_next.data_ptr() if self.lengths is not None else None, B, L,
                                                self.L_cap, Hq, Hkv, D, scale, 0, ws.data_ptr(), ws.numel(),
                                                _stream_ptr())
            else:
                if self.lengths is not None:
                    raise ValueError(f"{fn}: several tokens at once only while the sequences advance in lock step")
                if lse is None:
                    raise ValueError(f"{fn}: lse is required for n_new > 1")
                rc = lib.b200attn_fwd_kvcache_at(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ctx.data_ptr(),
                                                 lse.data_ptr(), B, n_new, self.length, self.L_cap, Hq, Hkv, D,
                                                 _lib.LAYOUTS["BHTD"], scale, _stream_ptr())
        _lib.check(rc, fn)

    def advance(self, n_new: int = 1) -> None:
        """Call once per step, after every layer has appended and attended."""
        if n_new <= 0 or self.length + n_new > self.L_cap:
            raise ValueError("KVCache.advance: n_new out of range")
        self.length += n_new
        if self.lengths is not None:
            self._lengths_host = [x + n_new for x in self._lengths_host]
            self.lengths += n_new
            self._lens_next += n_new
