"""Host-side mirror of the reference's flash-attention operator interface.

Same names, argument order and error behaviour as
``modernllm::flash_attn_forward`` / ``flash_attn_backward``
(llm/src/model/flash_attn.h:25-28,47-52; validation llm/src/model/flash_attn.cu:386-407,
433-455) with torch CUDA tensors standing in for ``modernllm::Tensor``:

* caller allocates every input and output, outputs are overwritten in full;
* ``B`` in the two reference-shaped functions is batch x heads (the reference
  kernels know nothing of heads); the ``*_gqa`` variants take (B, T, Hq, Hkv, D)
  and a layout and index the shared KV head directly;
* ``tile_kv`` / ``tile`` are accepted for source compatibility, validated like the
  reference (``<= 0`` raises) and otherwise ignored: tile shapes are compile-time
  properties of the sm_100a kernels;
* bad dtype / device / shape raise ValueError (std::invalid_argument in the
  reference), CUDA failures raise RuntimeError (std::runtime_error).

Tensors are BF16 (the reference's BF16 storage, llm/src/core/dtype.h:34-49), the
logsumexp tensor is FP32.  Everything runs on the current CUDA stream of torch.
There is no CPU or PyTorch fallback.
"""
from __future__ import annotations

import torch

from . import _lib

_workspaces: dict[tuple[int, str, int], torch.Tensor] = {}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _workspace(kind: str, nbytes: int, device: torch.device) -> torch.Tensor:
    """Private temporaries of the operator (the reference allocates its D vector per
    call, llm/src/model/flash_attn.cu:463); kept and grown per (device, stream) instead, so
    that calls issued on different torch streams never share scratch memory."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), kind, _stream_ptr())
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _check_tensors(fn: str, items) -> None:
    """items: (tensor, name, dtype).  Like the reference (llm/src/model/flash_attn.cu:386-397):
    every dtype is checked first, then every device."""
    for t, name, dtype in items:
        if not isinstance(t, torch.Tensor):
            raise ValueError(f"{fn}: {name} must be a tensor")
        if t.dtype != dtype:
            want = {torch.bfloat16: "BF16", torch.float32: "FP32"}.get(dtype, str(dtype))
            raise ValueError(f"{fn}: {name} must be {want}")
    for t, name, _ in items:
        if not t.is_cuda:
            raise ValueError(f"{fn}: {name} must be CUDA")
    for t, name, _ in items:
        if not t.is_contiguous():
            raise ValueError(f"{fn}: {name} must be contiguous")


def _dims_ok(B: int, T: int, D: int) -> bool:
    return B > 0 and T > 0 and D > 0


# ----------------------------------------------------------------------------
# GQA-aware entry points (what ModernGPT's attention chain would call)
# ----------------------------------------------------------------------------
def flash_attn_forward_gqa(q, k, v, ctx, L, B, T, Hq, Hkv, D, layout="BHTD", softmax_scale=None):
    """ctx = causal softmax(scale q k^T) v, L = logsumexp rows.  q, ctx: B*Hq*T*D BF16
    elements in `layout`; k, v: B*Hkv*T*D; L: [B, Hq, T] FP32."""
    fn = "flash_attn_forward"
    bf = torch.bfloat16
    _check_tensors(fn, [(q, "q", bf), (k, "k", bf), (v, "v", bf), (ctx, "ctx", bf), (L, "L", torch.float32)])
    if layout not in _lib.LAYOUTS:
        raise ValueError(f"{fn}: layout must be BHTD or BTHD")
    nq, nkv = B * Hq * T * D, B * Hkv * T * D
    if q.numel() != nq or ctx.numel() != nq or k.numel() != nkv or v.numel() != nkv:
        raise ValueError(f"{fn}: shape mismatch (qkv/ctx)")
    if L.numel() != B * Hq * T:
        raise ValueError(f"{fn}: L must be [B, T]")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        rc = lib.b200attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), ctx.data_ptr(), L.data_ptr(), B, T, Hq, Hkv, D,
                              _lib.LAYOUTS[layout], float(softmax_scale or 0.0), _stream_ptr())
    _lib.check(rc, fn)


def flash_attn_backward_gqa(q, k, v, ctx, L, d_ctx, d_q, d_k, d_v, B, T, Hq, Hkv, D, layout="BHTD",
                            softmax_scale=None, mode="auto"):
    """d_q, d_k, d_v (overwritten) for the forward above.  d_k, d_v are Hkv-wide: the
    sum over each group's query heads is done inside the kernel.  mode: "auto", "two_pass" (the
    reference's structure, llm/src/model/flash_attn.cu:475-503, every output bit-reproducible) or
    "one_pass" (D = 64: scores computed once, d_q summed by reduce-adds in no fixed order)."""
    fn = "flash_attn_backward"
    bf = torch.bfloat16
    _check_tensors(fn, [(q, "q", bf), (k, "k", bf), (v, "v", bf), (ctx, "ctx", bf), (L, "L", torch.float32),
                        (d_ctx, "d_ctx", bf), (d_q, "d_q", bf), (d_k, "d_k", bf), (d_v, "d_v", bf)])
    if layout not in _lib.LAYOUTS:
        raise ValueError(f"{fn}: layout must be BHTD or BTHD")
    nq, nkv = B * Hq * T * D, B * Hkv * T * D
    if any(t.numel() != nq for t in (q, ctx, d_ctx, d_q)) or any(t.numel() != nkv for t in (k, v, d_k, d_v)):
        raise ValueError(f"{fn}: shape mismatch")
    if L.numel() != B * Hq * T:
        raise ValueError(f"{fn}: L must be [B, T]")
    if mode not in _lib.BWD_MODES:
        raise ValueError(f"{fn}: mode must be auto, two_pass or one_pass")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        m = _lib.BWD_MODES[mode]
        nbytes = int(lib.b200attn_bwd_workspace_bytes_mode(B, T, Hq, Hkv, D, m))
        ws = _workspace("bwd", nbytes, q.device)
        rc = lib.b200attn_bwd_mode(q.data_ptr(), k.data_ptr(), v.data_ptr(), ctx.data_ptr(), L.data_ptr(),
                                   d_ctx.data_ptr(), d_q.data_ptr(), d_k.data_ptr(), d_v.data_ptr(), B, T, Hq, Hkv, D,
                                   _lib.LAYOUTS[layout], float(softmax_scale or 0.0), m, ws.data_ptr(), ws.numel(),
                                   _stream_ptr())
    _lib.check(rc, fn)


# ----------------------------------------------------------------------------
# Reference-shaped entry points: [B, T, D] with B = batch x heads
# ----------------------------------------------------------------------------
def flash_attn_forward(q, k, v, ctx, L, B, T, D, tile_kv=32):
    """Signature of modernllm::flash_attn_forward (llm/src/model/flash_attn.h:25-28)."""
    if tile_kv <= 0:
        raise ValueError("flash_attn_forward: tile_kv must be > 0")
    if not _dims_ok(B, T, D):
        raise ValueError("flash_attn_forward: shape mismatch (qkv/ctx)")
    flash_attn_forward_gqa(q, k, v, ctx, L, B, T, 1, 1, D, "BHTD")


def flash_attn_backward(q, k, v, ctx, L, d_ctx, d_q, d_k, d_v, B, T, D, tile=16):
    """Signature of modernllm::flash_attn_backward (llm/src/model/flash_attn.h:47-52)."""
    if tile <= 0:
        raise ValueError("flash_attn_backward: tile must be > 0")
    if not _dims_ok(B, T, D):
        raise ValueError("flash_attn_backward: shape mismatch")
    flash_attn_backward_gqa(q, k, v, ctx, L, d_ctx, d_q, d_k, d_v, B, T, 1, 1, D, "BHTD")


# ----------------------------------------------------------------------------
# Decode against a KV cache (the single-token path infer_modern_gpt lacks,
# llm/apps/infer_modern_gpt.cu:253-255)
# ----------------------------------------------------------------------------
def flash_attn_decode(q, kcache, vcache, o, lse, B, L, Hq, Hkv, D, softmax_scale=None, n_splits=0):
    """o[b, h] = softmax(scale q[b, h] . K[b, h/g, :L]) V[b, h/g, :L]; q, o [B, Hq, D] BF16,
    caches [B, Hkv, L, D] BF16, lse [B, Hq] FP32 or None."""
    fn = "flash_attn_decode"
    bf = torch.bfloat16
    items = [(q, "q", bf), (kcache, "kcache", bf), (vcache, "vcache", bf), (o, "o", bf)]
    if lse is not None:
        items.append((lse, "lse", torch.float32))
    _check_tensors(fn, items)
    if lse is not None:
        if lse.numel() != B * Hq:
            raise ValueError(f"{fn}: lse must be [B, Hq]")
    if q.numel() != B * Hq * D or o.numel() != B * Hq * D:
        raise ValueError(f"{fn}: shape mismatch (q/o)")
    if kcache.numel() != B * Hkv * L * D or vcache.numel() != B * Hkv * L * D:
        raise ValueError(f"{fn}: shape mismatch (cache)")
    lib = _lib.load()
    with torch.cuda.device(q.device):
        nbytes = int(lib.b200attn_decode_workspace_bytes(B, L, Hq, Hkv, D, int(n_splits)))
        ws = _workspace("decode", nbytes, q.device)
        rc = lib.b200attn_decode(q.data_ptr(), kcache.data_ptr(), vcache.data_ptr(), o.data_ptr(),
                                 lse.data_ptr() if lse is not None else None, B, L, Hq, Hkv, D,
                                 float(softmax_scale or 0.0), int(n_splits), ws.data_ptr(), ws.numel(), _stream_ptr())
    _lib.check(rc, fn)


def device_status() -> int:
    """Synchronises the current stream and raises RuntimeError if a kernel gave up on a
    bounded wait since the last check; returns 0 otherwise."""
    rc = _lib.load().b200attn_last_device_status(_stream_ptr())
    _lib.check(rc, "device_status")
    return rc
