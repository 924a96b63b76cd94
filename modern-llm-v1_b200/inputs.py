"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (stand-ins for activations of a training run; no dataset is involved).

Construction of q and k follows the reference's attention chain
(llm/src/model/modern_gpt.cu:358-370): RoPE on interleaved pairs
(llm/src/model/rope.cu:25-44, table :112-128) and a per-head RMSNorm with gamma = 1,
eps = 1e-5 (llm/src/model/rmsnorm.cu:24-53).  The reference applies RoPE first and the
norm second; a rotation keeps the row's sum of squares, so with gamma = 1 both orders
give the same values up to FP32 rounding.  Here the order is the reference's.

Everything is generated on the CPU from a torch generator, so every rank and the CPU
baseline see identical bytes for a given seed, then rounded to BF16
(round-to-nearest-even, llm/src/core/dtype.h:34-42; torch's conversion is the same rule).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class AttnConfig:
    name: str
    B: int
    T: int
    Hq: int
    Hkv: int
    D: int
    kind: str = "train"  # "train" (fwd+bwd) or "decode" (T is the cache length)
    qk_norm_rope: bool = True
    dout_std: float = 0.1  # dO ~ N(0, 1e-2): variance 1e-2

    @property
    def group(self) -> int:
        return self.Hq // self.Hkv

    @property
    def units(self) -> int:
        """Independent (batch, KV head) shards."""
        return self.B * self.Hkv

    def fwd_flops(self) -> float:
        return 4.0 * self.B * self.Hq * self.T * self.T * self.D / 2.0

    def fwd_bwd_flops(self) -> float:
        return 3.5 * self.fwd_flops()

    def decode_bytes(self) -> int:
        """K and V cache plus q and o, BF16."""
        return 2 * self.B * self.Hkv * self.T * self.D * 2 + 2 * self.B * self.Hq * self.D * 2


CONFIGS = {
    "c1_cpu_plumbing": AttnConfig("c1_cpu_plumbing", 2, 128, 6, 2, 64, qk_norm_rope=False, dout_std=1.0),
    "c2_50m_train": AttnConfig("c2_50m_train", 32, 512, 6, 2, 64),
    "c3_300m_class": AttnConfig("c3_300m_class", 16, 1024, 16, 4, 64),
    "c4_long_context": AttnConfig("c4_long_context", 4, 8192, 16, 4, 128),
    "c5_decode": AttnConfig("c5_decode", 64, 4096, 16, 4, 64, kind="decode"),
}


def rope_(x: torch.Tensor, base: float = 10000.0, pos0: int = 0) -> torch.Tensor:
    """In-place RoPE on x[..., T, D] (FP32), interleaved pairs (2i, 2i+1), token t at
    position pos0 + t; theta_i = base^(-2i/D) evaluated in float like the reference."""
    T, D = x.shape[-2], x.shape[-1]
    half = D // 2
    i = torch.arange(half, dtype=torch.float32)
    theta = torch.pow(torch.tensor(base, dtype=torch.float32), -(2.0 * i) / float(D))
    ang = (torch.arange(T, dtype=torch.float32) + float(pos0))[:, None] * theta[None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    x0 = x[..., 0::2].clone()
    x1 = x[..., 1::2].clone()
    x[..., 0::2] = x0 * c - x1 * s
    x[..., 1::2] = x0 * s + x1 * c
    return x


def rmsnorm_(x: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """In-place RMSNorm over the last axis with gamma = 1."""
    ms = (x.double() ** 2).mean(dim=-1, keepdim=True).float()
    x.mul_(1.0 / torch.sqrt(ms + eps))
    return x


def _qk(shape, gen, normed: bool, pos0: int = 0) -> torch.Tensor:
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    if normed:
        rope_(x, pos0=pos0)
        rmsnorm_(x)
    return x


def make_train_inputs(cfg: AttnConfig, seed: int, unit_lo: int = 0, unit_hi: int | None = None, bf16: bool = True):
    """q, k, v, dout in [B', H, T, D] layout for the (batch, KV head) units [unit_lo, unit_hi).

    Units are numbered b * Hkv + h_kv.  A slice keeps whole batches when it can and
    otherwise returns a tensor with B' = number of units and Hkv' = 1 (each unit is
    independent, so a shard may always be presented as a batch of single-KV-head items).
    Every unit's values depend only on (seed, unit index), never on the slice.
    Returns (q, k, v, dout, Hq', Hkv').
    """
    unit_hi = cfg.units if unit_hi is None else unit_hi
    n = unit_hi - unit_lo
    g, T, D = cfg.group, cfg.T, cfg.D
    q = torch.empty(n, g, T, D)
    k = torch.empty(n, 1, T, D)
    v = torch.empty(n, 1, T, D)
    do = torch.empty(n, g, T, D)
    for u in range(unit_lo, unit_hi):
        gen = torch.Generator().manual_seed(seed * 1_000_003 + u)
        q[u - unit_lo] = _qk((g, T, D), gen, cfg.qk_norm_rope)
        k[u - unit_lo] = _qk((1, T, D), gen, cfg.qk_norm_rope)
        v[u - unit_lo] = torch.randn((1, T, D), generator=gen)
        do[u - unit_lo] = torch.randn((g, T, D), generator=gen) * cfg.dout_std
    if unit_lo % cfg.Hkv == 0 and n % cfg.Hkv == 0:
        nb = n // cfg.Hkv
        q = q.view(nb, cfg.Hkv * g, T, D)
        do = do.view(nb, cfg.Hkv * g, T, D)
        k = k.view(nb, cfg.Hkv, T, D)
        v = v.view(nb, cfg.Hkv, T, D)
        hq, hkv = cfg.Hq, cfg.Hkv
    else:
        hq, hkv = g, 1
    if bf16:
        q, k, v, do = (t.bfloat16() for t in (q, k, v, do))
    return q.contiguous(), k.contiguous(), v.contiguous(), do.contiguous(), hq, hkv


def make_decode_inputs(cfg: AttnConfig, seed: int, unit_lo: int = 0, unit_hi: int | None = None, bf16: bool = True):
    """q [B', Hq', D], kcache, vcache [B', Hkv', L, D] for units [unit_lo, unit_hi): the cache
    holds normed + RoPE'd keys at positions 0..L-1, q is normed + RoPE'd at position L-1
    (the cache already contains the current token).  Returns (q, kc, vc, Hq', Hkv')."""
    unit_hi = cfg.units if unit_hi is None else unit_hi
    n = unit_hi - unit_lo
    g, L, D = cfg.group, cfg.T, cfg.D
    q = torch.empty(n, g, D)
    kc = torch.empty(n, 1, L, D)
    vc = torch.empty(n, 1, L, D)
    for u in range(unit_lo, unit_hi):
        gen = torch.Generator().manual_seed(seed * 1_000_003 + u)
        q[u - unit_lo] = _qk((g, 1, D), gen, cfg.qk_norm_rope, pos0=L - 1)[:, 0]
        kc[u - unit_lo] = _qk((1, L, D), gen, cfg.qk_norm_rope)
        vc[u - unit_lo] = torch.randn((1, L, D), generator=gen)
    if unit_lo % cfg.Hkv == 0 and n % cfg.Hkv == 0:
        nb = n // cfg.Hkv
        q = q.view(nb, cfg.Hkv * g, D)
        kc = kc.view(nb, cfg.Hkv, L, D)
        vc = vc.view(nb, cfg.Hkv, L, D)
        hq, hkv = cfg.Hq, cfg.Hkv
    else:
        hq, hkv = g, 1
    if bf16:
        q, kc, vc = (t.bfloat16() for t in (q, kc, vc))
    return q.contiguous(), kc.contiguous(), vc.contiguous(), hq, hkv
