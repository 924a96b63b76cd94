"""Shared helpers of the GPU parity tests (imported by test modules; not collected)."""
import numpy as np
import torch

import modern_llm_v1_b200 as m
from oracle import attn_oracle as ao

# Tolerances of the parity bar, versus FP32-math attention on identical BF16-rounded inputs.
TOL_MAX_ABS = 2e-2
TOL_REL_L2 = 1e-2
TOL_LSE = 1e-3


def to_layout(x, layout):
    return x.transpose(1, 2).contiguous() if layout == "BTHD" else x.contiguous()


def from_layout(x, layout):
    return x.transpose(1, 2) if layout == "BTHD" else x


def run_fwd(q, k, v, layout="BHTD", scale=None):
    """q [B,Hq,T,D], k/v [B,Hkv,T,D] BF16 CUDA (logical BHTD).  Returns O (logical BHTD), LSE."""
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    qa, ka, va = (to_layout(x, layout) for x in (q, k, v))
    o = torch.full_like(qa, float("nan"))
    lse = torch.full((B, Hq, T), float("nan"), device=q.device)
    m.flash_attn_forward_gqa(qa, ka, va, o, lse, B, T, Hq, Hkv, D, layout, scale)
    return from_layout(o, layout), lse


def run_fwd_bwd(q, k, v, do, layout="BHTD", scale=None, mode="auto"):
    B, Hq, T, D = q.shape
    Hkv = k.shape[1]
    qa, ka, va, doa = (to_layout(x, layout) for x in (q, k, v, do))
    o = torch.full_like(qa, float("nan"))
    lse = torch.full((B, Hq, T), float("nan"), device=q.device)
    dq = torch.full_like(qa, float("nan"))
    dk = torch.full_like(ka, float("nan"))
    dv = torch.full_like(va, float("nan"))
    m.flash_attn_forward_gqa(qa, ka, va, o, lse, B, T, Hq, Hkv, D, layout, scale)
    m.flash_attn_backward_gqa(qa, ka, va, o, lse, doa, dq, dk, dv, B, T, Hq, Hkv, D, layout, scale, mode)
    m.device_status()
    return tuple(from_layout(x, layout) for x in (o,)) + (lse,) + tuple(from_layout(x, layout) for x in (dq, dk, dv))


def np32(x):
    return x.detach().float().cpu().numpy()


def assert_close(name, got, want, max_abs=TOL_MAX_ABS, rel_l2=TOL_REL_L2):
    got, want = np32(got) if isinstance(got, torch.Tensor) else got, np.asarray(want)
    assert not np.isnan(got).any(), f"{name}: NaN in output (an element was never written)"
    ea, er = ao.max_abs(got, want), ao.rel_l2(got, want)
    assert ea <= max_abs, f"{name}: max-abs {ea:.3e} > {max_abs}"
    assert er <= rel_l2, f"{name}: rel-L2 {er:.3e} > {rel_l2}"


def check_against_oracle(q, k, v, do, layout="BHTD", mode="auto"):
    """Runs the CUDA path through the C ABI and the oracle on the same BF16-rounded inputs."""
    got = run_fwd_bwd(q, k, v, do, layout, mode=mode)
    want = ao.attn_fwd_bwd_c(np32(q), np32(k), np32(v), np32(do))
    assert_close("O", got[0], want[0])
    assert_close("LSE", got[1], want[1], max_abs=TOL_LSE, rel_l2=1.0)
    assert_close("dQ", got[2], want[2])
    assert_close("dK", got[3], want[3])
    assert_close("dV", got[4], want[4])
    return got, want


def randn_bf16(shape, seed, std=1.0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * std).bfloat16().to(device)
