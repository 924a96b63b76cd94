"""The oracle of the fused RoPE + QK-Norm operator against the reference's own host functions
(rope_host then rmsnorm_host, golden vectors in tests/golden/reference_host.npz), its backward against
finite differences of that pinned forward, and the host-side argument checks of the operator mirror."""
import numpy as np
import pytest
import torch

import modern_llm_v1_b200 as m
from oracle import attn_oracle as ao


@pytest.mark.parametrize("tag", ["ropenorm64", "ropenorm128"])
def test_forward_matches_reference_host_chain(golden, tag):
    y, rstd = ao.rope_norm_fwd(golden[tag + "_x"], golden[tag + "_g"])
    assert ao.max_abs(y, golden[tag + "_y"]) < 2e-6
    # rstd is what the reference's kernel stores: 1 / sqrt(mean r^2 + eps); RoPE keeps the norm of x
    x = golden[tag + "_x"].astype(np.float64)
    want = 1.0 / np.sqrt((x * x).mean(-1) + 1e-5)
    assert ao.max_abs(rstd, want.astype(np.float32)) < 1e-5


def test_forward_equals_pinned_rope_then_rmsnorm():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 3, 11, 64)).astype(np.float32)
    g = (1 + 0.3 * rng.standard_normal(64)).astype(np.float32)
    y, _ = ao.rope_norm_fwd(x, g)
    assert ao.max_abs(y, ao.rmsnorm(ao.rope(x)) * g) < 2e-6


@pytest.mark.parametrize("D", [64, 128])
def test_backward_matches_finite_differences(D):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((2, 2, 6, D)).astype(np.float32)
    g = (1 + 0.3 * rng.standard_normal(D)).astype(np.float32)
    dy = rng.standard_normal(x.shape).astype(np.float32)
    _, rstd = ao.rope_norm_fwd(x, g)
    dx, dg = ao.rope_norm_bwd(dy, x, g, rstd)

    def loss(xx, gg):
        yy, _ = ao.rope_norm_fwd(xx, gg)
        return float((yy.astype(np.float64) * dy).sum())

    eps = 1e-2
    for idx in [(0, 0, 0, 0), (1, 1, 5, D - 1), (0, 1, 3, 17), (1, 0, 2, 40)]:
        xp, xm = x.copy(), x.copy()
        xp[idx] += eps
        xm[idx] -= eps
        fd = (loss(xp, g) - loss(xm, g)) / (2 * eps)
        assert abs(fd - dx[idx]) < 5e-3 * max(1.0, abs(fd))  # the reference's finite-difference bar (5e-3)
    for d in (0, 9, D - 1):
        gp, gm = g.copy(), g.copy()
        gp[d] += eps
        gm[d] -= eps
        fd = (loss(x, gp) - loss(x, gm)) / (2 * eps)
        assert abs(fd - dg[d]) < 5e-3 * max(1.0, abs(fd))


def test_backward_accumulates_into_d_gamma():
    # llm/src/model/rmsnorm.h:17: "d_gamma is accumulated into"
    rng = np.random.default_rng(5)
    x = rng.standard_normal((1, 2, 4, 64)).astype(np.float32)
    g = np.ones(64, np.float32)
    dy = rng.standard_normal(x.shape).astype(np.float32)
    _, rstd = ao.rope_norm_fwd(x, g)
    _, dg1 = ao.rope_norm_bwd(dy, x, g, rstd)
    _, dg2 = ao.rope_norm_bwd(2 * dy, x, g, rstd)
    assert ao.max_abs(dg2, 2 * dg1) < 1e-5


def test_operator_argument_checks_come_before_any_cuda_call():
    x = torch.zeros(2, 4, 3, 64, dtype=torch.bfloat16)
    y = torch.zeros_like(x)
    cos = torch.zeros(4, 32)
    rstd = torch.zeros(2, 3, 4)
    g = torch.ones(64)
    with pytest.raises(ValueError, match="must be CUDA"):
        m.rope_qknorm_forward(x, cos, cos, g, 1e-5, y, rstd, 2, 4, 3, 64)
    with pytest.raises(ValueError, match="BF16 or FP32"):
        m.rope_qknorm_forward(x.to(torch.float16), cos, cos, g, 1e-5, y, rstd, 2, 4, 3, 64)
    with pytest.raises(ValueError, match="gamma must be FP32"):
        m.rope_qknorm_forward(x, cos, cos, g.double(), 1e-5, y, rstd, 2, 4, 3, 64)
