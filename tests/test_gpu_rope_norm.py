"""Fused RoPE + QK-Norm (forward and backward) through the C ABI against the CPU oracle, which is pinned
against the reference's rope_host / rmsnorm_host (tests/test_rope_norm_oracle.py).  Bars: y (BF16) and BF16
d_x: max-abs <= 2e-2 and rel-L2 <= 1e-2 like the attention outputs; FP32 d_x, rstd and d_gamma: rel-L2 <= 1e-4."""
import numpy as np
import pytest
import torch

import modern_llm_v1_b200 as m
from oracle import attn_oracle as ao

from gpu_util import assert_close

pytestmark = pytest.mark.gpu


def _to(x_bhtd, layout):
    return x_bhtd.transpose(1, 2).contiguous() if layout == "BTHD" else x_bhtd.contiguous()


def _from(x, layout):
    return x.transpose(1, 2) if layout == "BTHD" else x


def _case(B, T, H, D, x_dtype, x_layout, y_layout, seed=0):
    g = torch.Generator().manual_seed(20260100 + seed)
    x = torch.randn(B, H, T, D, generator=g).to(x_dtype)        # logical [B, H, T, D]
    dy = (0.5 * torch.randn(B, H, T, D, generator=g)).bfloat16()
    gamma = 1.0 + 0.2 * torch.randn(D, generator=g)
    cos, sin = m.make_rope_cache(T, D, 10000.0)
    xd, dyd, gd = _to(x, x_layout).cuda(), _to(dy, y_layout).cuda(), gamma.cuda()
    y = torch.full((B, H, T, D) if y_layout == "BHTD" else (B, T, H, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    rstd = torch.full((B, H, T), float("nan"), device="cuda")
    m.rope_qknorm_forward(xd, cos, sin, gd, 1e-5, y, rstd, B, T, H, D, x_layout, y_layout)
    dx = torch.full_like(xd, float("nan"))
    dg = torch.zeros(D, device="cuda")
    m.rope_qknorm_backward(dyd, xd, cos, sin, gd, rstd, dx, dg, B, T, H, D, x_layout, y_layout)
    m.device_status()
    # oracle on the values as stored
    xo, dyo = x.float().numpy(), dy.float().numpy()
    yo, rso = ao.rope_norm_fwd(xo, gamma.numpy())
    dxo, dgo = ao.rope_norm_bwd(dyo, xo, gamma.numpy(), rso)
    return (_from(y, y_layout), rstd, _from(dx, x_layout), dg), (yo, rso, dxo, dgo)


@pytest.mark.parametrize("x_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("x_layout,y_layout", [("BTHD", "BHTD"), ("BHTD", "BHTD"), ("BTHD", "BTHD"), ("BHTD", "BTHD")])
@pytest.mark.parametrize("B,T,H,D", [(2, 128, 6, 64), (1, 77, 3, 64), (2, 50, 4, 128), (1, 1, 1, 64)])
def test_matches_oracle(B, T, H, D, x_dtype, x_layout, y_layout):
    got, want = _case(B, T, H, D, x_dtype, x_layout, y_layout)
    assert_close("y", got[0], want[0])
    assert_close("rstd", got[1], want[1], max_abs=1e-4, rel_l2=1e-5)
    if x_dtype == torch.float32:
        assert_close("d_x", got[2], want[2], max_abs=1e-4, rel_l2=1e-4)
    else:
        assert_close("d_x", got[2], want[2])
    assert_close("d_gamma", got[3], want[3], max_abs=1e-2 * max(1.0, float(np.abs(want[3]).max())), rel_l2=1e-4)


def test_full_size_bit_reproducible_and_accumulating():
    # q of the 50M training shape; d_gamma is summed without atomics and accumulated into
    B, T, H, D = 32, 512, 6, 64
    g = torch.Generator().manual_seed(20260101)
    x = torch.randn(B, T, H, D, generator=g).bfloat16().cuda()
    dy = torch.randn(B, H, T, D, generator=g).bfloat16().cuda()
    gamma = (1.0 + 0.2 * torch.randn(D, generator=g)).cuda()
    cos, sin = m.make_rope_cache(T, D)
    outs = []
    for _ in range(2):
        y = torch.empty(B, H, T, D, dtype=torch.bfloat16, device="cuda")
        rstd = torch.empty(B, H, T, device="cuda")
        dx = torch.empty_like(x)
        dg = torch.zeros(D, device="cuda")
        m.rope_qknorm_forward(x, cos, sin, gamma, 1e-5, y, rstd, B, T, H, D)
        m.rope_qknorm_backward(dy, x, cos, sin, gamma, rstd, dx, dg, B, T, H, D)
        outs.append((y, rstd, dx, dg.clone()))
        m.rope_qknorm_backward(dy, x, cos, sin, gamma, rstd, dx, dg, B, T, H, D)
        assert torch.allclose(dg, 2 * outs[-1][3], rtol=1e-6, atol=0)
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    # rows keep their norm: |y / gamma| = sqrt(D) up to BF16 rounding
    n = (outs[0][0].float() / gamma).pow(2).sum(-1).sqrt()
    assert (n - D ** 0.5).abs().max().item() < 0.05


def test_output_feeds_attention_like_the_input_builder():
    # the builder of the benchmark inputs does RoPE -> RMSNorm (gamma 1) -> BF16 in torch on the CPU
    from modern_llm_v1_b200 import inputs

    B, T, H, D = 2, 256, 6, 64
    g = torch.Generator().manual_seed(7)
    x = torch.randn(B, H, T, D, generator=g)
    want = inputs.rmsnorm_(inputs.rope_(x.clone())).bfloat16()
    cos, sin = m.make_rope_cache(T, D)
    y = torch.empty(B, H, T, D, dtype=torch.bfloat16, device="cuda")
    rstd = torch.empty(B, H, T, device="cuda")
    m.rope_qknorm_forward(x.cuda(), cos, sin, torch.ones(D, device="cuda"), 1e-5, y, rstd, B, T, H, D, "BHTD", "BHTD")
    diff = (y.float().cpu() - want.float()).abs()
    assert diff.max().item() <= 2 ** -6  # at most one BF16 step for |y| < 4
    assert (diff > 0).float().mean().item() < 0.01


@pytest.mark.parametrize("x_dtype", [torch.bfloat16, torch.float32])
def test_q_and_k_in_one_launch_equal_two_calls(x_dtype):
    B, T, Hq, Hkv, D = 2, 300, 6, 2, 64
    g = torch.Generator().manual_seed(11)
    xs = [torch.randn(B, T, H, D, generator=g).to(x_dtype).cuda() for H in (Hq, Hkv)]
    dys = [torch.randn(B, H, T, D, generator=g).bfloat16().cuda() for H in (Hq, Hkv)]
    gms = [(1.0 + 0.2 * torch.randn(D, generator=g)).cuda() for _ in range(2)]
    cos, sin = m.make_rope_cache(T, D)
    single, fused = [], []
    for x, dy, gm, H in zip(xs, dys, gms, (Hq, Hkv)):
        y = torch.empty(B, H, T, D, dtype=torch.bfloat16, device="cuda")
        rstd = torch.empty(B, H, T, device="cuda")
        dx, dg = torch.empty_like(x), torch.zeros(D, device="cuda")
        m.rope_qknorm_forward(x, cos, sin, gm, 1e-5, y, rstd, B, T, H, D)
        m.rope_qknorm_backward(dy, x, cos, sin, gm, rstd, dx, dg, B, T, H, D)
        single += [y, rstd, dx, dg]
    ys = [torch.empty(B, H, T, D, dtype=torch.bfloat16, device="cuda") for H in (Hq, Hkv)]
    rs = [torch.empty(B, H, T, device="cuda") for H in (Hq, Hkv)]
    dxs = [torch.empty_like(x) for x in xs]
    dgs = [torch.zeros(D, device="cuda") for _ in range(2)]
    m.rope_qknorm_forward_qk(xs[0], xs[1], cos, sin, gms[0], gms[1], 1e-5, ys[0], ys[1], rs[0], rs[1], B, T, Hq, Hkv, D)
    m.rope_qknorm_backward_qk(dys[0], dys[1], xs[0], xs[1], cos, sin, gms[0], gms[1], rs[0], rs[1], dxs[0], dxs[1],
                              dgs[0], dgs[1], B, T, Hq, Hkv, D)
    m.device_status()
    for i in range(2):
        fused += [ys[i], rs[i], dxs[i], dgs[i]]
    for a, b in zip(single[:3] + single[4:7], fused[:3] + fused[4:7]):
        assert torch.equal(a, b)
    # d_gamma: the partial sums depend on the grid, which differs between the two forms: equal up to rounding
    for a, b in ((single[3], fused[3]), (single[7], fused[7])):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)
