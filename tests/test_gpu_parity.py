"""Parity of the CUDA path (called through the C ABI) with the CPU oracle: bit-identical
BF16-rounded inputs, FP32/FP64 reference math.  Bar: O, dQ, dK, dV max-abs <= 2e-2 and
rel-L2 <= 1e-2; logsumexp max-abs <= 1e-3."""
import numpy as np
import pytest
import torch

import modern_llm_v1_b200 as m
from modern_llm_v1_b200 import inputs
from oracle import attn_oracle as ao

from gpu_util import (TOL_LSE, assert_close, check_against_oracle, np32, randn_bf16, run_fwd, run_fwd_bwd)

pytestmark = pytest.mark.gpu


def _case(B, T, Hq, Hkv, D, seed=0, dout_std=0.1):
    # dO ~ N(0, 1e-2) as in the benchmark configurations: the absolute bar (2e-2) presumes gradients
    # of that magnitude (BF16 output rounding alone is 1.6e-2 once |x| >= 4)
    return (randn_bf16((B, Hq, T, D), seed), randn_bf16((B, Hkv, T, D), seed + 1), randn_bf16((B, Hkv, T, D), seed + 2),
            randn_bf16((B, Hq, T, D), seed + 3, dout_std))


def test_config1_cpu_plumbing_shape():
    # B=2, T=128, Hq=6, Hkv=2, D=64; q,k,v,dO ~ N(0,1), scale 1/sqrt(64)
    cfg = inputs.CONFIGS["c1_cpu_plumbing"]
    q, k, v, do, _, _ = inputs.make_train_inputs(cfg, 20260001)
    check_against_oracle(q.cuda(), k.cuda(), v.cuda(), do.cuda())


@pytest.mark.parametrize("T", [1, 2, 63, 77, 127, 128, 129, 200, 257, 384])
def test_ragged_lengths(T):
    check_against_oracle(*_case(2, T, 4, 2, 64, seed=T))


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (4, 4), (6, 2), (8, 1), (16, 4)])
def test_gqa_groupings(Hq, Hkv):
    check_against_oracle(*_case(2, 160, Hq, Hkv, 64, seed=Hq * 10 + Hkv))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("layout", ["BHTD", "BTHD"])
def test_layouts_and_head_dims(D, layout):
    check_against_oracle(*_case(2, 300, 4, 2, D, seed=D), layout=layout)


def test_reference_test_shapes_with_d64():
    # the D=64 shape of llm/tests/test_flash_attn.cu:72 ([B'=4, T=128, D=64], B' = batch x heads)
    # through the reference-shaped entry points
    B, T, D = 4, 128, 64
    g = torch.Generator().manual_seed(0)
    q, k, v, do = ((torch.rand(B, T, D, generator=g) * 2 - 1).bfloat16().cuda() for _ in range(4))
    ctx, L = torch.empty_like(q), torch.empty(B, T, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
    m.flash_attn_forward(q, k, v, ctx, L, B, T, D, tile_kv=16)
    m.flash_attn_backward(q, k, v, ctx, L, do, dq, dk, dv, B, T, D, tile=16)
    want = ao.attn_fwd_bwd_c(*(np32(x)[:, None] for x in (q, k, v, do)))
    assert_close("ctx", ctx, want[0][:, 0])
    assert_close("L", L, want[1][:, 0], max_abs=TOL_LSE, rel_l2=1.0)
    assert_close("d_q", dq, want[2][:, 0])
    assert_close("d_k", dk, want[3][:, 0])
    assert_close("d_v", dv, want[4][:, 0])


def test_golden_fixture_of_reference_attn_host(golden):
    # [1,128,64] case produced by the reference's attn_host; inputs rounded to BF16 for the GPU,
    # so the comparison carries that rounding too (still inside the bar)
    q, k, v = (torch.from_numpy(golden[f"attn4_{n}"]).bfloat16().cuda()[:, None] for n in "qkv")
    o, lse = run_fwd(q, k, v)
    assert_close("ctx", o[:, 0], golden["attn4_ctx"])


def test_mha_golden_layout_bthd(golden):
    # reference mha_host reads [B, T, H*d] directly; pad d=6 is unsupported, so check the
    # layout path with the D=64 oracle instead: BTHD result == BHTD result bit for bit
    q, k, v, do = _case(2, 130, 4, 2, 64, seed=5)
    a = run_fwd_bwd(q, k, v, do, "BHTD")
    b = run_fwd_bwd(q, k, v, do, "BTHD")
    for x, y in zip(a, b):
        assert torch.equal(x.contiguous(), y.contiguous())


@pytest.mark.parametrize("name,units", [("c2_50m_train", [0, 31, 63]), ("c3_300m_class", [0, 63])])
def test_benchmark_configs_against_oracle_on_sampled_units(name, units):
    # QK-normed + RoPE'd q,k; v ~ N(0,1); dO ~ N(0,1e-2).  Full problem on the GPU, the oracle on
    # a sample of (batch, KV head) units.
    cfg = inputs.CONFIGS[name]
    q, k, v, do, _, _ = inputs.make_train_inputs(cfg, 20260002)
    got = run_fwd_bwd(q.cuda(), k.cuda(), v.cuda(), do.cuda())
    g = cfg.group
    for u in units:
        b, hk = divmod(u, cfg.Hkv)
        hs = slice(hk * g, hk * g + g)
        want = ao.attn_fwd_bwd_c(np32(q[b:b + 1, hs]), np32(k[b:b + 1, hk:hk + 1]), np32(v[b:b + 1, hk:hk + 1]),
                                 np32(do[b:b + 1, hs]))
        assert_close("O", got[0][b:b + 1, hs], want[0])
        assert_close("LSE", got[1][b:b + 1, hs], want[1], max_abs=TOL_LSE, rel_l2=1.0)
        assert_close("dQ", got[2][b:b + 1, hs], want[2])
        assert_close("dK", got[3][b:b + 1, hk:hk + 1], want[3])
        assert_close("dV", got[4][b:b + 1, hk:hk + 1], want[4])


def test_long_context_config_sampled_rows():
    # B=4, T=8192, Hq=16, Hkv=4, D=128: forward rows of one unit against the oracle's decode
    # form (row t of the causal forward = decode over keys 0..t), plus logsumexp stability
    cfg = inputs.CONFIGS["c4_long_context"]
    q, k, v, do, hq, hkv = inputs.make_train_inputs(cfg, 20260004, 5, 6)  # one unit: [1, 4, T, D]
    o, lse = run_fwd(q.cuda(), k.cuda(), v.cuda())
    assert torch.isfinite(lse).all() and torch.isfinite(o.float()).all()
    for t in (0, 127, 128, 4095, 8191):
        od, ld = ao.decode_c(np32(q[:, :, t]), np32(k[:, :, :t + 1]), np32(v[:, :, :t + 1]))
        assert_close(f"O[{t}]", o[:, :, t], od)
        assert_close(f"LSE[{t}]", lse[:, :, t], ld, max_abs=TOL_LSE, rel_l2=1.0)


def test_long_context_config_backward_on_one_unit():
    # The whole C4 problem (B=4, T=8192, Hq=16, Hkv=4, D=128: 64 key tiles per item, the device-wide item counter at
    # D=128, P recomputed from the logsumexp over 8k keys) forward + backward on the GPU; O, logsumexp, dQ, dK, dV
    # of one (batch, KV head) unit against the oracle.
    cfg = inputs.CONFIGS["c4_long_context"]
    q, k, v, do, _, _ = inputs.make_train_inputs(cfg, 20260004)
    got = run_fwd_bwd(q.cuda(), k.cuda(), v.cuda(), do.cuda())
    g = cfg.group
    b, hk = 2, 1
    hs = slice(hk * g, hk * g + g)
    want = ao.attn_fwd_bwd_c(np32(q[b:b + 1, hs]), np32(k[b:b + 1, hk:hk + 1]), np32(v[b:b + 1, hk:hk + 1]),
                             np32(do[b:b + 1, hs]))
    assert_close("O", got[0][b:b + 1, hs], want[0])
    assert_close("LSE", got[1][b:b + 1, hs], want[1], max_abs=TOL_LSE, rel_l2=1.0)
    assert_close("dQ", got[2][b:b + 1, hs], want[2])
    assert_close("dK", got[3][b:b + 1, hk:hk + 1], want[3])
    assert_close("dV", got[4][b:b + 1, hk:hk + 1], want[4])


def test_head_dim_128_with_several_items_per_cta():
    # B=4, T=2048, Hq=8, Hkv=2, D=128: 512 forward items on 296 persistent CTAs (single Q buffer, two S buffers),
    # 128-key-tile dQ pass, persistent dK/dV pass with one K/V buffer.  Full problem on the GPU, the oracle on two
    # (batch, KV head) units.
    B, T, Hq, Hkv, D = 4, 2048, 8, 2, 128
    q, k, v, do = _case(B, T, Hq, Hkv, D, seed=128)
    got = run_fwd_bwd(q, k, v, do)
    g = Hq // Hkv
    for b, hk in ((0, 1), (3, 0)):
        hs = slice(hk * g, hk * g + g)
        want = ao.attn_fwd_bwd_c(np32(q[b:b + 1, hs]), np32(k[b:b + 1, hk:hk + 1]), np32(v[b:b + 1, hk:hk + 1]),
                                 np32(do[b:b + 1, hs]))
        assert_close("O", got[0][b:b + 1, hs], want[0])
        assert_close("LSE", got[1][b:b + 1, hs], want[1], max_abs=TOL_LSE, rel_l2=1.0)
        assert_close("dQ", got[2][b:b + 1, hs], want[2])
        assert_close("dK", got[3][b:b + 1, hk:hk + 1], want[3])
        assert_close("dV", got[4][b:b + 1, hk:hk + 1], want[4])
