"""The one-pass backward (mode "one_pass", D = 64: scores computed once, dq summed by reduce-adds into an FP32
accumulator) against the CPU oracle, through the C ABI, at the same bar as the two-pass backward: dQ, dK, dV
max-abs <= 2e-2 and rel-L2 <= 1e-2.  dk and dv are summed in a fixed order inside one CTA and must be
bit-reproducible; the order of the dq additions is not fixed, so dq is held to FP32-rounding closeness between
runs and between the two modes."""
import pytest
import torch

import modern_llm_v1_b200 as m
from modern_llm_v1_b200 import inputs
from oracle import attn_oracle as ao

from gpu_util import assert_close, check_against_oracle, np32, randn_bf16, run_fwd_bwd

pytestmark = pytest.mark.gpu


def _case(B, T, Hq, Hkv, seed=0):
    return (randn_bf16((B, Hq, T, 64), seed), randn_bf16((B, Hkv, T, 64), seed + 1), randn_bf16((B, Hkv, T, 64), seed + 2),
            randn_bf16((B, Hq, T, 64), seed + 3, 0.1))


@pytest.mark.parametrize("T", [1, 63, 127, 128, 129, 200, 257, 384, 700])
def test_ragged_lengths(T):
    check_against_oracle(*_case(2, T, 4, 2, seed=T), mode="one_pass")


@pytest.mark.parametrize("Hq,Hkv", [(1, 1), (4, 4), (6, 2), (8, 1), (16, 4)])
def test_gqa_groupings(Hq, Hkv):
    check_against_oracle(*_case(2, 160, Hq, Hkv, seed=Hq * 10 + Hkv), mode="one_pass")


def test_projection_layout():
    check_against_oracle(*_case(2, 300, 4, 1, seed=9), layout="BTHD", mode="one_pass")


@pytest.mark.parametrize("name,units", [("c2_50m_train", [0, 31, 63]), ("c3_300m_class", [63])])
def test_benchmark_configs_on_sampled_units(name, units):
    cfg = inputs.CONFIGS[name]
    q, k, v, do, _, _ = inputs.make_train_inputs(cfg, 20260002)
    got = run_fwd_bwd(q.cuda(), k.cuda(), v.cuda(), do.cuda(), mode="one_pass")
    g = cfg.group
    for u in units:
        b, hk = divmod(u, cfg.Hkv)
        hs = slice(hk * g, hk * g + g)
        want = ao.attn_fwd_bwd_c(np32(q[b:b + 1, hs]), np32(k[b:b + 1, hk:hk + 1]), np32(v[b:b + 1, hk:hk + 1]),
                                 np32(do[b:b + 1, hs]))
        assert_close("dQ", got[2][b:b + 1, hs], want[2])
        assert_close("dK", got[3][b:b + 1, hk:hk + 1], want[3])
        assert_close("dV", got[4][b:b + 1, hk:hk + 1], want[4])


def test_two_runs_and_two_modes():
    # several items per CTA (device-wide item counter) and several key tiles per query tile
    q, k, v, do = _case(8, 1024, 8, 2, seed=77)
    a = run_fwd_bwd(q, k, v, do, mode="one_pass")
    b = run_fwd_bwd(q, k, v, do, mode="one_pass")
    two = run_fwd_bwd(q, k, v, do, mode="two_pass")
    # dK, dV: one CTA sums them in a fixed order
    assert torch.equal(a[3], b[3]) and torch.equal(a[4], b[4])
    # dQ: the same contributions added in another order differ by FP32 rounding, i.e. by at most a BF16 ulp or so
    for x, y in ((a[2], b[2]), (a[2], two[2])):
        assert_close("dQ", x, np32(y), max_abs=2e-3, rel_l2=1e-3)
    assert_close("dK", a[3], np32(two[3]), max_abs=2e-3, rel_l2=1e-3)
    assert_close("dV", a[4], np32(two[4]), max_abs=2e-3, rel_l2=1e-3)


def test_zero_upstream_gradient_gives_exact_zeros():
    q, k, v, do = _case(2, 300, 6, 2, seed=5)
    out = run_fwd_bwd(q, k, v, torch.zeros_like(do), mode="one_pass")
    for x in out[2:]:
        assert (x.float() == 0).all()


def test_head_dim_128_is_refused():
    q, k, v = (randn_bf16((1, 2, 128, 128), s) for s in (1, 2, 3))
    o, lse = torch.empty_like(q), torch.empty(1, 2, 128, device="cuda")
    m.flash_attn_forward_gqa(q, k, v, o, lse, 1, 128, 2, 2, 128)
    with pytest.raises(ValueError, match="unsupported"):
        m.flash_attn_backward_gqa(q, k, v, o, lse, q, torch.empty_like(q), torch.empty_like(k), torch.empty_like(v),
                                  1, 128, 2, 2, 128, mode="one_pass")
    with pytest.raises(ValueError, match="mode must be"):
        m.flash_attn_backward_gqa(q, k, v, o, lse, q, torch.empty_like(q), torch.empty_like(k), torch.empty_like(v),
                                  1, 128, 2, 2, 128, mode="three_pass")
    assert m.device_status() == 0
