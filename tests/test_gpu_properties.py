"""Size-independent properties at the benchmark's full sizes, and memory-safety checks that
stand in for a sanitizer: NaN-poisoned outputs, guard bands, run-twice bit equality."""
import pytest
import torch

import modern_llm_v1_b200 as m
from modern_llm_v1_b200 import inputs

from gpu_util import randn_bf16, run_fwd, run_fwd_bwd

pytestmark = pytest.mark.gpu

FULL = ["c2_50m_train", "c3_300m_class"]


def _cfg_inputs(name, seed=20260002):
    cfg = inputs.CONFIGS[name]
    q, k, v, do, _, _ = inputs.make_train_inputs(cfg, seed)
    return cfg, q.cuda(), k.cuda(), v.cuda(), do.cuda()


@pytest.mark.parametrize("name", FULL)
def test_two_runs_are_bit_identical(name):
    # the design has no atomics; a difference between runs means a missing barrier
    _, q, k, v, do = _cfg_inputs(name)
    a = run_fwd_bwd(q, k, v, do)
    b = run_fwd_bwd(q, k, v, do)
    for x, y in zip(a, b):
        assert torch.equal(x, y)


@pytest.mark.parametrize("name", FULL)
def test_softmax_rows_sum_to_one(name):
    # V = 1 everywhere -> O = 1 exactly up to BF16 rounding of P and of O
    _, q, k, v, _ = _cfg_inputs(name)
    o, lse = run_fwd(q, k, torch.ones_like(v))
    assert (o.float() - 1.0).abs().max().item() <= 1.0 / 64
    assert torch.isfinite(lse).all()


@pytest.mark.parametrize("name", FULL)
def test_backward_is_linear_in_dout(name):
    # scaling dO by a power of two scales every product exactly: gradients double bit for bit
    _, q, k, v, do = _cfg_inputs(name)
    a = run_fwd_bwd(q, k, v, do)
    b = run_fwd_bwd(q, k, v, (do.float() * 2).bfloat16())
    for x, y in zip(a[2:], b[2:]):
        assert torch.equal((x.float() * 2).bfloat16(), y)
    # and dO = 0 gives exactly zero gradients
    c = run_fwd_bwd(q, k, v, torch.zeros_like(do))
    for x in c[2:]:
        assert (x.float() == 0).all()


def test_value_gradient_of_first_key_collects_every_row():
    # dV[j] = sum_i P[i,j] dO[i]; with dO = 1: sum_j dV[j, d] = T per head-dim column (rows of P sum to 1),
    # summed over the group's query heads
    cfg, q, k, v, do = _cfg_inputs("c2_50m_train")
    out = run_fwd_bwd(q, k, v, torch.ones_like(do))
    tot = out[4].float().sum(dim=2)  # [B, Hkv, D]
    want = float(cfg.T * cfg.group)
    assert ((tot - want).abs() / want).max().item() < 5e-3


def test_causality_future_tokens_do_not_matter():
    q, k, v = randn_bf16((2, 4, 300, 64), 1), randn_bf16((2, 2, 300, 64), 2), randn_bf16((2, 2, 300, 64), 3)
    o1, l1 = run_fwd(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 200:] = 7.0
    v2[:, :, 200:] = -3.0
    o2, l2 = run_fwd(q, k2, v2)
    assert torch.equal(o1[:, :, :200], o2[:, :, :200]) and torch.equal(l1[:, :, :200], l2[:, :, :200])


@pytest.mark.parametrize("T,D", [(77, 64), (200, 128), (512, 64)])
def test_guard_bands_stay_untouched(T, D):
    # outputs live inside larger poisoned buffers; nothing outside them may change
    B, Hq, Hkv, pad = 2, 4, 2, 4096
    q, k, v, do = (randn_bf16((B, h, T, D), s) for s, h in ((1, Hq), (2, Hkv), (3, Hkv), (4, Hq)))

    def guarded(n, dtype):
        buf = torch.full((n + 2 * pad,), 12345.0 if dtype == torch.float32 else 123.0, dtype=dtype, device="cuda")
        return buf, buf[pad:pad + n]

    nq, nkv = B * Hq * T * D, B * Hkv * T * D
    bo, o = guarded(nq, torch.bfloat16)
    bl, L = guarded(B * Hq * T, torch.float32)
    bdq, dq = guarded(nq, torch.bfloat16)
    bdk, dk = guarded(nkv, torch.bfloat16)
    bdv, dv = guarded(nkv, torch.bfloat16)
    m.flash_attn_forward_gqa(q, k, v, o, L, B, T, Hq, Hkv, D)
    m.flash_attn_backward_gqa(q, k, v, o, L, do, dq, dk, dv, B, T, Hq, Hkv, D)
    m.device_status()
    for buf, n in ((bo, nq), (bl, B * Hq * T), (bdq, nq), (bdk, nkv), (bdv, nkv)):
        fill = buf[0].item()
        assert (buf[:pad] == fill).all() and (buf[pad + n:] == fill).all()
        assert torch.isfinite(buf[pad:pad + n].float()).all()


def test_shape_errors_raise_value_error_on_gpu_tensors():
    q = randn_bf16((2, 128, 64), 0)
    L = torch.empty(2, 128, device="cuda")
    with pytest.raises(ValueError, match="shape mismatch"):
        m.flash_attn_forward(q, q, q[:1], q.clone(), L, 2, 128, 64)
    with pytest.raises(ValueError, match=r"L must be \[B, T\]"):
        m.flash_attn_forward(q, q, q, q.clone(), L[:1], 2, 128, 64)
    q32 = randn_bf16((1, 128, 32), 0)
    with pytest.raises(ValueError, match="unsupported head dimension"):
        m.flash_attn_forward(q32, q32, q32, q32.clone(), torch.empty(1, 128, device="cuda"), 1, 128, 32)
    assert m.device_status() == 0
