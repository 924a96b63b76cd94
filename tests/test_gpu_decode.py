"""Split-KV decode through the C ABI against the oracle (row L-1 of causal attention)."""
import pytest
import torch

import modern_llm_v1_b200 as m
from modern_llm_v1_b200 import inputs
from oracle import attn_oracle as ao

from gpu_util import TOL_LSE, assert_close, np32, randn_bf16, run_fwd

pytestmark = pytest.mark.gpu


def _decode(q, kc, vc, n_splits=0, want_lse=True):
    B, Hq, D = q.shape
    Hkv, L = kc.shape[1], kc.shape[2]
    o = torch.full_like(q, float("nan"))
    lse = torch.full((B, Hq), float("nan"), device=q.device) if want_lse else None
    m.flash_attn_decode(q, kc, vc, o, lse, B, L, Hq, Hkv, D, n_splits=n_splits)
    m.device_status()
    return o, lse


@pytest.mark.parametrize("B,L,Hq,Hkv,D,splits", [
    (1, 1, 1, 1, 64, 0), (2, 100, 4, 2, 64, 0), (2, 128, 6, 2, 64, 0), (2, 1000, 6, 2, 64, 0),
    (3, 777, 16, 4, 128, 0), (2, 513, 16, 1, 64, 0), (2, 300, 12, 2, 64, 0), (2, 300, 5, 1, 128, 2),
    (2, 2048, 16, 4, 64, 1), (2, 2048, 16, 4, 64, 16), (1, 700, 7, 7, 64, 3), (1, 640, 11, 1, 64, 0),
])
def test_decode_matches_oracle(B, L, Hq, Hkv, D, splits):
    q, kc, vc = randn_bf16((B, Hq, D), 1), randn_bf16((B, Hkv, L, D), 2), randn_bf16((B, Hkv, L, D), 3)
    o, lse = _decode(q, kc, vc, splits)
    wo, wl = ao.decode_c(np32(q), np32(kc), np32(vc))
    assert_close("O", o, wo)
    assert_close("LSE", lse, wl, max_abs=TOL_LSE, rel_l2=1.0)


def test_decode_config5_sampled_units():
    # B=64, cache 4096, Hq=16, Hkv=4, D=64; keys normed + RoPE'd at their true positions
    cfg = inputs.CONFIGS["c5_decode"]
    q, kc, vc, _, _ = inputs.make_decode_inputs(cfg, 20260005)
    o, lse = _decode(q.cuda(), kc.cuda(), vc.cuda())
    for b in (0, 37, 63):
        wo, wl = ao.decode_c(np32(q[b:b + 1]), np32(kc[b:b + 1]), np32(vc[b:b + 1]))
        assert_close("O", o[b:b + 1], wo)
        assert_close("LSE", lse[b:b + 1], wl, max_abs=TOL_LSE, rel_l2=1.0)


def test_decode_equals_last_row_of_the_forward_kernel():
    B, L, Hq, Hkv, D = 2, 900, 8, 2, 64
    q, k, v = randn_bf16((B, Hq, L, D), 4), randn_bf16((B, Hkv, L, D), 5), randn_bf16((B, Hkv, L, D), 6)
    o, lse = run_fwd(q, k, v)
    od, ld = _decode(q[:, :, -1].contiguous(), k, v)
    assert (od.float() - o[:, :, -1].float()).abs().max().item() <= 1e-2
    assert (ld - lse[:, :, -1]).abs().max().item() <= 1e-3


def test_decode_without_lse_and_split_invariance():
    q, kc, vc = randn_bf16((2, 8, 64), 7), randn_bf16((2, 2, 1500, 64), 8), randn_bf16((2, 2, 1500, 64), 9)
    o0, _ = _decode(q, kc, vc, 1, want_lse=False)
    for s in (2, 5, 12):
        o1, _ = _decode(q, kc, vc, s)
        assert (o0.float() - o1.float()).abs().max().item() <= 4e-3


def test_decode_is_bit_repeatable():
    # the producer re-fills a K/V stage the moment the last warp has released it: a stage that was still being read
    # would show as a run that differs from the first
    q, kc, vc = randn_bf16((16, 16, 64), 4), randn_bf16((16, 4, 3000, 64), 5), randn_bf16((16, 4, 3000, 64), 6)
    first = _decode(q, kc, vc)
    for _ in range(100):
        o, lse = _decode(q, kc, vc)
        assert torch.equal(o, first[0]) and torch.equal(lse, first[1])
