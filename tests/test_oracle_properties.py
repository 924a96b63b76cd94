"""Self-consistency of the oracle: C vs numpy, finite differences (the reference's own
backward check, llm/tests/test_attention.cu:125-197), GQA by definition, decode, layouts."""
import numpy as np
import pytest

from oracle import attn_oracle as ao


def _rand(rng, *shape, lo=-1.0, hi=1.0):
    return rng.uniform(lo, hi, size=shape).astype(np.float32)


@pytest.mark.parametrize("B,Hq,Hkv,T,D", [(2, 6, 2, 33, 16), (1, 4, 4, 17, 8), (2, 8, 1, 20, 32), (1, 1, 1, 1, 4)])
def test_c_matches_numpy(B, Hq, Hkv, T, D):
    rng = np.random.default_rng(1)
    q, k, v, do = _rand(rng, B, Hq, T, D), _rand(rng, B, Hkv, T, D), _rand(rng, B, Hkv, T, D), _rand(rng, B, Hq, T, D)
    for a, b in zip(ao.attn_fwd_bwd_c(q, k, v, do), ao.attn_fwd_bwd_np(q, k, v, do)):
        assert ao.max_abs(a, b) < 2e-6


def test_backward_matches_finite_differences():
    # same construction as the reference: loss = sum(ctx * upstream), central differences, eps 1e-3, tol 5e-3
    rng = np.random.default_rng(7)
    B, Hq, Hkv, T, D = 1, 2, 1, 4, 5
    q, k, v = (_rand(rng, B, h, T, D, lo=-0.5, hi=0.5) for h in (Hq, Hkv, Hkv))
    up = _rand(rng, B, Hq, T, D, lo=-0.5, hi=0.5)
    _, _, dq, dk, dv = ao.attn_fwd_bwd_c(q, k, v, up)

    def loss(q_, k_, v_):
        o, _ = ao.attn_fwd_bwd_np(q_, k_, v_)
        return float((o * up).sum())

    eps = 1e-3
    for name, x, g in (("q", q, dq), ("k", k, dk), ("v", v, dv)):
        fd = np.zeros_like(x, dtype=np.float64)
        for idx in np.ndindex(x.shape):
            xp, xm = x.astype(np.float64), x.astype(np.float64)
            xp[idx] += eps
            xm[idx] -= eps
            args_p = {"q": q, "k": k, "v": v, name: xp}
            args_m = {"q": q, "k": k, "v": v, name: xm}
            fd[idx] = (loss(args_p["q"], args_p["k"], args_p["v"]) - loss(args_m["q"], args_m["k"], args_m["v"])) / (2 * eps)
        assert ao.max_abs(g, fd) < 5e-3, name


def test_gqa_equals_mha_on_repeated_kv_with_group_sum():
    # definition: repeat_kv_heads then per-head attention, dK/dV summed back (attention.cu:393-429)
    rng = np.random.default_rng(3)
    B, Hq, Hkv, T, D = 2, 6, 2, 19, 8
    g = Hq // Hkv
    q, k, v, do = _rand(rng, B, Hq, T, D), _rand(rng, B, Hkv, T, D), _rand(rng, B, Hkv, T, D), _rand(rng, B, Hq, T, D)
    o, lse, dq, dk, dv = ao.attn_fwd_bwd_c(q, k, v, do)
    kf, vf = np.repeat(k, g, axis=1), np.repeat(v, g, axis=1)
    o2, lse2, dq2, dk2, dv2 = ao.attn_fwd_bwd_c(q, kf, vf, do)
    assert ao.max_abs(o, o2) < 1e-6 and ao.max_abs(lse, lse2) < 1e-6 and ao.max_abs(dq, dq2) < 1e-6
    assert ao.max_abs(dk, dk2.reshape(B, Hkv, g, T, D).sum(2)) < 2e-6
    assert ao.max_abs(dv, dv2.reshape(B, Hkv, g, T, D).sum(2)) < 2e-6


def test_layouts_agree():
    rng = np.random.default_rng(4)
    B, Hq, Hkv, T, D = 2, 4, 2, 13, 8
    q, k, v, do = _rand(rng, B, Hq, T, D), _rand(rng, B, Hkv, T, D), _rand(rng, B, Hkv, T, D), _rand(rng, B, Hq, T, D)
    a = ao.attn_fwd_bwd_c(q, k, v, do)
    t = lambda x: np.ascontiguousarray(x.transpose(0, 2, 1, 3))
    b = ao.attn_fwd_bwd_c(t(q), t(k), t(v), t(do), layout="BTHD")
    for i in (0, 2, 3, 4):
        assert ao.max_abs(a[i], b[i].transpose(0, 2, 1, 3)) < 1e-7
    assert ao.max_abs(a[1], b[1]) < 1e-7


def test_decode_is_last_row_of_causal_forward():
    rng = np.random.default_rng(5)
    B, Hq, Hkv, L, D = 2, 8, 2, 37, 16
    q, k, v = _rand(rng, B, Hq, L, D), _rand(rng, B, Hkv, L, D), _rand(rng, B, Hkv, L, D)
    o, lse = ao.attn_fwd_c(q, k, v)
    od, ld = ao.decode_c(q[:, :, -1], k, v)
    assert ao.max_abs(od, o[:, :, -1]) < 1e-6 and ao.max_abs(ld, lse[:, :, -1]) < 1e-6


def test_first_row_attends_only_to_itself():
    rng = np.random.default_rng(6)
    q, k, v = _rand(rng, 1, 2, 9, 4), _rand(rng, 1, 2, 9, 4), _rand(rng, 1, 2, 9, 4)
    o, lse = ao.attn_fwd_c(q, k, v)
    assert ao.max_abs(o[:, :, 0], v[:, :, 0]) < 1e-7
    s00 = (q[:, :, 0] * k[:, :, 0]).sum(-1) / np.sqrt(np.float32(4))
    assert ao.max_abs(lse[:, :, 0], s00) < 1e-6


def test_rows_of_softmax_sum_to_one_via_constant_v():
    rng = np.random.default_rng(8)
    q, k = _rand(rng, 1, 3, 21, 8), _rand(rng, 1, 1, 21, 8)
    v = np.ones((1, 1, 21, 8), np.float32)
    o, _ = ao.attn_fwd_c(q, k, v)
    assert ao.max_abs(o, np.ones_like(o)) < 1e-6
