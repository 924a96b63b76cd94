"""Host-side mirror of the reference operator interface, input builders and shard
arithmetic — everything that needs no GPU."""
import numpy as np
import pytest
import torch

import modern_llm_v1_b200 as m
from modern_llm_v1_b200 import inputs, sharding
from oracle import attn_oracle as ao


def _t(*shape, dtype=torch.bfloat16):
    return torch.zeros(*shape, dtype=dtype)


def test_forward_rejects_like_the_reference():
    B, T, D = 2, 8, 64
    q, k, v, c, L = _t(B, T, D), _t(B, T, D), _t(B, T, D), _t(B, T, D), _t(B, T, dtype=torch.float32)
    # tensors must be CUDA (llm/src/model/flash_attn.cu:392-397)
    with pytest.raises(ValueError, match="must be CUDA"):
        m.flash_attn_forward(q, k, v, c, L, B, T, D)
    # tile_kv must be > 0 (:398-399)
    with pytest.raises(ValueError, match="tile_kv must be > 0"):
        m.flash_attn_forward(q, k, v, c, L, B, T, D, tile_kv=0)
    # dtype check comes first (:386-391)
    with pytest.raises(ValueError, match="must be BF16"):
        m.flash_attn_forward(q.float(), k, v, c, L, B, T, D)
    with pytest.raises(ValueError, match="L must be FP32"):
        m.flash_attn_forward(q, k, v, c, L.bfloat16(), B, T, D)


def test_backward_rejects_like_the_reference():
    B, T, D = 2, 8, 64
    x = [_t(B, T, D) for _ in range(9)]
    L = _t(B, T, dtype=torch.float32)
    with pytest.raises(ValueError, match="tile must be > 0"):
        m.flash_attn_backward(x[0], x[1], x[2], x[3], L, x[4], x[5], x[6], x[7], B, T, D, tile=-1)
    with pytest.raises(ValueError, match="must be CUDA"):
        m.flash_attn_backward(x[0], x[1], x[2], x[3], L, x[4], x[5], x[6], x[7], B, T, D)


def test_unit_ranges_partition_exactly():
    for n in (0, 1, 7, 16, 64, 256):
        for world in (1, 2, 3, 4, 8):
            got = [sharding.unit_range(n, r, world) for r in range(world)]
            assert got[0][0] == 0 and got[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
            sizes = [hi - lo for lo, hi in got]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.unit_range(4, 4, 4)
    assert sharding.unit_to_batch_head(5, 2) == (2, 1)
    assert list(sharding.query_heads_of_unit(5, 6, 2)) == [3, 4, 5]


def test_every_config_divides_over_1_2_4_8_gpus():
    for cfg in inputs.CONFIGS.values():
        if cfg.name == "c1_cpu_plumbing":
            continue
        for n in (1, 2, 4, 8):
            assert cfg.units % n == 0


def test_flop_and_byte_model():
    c2 = inputs.CONFIGS["c2_50m_train"]
    assert c2.fwd_flops() == pytest.approx(6.442e9, rel=1e-3)
    assert c2.fwd_bwd_flops() == pytest.approx(2.255e10, rel=1e-3)
    assert inputs.CONFIGS["c4_long_context"].fwd_flops() == pytest.approx(1.0995e12, rel=1e-3)
    assert inputs.CONFIGS["c5_decode"].decode_bytes() == 268_697_600


def test_input_builders_follow_reference_rope_and_rmsnorm():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(3, 40, 64, generator=g)
    y = inputs.rope_(x.clone())
    assert ao.max_abs(y.numpy(), ao.rope(x.numpy())) < 2e-6
    y = inputs.rope_(x.clone(), pos0=17)
    assert ao.max_abs(y.numpy(), ao.rope(x.numpy(), pos0=17)) < 2e-5
    z = inputs.rmsnorm_(x.clone())
    assert ao.max_abs(z.numpy(), ao.rmsnorm(x.numpy())) < 2e-6
    # torch's BF16 conversion is the reference's round-to-nearest-even
    assert np.array_equal(x.bfloat16().float().numpy(), ao.round_bf16(x.numpy()))


def test_shard_inputs_do_not_depend_on_the_slice():
    cfg = inputs.AttnConfig("t", 3, 16, 6, 2, 64)
    q, k, v, do, hq, hkv = inputs.make_train_inputs(cfg, 5)
    assert (hq, hkv) == (6, 2) and q.shape == (3, 6, 16, 64) and k.shape == (3, 2, 16, 64)
    # units 1..3 = (b0,h1), (b1,h0): not whole batches -> one KV head per item
    q2, k2, v2, do2, hq2, hkv2 = inputs.make_train_inputs(cfg, 5, 1, 3)
    assert (hq2, hkv2) == (3, 1)
    assert torch.equal(q2[0], q[0, 3:6]) and torch.equal(k2[0, 0], k[0, 1])
    assert torch.equal(q2[1], q[1, 0:3]) and torch.equal(v2[1, 0], v[1, 0]) and torch.equal(do2[1], do[1, 0:3])
    # normed + RoPE'd rows have unit RMS
    qf = q.float()
    assert torch.allclose((qf * qf).mean(-1), torch.ones(3, 6, 16), atol=2e-2)


def test_decode_inputs_match_the_training_construction():
    cfg = inputs.AttnConfig("d", 2, 24, 4, 2, 64, kind="decode")
    q, kc, vc, hq, hkv = inputs.make_decode_inputs(cfg, 9)
    assert q.shape == (2, 4, 64) and kc.shape == (2, 2, 24, 64) and (hq, hkv) == (4, 2)
    q1, kc1, vc1, _, _ = inputs.make_decode_inputs(cfg, 9, 2, 4)
    assert torch.equal(q1[0], q[1]) and torch.equal(kc1[0], kc[1]) and torch.equal(vc1[0], vc[1])
