"""The oracle of the KV-cache append against the reference's own host functions (rope_host then
rmsnorm_host at the tokens' true positions, golden vectors in tests/golden/reference_host.npz), its
chunk invariance, and the host-side argument checks of KVCache."""
import numpy as np
import pytest
import torch

import modern_llm_v1_b200 as m
from oracle import attn_oracle as ao


@pytest.mark.parametrize("tag,chunks", [("ropenorm64", (0, 1, 2, 17, 32, 33)), ("ropenorm128", (0, 4, 9))])
def test_append_in_chunks_matches_reference_host_chain(golden, tag, chunks):
    # golden x, y: [n, T, D] with row t rotated at position t by the reference's rope_host
    x, g, y = golden[tag + "_x"], golden[tag + "_g"], golden[tag + "_y"]
    n, T, D = x.shape
    xk = np.ascontiguousarray(x.transpose(1, 0, 2))[None]  # [B=1, T, H=n, D]
    kc = np.zeros((1, n, T + 3, D), np.float32)
    vc = np.zeros_like(kc)
    for a, b in zip(chunks[:-1], chunks[1:]):
        q = ao.kv_append(xk[:, a:b], xk[:, a:b], xk[:, a:b], g, g, kc, vc, a)
        assert ao.max_abs(q[0], y[:, a:b]) < 2e-6  # q rows get the same chain
    assert ao.max_abs(kc[0, :, :T], y) < 2e-6
    assert np.array_equal(vc[0, :, :T], x)  # v is only re-laid
    assert not kc[0, :, T:].any() and not vc[0, :, T:].any()  # rows beyond the appended ones are untouched


def test_append_equals_rope_norm_fwd_rows():
    rng = np.random.default_rng(11)
    B, T, Hq, Hkv, D = 2, 10, 4, 2, 64
    xq = rng.standard_normal((B, T, Hq, D)).astype(np.float32)
    xk = rng.standard_normal((B, T, Hkv, D)).astype(np.float32)
    xv = rng.standard_normal((B, T, Hkv, D)).astype(np.float32)
    gq = (1 + 0.3 * rng.standard_normal(D)).astype(np.float32)
    gk = (1 + 0.3 * rng.standard_normal(D)).astype(np.float32)
    kc = np.zeros((B, Hkv, 16, D), np.float32)
    vc = np.zeros_like(kc)
    qs = [ao.kv_append(xq[:, a:b], xk[:, a:b], xv[:, a:b], gq, gk, kc, vc, a) for a, b in ((0, 7), (7, 8), (8, 10))]
    yq, _ = ao.rope_norm_fwd(np.swapaxes(xq, 1, 2), gq)
    yk, _ = ao.rope_norm_fwd(np.swapaxes(xk, 1, 2), gk)
    assert np.array_equal(np.concatenate(qs, axis=2), yq)
    assert np.array_equal(kc[:, :, :T], yk)
    assert np.array_equal(vc[:, :, :T], np.swapaxes(xv, 1, 2))


def test_decode_over_appended_cache_is_last_row_of_causal_attention():
    rng = np.random.default_rng(12)
    B, T, Hq, Hkv, D = 1, 9, 4, 2, 64
    xq = rng.standard_normal((B, T, Hq, D)).astype(np.float32)
    xk = rng.standard_normal((B, T, Hkv, D)).astype(np.float32)
    xv = rng.standard_normal((B, T, Hkv, D)).astype(np.float32)
    g = np.ones(D, np.float32)
    kc = np.zeros((B, Hkv, T, D), np.float32)
    vc = np.zeros_like(kc)
    q = ao.kv_append(xq, xk, xv, g, g, kc, vc, 0)
    o, lse = ao.attn_fwd_c(q, kc, vc)
    od, ld = ao.decode_c(np.ascontiguousarray(q[:, :, -1]), kc, vc)
    assert ao.max_abs(od, o[:, :, -1]) < 1e-6 and ao.max_abs(ld, lse[:, :, -1]) < 1e-6


def test_kvcache_needs_the_cuda_library_and_checks_sizes():
    with pytest.raises(ValueError, match="multiple of Hkv"):
        m.KVCache(1, 1, 3, 2, 64, 16, device="cpu")
    with pytest.raises(ValueError, match="64 or 128"):
        m.KVCache(1, 1, 2, 2, 32, 16, device="cpu")


def test_kvcache_argument_checks_come_before_any_cuda_call():
    # built without __init__ so that no device buffer is needed on a CPU-only machine
    c = m.KVCache.__new__(m.KVCache)
    c.n_layers, c.B, c.Hq, c.Hkv, c.D, c.L_cap, c.eps, c.length = 2, 2, 4, 2, 64, 8, 1e-5, 0
    c.device = torch.device("cpu")
    c.lengths = c._lens_next = c._lengths_host = None
    xq = torch.zeros(2, 1, 4, 64)
    xk = torch.zeros(2, 1, 2, 64)
    g = torch.ones(64)
    qo = torch.zeros(2, 4, 1, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="layer 2 out of range"):
        c.append(2, xq, xk, xk, g, g, qo)
    with pytest.raises(ValueError, match="BF16 or FP32"):
        c.append(0, xq.half(), xk, xk, g, g, qo)
    with pytest.raises(ValueError, match="xk must be FP32"):
        c.append(0, xq, xk.bfloat16(), xk, g, g, qo)
    with pytest.raises(ValueError, match="q_out must be BF16"):
        c.append(0, xq, xk, xk, g, g, qo.float())
    with pytest.raises(ValueError, match="must be CUDA"):
        c.append(0, xq, xk, xk, g, g, qo)
    with pytest.raises(ValueError, match="must be CUDA"):
        c.attend(0, qo, qo, None)
    with pytest.raises(ValueError, match="n_new out of range"):
        c.advance(9)
    c.advance(8)
    assert c.length == 8
    with pytest.raises(ValueError, match="n_new out of range"):
        c.advance(1)
    c.reset()
    assert c.length == 0
    with pytest.raises(ValueError, match="B lengths"):
        c.set_lengths([1, 2, 3])
    with pytest.raises(ValueError, match="B lengths"):
        c.set_lengths([1, 9])
