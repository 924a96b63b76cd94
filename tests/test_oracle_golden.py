"""The CPU oracle against fixtures produced by the reference's own host code
(tests/golden/make_golden.py: attn_host, mha_host, rope_host, rmsnorm_host, BF16 helpers)."""
import numpy as np

from oracle import attn_oracle as ao

ATTN_CASES = 5


def test_forward_matches_reference_attn_host(golden):
    # tolerance of the reference's own forward test (llm/tests/test_attention.cu:121: 1e-4)
    for i in range(ATTN_CASES):
        q, k, v = golden[f"attn{i}_q"], golden[f"attn{i}_k"], golden[f"attn{i}_v"]
        o, _ = ao.attn_fwd_c(q[:, None], k[:, None], v[:, None])  # [B',T,D] -> [B',1,T,D]
        assert ao.max_abs(o[:, 0], golden[f"attn{i}_ctx"]) < 1e-5
        o2, _ = ao.attn_fwd_bwd_np(q[:, None], k[:, None], v[:, None])
        assert ao.max_abs(o2[:, 0], golden[f"attn{i}_ctx"]) < 1e-5


def test_logsumexp_reproduces_reference_probs(golden):
    # probs[i, j] of the reference equals exp(scale * q_i.k_j - L_i) for the oracle's L
    for i in range(ATTN_CASES):
        q, k, v = golden[f"attn{i}_q"], golden[f"attn{i}_k"], golden[f"attn{i}_v"]
        D = q.shape[-1]
        _, lse = ao.attn_fwd_c(q[:, None], k[:, None], v[:, None])
        s = np.einsum("bid,bjd->bij", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(np.float32(D))
        p = np.tril(np.exp(s - lse[:, 0, :, None]))
        assert ao.max_abs(p, golden[f"attn{i}_probs"]) < 1e-5  # llm/tests/test_attention.cu:122


def test_bthd_layout_matches_reference_mha_host(golden):
    B, T, H, d = (int(x) for x in golden["mha_dims"])
    q, k, v = (golden[n].reshape(B, T, H, d) for n in ("mha_q", "mha_k", "mha_v"))
    o, _ = ao.attn_fwd_c(q, k, v, layout="BTHD")
    assert ao.max_abs(o.reshape(B, T, H * d), golden["mha_ctx"]) < 1e-5


def test_rope_matches_reference(golden):
    assert ao.max_abs(ao.rope(golden["rope_x"]), golden["rope_y"]) < 1e-6
    assert ao.max_abs(ao.rope(golden["rope64_x"]), golden["rope64_y"]) < 1e-6


def test_rmsnorm_matches_reference(golden):
    assert ao.max_abs(ao.rmsnorm(golden["rms_x"]), golden["rms_y"]) < 1e-6


def test_bf16_rounding_is_bit_exact(golden):
    bits = ao.to_bf16_bits(golden["bf16_x"])
    assert np.array_equal(bits, golden["bf16_bits"])
    assert np.array_equal(ao.from_bf16_bits(bits), golden["bf16_back"])
    assert np.array_equal(ao.round_bf16(golden["bf16_x"]), golden["bf16_back"])
