"""KV-cache append, prefill over the cache and cached decode through the C ABI against the oracle."""
import numpy as np
import pytest
import torch

import modern_llm_v1_b200 as m
from oracle import attn_oracle as ao

from gpu_util import TOL_LSE, assert_close, np32

pytestmark = pytest.mark.gpu


def _inputs(B, T, Hq, Hkv, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    xq = torch.randn((B, T, Hq, D), generator=g).to(dtype).cuda()
    xk = torch.randn((B, T, Hkv, D), generator=g).to(dtype).cuda()
    xv = torch.randn((B, T, Hkv, D), generator=g).to(dtype).cuda()
    gq = (1 + 0.3 * torch.randn(D, generator=g)).cuda()
    gk = (1 + 0.3 * torch.randn(D, generator=g)).cuda()
    return xq, xk, xv, gq, gk


def _append(cache, layer, xq, xk, xv, gq, gk):
    q = torch.full((cache.B, cache.Hq, xq.shape[1], cache.D), float("nan"), dtype=torch.bfloat16, device="cuda")
    cache.append(layer, xq.contiguous(), xk.contiguous(), xv.contiguous(), gq, gk, q)
    return q


@pytest.mark.parametrize("B,T,Hq,Hkv,D,dtype,chunks", [
    (2, 33, 6, 2, 64, torch.float32, (0, 33)),
    (2, 33, 6, 2, 64, torch.bfloat16, (0, 1, 2, 20, 33)),
    (3, 40, 16, 4, 128, torch.float32, (0, 7, 39, 40)),
    (1, 5, 3, 3, 128, torch.bfloat16, (0, 5)),
    (64, 1, 16, 4, 64, torch.float32, (0, 1)),
])
def test_append_matches_oracle(B, T, Hq, Hkv, D, dtype, chunks):
    xq, xk, xv, gq, gk = _inputs(B, T, Hq, Hkv, D, dtype, 100 + T)
    L_cap = T + 5
    cache = m.KVCache(2, B, Hq, Hkv, D, L_cap)
    cache.k.fill_(7.0)
    cache.v.fill_(7.0)
    kc = np.zeros((B, Hkv, L_cap, D), np.float32)
    vc = np.zeros_like(kc)
    for a, b in zip(chunks[:-1], chunks[1:]):
        q = _append(cache, 1, xq[:, a:b], xk[:, a:b], xv[:, a:b], gq, gk)
        cache.advance(b - a)
        wq = ao.kv_append(np32(xq[:, a:b]), np32(xk[:, a:b]), np32(xv[:, a:b]), np32(gq), np32(gk), kc, vc, a)
        assert_close("q", q, wq)
    m.device_status()
    assert cache.length == T
    assert_close("K", cache.k[1, :, :, :T], kc[:, :, :T])
    # v is a conversion to BF16: exact
    assert torch.equal(cache.v[1, :, :, :T].float().cpu(), torch.from_numpy(ao.round_bf16(vc[:, :, :T].copy())))
    # nothing else was written: the other layer, and the rows beyond the length
    assert (cache.k[0] == 7.0).all() and (cache.v[0] == 7.0).all()
    assert (cache.k[1, :, :, T:] == 7.0).all() and (cache.v[1, :, :, T:] == 7.0).all()


@pytest.mark.parametrize("D,dtype", [(64, torch.float32), (64, torch.bfloat16), (128, torch.float32)])
def test_append_gives_the_bits_of_the_training_operator(D, dtype):
    B, T, Hq, Hkv = 2, 50, 8, 2
    xq, xk, xv, gq, gk = _inputs(B, T, Hq, Hkv, D, dtype, 7)
    cos, sin = m.make_rope_cache(T, D)
    yq = torch.empty((B, Hq, T, D), dtype=torch.bfloat16, device="cuda")
    yk = torch.empty((B, Hkv, T, D), dtype=torch.bfloat16, device="cuda")
    rq = torch.empty((B, Hq, T), device="cuda")
    rk = torch.empty((B, Hkv, T), device="cuda")
    m.rope_qknorm_forward_qk(xq, xk, cos, sin, gq, gk, 1e-5, yq, yk, rq, rk, B, T, Hq, Hkv, D)
    cache = m.KVCache(1, B, Hq, Hkv, D, T)
    qs = []
    for a, b in ((0, 31), (31, 32), (32, 50)):
        qs.append(_append(cache, 0, xq[:, a:b], xk[:, a:b], xv[:, a:b], gq, gk))
        cache.advance(b - a)
    assert torch.equal(torch.cat(qs, dim=2), yq)
    assert torch.equal(cache.k[0], yk)


@pytest.mark.parametrize("B,T,Hq,Hkv,D,L_cap", [(2, 300, 6, 2, 64, 300), (2, 300, 6, 2, 64, 1000), (1, 200, 8, 2, 128, 257)])
def test_prefill_over_the_cache_equals_the_forward_on_dense_tensors(B, T, Hq, Hkv, D, L_cap):
    xq, xk, xv, gq, gk = _inputs(B, T, Hq, Hkv, D, torch.float32, 9)
    cache = m.KVCache(1, B, Hq, Hkv, D, L_cap)
    cache.k.fill_(float("nan"))  # rows beyond T must never reach a result
    cache.v.fill_(float("nan"))
    q = _append(cache, 0, xq, xk, xv, gq, gk)
    ctx = torch.full_like(q, float("nan"))
    lse = torch.full((B, Hq, T), float("nan"), device="cuda")
    cache.attend(0, q, ctx, lse, n_new=T)
    cache.advance(T)
    m.device_status()
    k, v = cache.k[0, :, :, :T].contiguous(), cache.v[0, :, :, :T].contiguous()
    ctx2, lse2 = torch.empty_like(ctx), torch.empty_like(lse)
    m.flash_attn_forward_gqa(q, k, v, ctx2, lse2, B, T, Hq, Hkv, D)
    m.device_status()
    assert torch.equal(ctx, ctx2) and torch.equal(lse, lse2)
    wo, wl = ao.attn_fwd_c(np32(q), np32(k), np32(v))
    assert_close("O", ctx, wo)
    assert_close("LSE", lse, wl, max_abs=TOL_LSE, rel_l2=1.0)


@pytest.mark.parametrize("B,Hq,Hkv,D,chunks,L_cap", [
    (2, 6, 2, 64, (200, 1, 130, 57, 300), 700),     # prompt in chunks of uneven size, one of a single token
    (1, 8, 2, 128, (129, 128, 64), 400),
    (3, 4, 4, 64, (64, 64, 64, 64), 256),           # chunk boundaries on the 64-key tile boundaries
])
def test_chunked_prefill_equals_the_rows_of_the_whole_forward(B, Hq, Hkv, D, chunks, L_cap):
    # several new tokens against a non-empty cache: every chunk's rows must be the rows of one causal forward over
    # the whole prompt (oracle on the cached, BF16-rounded q, k, v)
    T = sum(chunks)
    xq, xk, xv, gq, gk = _inputs(B, T, Hq, Hkv, D, torch.float32, 21)
    cache = m.KVCache(1, B, Hq, Hkv, D, L_cap)
    cache.k.fill_(float("nan"))  # rows that are not cached yet must never reach a result
    cache.v.fill_(float("nan"))
    qs, ctxs, lses = [], [], []
    pos = 0
    for n in chunks:
        sl = slice(pos, pos + n)
        q = _append(cache, 0, xq[:, sl], xk[:, sl], xv[:, sl], gq, gk)
        ctx = torch.full_like(q, float("nan"))
        lse = torch.full((B, Hq, n), float("nan"), device="cuda")
        cache.attend(0, q, ctx, lse, n_new=n)
        cache.advance(n)
        qs.append(q), ctxs.append(ctx), lses.append(lse)
        pos += n
    m.device_status()
    q, ctx, lse = torch.cat(qs, 2), torch.cat(ctxs, 2), torch.cat(lses, 2)
    k, v = cache.k[0, :, :, :T].contiguous(), cache.v[0, :, :, :T].contiguous()
    wo, wl = ao.attn_fwd_c(np32(q), np32(k), np32(v))
    assert_close("O", ctx, wo)
    assert_close("LSE", lse, wl, max_abs=TOL_LSE, rel_l2=1.0)
    # and close to the one-shot forward of this library (the tiles fall differently, so not bit for bit)
    ctx2, lse2 = torch.empty_like(ctx), torch.empty_like(lse)
    m.flash_attn_forward_gqa(q.contiguous(), k, v, ctx2, lse2, B, T, Hq, Hkv, D)
    m.device_status()
    assert_close("O vs one-shot", ctx, np32(ctx2), max_abs=1e-2, rel_l2=3e-3)


def test_generation_loop_matches_the_full_forward_per_token():
    """Prompt of 70 tokens, then 30 single-token steps: every step's output equals the last row of a full
    causal forward over the tokens so far (what the reference's sampler computes each step), inside the bar."""
    B, Hq, Hkv, D, T0, steps, L_cap = 2, 6, 2, 64, 70, 30, 128
    T = T0 + steps
    xq, xk, xv, gq, gk = _inputs(B, T, Hq, Hkv, D, torch.float32, 21)
    cache = m.KVCache(1, B, Hq, Hkv, D, L_cap)
    q = _append(cache, 0, xq[:, :T0], xk[:, :T0], xv[:, :T0], gq, gk)
    ctx = torch.empty_like(q)
    lse = torch.empty((B, Hq, T0), device="cuda")
    cache.attend(0, q, ctx, lse, n_new=T0)
    cache.advance(T0)
    outs, lses = [], []
    for t in range(T0, T):
        q1 = _append(cache, 0, xq[:, t:t + 1], xk[:, t:t + 1], xv[:, t:t + 1], gq, gk)
        o1 = torch.full_like(q1, float("nan"))
        l1 = torch.full((B, Hq, 1), float("nan"), device="cuda")
        cache.attend(0, q1, o1, l1)
        cache.advance()
        outs.append(o1)
        lses.append(l1)
    m.device_status()
    assert cache.length == T
    # oracle: the whole sequence at once
    kc = np.zeros((B, Hkv, T, D), np.float32)
    vc = np.zeros_like(kc)
    wq = ao.kv_append(np32(xq), np32(xk), np32(xv), np32(gq), np32(gk), kc, vc, 0)
    wo, wl = ao.attn_fwd_c(ao.round_bf16(wq), ao.round_bf16(kc), ao.round_bf16(vc))
    assert_close("O", torch.cat(outs, dim=2), wo[:, :, T0:])
    assert_close("LSE", torch.cat(lses, dim=2), wl[:, :, T0:], max_abs=2 * TOL_LSE, rel_l2=1.0)


def test_cached_decode_ignores_rows_beyond_the_length():
    B, Hq, Hkv, D, L, L_cap = 2, 16, 4, 64, 777, 2048
    g = torch.Generator().manual_seed(5)
    kc = torch.randn((B, Hkv, L_cap, D), generator=g).bfloat16().cuda()
    vc = torch.randn((B, Hkv, L_cap, D), generator=g).bfloat16().cuda()
    q = torch.randn((B, Hq, D), generator=g).bfloat16().cuda()
    kc[:, :, L:] = float("nan")
    vc[:, :, L:] = float("nan")
    cache = m.KVCache(1, B, Hq, Hkv, D, L_cap)
    cache.k[0].copy_(kc)
    cache.v[0].copy_(vc)
    cache.length = L - 1  # the newest token's row is already in place
    o = torch.full((B, Hq, 1, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    lse = torch.full((B, Hq, 1), float("nan"), device="cuda")
    cache.attend(0, q.view(B, Hq, 1, D), o, lse)
    m.device_status()
    o2, lse2 = torch.empty_like(q), torch.empty((B, Hq), device="cuda")
    m.flash_attn_decode(q, kc[:, :, :L].contiguous(), vc[:, :, :L].contiguous(), o2, lse2, B, L, Hq, Hkv, D)
    m.device_status()
    assert torch.equal(o.view(B, Hq, D), o2) and torch.equal(lse.view(B, Hq), lse2)
    wo, wl = ao.decode_c(np32(q), np32(kc[:, :, :L]), np32(vc[:, :, :L]))
    assert_close("O", o2, wo)


def test_capacity_and_argument_errors():
    cache = m.KVCache(1, 1, 2, 1, 64, 4)
    xq = torch.zeros((1, 3, 2, 64), device="cuda")
    xk = torch.zeros((1, 3, 1, 64), device="cuda")
    g = torch.ones(64, device="cuda")
    q = torch.zeros((1, 2, 3, 64), dtype=torch.bfloat16, device="cuda")
    cache.append(0, xq, xk, xk, g, g, q)
    cache.advance(3)
    with pytest.raises(ValueError, match="exceed the capacity"):
        cache.append(0, xq, xk, xk, g, g, q)
    with pytest.raises(ValueError, match="n_new out of range"):
        cache.length = 2
        cache.attend(0, q, q, torch.zeros((1, 2, 3), device="cuda"), n_new=3)  # 2 + 3 tokens > capacity 4
    cache.length = 3
    lib = m._lib.load()
    rc = lib.b200attn_kv_append(xq.data_ptr(), xk.data_ptr(), xk.data_ptr(), 0, q.data_ptr(), cache.k.data_ptr(),
                                cache.v.data_ptr(), g.data_ptr(), g.data_ptr(), cache.cos.data_ptr(),
                                cache.sin.data_ptr(), 1, 3, 2, 4, 2, 1, 64, 1e-5, None)
    assert rc == 1  # B200ATTN_ERR_INVALID_ARG: pos0 + n_new > L_cap
    rc = lib.b200attn_decode_cached(q.data_ptr(), cache.k.data_ptr(), cache.v.data_ptr(), q.data_ptr(), None, 1, 5, 4, 2,
                                    1, 64, 0.0, 0, cache.k.data_ptr(), 1 << 20, None)
    assert rc == 1  # L > L_cap
    m.device_status()


@pytest.mark.parametrize("B,Hq,Hkv,D,lens", [
    (5, 6, 2, 64, (1, 128, 129, 777, 300)),
    (4, 16, 4, 128, (513, 2, 64, 1000)),
    (3, 8, 8, 64, (255, 256, 257)),
])
def test_sequences_of_different_lengths_match_the_oracle_one_by_one(B, Hq, Hkv, D, lens):
    """Per-sequence lengths: the new token of sequence b is rotated at position lens[b] - 1, lands in row
    lens[b] - 1 of its cache and attends to lens[b] rows; every sequence is checked against the oracle alone."""
    L_cap = 1024
    g = torch.Generator().manual_seed(31)
    kc = torch.randn((B, Hkv, L_cap, D), generator=g).bfloat16().cuda()
    vc = torch.randn((B, Hkv, L_cap, D), generator=g).bfloat16().cuda()
    xq, xk, xv, gq, gk = _inputs(B, 1, Hq, Hkv, D, torch.float32, 32)
    cache = m.KVCache(1, B, Hq, Hkv, D, L_cap)
    cache.k[0].copy_(kc)
    cache.v[0].copy_(vc)
    cache.set_lengths([n - 1 for n in lens])  # the tokens before the new one
    q = _append(cache, 0, xq, xk, xv, gq, gk)
    o = torch.full_like(q, float("nan"))
    lse = torch.full((B, Hq, 1), float("nan"), device="cuda")
    cache.attend(0, q, o, lse)
    cache.advance()
    m.device_status()
    assert cache._lengths_host == list(lens) and cache.lengths.tolist() == list(lens)
    for b, n in enumerate(lens):
        kb, vb = np32(kc[b:b + 1]).copy(), np32(vc[b:b + 1]).copy()
        wq = ao.kv_append(np32(xq[b:b + 1]), np32(xk[b:b + 1]), np32(xv[b:b + 1]), np32(gq), np32(gk), kb, vb, n - 1)
        assert_close(f"q[{b}]", q[b:b + 1], wq)
        assert_close(f"K row[{b}]", cache.k[0, b, :, n - 1], kb[0, :, n - 1])
        # only row n - 1 of the sequence's caches changed
        keep = torch.ones(L_cap, dtype=torch.bool)
        keep[n - 1] = False
        assert torch.equal(cache.k[0, b][:, keep.cuda()], kc[b][:, keep.cuda()])
        assert torch.equal(cache.v[0, b][:, keep.cuda()], vc[b][:, keep.cuda()])
        wo, wl = ao.decode_c(ao.round_bf16(wq[:, :, 0]), ao.round_bf16(kb[:, :, :n]), ao.round_bf16(vb[:, :, :n]))
        assert_close(f"O[{b}]", o[b:b + 1, :, 0], wo)
        assert_close(f"LSE[{b}]", lse[b:b + 1, :, 0], wl, max_abs=2 * TOL_LSE, rel_l2=1.0)


def test_a_position_beyond_the_capacity_is_reported_and_skipped():
    B, Hq, Hkv, D, L_cap = 2, 2, 1, 64, 8
    xq, xk, xv, gq, gk = _inputs(B, 1, Hq, Hkv, D, torch.float32, 33)
    cache = m.KVCache(1, B, Hq, Hkv, D, L_cap)
    cache.set_lengths([3, 7])
    cache.lengths[1] = 8  # the device copy says "full" behind the host's back
    q = _append(cache, 0, xq, xk, xv, gq, gk)
    with pytest.raises(RuntimeError, match="exceeds the cache capacity"):
        m.device_status()
    assert m.device_status() == 0  # reported once, then cleared
    assert cache.k[0, 0, :, 3].abs().sum().item() > 0 and cache.k[0, 1].abs().sum().item() == 0
