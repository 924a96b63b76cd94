"""b200attn_bwd_static: the backward for callers that cannot allocate device memory.

Some callers of this library have no way to get a workspace at the point where they call the
backward: a training step running under a caching allocator that must never see a raw
cudaMalloc (it synchronises the whole device), a serving loop that forbids allocation after
start-up, a host without an allocator of its own.  For them the library keeps the backward's two
per-row vectors in a fixed 4 MiB array of its own device image and allocates nothing.

This test calls that entry point through the C ABI and holds it to the regular entry point
(b200attn_bwd_mode, two-pass, with a caller workspace) and to the CPU oracle on two calls in a row.  The second call is a smaller
problem, so the array still holds the first call's rows beyond what the second one rewrites:
stale contents must not leak into the result.  Both entry points run the same kernels, so the
results have to be bit-identical.  The file is named so that pytest collects it last.
"""
import pytest
import torch

import modern_llm_v1_b200 as m
from modern_llm_v1_b200 import _lib
from oracle import attn_oracle as ao

from gpu_util import assert_close, np32

pytestmark = pytest.mark.gpu


def _inputs(B, T, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, T, D, generator=g).bfloat16().cuda()
    k = torch.randn(B, Hkv, T, D, generator=g).bfloat16().cuda()
    v = torch.randn(B, Hkv, T, D, generator=g).bfloat16().cuda()
    do = (torch.randn(B, Hq, T, D, generator=g) * 0.1).bfloat16().cuda()
    return q, k, v, do


def _both_backwards(lib, B, T, Hq, Hkv, D, seed):
    q, k, v, do = _inputs(B, T, Hq, Hkv, D, seed)
    o, lse = torch.empty_like(q), torch.empty(B, Hq, T, device="cuda")
    m.flash_attn_forward_gqa(q, k, v, o, lse, B, T, Hq, Hkv, D)
    # regular entry point, caller-owned workspace
    want = [torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
    m.flash_attn_backward_gqa(q, k, v, o, lse, do, want[0], want[1], want[2], B, T, Hq, Hkv, D, mode="two_pass")
    # allocation-free entry point, straight through the C ABI
    got = [torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))]
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.b200attn_bwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                 do.data_ptr(), got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), B, T, Hq, Hkv,
                                 D, _lib.LAYOUT_BHTD, 0.0, stream)
    assert rc == _lib.OK, _lib.strerror(rc)
    m.device_status()
    # and not only against the sibling entry point: the oracle on the same inputs, at the bar of every parity test
    ref = ao.attn_fwd_bwd_c(np32(q), np32(k), np32(v), np32(do))
    for name, x, y in zip(("dq", "dk", "dv"), got, ref[2:]):
        assert_close(name, x, y)
    return got, want


def test_static_scratch_backward_matches_workspace_backward_twice_in_a_row(lib):
    # first call: 2*6*384 = 4608 rows of the array; second call: 1*4*(200 -> 256) = 1024 rows; third call: a ragged
    # last tile at D = 64, 1*6*(77 -> 128) = 768 rows
    for B, T, Hq, Hkv, D, seed in ((2, 384, 6, 2, 64, 1), (1, 200, 4, 2, 128, 2), (1, 77, 6, 2, 64, 3)):
        got, want = _both_backwards(lib, B, T, Hq, Hkv, D, seed)
        for name, a, b in zip(("dq", "dk", "dv"), got, want):
            assert torch.isfinite(a.float()).all(), name
            assert torch.equal(a, b), f"{name}: static-scratch backward differs from the workspace backward"


def test_static_scratch_backward_leaves_free_device_memory_unchanged(lib):
    # what the entry point promises: after a first call (which loads the kernels) a call takes no device memory
    B, T, Hq, Hkv, D = 2, 256, 6, 2, 64
    q, k, v, do = _inputs(B, T, Hq, Hkv, D, 4)
    o, lse = torch.empty_like(q), torch.empty(B, Hq, T, device="cuda")
    m.flash_attn_forward_gqa(q, k, v, o, lse, B, T, Hq, Hkv, D)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = lib.b200attn_bwd_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(),
                                     do.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, T, Hq, Hkv, D,
                                     _lib.LAYOUT_BHTD, 0.0, stream)
        assert rc == _lib.OK, _lib.strerror(rc)
        torch.cuda.synchronize()

    call()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    assert m.device_status() == 0


def test_problems_beyond_the_fixed_scratch_are_refused(lib):
    # B * Hq * ceil(T/128)*128 = 8 * 16 * 8192 = 1048576 rows > 524288: refused before anything is launched
    dummy = torch.zeros(64, dtype=torch.bfloat16, device="cuda")
    p = dummy.data_ptr()
    rc = lib.b200attn_bwd_static(p, p, p, p, p, p, p, p, p, 8, 8192, 16, 4, 128, _lib.LAYOUT_BHTD, 0.0, None)
    assert rc == _lib.ERR_TOO_LARGE
    assert "524288" in _lib.strerror(rc)
    with pytest.raises(ValueError):
        _lib.check(rc, "b200attn_bwd_static")
    assert m.device_status() == 0
