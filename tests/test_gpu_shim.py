"""The C++ boundary executed: modern-llm-v1_b200/csrc/modernllm_shim.{h,cc} compiled against the reference's own
Tensor (llm/src/core/tensor.h:25-97) into oracle/_ref/libshim_gpu.so and called with reference Tensors, the way
the reference's tests and benchmark call flash_attn_forward / flash_attn_backward
(llm/tests/test_flash_attn.cu:51,99,170,174; llm/tests/bench_flash_attn.cu:73,82,91).  Checked against the CPU
oracle at the parity bar, against the reference's exception behaviour (llm/src/model/flash_attn.cu:386-407), and
for the absence of allocations in steady state.  Skipped where the library was not built (it needs the reference
tree at build time)."""
import ctypes
import os

import pytest
import torch

import modern_llm_v1_b200 as m
from oracle import attn_oracle as ao

from gpu_util import TOL_LSE, assert_close, np32, randn_bf16

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libshim_gpu.so")
OK, INVALID_ARGUMENT, RUNTIME_ERROR = 0, 1, 2


@pytest.fixture(scope="module")
def shim(lib):
    if not os.path.exists(LIB):
        pytest.skip("oracle/_ref/libshim_gpu.so not built")
    L = ctypes.CDLL(LIB)
    vp, i = ctypes.c_void_p, ctypes.c_int
    L.shim_flash_attn_forward.argtypes = [vp] * 5 + [i] * 5 + [vp]
    L.shim_flash_attn_backward.argtypes = [vp] * 9 + [i] * 5 + [vp]
    L.shim_flash_attn_forward_gqa.argtypes = [vp] * 5 + [i] * 6 + [vp]
    L.shim_flash_attn_backward_gqa.argtypes = [vp] * 9 + [i] * 6 + [vp]
    L.shim_flash_attn_decode.argtypes = [vp] * 4 + [i] * 5 + [vp]
    L.shim_last_error.restype = ctypes.c_char_p
    return L


def _p(t):
    return t.data_ptr()


def test_reference_shaped_entry_points_at_the_reference_test_shape(shim):
    # [B' = 4, T = 128, D = 64], uniform(-1, 1) inputs, tile arguments as the reference test passes them
    # (llm/tests/test_flash_attn.cu:69-72)
    B, T, D = 4, 128, 64
    g = torch.Generator().manual_seed(0)
    q, k, v, do = ((torch.rand(B, T, D, generator=g) * 2 - 1).bfloat16().cuda() for _ in range(4))
    ctx, L = torch.full_like(q, float("nan")), torch.full((B, T), float("nan"), device="cuda")
    dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
    assert shim.shim_flash_attn_forward(_p(q), _p(k), _p(v), _p(ctx), _p(L), B, T, D, 16, 0, None) == OK
    assert shim.shim_flash_attn_backward(_p(q), _p(k), _p(v), _p(ctx), _p(L), _p(do), _p(dq), _p(dk), _p(dv), B, T, D, 16, 0,
                                         None) == OK
    m.device_status()
    want = ao.attn_fwd_bwd_c(*(np32(x)[:, None] for x in (q, k, v, do)))
    assert_close("ctx", ctx, want[0][:, 0])
    assert_close("L", L, want[1][:, 0], max_abs=TOL_LSE, rel_l2=1.0)
    assert_close("d_q", dq, want[2][:, 0])
    assert_close("d_k", dk, want[3][:, 0])
    assert_close("d_v", dv, want[4][:, 0])


@pytest.mark.parametrize("layout", [0, 1])
def test_gqa_overloads(shim, layout):
    B, T, Hq, Hkv, D = 2, 300, 6, 2, 64
    q, k, v = randn_bf16((B, Hq, T, D), 1), randn_bf16((B, Hkv, T, D), 2), randn_bf16((B, Hkv, T, D), 3)
    do = randn_bf16((B, Hq, T, D), 4, 0.1)
    lay = (lambda x: x.transpose(1, 2).contiguous()) if layout == 1 else (lambda x: x.contiguous())
    unlay = (lambda x: x.transpose(1, 2)) if layout == 1 else (lambda x: x)
    qa, ka, va, doa = lay(q), lay(k), lay(v), lay(do)
    ctx, L = torch.full_like(qa, float("nan")), torch.full((B, Hq, T), float("nan"), device="cuda")
    dq, dk, dv = torch.full_like(qa, float("nan")), torch.full_like(ka, float("nan")), torch.full_like(va, float("nan"))
    side = torch.cuda.Stream()  # a stream of the caller's: the shim must launch there, with a kept workspace
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        st = side.cuda_stream
        assert shim.shim_flash_attn_forward_gqa(_p(qa), _p(ka), _p(va), _p(ctx), _p(L), B, T, Hq, Hkv, D, layout, st) == OK
        assert shim.shim_flash_attn_backward_gqa(_p(qa), _p(ka), _p(va), _p(ctx), _p(L), _p(doa), _p(dq), _p(dk), _p(dv), B, T,
                                                 Hq, Hkv, D, layout, st) == OK
    side.synchronize()
    m.device_status()
    want = ao.attn_fwd_bwd_c(np32(q), np32(k), np32(v), np32(do))
    assert_close("ctx", unlay(ctx), want[0])
    assert_close("L", L, want[1], max_abs=TOL_LSE, rel_l2=1.0)
    assert_close("d_q", unlay(dq), want[2])
    assert_close("d_k", unlay(dk), want[3])
    assert_close("d_v", unlay(dv), want[4])


def test_reference_exceptions(shim):
    B, T, D = 2, 128, 64
    q = randn_bf16((B, T, D), 0)
    q32 = q.float()
    L = torch.empty(B, T, device="cuda")
    # FP32 tensors are what the reference's kernels take; this engine's I/O type is BF16: invalid_argument,
    # as the reference throws for a wrong dtype (llm/src/model/flash_attn.cu:386-391)
    assert shim.shim_flash_attn_forward(_p(q32), _p(q32), _p(q32), _p(q32), _p(L), B, T, D, 32, 1, None) == INVALID_ARGUMENT
    assert b"must be BF16" in shim.shim_last_error()
    # tile <= 0 (llm/src/model/flash_attn.cu:398, 445)
    assert shim.shim_flash_attn_forward(_p(q), _p(q), _p(q), _p(q), _p(L), B, T, D, 0, 0, None) == INVALID_ARGUMENT
    assert b"tile_kv must be > 0" in shim.shim_last_error()
    assert shim.shim_flash_attn_backward(*([_p(q)] * 4), _p(L), *([_p(q)] * 4), B, T, D, -1, 0, None) == INVALID_ARGUMENT
    assert b"tile must be > 0" in shim.shim_last_error()
    # numel mismatch (llm/src/model/flash_attn.cu:400-404): the tensors hold B*T*D elements, the call says 2B
    assert shim.shim_flash_attn_forward_gqa(_p(q), _p(q), _p(q), _p(q), _p(L), B, T, 2, 1, 32, 0, None) == INVALID_ARGUMENT
    # a head dimension the engine does not have: also invalid_argument
    assert m.device_status() == 0


def test_steady_state_backward_allocates_nothing_and_does_not_synchronise(shim):
    B, T, Hq, Hkv, D = 4, 512, 6, 2, 64
    q, k, v = randn_bf16((B, Hq, T, D), 1), randn_bf16((B, Hkv, T, D), 2), randn_bf16((B, Hkv, T, D), 3)
    do = randn_bf16((B, Hq, T, D), 4, 0.1)
    ctx, L = torch.empty_like(q), torch.empty(B, Hq, T, device="cuda")
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    side = torch.cuda.Stream()

    def both(st):
        assert shim.shim_flash_attn_forward_gqa(_p(q), _p(k), _p(v), _p(ctx), _p(L), B, T, Hq, Hkv, D, 0, st) == OK
        assert shim.shim_flash_attn_backward_gqa(_p(q), _p(k), _p(v), _p(ctx), _p(L), _p(do), _p(dq), _p(dk), _p(dv), B, T, Hq,
                                                 Hkv, D, 0, st) == OK

    for st in (None, side.cuda_stream):  # legacy default stream: the library's fixed scratch; a stream: a kept workspace
        both(st)  # the first call on a stream may allocate its workspace
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        # a long kernel in front on the same stream: if the shim synchronised, the host would wait for it
        torch.cuda._sleep(200_000_000) if st is None else None
        import time

        t0 = time.perf_counter()
        for _ in range(5):
            both(st)
        host_s = time.perf_counter() - t0
        torch.cuda.synchronize()
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0, "the steady-state shim call changed the amount of free device memory"
        if st is None:
            assert host_s < 0.05, f"the shim blocked the host for {host_s:.3f} s behind queued work"
    assert m.device_status() == 0


def test_decode_through_the_shim(shim):
    B, Lc, Hq, Hkv, D = 3, 700, 8, 2, 64
    q, kc, vc = randn_bf16((B, Hq, D), 1), randn_bf16((B, Hkv, Lc, D), 2), randn_bf16((B, Hkv, Lc, D), 3)
    o = torch.full_like(q, float("nan"))
    assert shim.shim_flash_attn_decode(_p(q), _p(kc), _p(vc), _p(o), B, Lc, Hq, Hkv, D, None) == OK
    m.device_status()
    od, _ = ao.decode_c(np32(q), np32(kc), np32(vc))
    assert_close("o", o, od)
