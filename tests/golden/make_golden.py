"""Generates tests/golden/reference_host.npz from the reference's OWN host functions.

Run in a container where the reference tree is mounted:

    make -C oracle ref          # builds oracle/_ref/libref_host.so from the reference sources
    python tests/golden/make_golden.py

The library wraps, unchanged, attn_host (llm/tests/test_attention.cu:21-75), mha_host
(llm/tests/test_mha.cu:24-72), rope_host (llm/tests/test_rope.cu:18-38), rmsnorm_host
(llm/tests/test_rmsnorm.cu:16-27) and f32_to_bf16 / bf16_to_f32 (llm/src/core/dtype.h:34-49).
Inputs are seeded numpy draws with the distributions of the reference's tests (U(-1,1));
the shapes are the reference's test shapes (llm/tests/test_attention.cu:82,
llm/tests/test_mha.cu:107, llm/tests/test_flash_attn.cu:69-72).  The fixture travels with
the repository; the reference tree does not.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LIB = os.path.join(ROOT, "oracle", "_ref", "libref_host.so")


def fp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def main():
    L = ctypes.CDLL(LIB)
    rng = np.random.default_rng(20260001)
    out = {}

    def u(*shape):
        return rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)

    # attn_host on [B', T, D]; shapes of test_attention.cu and test_flash_attn.cu
    for i, (B, T, D) in enumerate([(2, 5, 6), (2, 8, 4), (2, 16, 8), (2, 64, 16), (1, 128, 64)]):
        q, k, v = u(B, T, D), u(B, T, D), u(B, T, D)
        ctx = np.zeros((B, T, D), np.float32)
        probs = np.zeros((B, T, T), np.float32)
        L.ref_attn_host(fp(q), fp(k), fp(v), B, T, D, fp(ctx), fp(probs))
        out.update({f"attn{i}_q": q, f"attn{i}_k": k, f"attn{i}_v": v, f"attn{i}_ctx": ctx, f"attn{i}_probs": probs})
    # mha_host on [B, T, H*d]
    B, T, H, d = 2, 5, 4, 6
    q, k, v = u(B, T, H * d), u(B, T, H * d), u(B, T, H * d)
    ctx = np.zeros((B, T, H * d), np.float32)
    L.ref_mha_host(fp(q), fp(k), fp(v), B, T, H, d, fp(ctx))
    out.update({"mha_q": q, "mha_k": k, "mha_v": v, "mha_ctx": ctx, "mha_dims": np.array([B, T, H, d])})
    # rope_host, base 10000
    N, T, d = 3, 7, 8
    x = u(N, T, d)
    y = np.zeros_like(x)
    L.ref_rope_host(fp(x), fp(y), N, T, d, ctypes.c_float(10000.0))
    out.update({"rope_x": x, "rope_y": y})
    N, T, d = 2, 40, 64
    x = u(N, T, d)
    y = np.zeros_like(x)
    L.ref_rope_host(fp(x), fp(y), N, T, d, ctypes.c_float(10000.0))
    out.update({"rope64_x": x, "rope64_y": y})
    # rmsnorm_host, gamma = 1, eps = 1e-5
    N, D = 5, 16
    x = u(N, D)
    g = np.ones(D, np.float32)
    y = np.zeros_like(x)
    L.ref_rmsnorm_host(fp(x), fp(g), fp(y), N, D, ctypes.c_float(1e-5))
    out.update({"rms_x": x, "rms_y": y})
    # BF16 rounding, including ties and values next to them
    x = np.concatenate([u(4096) * 3.0, np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 0.0, 65280.0, 3.0e38],
                                                np.float32)])
    bits = x.view(np.uint32).copy()
    bits[:2048] = (bits[:2048] & 0xFFFF0000) | 0x8000  # exact ties
    x = bits.view(np.float32)
    y = np.zeros(x.shape, np.uint16)
    L.ref_f32_to_bf16(fp(x), y.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), x.size)
    z = np.zeros(x.shape, np.float32)
    L.ref_bf16_to_f32(y.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16)), fp(z), x.size)
    out.update({"bf16_x": x, "bf16_bits": y, "bf16_back": z})
    # rope_host followed by rmsnorm_host with a non-trivial gamma: the chain the model runs on q and k
    # (llm/src/model/modern_gpt.cu:358-370), for the fused RoPE + QK-Norm kernel
    for tag, (N, T, d) in {"ropenorm64": (3, 33, 64), "ropenorm128": (2, 9, 128)}.items():
        x = u(N, T, d)
        r = np.zeros_like(x)
        L.ref_rope_host(fp(x), fp(r), N, T, d, ctypes.c_float(10000.0))
        g = (1.0 + 0.2 * u(d)).astype(np.float32)
        y = np.zeros_like(x)
        L.ref_rmsnorm_host(fp(r), fp(g), fp(y), N * T, d, ctypes.c_float(1e-5))
        out.update({f"{tag}_x": x, f"{tag}_g": g, f"{tag}_y": y})
    np.savez_compressed(os.path.join(HERE, "reference_host.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_host.npz"), sum(a.nbytes for a in out.values()), "bytes raw")


if __name__ == "__main__":
    main()
