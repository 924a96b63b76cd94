"""Child process of test_gpu_item_scheduling.py (not collected): runs forward + backward on seeded inputs
and prints one SHA-256 per output, so that runs under different B200ATTN_ITEMS settings (the library reads
the variable once per process) can be compared bit for bit."""
import hashlib
import sys

import torch

import modern_llm_v1_b200 as m


def main():
    B, T, Hq, Hkv, D, reps = (int(x) for x in sys.argv[1:7])
    g = torch.Generator().manual_seed(20260003)
    mk = lambda *s, std=1.0: (torch.randn(*s, generator=g) * std).bfloat16().cuda()
    q, k, v, do = mk(B, Hq, T, D), mk(B, Hkv, T, D), mk(B, Hkv, T, D), mk(B, Hq, T, D, std=0.1)
    first = digests = None
    for _ in range(reps):  # more launches than the library has counter pairs: every pair is used again
        o = torch.full_like(q, float("nan"))
        lse = torch.full((B, Hq, T), float("nan"), device="cuda")
        dq, dk, dv = torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))
        m.flash_attn_forward_gqa(q, k, v, o, lse, B, T, Hq, Hkv, D)
        m.flash_attn_backward_gqa(q, k, v, o, lse, do, dq, dk, dv, B, T, Hq, Hkv, D)
        m.device_status()
        outs = [o, lse, dq, dk, dv]
        if first is None:
            assert not any(torch.isnan(x.float()).any().item() for x in outs), "an output element was never written"
            first = outs
            digests = [hashlib.sha256(x.cpu().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest() for x in outs]
        for name, x, y in zip(("O", "LSE", "dQ", "dK", "dV"), outs, first):
            # compared on the device, bit for bit (NaN never equals itself, so an unwritten element fails too)
            assert torch.equal(x, y), f"two runs in one process differ in {name}"
    print(" ".join(digests))


if __name__ == "__main__":
    main()
