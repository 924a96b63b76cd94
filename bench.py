#!/usr/bin/env python3
"""Benchmark of the causal GQA attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config NAME]

One "step" is one forward (O + logsumexp) and one backward (dQ, dK, dV) over one batch of
seeded synthetic activations of the named configuration (default: the 50M training shape,
B=32, T=512, Hq=6, Hkv=2, D=64, BF16 I/O, FP32 accumulation).  Prints ONE JSON line.

* value      whole-job TFLOP/s with inputs resident in HBM (4*B*Hq*T^2*D/2 forward FLOPs,
             2.5x that for backward), device-timed, max over ranks.
* e2e        the same metric through the public operator API with HOST buffers: every step
             copies its inputs from pinned host memory and reads its results back.
* roofline   the dominant kernel's tensor throughput against the measured BF16 peak.
* cpu_baseline  the CPU oracle (a port of the reference's host attention) on the box's cores.

Multi-GPU (launched by torchrun, one rank per GPU): every rank runs the full configuration on
its own seed — (batch, KV head) shards are independent, no collective is on the data path —
so scaling is "weak"; NCCL only carries the timing reduction and a checksum gather.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}

# DRAM traffic of the dominant kernel per launch at the default workload, from the committed ncu
# summary (profiles/); None until a capture exists for the current kernel.
# (dram read + write per launch of each kernel, profiles/attn_fwd_bwd_c2_50m_train.md)
NCU_TRAFFIC_BYTES = {"c2_50m_train": {"attn_fwd_kernel": 21033728, "attn_bwd_dq_kernel": 46777088,
                                      "attn_bwd_dkdv_kernel": 34416896},
                     # profiles/attn_fwd_bwd_c3_300m_class.md
                     "c3_300m_class": {"attn_fwd_kernel": 53215488, "attn_bwd_dq_kernel": 132836864,
                                       "attn_bwd_dkdv_kernel": 96702208},
                     # profiles/attn_fwd_bwd_c4_long_context.md (the dK/dV pass streams Q and dO once per key tile: the
                     # re-reads hit L2 at 78 %, the rest comes from DRAM again)
                     "c4_long_context": {"attn_fwd_kernel": 473484288, "attn_bwd_dq_kernel": 1000673280,
                                         "attn_bwd_dkdv_kernel": 1197408512}}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2_50m_train")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="issue every launch of the timed region from Python instead of replaying CUDA graphs")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak (default): every rank runs the whole config; strong: the config's batch is split over "
                         "the ranks (contiguous (batch, KV head) units), so the total work is fixed")
    ap.add_argument("--backward", default="two_pass", choices=["two_pass", "one_pass"],
                    help="two_pass (default, bit-reproducible): dQ pass + dK/dV pass; one_pass (D = 64): scores computed "
                         "once, dQ summed by reduce-adds (row-vector kernel, fused kernel, dQ conversion)")
    ap.add_argument("--op", default="attention", choices=["attention", "qkprep", "decode_step"],
                    help="qkprep: the fused RoPE + QK-Norm operator on the config's q and k (HBM GB/s); "
                         "decode_step (with --config c5_decode): one cached sampling step of a layer, KV-cache "
                         "append + split-KV decode (HBM GB/s)")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------
# clocks: sampled through NVML while the timed region runs
# ------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        self.period = period_s
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if r & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ------------------------------------------------------------------------------------------
# CPU side: the oracle port timed on the host cores (cpu_baseline leg and --impl reference)
# ------------------------------------------------------------------------------------------
class StepGraphs:
    """Runs exactly K steps from CUDA graphs.  A step is a few short launches (2-3 kernels of 25-45 us); issued one
    by one from Python the host can set the pace (15-25 us per call on a slow host), so one round over the buffer
    sets is captured in a graph and replayed; a remainder of K % round steps comes from single-step graphs.  The
    launches inside a graph keep their programmatic-dependent-launch edges."""

    def __init__(self, step_fn, round_len: int):
        import torch

        self.torch, self.step_fn, self.round_len = torch, step_fn, round_len
        self.singles = {}
        self.round = self._capture(range(round_len))

    def _capture(self, indices):
        torch = self.torch
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for i in indices:
                    self.step_fn(i)
        torch.cuda.current_stream().wait_stream(side)
        return graph

    def prepare(self, k: int) -> None:
        for i in range(k % self.round_len):
            if i not in self.singles:
                self.singles[i] = self._capture([i])
        self.round.replay()  # warm
        for g in self.singles.values():
            g.replay()

    def run(self, k: int) -> None:
        rounds, rem = divmod(k, self.round_len)
        for _ in range(rounds):
            self.round.replay()
        for i in range(rem):
            self.singles[i].replay()


def cpu_prepare(cfg, seed, n_units, one_head=False):
    """FP32 copies of the BF16-rounded inputs of the first `n_units` (batch, KV head) units; with
    one_head only the first query head of the first unit (the smallest sample there is)."""
    from modern_llm_v1_b200 import inputs

    q, k, v, do, hq, hkv = inputs.make_train_inputs(cfg, seed, 0, n_units, bf16=True)
    arrs = [t.float().numpy() for t in (q, k, v, do)]
    frac = n_units / cfg.units
    if one_head:
        arrs = [arrs[0][:1, :1].copy(), arrs[1][:1, :1].copy(), arrs[2][:1, :1].copy(), arrs[3][:1, :1].copy()]
        frac = 1.0 / (cfg.units * cfg.group)
    return arrs, cfg.fwd_bwd_flops() * frac


def cpu_time_units(cfg, seed, n_units, repeats=1):
    """Seconds for one forward+backward of `n_units` (batch, KV head) units on the CPU oracle
    (all host threads), and the FLOPs those units stand for."""
    from oracle import attn_oracle as ao

    arrs, flops = cpu_prepare(cfg, seed, n_units)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        ao.attn_fwd_bwd_c(*arrs)
        best = min(best, time.perf_counter() - t0)
    return best, flops


def use_all_host_cores():
    """torchrun exports OMP_NUM_THREADS=1; the CPU legs want every core this process may run on."""
    from oracle import attn_oracle as ao

    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    ao.set_num_threads(n)
    return ao.num_threads()


def cpu_baseline(cfg, seed):
    from oracle import attn_oracle as ao

    cores = use_all_host_cores()
    # about 20 core-seconds of work at ~1.9 GFLOP/s per core of this scalar double-precision port
    unit_flops = cfg.fwd_bwd_flops() / cfg.units
    n_units = int(max(1, min(cfg.units, 20.0 * 1.9e9 / unit_flops)))
    t, flops = cpu_time_units(cfg, seed, n_units)
    heads = n_units * cfg.group
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": min(cores, heads), "kind": "port",
            "sample": f"{n_units} of {cfg.units} (batch, KV head) units of {cfg.name}, forward+backward once, "
                      f"{t:.2f} s wall on {min(cores, heads)} threads (OpenMP over batch x query head)"}


def run_reference_arm(args, cfg, cfg_full, rank, world):
    """--impl reference: the reference's host attention algorithm (oracle port: the reference's own
    host function is forward-only and single-threaded) on this box's cores, bounded sample per step."""
    if rank != 0:
        return
    from oracle import attn_oracle as ao

    cores = use_all_host_cores()
    seed = 20260002
    # calibrate on a few units, then size the per-step sample so that the run ends within ~2 minutes
    n_cal = min(cfg.units, max(2, min(cores, 8)))
    t_cal, _ = cpu_time_units(cfg, seed, n_cal)
    budget = 100.0 / max(1, args.steps + args.warmup)  # seconds per step
    waves = lambda n: -(-(n * cfg.group) // cores)     # heads are spread over the threads in waves
    t_head = t_cal / waves(n_cal)                      # wall time of one wave of heads
    n_units, one_head = 1, True
    if t_head * waves(1) <= budget:
        one_head = False
        while n_units * 2 <= cfg.units and t_head * waves(n_units * 2) <= budget:
            n_units *= 2
    arrs, step_flops = cpu_prepare(cfg, seed, n_units, one_head)
    for _ in range(args.warmup):
        ao.attn_fwd_bwd_c(*arrs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ao.attn_fwd_bwd_c(*arrs)
    dt = time.perf_counter() - t0
    val = step_flops * args.steps / dt / 1e12
    threads = 1 if one_head else min(cores, n_units * cfg.group)
    sample = ("one query head of one unit" if one_head else f"{n_units} of {cfg.units} (batch, KV head) units") + \
             f" of {cfg.name} per step, forward+backward on the CPU oracle"
    line = {
        "impl": "reference", "metric": "causal_gqa_attn_fwd_bwd_tflops", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": workload_config(cfg_full, world, args.scaling),
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU side
# ------------------------------------------------------------------------------------------
class BufferSet:
    """Device tensors of one step: inputs, outputs and gradients (BHTD layout)."""

    def __init__(self, cfg, host, device):
        import torch

        self.q, self.k, self.v, self.do = (t.to(device, non_blocking=True) for t in host)
        self.o = torch.empty_like(self.q)
        self.lse = torch.empty(cfg.B, cfg.Hq, cfg.T, dtype=torch.float32, device=device)
        self.dq = torch.empty_like(self.q)
        self.dk = torch.empty_like(self.k)
        self.dv = torch.empty_like(self.v)

    def nbytes(self):
        return sum(t.numel() * t.element_size() for t in
                   (self.q, self.k, self.v, self.do, self.o, self.lse, self.dq, self.dk, self.dv))


BWD_MODE = "two_pass"  # set from --backward


def step(m, cfg, s):
    """One forward + one backward (two-pass backward: three kernel launches per step; one-pass: four)."""
    m.flash_attn_forward_gqa(s.q, s.k, s.v, s.o, s.lse, cfg.B, cfg.T, cfg.Hq, cfg.Hkv, cfg.D)
    m.flash_attn_backward_gqa(s.q, s.k, s.v, s.o, s.lse, s.do, s.dq, s.dk, s.dv, cfg.B, cfg.T, cfg.Hq, cfg.Hkv, cfg.D,
                              mode=BWD_MODE)


def set_bytes(cfg):
    """Bytes of one step's device tensors: q, dO, O, dQ (Hq heads), k, v, dK, dV (Hkv heads), BF16, and the logsumexp."""
    return 2 * cfg.B * cfg.T * cfg.D * (4 * cfg.Hq + 4 * cfg.Hkv) + 4 * cfg.B * cfg.Hq * cfg.T


def n_buffer_sets(cfg):
    return max(2, int(2 * 126e6 // set_bytes(cfg)) + 1)


def workload_config(cfg_full, world, scaling):
    """What both arms print under "config": the workload, identical for the two arms (how an arm ran it is in "run")."""
    per_gpu = cfg_full if scaling == "weak" else dataclasses.replace(cfg_full, B=cfg_full.B // world)
    n = n_buffer_sets(per_gpu)
    return {"workload": cfg_full.name, "B_per_gpu": per_gpu.B,
            "global_B": cfg_full.B * world if scaling == "weak" else cfg_full.B, "T": cfg_full.T, "Hq": cfg_full.Hq,
            "Hkv": cfg_full.Hkv, "D": cfg_full.D, "layout": "BHTD",
            "parallelism": f"{world} x independent (batch, KV head) shards",
            "l2": f"on a GPU consecutive steps rotate over {n} distinct buffer sets, {n * set_bytes(per_gpu) / 1e6:.0f} MB "
                  "> 126 MB L2",
            "inputs": "q,k: N(0,1) -> RoPE(base 1e4) -> per-head RMSNorm(gamma 1); v: N(0,1); dO: N(0,1e-2) "
                      "(sigma 0.1; the kernels' time does not depend on the scale of dO); rounded to BF16"}


def kernel_breakdown(m, cfg, sets, steps):
    """Average device time of each kernel of a step, CUDA events on the launching stream."""
    import torch

    lib = m._lib.load()
    n = min(steps, 200)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(6)] for _ in range(n)]
    for row in evs:  # events get their CUDA handle on first record
        for e in row:
            e.record()
    torch.cuda.synchronize()
    for i in range(n):
        s = sets[i % len(sets)]
        e = evs[i]
        m._lib.check(lib.b200attn_set_bwd_profile_events4(e[2].cuda_event, e[3].cuda_event, e[4].cuda_event,
                                                           e[5].cuda_event), "set_bwd_profile_events4")
        e[0].record()
        m.flash_attn_forward_gqa(s.q, s.k, s.v, s.o, s.lse, cfg.B, cfg.T, cfg.Hq, cfg.Hkv, cfg.D)
        e[1].record()
        m.flash_attn_backward_gqa(s.q, s.k, s.v, s.o, s.lse, s.do, s.dq, s.dk, s.dv, cfg.B, cfg.T, cfg.Hq, cfg.Hkv,
                                  cfg.D, mode=BWD_MODE)
    lib.b200attn_set_bwd_profile_events4(None, None, None, None)
    torch.cuda.synchronize()
    if BWD_MODE == "one_pass":
        names = ["attn_fwd_kernel", "attn_bwd_prep_kernel", "attn_bwd_onepass_kernel", "attn_bwd_dq_convert_kernel"]
        pairs = [(0, 1), (2, 3), (3, 4), (4, 5)]
    else:
        names = ["attn_fwd_kernel", "attn_bwd_dq_kernel", "attn_bwd_dkdv_kernel"]
        pairs = [(0, 1), (2, 3), (3, 4)]
    out = {}
    for name, (a, b) in zip(names, pairs):
        out[name] = sum(e[a].elapsed_time(e[b]) for e in evs) / n  # ms
    return out


def bind_near_gpu(index):
    """Binds this process to the host cores NVML names as close to GPU `index` (those of them the process may
    run on), so that the pinned buffers allocated afterwards are first touched on that side of the host.  A host
    setting of this process only; nothing on the GPU changes.  Returns the number of cores bound, or None."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (max(allowed) // 64) + 1)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        pick = near & allowed
        if pick and pick != allowed:
            os.sched_setaffinity(0, pick)
            return len(pick)
        return len(allowed) if pick else None
    except Exception:
        return None


class PackedStep:
    """Device tensors of one step carved out of two allocations (inputs q|k|v|dO and outputs O|dQ|dK|dV), so that
    a step's inputs cross the host link in ONE copy and its results in one."""

    def __init__(self, cfg, device):
        import torch

        nq, nk = cfg.B * cfg.Hq * cfg.T * cfg.D, cfg.B * cfg.Hkv * cfg.T * cfg.D
        self.inp = torch.empty(2 * nq + 2 * nk, dtype=torch.bfloat16, device=device)
        self.out = torch.empty(2 * nq + 2 * nk, dtype=torch.bfloat16, device=device)
        qs, ks = (cfg.B, cfg.Hq, cfg.T, cfg.D), (cfg.B, cfg.Hkv, cfg.T, cfg.D)
        self.q, self.k = self.inp[:nq].view(qs), self.inp[nq:nq + nk].view(ks)
        self.v, self.do = self.inp[nq + nk:nq + 2 * nk].view(ks), self.inp[nq + 2 * nk:].view(qs)
        self.o, self.dq = self.out[:nq].view(qs), self.out[nq:2 * nq].view(qs)
        self.dk, self.dv = self.out[2 * nq:2 * nq + nk].view(ks), self.out[2 * nq + nk:].view(ks)
        self.lse = torch.empty(cfg.B, cfg.Hq, cfg.T, dtype=torch.float32, device=device)


def e2e_measure(m, cfg, host_sets, steps, warmup, device):
    """ms per step through the operator API with HOST buffers: one H2D copy of q|k|v|dO from pinned memory, forward,
    backward, one D2H copy of O|dQ|dK|dV into pinned memory; three streams, two device buffer sets in flight.  Also
    the same copies with no kernels in between (what the host link alone allows)."""
    import torch

    n_buf = 2
    dev = [PackedStep(cfg, device) for _ in range(n_buf)]
    packed_in = []
    for h in host_sets:
        buf = torch.empty(dev[0].inp.numel(), dtype=torch.bfloat16, pin_memory=True)
        torch.cat([t.reshape(-1) for t in (h[0], h[1], h[2], h[3])], out=buf)
        packed_in.append(buf)
    outs = [torch.empty(dev[0].out.numel(), dtype=torch.bfloat16, pin_memory=True) for _ in range(n_buf)]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(n_buf)]
    ev_cmp = [torch.cuda.Event() for _ in range(n_buf)]
    ev_out = [torch.cuda.Event() for _ in range(n_buf)]
    torch.cuda.synchronize()

    def one(i, compute=True):
        b = i % n_buf
        d = dev[b]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[b])  # the previous use of these device inputs has been consumed
            d.inp.copy_(packed_in[i % len(packed_in)], non_blocking=True)
            ev_in[b].record()
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[b])
            s_cmp.wait_event(ev_out[b])  # the previous outputs of this set have left the device
            if compute:
                step(m, cfg, d)
            ev_cmp[b].record()
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[b])
            outs[b].copy_(d.out, non_blocking=True)
            ev_out[b].record()

    def timed(compute):
        for i in range(warmup):
            one(i, compute)
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(steps):
            one(i, compute)
        for st in (s_in, s_cmp, s_out):
            torch.cuda.current_stream().wait_stream(st)
        t1.record()
        torch.cuda.synchronize()
        return t0.elapsed_time(t1) / steps

    ms = timed(True)
    ms_copy = timed(False)
    nbytes = dev[0].inp.numel() * 2
    return ms, ms_copy, nbytes, nbytes


def run_decode(m, cfg, args, rank, world, device, peaks, warmup, steps, barrier):
    """Split-KV decode (one query token per sequence against the KV cache): HBM GB/s.  Algorithmic bytes
    per step = K cache + V cache + q + o.  The cache (268 MB at the default shape) is larger than L2."""
    import torch
    import torch.distributed as dist
    from modern_llm_v1_b200 import inputs

    q, kc, vc, _, _ = inputs.make_decode_inputs(cfg, 20260005 + 1000 * rank)
    q, kc, vc = q.to(device), kc.to(device), vc.to(device)
    o = torch.empty_like(q)
    lse = torch.empty(cfg.B, cfg.Hq, dtype=torch.float32, device=device)

    def step():
        m.flash_attn_decode(q, kc, vc, o, lse, cfg.B, cfg.T, cfg.Hq, cfg.Hkv, cfg.D)

    for _ in range(warmup):
        step()
    m.device_status()
    graphs = None
    if not args.no_graph:
        graphs = StepGraphs(lambda i: step(), 8)
        graphs.prepare(steps)
        m.device_status()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    if graphs is not None:
        graphs.run(steps)
    else:
        for _ in range(steps):
            step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    m.device_status()
    # end to end: q from pinned host memory, o back to pinned host memory, a stream synchronise per step
    q_host, o_host = q.cpu().pin_memory(), torch.empty(q.shape, dtype=q.dtype).pin_memory()
    n_e2e = max(10, steps // 10)
    barrier()
    e0.record()
    for _ in range(n_e2e):
        q.copy_(q_host, non_blocking=True)
        step()
        o_host.copy_(o, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    if world > 1:
        t = torch.tensor([ms_e2e], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    nbytes = cfg.decode_bytes()
    gbs = world * nbytes / (ms * 1e-3) / 1e9
    peak = float(peaks["hbm_gbs"])
    if rank == 0:
        print(json.dumps({
            "metric": "decode_attn_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": cfg.name, "B_per_gpu": cfg.B, "cache_len": cfg.T, "Hq": cfg.Hq, "Hkv": cfg.Hkv,
                       "D": cfg.D, "l2": f"cache of {nbytes / 1e6:.0f} MB > 126 MB L2"},
            "clocks": clocks, "gpu_launches": 2 * steps,
            "e2e": {"value": world * nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": q.numel() * 2, "d2h_bytes_per_step": q.numel() * 2,
                    "note": "q from pinned host memory, o read back, a stream synchronise per step; the cache stays "
                            "on the device, as it does between the tokens of a sampling loop"},
            "roofline": {"bound": "hbm", "kernel": "attn_decode_kernel", "achieved": gbs / world, "peak": peak,
                         "unit": "GB/s", "frac": gbs / world / peak,
                         "traffic": 273341184 if cfg.name == "c5_decode" else None,  # profiles/attn_decode_c5_decode.md
                         "peak_source": f"hbm_gbs of {peaks['_source']}", "bytes_per_launch": nbytes,
                         "note": "time includes the combine kernel (2 launches per step)"},
        }), flush=True)


def run_qkprep(m, cfg, args, rank, world, device, peaks, warmup, steps, barrier):
    """Fused RoPE + QK-Norm, forward and backward, on q ([B,T,Hq,D]) and k ([B,T,Hkv,D]) of the config, BF16 in
    the projection-output layout, BF16 out in the attention layout: HBM GB/s.  Algorithmic bytes per step =
    forward (x read, y written, rstd written) + backward (x, dy, rstd read, dx written); the step rotates over
    buffer sets larger than L2."""
    import numpy as np
    import torch
    import torch.distributed as dist

    B, T, D = cfg.B, cfg.T, cfg.D
    heads = (cfg.Hq, cfg.Hkv)
    g = torch.Generator().manual_seed(20260006 + 1000 * rank)
    n_sets = 4
    cos, sin = m.make_rope_cache(T, D, 10000.0, device)
    gamma = [(1.0 + 0.1 * torch.randn(D, generator=g)).to(device) for _ in heads]
    sets = []
    for _ in range(n_sets):
        s = []
        for H in heads:
            x = torch.randn(B, T, H, D, generator=g).bfloat16().to(device)
            dy = torch.randn(B, H, T, D, generator=g).bfloat16().to(device)
            s.append(dict(x=x, dy=dy, y=torch.empty(B, H, T, D, dtype=torch.bfloat16, device=device),
                          rstd=torch.empty(B, H, T, device=device), dx=torch.empty_like(x),
                          dg=torch.zeros(D, device=device)))
        sets.append(s)

    def step(i):
        tq, tk = sets[i % n_sets]
        m.rope_qknorm_forward_qk(tq["x"], tk["x"], cos, sin, gamma[0], gamma[1], 1e-5, tq["y"], tk["y"], tq["rstd"],
                                 tk["rstd"], B, T, cfg.Hq, cfg.Hkv, D)
        m.rope_qknorm_backward_qk(tq["dy"], tk["dy"], tq["x"], tk["x"], cos, sin, gamma[0], gamma[1], tq["rstd"],
                                  tk["rstd"], tq["dx"], tk["dx"], tq["dg"], tk["dg"], B, T, cfg.Hq, cfg.Hkv, D)

    for i in range(warmup):
        step(i)
    m.device_status()
    # Three short launches per step: issued one by one from Python the host, not the GPU, sets the pace
    # (about 20 us per call), so one round over the buffer sets is captured in a CUDA graph and replayed.
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            for i in range(n_sets):
                step(i)
    torch.cuda.current_stream().wait_stream(side)
    steps = max(n_sets, steps // n_sets * n_sets)
    for _ in range(3):
        graph.replay()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(steps // n_sets):
        graph.replay()
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / steps
    if world > 1:
        t_ = torch.tensor([ms], device=device)
        dist.all_reduce(t_, op=dist.ReduceOp.MAX)
        ms = float(t_.item())
    m.device_status()
    rows = B * T * sum(heads)
    nbytes = rows * D * 2 * 2 + rows * 4 + rows * D * 2 * 3 + rows * 4  # fwd: x, y, rstd; bwd: x, dy, dx, rstd
    # end to end: x and dy of q and k from pinned host memory, y and dx back, a stream synchronise per step
    tq0, tk0 = sets[0]
    h_in = [t[k_].cpu().pin_memory() for t in (tq0, tk0) for k_ in ("x", "dy")]
    h_out = [torch.empty(t[k_].shape, dtype=t[k_].dtype).pin_memory() for t in (tq0, tk0) for k_ in ("y", "dx")]
    n_e2e = max(5, min(50, steps // 20))
    barrier()
    e0.record()
    for _ in range(n_e2e):
        for dst, src in zip([t[k_] for t in (tq0, tk0) for k_ in ("x", "dy")], h_in):
            dst.copy_(src, non_blocking=True)
        step(0)
        for dst, src in zip(h_out, [t[k_] for t in (tq0, tk0) for k_ in ("y", "dx")]):
            dst.copy_(src, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    e1.record()
    barrier()
    ms_e2e = e0.elapsed_time(e1) / n_e2e
    if world > 1:
        t_ = torch.tensor([ms_e2e], device=device)
        dist.all_reduce(t_, op=dist.ReduceOp.MAX)
        ms_e2e = float(t_.item())
    m.device_status()
    gbs = world * nbytes / (ms * 1e-3) / 1e9
    peak = float(peaks["hbm_gbs"])
    out = {
        "metric": "rope_qknorm_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": cfg.name + "_qkprep", "B_per_gpu": B, "T": T, "Hq": cfg.Hq, "Hkv": cfg.Hkv, "D": D,
                   "io": "x, dy, dx BF16 [B,T,H,D] / [B,H,T,D]; y BF16 [B,H,T,D]; rstd FP32",
                   "l2": f"rotating over {n_sets} buffer sets, {n_sets * rows * D * 2 * 4 / 1e6:.0f} MB > 126 MB L2",
                   "launch": "one round over the buffer sets captured in a CUDA graph and replayed"},
        "clocks": clocks, "gpu_launches": 3 * steps,
        "e2e": {"value": world * nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in h_in),
                "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in h_out),
                "note": "bound by the host link: every tensor crosses it once per step"},
        "roofline": {"bound": "hbm", "kernel": "rope_norm_fwd_kernel + rope_norm_bwd_kernel", "achieved": gbs / world,
                     "peak": peak, "unit": "GB/s", "frac": gbs / world / peak,
                     "traffic": 794041344 if cfg.name == "c4_long_context" else None,  # profiles/rope_norm_c4_long_context.md
                     "peak_source": f"hbm_gbs of {peaks['_source']}", "bytes_per_step": nbytes,
                     "note": "3 launches per step: q and k together, forward, backward, d_gamma sums"},
    }
    if rank == 0 and not args.no_cpu_baseline:
        from oracle import attn_oracle as ao
        use_all_host_cores()
        xs = np.random.default_rng(1).standard_normal((8, heads[0], T, D)).astype(np.float32)
        gs = np.ones(D, np.float32)
        t0 = time.perf_counter()
        yo, rs = ao.rope_norm_fwd(xs, gs)
        ao.rope_norm_bwd(yo, xs, gs, rs)
        dt = time.perf_counter() - t0
        srows = xs.shape[0] * heads[0] * T
        sbytes = srows * D * 2 * 5 + srows * 8
        out["cpu_baseline"] = {"value": sbytes / dt / 1e9, "unit": "GB/s (same byte convention)", "cores": ao.num_threads(),
                               "kind": "port", "sample": f"{srows} of {rows} rows, forward + backward once, {dt:.2f} s wall "
                               "(the backward's d_gamma sum is single-threaded by design)"}
    if rank == 0:
        print(json.dumps(out), flush=True)


def run_decode_step(m, cfg, args, rank, world, device, peaks, warmup, steps, barrier):
    """One cached sampling step of a layer: KVCache.append (split heads + RoPE at the true position + QK-Norm +
    cache write for the newest token of every sequence) followed by KVCache.attend (split-KV decode over the
    cache): HBM GB/s.  The cache length is held at the config's (each step rewrites row L-1 and reads L rows);
    algorithmic bytes per step = K and V cache + the new token's FP32 q, k, v rows in + BF16 q, k, v, o out."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from modern_llm_v1_b200 import inputs

    B, L, Hq, Hkv, D = cfg.B, cfg.T, cfg.Hq, cfg.Hkv, cfg.D
    _, kc, vc, _, _ = inputs.make_decode_inputs(cfg, 20260005 + 1000 * rank)
    cache = m.KVCache(1, B, Hq, Hkv, D, L, device=device)
    cache.k[0].copy_(kc)
    cache.v[0].copy_(vc)
    del kc, vc
    g = torch.Generator().manual_seed(20260007 + 1000 * rank)
    host = [torch.randn(B, 1, H, D, generator=g).pin_memory() for H in (Hq, Hkv, Hkv)]
    xq, xk, xv = (t.to(device) for t in host)
    gamma = torch.ones(D, device=device)
    q = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16, device=device)
    o = torch.empty_like(q)
    o_host = torch.empty(B, Hq, 1, D, dtype=torch.bfloat16).pin_memory()

    def step(e2e=False):
        cache.length = L - 1
        if e2e:
            for d, h in zip((xq, xk, xv), host):
                d.copy_(h, non_blocking=True)
        cache.append(0, xq, xk, xv, gamma, gamma, q)
        cache.attend(0, q, o, None)
        if e2e:
            o_host.copy_(o, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    graphs = None

    def timed(n, e2e=False):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        if graphs is not None and not e2e:
            graphs.run(n)
        else:
            for _ in range(n):
                step(e2e)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1) / n
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for _ in range(warmup):
        step()
    m.device_status()
    if not args.no_graph:
        graphs = StepGraphs(lambda i: step(), 8)
        graphs.prepare(steps)
        m.device_status()
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    ms = timed(steps)
    clocks = sampler.stop()
    m.device_status()
    ms_e2e = timed(max(10, steps // 10), e2e=True)
    m.device_status()
    rows = B * (Hq + 2 * Hkv)
    h2d, d2h = rows * D * 4, B * Hq * D * 2
    nbytes = cfg.decode_bytes() + rows * D * 4 + rows * D * 2
    gbs = world * nbytes / (ms * 1e-3) / 1e9
    peak = float(peaks["hbm_gbs"])
    out = {
        "metric": "decode_step_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg.name + "_step", "B_per_gpu": B, "cache_len": L, "Hq": Hq, "Hkv": Hkv, "D": D,
                   "io": "new token's q, k, v FP32 [B,1,H,D] in; caches BF16 [B,Hkv,L,D]; o BF16 out",
                   "l2": f"cache of {cfg.decode_bytes() / 1e6:.0f} MB > 126 MB L2"},
        "clocks": clocks, "gpu_launches": 3 * steps,
        "e2e": {"value": world * nbytes / (ms_e2e * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "the new token's rows from pinned host memory, o read back, a stream synchronise per step"},
        "roofline": {"bound": "hbm", "kernel": "attn_decode_kernel", "achieved": gbs / world, "peak": peak,
                     "unit": "GB/s", "frac": gbs / world / peak,
                     # the three kernels of a step, profiles/kv_append_decode_step_c5_decode.md
                     "traffic": 272819456 if cfg.name == "c5_decode" else None,
                     "peak_source": f"hbm_gbs of {peaks['_source']}", "bytes_per_step": nbytes,
                     "note": "3 launches per step: kv_append_kernel, attn_decode_kernel, attn_decode_combine_kernel"},
    }
    if rank == 0 and not args.no_cpu_baseline:
        from oracle import attn_oracle as ao
        use_all_host_cores()
        nb = min(B, 8)
        kc32, vc32 = cache.k[0, :nb].float().cpu().numpy(), cache.v[0, :nb].float().cpu().numpy()
        hq, hk, hv = (t[:nb].numpy() for t in host)
        ones = np.ones(D, np.float32)
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 5.0:
            q32 = ao.kv_append(hq, hk, hv, ones, ones, kc32, vc32, L - 1)
            ao.decode_c(np.ascontiguousarray(q32[:, :, 0]), kc32, vc32)
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        out["cpu_baseline"] = {"value": nbytes * nb / B / dt / 1e9, "unit": "GB/s (same byte convention)",
                               "cores": ao.num_threads(), "kind": "port",
                               "sample": f"{nb} of {B} sequences, {reps} steps, FP32 caches on the host"}
    if rank == 0:
        print(json.dumps(out), flush=True)


def main():
    args = parse_args()
    import modern_llm_v1_b200 as m
    from modern_llm_v1_b200 import inputs

    cfg = inputs.CONFIGS[args.config]
    global BWD_MODE
    BWD_MODE = args.backward
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    cfg_full = cfg
    global_B = cfg.B * world
    if args.scaling == "strong" and world > 1:
        if cfg.B % world != 0:
            raise SystemExit(f"--scaling strong: the batch {cfg.B} does not divide over {world} ranks")
        global_B = cfg.B
        cfg = dataclasses.replace(cfg, B=cfg.B // world)  # this rank's contiguous block of (batch, KV head) units

    if args.impl == "reference":
        run_reference_arm(args, cfg, cfg_full, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = load_peaks()
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.op == "qkprep":
        run_qkprep(m, cfg, args, rank, world, device, peaks, warmup, steps, barrier)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if args.op == "decode_step":
        if cfg.kind != "decode":
            raise SystemExit("--op decode_step needs a decode config (--config c5_decode)")
        run_decode_step(m, cfg, args, rank, world, device, peaks, warmup, steps, barrier)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    if cfg.kind == "decode":
        run_decode(m, cfg, args, rank, world, device, peaks, warmup, steps, barrier)
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # Distinct buffer sets so that the working set of consecutive steps exceeds the 126 MB L2.
    seed0 = 20260002 + 1000 * rank
    host0 = [t.pin_memory() for t in inputs.make_train_inputs(cfg, seed0)[:4]]
    probe = BufferSet(cfg, host0, device)
    n_sets = n_buffer_sets(cfg)
    host_sets = [host0] + [[t.pin_memory() for t in inputs.make_train_inputs(cfg, seed0 + i)[:4]]
                           for i in range(1, min(n_sets, 4))]
    sets = [probe] + [BufferSet(cfg, host_sets[i % len(host_sets)], device) for i in range(1, n_sets)]
    torch.cuda.synchronize()

    for i in range(warmup):
        step(m, cfg, sets[i % n_sets])
    m.device_status()
    barrier()

    # ONE launch protocol gives `value`: a round over the buffer sets captured in a CUDA graph and replayed (it does
    # not depend on how fast the host's Python issues three 25-30 us launches); --no-graph makes it direct calls.
    # The other way is timed too, over the same K steps, and only reported in config.ms_per_step_by_launch.
    graphs = None
    if not args.no_graph:
        graphs = StepGraphs(lambda i: step(m, cfg, sets[i % n_sets]), n_sets)
        graphs.prepare(steps)
        m.device_status()

    def timed_steps(run, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        run(n)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        m.device_status()
        if world > 1:
            t = torch.tensor([ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def run_direct(n):
        for i in range(n):
            step(m, cfg, sets[i % n_sets])

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_by_launch = {"direct": timed_steps(run_direct, steps)}
    if graphs is not None:
        ms_by_launch["graph"] = timed_steps(graphs.run, steps)
    clocks = sampler.stop()
    launch_how = "direct" if graphs is None else "graph"
    ms_step = ms_by_launch[launch_how] / steps
    flops_step = cfg.fwd_bwd_flops()
    value = world * flops_step / (ms_step * 1e-3) / 1e12

    # the same steps on ONE buffer set (inputs of 67 MB stay in the 126 MB L2 from step to step)
    warm_graph = StepGraphs(lambda i: step(m, cfg, sets[0]), 4) if graphs is not None else None
    if warm_graph is not None:
        warm_graph.prepare(steps)
        ms_warm = timed_steps(warm_graph.run, steps) / steps
    else:
        ms_warm = timed_steps(lambda n: [step(m, cfg, sets[0]) for _ in range(n)], steps) / steps

    # checksum gather: outside every timed region
    checksum = float(sets[0].dq.float().abs().sum().item())
    if world > 1:
        t = torch.tensor([checksum], device=device)
        parts = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        checksum = [float(p.item()) for p in parts]

    # per-kernel device times (same loop, events between the kernels)
    kt = kernel_breakdown(m, cfg, sets, steps)
    # FLOPs per launch.  Credited (the metric's convention: forward 2 products over the causal half, backward 5):
    # the backward's 5 are split over its two kernels in the ratio of what they execute (dQ pass 3 products,
    # dK/dV pass 4: both recompute the scores), so the credited shares add up to the metric's FLOPs.
    gemm = cfg.fwd_flops() / 2.0
    executed = {"attn_fwd_kernel": 2 * gemm, "attn_bwd_dq_kernel": 3 * gemm, "attn_bwd_dkdv_kernel": 4 * gemm,
                "attn_bwd_onepass_kernel": 5 * gemm, "attn_bwd_prep_kernel": 0.0, "attn_bwd_dq_convert_kernel": 0.0}
    credited = {"attn_fwd_kernel": 2 * gemm, "attn_bwd_dq_kernel": 5 * gemm * 3 / 7, "attn_bwd_dkdv_kernel": 5 * gemm * 4 / 7,
                "attn_bwd_onepass_kernel": 5 * gemm, "attn_bwd_prep_kernel": 0.0, "attn_bwd_dq_convert_kernel": 0.0}
    dom = max(kt, key=kt.get)
    burst, sustained = float(peaks["bf16_tflops"]), float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))
    achieved = credited[dom] / (kt[dom] * 1e-3) / 1e12
    bwd_ms = sum(v for k, v in kt.items() if k != "attn_fwd_kernel")
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": burst, "unit": "TFLOP/s", "frac": achieved / burst,
        "traffic": NCU_TRAFFIC_BYTES.get(cfg.name, {}).get(dom) if cfg.B == inputs.CONFIGS[args.config].B else None,
        "peak_source": f"bf16_tflops (burst) of {peaks['_source']}: the timed region lasts milliseconds at full clocks; "
                       f"sustained {sustained}",
        "flops_per_launch": credited[dom], "ms_per_launch": kt[dom],
        "flops_convention": "credited: forward 2 products per score block, backward 5, the backward's split 3:4 over "
                            "the dQ and dK/dV passes",
        "executed": {"flops_per_launch": executed[dom], "achieved": executed[dom] / (kt[dom] * 1e-3) / 1e12,
                     "frac_of_burst": executed[dom] / (kt[dom] * 1e-3) / 1e12 / burst,
                     "frac_of_sustained": executed[dom] / (kt[dom] * 1e-3) / 1e12 / sustained},
        "kernels_ms": kt,
        "fwd": {"ms": kt["attn_fwd_kernel"], "tflops": cfg.fwd_flops() / (kt["attn_fwd_kernel"] * 1e-3) / 1e12,
                "frac_of_burst": cfg.fwd_flops() / (kt["attn_fwd_kernel"] * 1e-3) / 1e12 / burst},
        "bwd": {"ms": bwd_ms, "tflops": 2.5 * cfg.fwd_flops() / (bwd_ms * 1e-3) / 1e12,
                "frac_of_burst": 2.5 * cfg.fwd_flops() / (bwd_ms * 1e-3) / 1e12 / burst,
                "note": "kernels timed one by one with events between them; back to back they overlap a little"},
        "whole_step": {"achieved": value / world, "frac": value / world / burst, "frac_of_sustained": value / world / sustained,
                       "l2_warm_ms_per_step": ms_warm,
                       "l2_warm_tflops": flops_step / (ms_warm * 1e-3) / 1e12},
    }
    # the HBM roof beside the tensor roof: with L2-cold inputs a step cannot move fewer bytes than
    # forward q,k,v,o,lse and backward q,k,v,o,lse,dO,dq,dk,dv (BF16, FP32 lse)
    qb, kb = cfg.B * cfg.Hq * cfg.T * cfg.D * 2, cfg.B * cfg.Hkv * cfg.T * cfg.D * 2
    lb = cfg.B * cfg.Hq * cfg.T * 4
    min_bytes = (2 * qb + 2 * kb + lb) + (4 * qb + 4 * kb + lb)
    hbm_ms = min_bytes / (float(peaks["hbm_gbs"]) * 1e9) * 1e3
    roofline["hbm_roof"] = {"min_bytes_per_step": min_bytes, "ms_per_step_at_hbm_peak": hbm_ms,
                            "tflops_ceiling": cfg.fwd_bwd_flops() / (hbm_ms * 1e-3) / 1e12,
                            "frac_of_ceiling": (value / world) / (cfg.fwd_bwd_flops() / (hbm_ms * 1e-3) / 1e12)}

    # strong scaling and the (batch, KV head) partition on hardware: every N > 1 run carries it
    strong = None
    if world > 1 and args.scaling == "weak":
        strong = {}
        for name in dict.fromkeys([cfg_full.name, "c3_300m_class"]):
            full = inputs.CONFIGS[name] if name != cfg_full.name else cfg_full
            t_full = ms_step if name == cfg_full.name else None
            strong[name] = measure_strong(m, full, rank, world, device, min(steps, 400), barrier, t_full,
                                          sets[0] if (name == cfg_full.name and rank == 0) else None)

    # end to end with host buffers
    near = bind_near_gpu(local_rank)
    e2e_steps = max(20, min(steps, 200))
    e2e_ms, copy_ms, h2d, d2h = e2e_measure(m, cfg, host_sets, e2e_steps, 5, device)
    if world > 1:
        t = torch.tensor([e2e_ms, copy_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms, copy_ms = float(t[0].item()), float(t[1].item())
    e2e = {"value": world * flops_step / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
           "copy_only_ms_per_step": copy_ms,
           "host_link_gbs_per_direction": h2d / (copy_ms * 1e-3) / 1e9,
           "host_cores_bound_near_gpu": near,
           "what": "pinned host q|k|v|dO -> device in one copy, forward, backward, O|dQ|dK|dV -> pinned host in one copy; "
                   "copies and compute of consecutive steps overlap on three streams; copy_only is the same loop "
                   "without the kernels (what the host link allows)"}
    m.device_status()

    cpu = ref_gpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline(cfg, seed0)
        ref_gpu = reference_gpu_paths(m, cfg, sets[0])

    if rank == 0:
        config = workload_config(cfg_full, world, args.scaling)
        run = {
            "launch": ("one round over the buffer sets captured in a CUDA graph and replayed" if launch_how == "graph"
                       else "every launch issued from Python"),
            "ms_per_step_by_launch": {k: v / steps for k, v in ms_by_launch.items()},
            "backward": ("two-pass (dQ pass, dK/dV pass): bit-reproducible" if BWD_MODE == "two_pass" else
                         "one-pass (row-vector kernel, fused kernel, dQ conversion): dQ summed by reduce-adds"),
            "buffer_sets": n_sets}
        line = {
            "metric": "causal_gqa_attn_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling,
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config, "run": run,
            "per_gpu_tflops": value / world,
            "pct_of_bf16_peak": {"burst": 100 * value / world / burst, "sustained": 100 * value / world / sustained,
                                 "source": peaks["_source"]},
            "clocks": clocks, "e2e": e2e, "gpu_launches": (3 if BWD_MODE == "two_pass" else 4) * steps, "roofline": roofline,
            "checksum_dq_abs_sum": checksum,
        }
        if strong is not None:
            line["strong"] = strong
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if ref_gpu is not None:
            line["reference_gpu"] = ref_gpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def measure_strong(m, full, rank, world, device, steps, barrier, t_full_ms, full_result):
    """The whole configuration `full` split over the ranks by (batch, KV head) units (sharding.unit_range): every
    rank runs its contiguous block, nothing is exchanged.  Device time of a step is the max over ranks; efficiency is
    against the time of the whole configuration on one GPU (t_full_ms, measured in this run when the configuration
    is the bench's own, else taken by rank 0 here).  Outside the timed region every rank's O, dQ, dK, dV are gathered
    over NCCL (sharding.gather_units) and rank 0 compares them, bit for bit, with its own run of the whole
    configuration."""
    import torch
    import torch.distributed as dist
    from modern_llm_v1_b200 import inputs, sharding

    seed = 20260002
    lo, hi = sharding.unit_range(full.units, rank, world)
    if (hi - lo) % full.Hkv or lo % full.Hkv:
        return {"skipped": f"{full.units} units do not split into whole batches over {world} ranks"}
    mine = dataclasses.replace(full, B=(hi - lo) // full.Hkv)
    host = [t.pin_memory() for t in inputs.make_train_inputs(full, seed, lo, hi)[:4]]
    one = BufferSet(mine, host, device)
    n_sets = max(2, int(2 * 126e6 // one.nbytes()) + 1)
    sets = [one] + [BufferSet(mine, host, device) for _ in range(n_sets - 1)]
    for i in range(3):
        step(m, mine, sets[i % n_sets])
    graphs = StepGraphs(lambda i: step(m, mine, sets[i % n_sets]), n_sets)
    graphs.prepare(steps)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    graphs.run(steps)
    e1.record()
    barrier()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    m.device_status()
    # the whole configuration on one GPU, for the efficiency and for the comparison
    ref = None
    if rank == 0:
        if full_result is None:
            hf = inputs.make_train_inputs(full, seed)[:4]
            fs = [BufferSet(full, hf, device) for _ in range(max(2, int(2 * 126e6 // (one.nbytes() * world)) + 1))]
            for s_ in fs[:2]:
                step(m, full, s_)
            gf = StepGraphs(lambda i: step(m, full, fs[i % len(fs)]), len(fs))
            gf.prepare(steps)
            torch.cuda.synchronize()
            e0.record()
            gf.run(steps)
            e1.record()
            torch.cuda.synchronize()
            t_full_ms = e0.elapsed_time(e1) / steps
            full_result = fs[0]
        ref = full_result
    tt = torch.tensor([t_full_ms if rank == 0 else 0.0], device=device)
    dist.broadcast(tt, 0)
    t_full_ms = float(tt.item())
    # verification gather (the only collective; not timed)
    g, T, D, Hkv = full.group, full.T, full.D, full.Hkv
    per_unit = lambda x, h: x.reshape(-1, Hkv, h, T, D).reshape(-1, h, T, D)
    ok, worst = True, 0.0
    for name, local, h in (("o", one.o, g), ("dq", one.dq, g), ("dk", one.dk, 1), ("dv", one.dv, 1)):
        got = sharding.gather_units(per_unit(local, h).contiguous(), full.units, rank, world)
        if rank == 0:
            want = per_unit(getattr(ref, name), h)
            same = torch.equal(got, want)
            ok = ok and same
            if not same:
                worst = max(worst, float((got.float() - want.float()).abs().max().item()))
    flops = full.fwd_bwd_flops()
    return {"ms_per_step": ms, "tflops_total": flops / (ms * 1e-3) / 1e12,
            "tflops_per_gpu": flops / (ms * 1e-3) / 1e12 / world, "one_gpu_ms_per_step": t_full_ms,
            "speedup": t_full_ms / ms, "efficiency": t_full_ms / ms / world,
            "units_per_gpu": hi - lo, "query_tiles_per_gpu": (hi - lo) * g * ((T + 127) // 128),
            "limiter": strong_limiter((hi - lo) * g * ((T + 127) // 128)),
            "parity_ok": bool(ok) if rank == 0 else None, "parity_max_abs_diff": worst,
            "parity": "O, dQ, dK, dV of every unit gathered over NCCL == the whole configuration run on rank 0, bit for bit"}


def strong_limiter(items):
    """Names what keeps a strong-scaling split below linear, from the forward / dQ-pass items left per GPU."""
    base = "per-kernel start-up and tail (about 6 us each of three kernels) do not shrink with the work"
    if items < 296:
        return f"{base}, and {items} forward items do not fill the 296 CTA slots of a GPU"
    if items < 4 * 296:
        return (f"{base}, and {items} forward items are {items / 296:.1f} per CTA slot: lists of one to three items "
                "cannot be balanced as evenly as the whole configuration's")
    return base


def reference_gpu_paths(m, cfg, s):
    """The reference's own two GPU attention paths (its per-row flash kernels and its cuBLAS path with
    repeat_kv_heads / accumulate_kv_grads, compiled unchanged for sm_100a into oracle/_ref/libref_gpu.so where the
    reference tree was present at build time) timed beside this library: forward + backward at the configuration, and
    forward / backward at the shapes of the reference's own benchmark (llm/tests/bench_flash_attn.cu:98-101:
    B' = 8 heads, D = 64, T = 128..512; B' = 4 at T = 1024).  Part of the CPU/reference baseline leg: never on the
    product path, never in a timed region of the arm."""
    import ctypes

    import torch

    path = os.path.join(ROOT, "oracle", "_ref", "libref_gpu.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/libref_gpu.so was not built (it needs the reference tree at build time)"}
    L = ctypes.CDLL(path)
    L.ref_gpu_attention.argtypes = [ctypes.c_int] + [ctypes.c_void_p] * 9 + [ctypes.c_int] * 5
    L.ref_gpu_attention.restype = ctypes.c_int

    def ms_of(fn, reps):
        fn()
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def ref_call(which, q, k, v, do, B, T, Hq, Hkv, D):
        qf, kf, vf = q.float().contiguous(), k.float().contiguous(), v.float().contiguous()
        dof = do.float().contiguous() if do is not None else None
        o, dq, dk, dv = torch.empty_like(qf), torch.empty_like(qf), torch.empty_like(kf), torch.empty_like(vf)
        lse = torch.zeros(B, Hq, T, device=q.device)

        def run():
            rc = L.ref_gpu_attention(which, qf.data_ptr(), kf.data_ptr(), vf.data_ptr(),
                                     dof.data_ptr() if dof is not None else None, o.data_ptr(), lse.data_ptr(), dq.data_ptr(),
                                     dk.data_ptr(), dv.data_ptr(), B, T, Hq, Hkv, D)
            if rc != 0:
                raise RuntimeError("the reference's GPU attention threw")
        return run

    out = {"what": "the reference's GPU paths compiled unchanged for sm_100a (FP32), its own GQA copies and allocations "
                   "included, on this GPU"}
    B, T, Hq, Hkv, D = cfg.B, cfg.T, cfg.Hq, cfg.Hkv, cfg.D
    flash = ms_of(ref_call(0, s.q, s.k, s.v, s.do, B, T, Hq, Hkv, D), 2)
    cublas = ms_of(ref_call(1, s.q, s.k, s.v, s.do, B, T, Hq, Hkv, D), 2)
    ours = ms_of(lambda: step(m, cfg, s), 20)
    out[cfg.name] = {"flash_ms": flash, "cublas_ms": cublas, "this_library_ms": ours}
    table = []
    for Bh, Tb in ((8, 128), (8, 256), (8, 512), (4, 1024)):
        g = torch.Generator().manual_seed(Tb)
        q, k, v, do = ((torch.rand(Bh, 1, Tb, 64, generator=g) * 2 - 1).bfloat16().to(s.q.device) for _ in range(4))
        o, lse = torch.empty_like(q), torch.empty(Bh, 1, Tb, device=q.device)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(q), torch.empty_like(q)
        row = {"B_heads": Bh, "T": Tb, "D": 64}
        for which, nm in ((0, "flash"), (1, "naive")):
            row[f"{nm}_fwd_ms"] = ms_of(ref_call(which, q, k, v, None, Bh, Tb, 1, 1, 64), 8)
            row[f"{nm}_fwd_bwd_ms"] = ms_of(ref_call(which, q, k, v, do, Bh, Tb, 1, 1, 64), 8)
        row["this_library_fwd_ms"] = ms_of(lambda: m.flash_attn_forward_gqa(q, k, v, o, lse, Bh, Tb, 1, 1, 64), 20)
        row["this_library_bwd_ms"] = ms_of(
            lambda: m.flash_attn_backward_gqa(q, k, v, o, lse, do, dq, dk, dv, Bh, Tb, 1, 1, 64, mode="two_pass"), 20)
        table.append(row)
    out["reference_bench_shapes"] = table
    m.device_status()
    return out


if __name__ == "__main__":
    main()
