"""The N>1 path on CPU: two gloo ranks each run the oracle on their (batch, KV head)
shard; the gathered result must equal the unsharded run.  No collective is part of the
data path, only of this verification."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from modern_llm_v1_b200 import inputs, sharding
from oracle import attn_oracle as ao

CFG = inputs.AttnConfig("gloo", 3, 24, 6, 2, 16)  # 6 units; world 2 -> 3 + 3, world 4 -> 2,2,1,1
SEED = 11


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ao.set_num_threads(1)
    lo, hi = sharding.unit_range(CFG.units, rank, world)
    # one unit at a time: [1, g, T, D] / [1, 1, T, D]
    outs = {k: [] for k in ("o", "dq", "dk", "dv")}
    for u in range(lo, hi):
        q, k, v, do, hq, hkv = inputs.make_train_inputs(CFG, SEED, u, u + 1)
        o, lse, dq, dk, dv = ao.attn_fwd_bwd_c(q.float().numpy(), k.float().numpy(), v.float().numpy(), do.float().numpy())
        for name, val in (("o", o), ("dq", dq), ("dk", dk), ("dv", dv)):
            outs[name].append(torch.from_numpy(val))
    full = {}
    for name, vals in outs.items():
        local = torch.cat(vals) if vals else torch.zeros((0,) + (CFG.group if name in ("o", "dq") else 1, CFG.T, CFG.D))
        full[name] = sharding.gather_units(local, CFG.units, rank, world)
    dist.barrier()
    if rank == 0:
        np.savez(os.path.join(out_dir, f"gathered_w{world}.npz"), **{k: v.numpy() for k, v in full.items()})
    dist.destroy_process_group()


def _run(world, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = np.load(os.path.join(str(tmp_path), f"gathered_w{world}.npz"))
    q, k, v, do, hq, hkv = inputs.make_train_inputs(CFG, SEED)
    o, lse, dq, dk, dv = ao.attn_fwd_bwd_c(q.float().numpy(), k.float().numpy(), v.float().numpy(), do.float().numpy())
    g, T, D = CFG.group, CFG.T, CFG.D
    # unit u = b * Hkv + hk owns query heads hk*g .. hk*g+g-1 of batch b
    assert ao.max_abs(got["o"], o.reshape(CFG.units, g, T, D)) == 0.0
    assert ao.max_abs(got["dq"], dq.reshape(CFG.units, g, T, D)) == 0.0
    assert ao.max_abs(got["dk"], dk.reshape(CFG.units, 1, T, D)) == 0.0
    assert ao.max_abs(got["dv"], dv.reshape(CFG.units, 1, T, D)) == 0.0


def test_two_ranks_equal_unsharded(tmp_path):
    _run(2, tmp_path)


def test_four_ranks_with_uneven_shards(tmp_path):
    _run(4, tmp_path)
