"""World-size-2 gloo tests (CPU) of the data-parallel host logic.  Per-rank gradients come from the
oracle, so what is tested is the sharding, the single all-reduce and the 1/world scaling."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from alphanesgpu_b200 import synth
from alphanesgpu_b200.dist import HostWatchdog, allreduce_sum_, broadcast_params_, shard_indices
from conftest import CFG


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle
    oracle.set_threads(2)
    pos, box, tipos = synth.water_frames("water96", [1000, 1001, 1002, 1003])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape)
    if rank != 0:
        theta = theta * 0  # must be overwritten by the broadcast
    th = broadcast_params_(torch.as_tensor(theta)).numpy()
    el, fl = synth.labels(4, shape.N)
    idx = shard_indices(4, rank, world)
    r = oracle.energy_force_grad(CFG, shape.desc(), pos[idx], box[idx], shape.type_map, th, emb, np.float64,
                                 with_grad=True, e_label=el[idx], f_label=fl[idx], pb=0.0)
    g = torch.as_tensor(r["grad"].copy())
    allreduce_sum_(g)
    g /= world
    if rank == 0:
        full = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, th, emb, np.float64,
                                        with_grad=True, e_label=el, f_label=fl, pb=0.0)
        q.put((idx.tolist(), float(np.abs(g.numpy() - full["grad"]).max() / np.abs(full["grad"]).max())))
    dist.barrier()
    dist.destroy_process_group()


def test_sharded_gradient_mean_equals_global_batch_gradient():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    idx, err = q.get(timeout=300)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert idx == [0, 2]  # idx[rank::world]
    assert err < 1e-12


def test_shard_indices_equal_counts():
    for n, w in ((64, 8), (10, 4), (7, 2)):
        parts = [shard_indices(n, r, w) for r in range(w)]
        assert len({len(p) for p in parts}) == 1
        assert len(set(np.concatenate(parts).tolist())) == sum(len(p) for p in parts)


def _wd_worker(rank, world, port, q):
    store = dist.TCPStore("127.0.0.1", port, world, rank == 0, timeout=__import__("datetime").timedelta(seconds=20))
    wd = HostWatchdog(store, rank, world, timeout_s=1.0)
    wd.beat(1)
    wd.check(1)  # both ranks publish step 1
    if rank == 1:
        q.put("rank1 leaves between steps")
        return  # a rank that never joins step 2 (it exits cleanly between steps)
    wd.beat(2)
    try:
        wd.check(2)
        q.put("no error")
    except RuntimeError as e:
        q.put("detected: %s" % e)


def test_host_watchdog_detects_missing_rank_without_hanging():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_wd_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    msgs = [q.get(timeout=60), q.get(timeout=60)]
    for p in procs:
        p.join(timeout=30)
    assert any(m.startswith("detected") and "[1]" in m for m in msgs), msgs
