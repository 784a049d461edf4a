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


def _connect_worker(rank, world, port, q, failing):
    """connect_collectively with stand-ins for the library calls: rank `failing` cannot create its block
    (or, failing = -2, rank 1 cannot map a peer's block); every rank must raise, and release what it made."""
    import ctypes as C
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from alphanesgpu_b200.dist import connect_collectively
    log = []

    def create():
        if rank == failing:
            raise RuntimeError("no memory on rank %d" % rank)
        log.append("create")
        return 1000 + rank

    def get_handle(h, buf):
        C.memmove(buf, bytes([rank]) * 64, 64)
        return 0

    def connect(h, blob):
        assert len(blob) == 64 * world and blob[64 * rank] == rank
        log.append("connect")
        return 5 if (failing == -2 and rank == 1) else 0  # a non-zero status of the library raises

    def destroy(h):
        log.append("destroy")

    try:
        h = connect_collectively(create, get_handle, connect, destroy, world, torch.device("cpu"), None, "fake")
        q.put((rank, "ok", h, log))
    except RuntimeError as exc:
        q.put((rank, "raised", str(exc), log))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("failing", [-1, 1, -2])
def test_peer_memory_set_up_fails_on_every_rank_alike(failing):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_connect_worker, args=(r, 2, port, q, failing)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict((r[0], r[1:]) for r in (q.get(timeout=120) for _ in range(2)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    if failing == -1:
        assert got[0][0] == "ok" and got[1][0] == "ok" and got[0][1] == 1000 and got[1][1] == 1001
        assert got[0][2] == ["create", "connect"]
    else:
        assert got[0][0] == "raised" and got[1][0] == "raised"
        for r in (0, 1):
            made = "create" in got[r][2]
            assert ("destroy" in got[r][2]) == made  # whatever was created is released
        if failing == 1:
            assert "connect" not in got[0][2]  # nobody maps anything when a block is missing
