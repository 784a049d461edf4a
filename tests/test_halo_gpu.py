"""stafb_halo_*: the slab decomposition's halo exchange over peer memory (positions stored into the neighbours'
atom arrays, ghost forces stored back, energies summed in rank order).

One GPU: 2, 3 and 4 ranks emulated in one process - every rank its own model and halo block, the blocks connected
directly; all ranks' pushes are issued before any wait and all returns before any collect, so that no kernel ever
waits for a kernel behind it on the same GPU.  The result must equal the evaluation of the whole box (the
reference's test/test-lammps-dd-parity: 1 vs 2 vs 4 ranks), over several evaluations with moving atoms and a ghost
set that is re-chosen in between - by the device-side planner (mailboxes in the peers' memory), by the same planner
run one evaluation ahead, and by a plan made on the host.
Two GPUs (skipped otherwise): two processes, CUDA IPC, the evaluation replayed as a CUDA graph.
A wait that runs out (a flag nobody sets) must leave a status and a usable context.
"""
import os
import socket

import numpy as np
import pytest
import torch

from alphanesgpu_b200 import synth
from conftest import CFG

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _system(dtype, dev, seed=3100):
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water768", [seed])
    shape = synth.baseline_shape(tipos)
    npdt = np.float32 if dtype == torch.float32 else np.float64
    theta, emb = synth.init_params(shape, dtype=npdt)
    gpos = torch.as_tensor(pos.reshape(-1, 3).astype(npdt)).to(dev)
    gtypes = torch.as_tensor(shape.type_map.astype(np.int32)).to(dev)
    full = StafModel(shape, CFG, theta, emb, 1, dtype=dtype, device=dev)
    return shape, theta, emb, box[0], gpos, gtypes, full


def _rank_model(shape, theta, emb, dtype, dev, cap):
    from alphanesgpu_b200.model import StafModel
    from alphanesgpu_b200.params import ModelShape
    sh = ModelShape(nt=shape.nt, tipos=[1] * shape.nt, Fr=shape.Fr, Fa=shape.Fa, widths=shape.widths)
    return StafModel(sh, CFG, theta, emb, 1, dtype=dtype, device=dev, n_max=cap)


def _evaluate_emulated(doms):
    for d in doms:
        d.phase_push()
    for d in doms:
        d.phase_wait()
    for d in doms:
        d.phase_eval_return()
    for d in doms:
        d.phase_collect()


@pytest.mark.parametrize("world,mode", [(2, "device"), (3, "device"), (4, "device"), (3, "host"), (3, "early"),
                                        (2, "early")])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.float64, 1e-12)])
def test_emulated_ranks_equal_the_whole_box(world, mode, dtype, tol):
    from alphanesgpu_b200.slab import PeerSlabDomain
    dev = torch.device("cuda:0")
    shape, theta, emb, box6, gpos, gtypes, full = _system(dtype, dev)
    N = shape.N
    cap = N
    skin = 0.2 if world == 2 else 0.3  # two ranks: the slab must be two halo widths wide (9.8 A >= 2 * 4.7 A)
    models = [_rank_model(shape, theta, emb, dtype, dev, cap) for _ in range(world)]
    doms = [PeerSlabDomain(models[r], box6, CFG["Rc"], r, world, cap_atoms=cap, cap_face=cap, skin=skin, local=True)
            for r in range(world)]
    PeerSlabDomain.connect_local(doms)
    own = [d.set_owned_from_global(gpos, gtypes) for d in doms]
    assert sum(len(o) for o in own) == N
    gen = torch.Generator(device="cpu").manual_seed(5)
    boxt = torch.as_tensor(np.asarray(box6)[None].astype(np.float64)).to(dev, dtype)
    for k in range(5):
        if k == 0 or (k == 3 and mode != "early"):
            # ghost sets re-chosen: on the device, or on the host and installed with stafb_halo_set_plan
            (PeerSlabDomain.plan_local_explicit if mode == "host" else PeerSlabDomain.plan_local)(doms)
        early = mode == "early" and k == 2
        if early:
            # the plan of evaluation 3 onwards prepared ahead of evaluation 2, which still runs under the old one
            for which in range(3):
                for d in doms:
                    d._plan_launch(which)
        _evaluate_emulated(doms)
        if early:
            for d in doms:
                d._plan_finish()
        torch.cuda.synchronize()
        for d in doms:
            d.check()
        e_full, f_full = full.energy_force(gpos.reshape(1, -1), boxt)
        f_full = f_full.reshape(N, 3)
        scale = float(f_full.abs().max())
        for r, d in enumerate(doms):
            n = d.pos.shape[0]
            assert float((d.force[:n] - f_full[own[r]]).abs().max()) <= tol * scale, (k, r)
            assert abs(float(d.e_total[0]) - float(e_full[0])) <= 10 * tol * abs(float(e_full[0])), (k, r)
            assert float(d.e_total[0]) == float(doms[0].e_total[0])  # summed in rank order: the same bits everywhere
        # the atoms move by at most 0.02 A per coordinate and evaluation: well inside half the skin between plans
        gpos += ((torch.rand(N, 3, generator=gen, dtype=torch.float64) - 0.5) * 0.04).to(dev, dtype)
        for r, d in enumerate(doms):
            d.pos.copy_(gpos[own[r]])
    for d in doms:
        d.close()
    for m in models:
        m.close()
    full.close()


def test_a_wait_that_runs_out_leaves_a_status_and_a_usable_context():
    from alphanesgpu_b200 import _lib
    from alphanesgpu_b200.slab import PeerSlabDomain
    dev = torch.device("cuda:0")
    dtype = torch.float32
    shape, theta, emb, box6, gpos, gtypes, full = _system(dtype, dev)
    world, cap = 3, shape.N
    models = [_rank_model(shape, theta, emb, dtype, dev, cap) for _ in range(world)]
    doms = [PeerSlabDomain(models[r], box6, CFG["Rc"], r, world, cap_atoms=cap, cap_face=cap, local=True)
            for r in range(world)]
    PeerSlabDomain.connect_local(doms)
    for d in doms:
        d.set_owned_from_global(gpos, gtypes)
    PeerSlabDomain.plan_local(doms)
    d0 = doms[0]
    d0.set_wait_ms(1)
    # rank 0 alone: nobody publishes positions or forces for it
    d0.phase_push()
    d0.phase_wait()
    d0.phase_collect()
    torch.cuda.synchronize()
    assert _lib.lib().stafb_halo_status(d0.h) == 9  # STAFB_ERR_PEER_TIMEOUT
    with pytest.raises(_lib.StafbError):
        d0.check()
    # the device is still there and the other ranks' evaluation number has not moved
    boxt = torch.as_tensor(np.asarray(box6)[None].astype(np.float32)).to(dev)
    e, f = full.energy_force(gpos.reshape(1, -1), boxt)
    assert torch.isfinite(e).all() and torch.isfinite(f).all()
    for d in doms:
        d.close()
    for m in models:
        m.close()
    full.close()


def _worker(rank, world, port, q, halo_every=4, use_graph=True):
    import torch.distributed as dist
    from alphanesgpu_b200.slab import PeerSlabDomain
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    dtype = torch.float32
    shape, theta, emb, box6, gpos, gtypes, full = _system(dtype, dev)
    N = shape.N
    model = _rank_model(shape, theta, emb, dtype, dev, N)
    dom = PeerSlabDomain(model, box6, CFG["Rc"], rank, world, cap_atoms=N, cap_face=N, skin=0.2,
                         halo_every=halo_every, use_graph=use_graph)
    own = dom.set_owned_from_global(gpos, gtypes)
    boxt = torch.as_tensor(np.asarray(box6)[None].astype(np.float32)).to(dev)
    worst = 0.0
    gen = torch.Generator(device="cpu").manual_seed(7)  # the same walk on both ranks
    for k in range(9):  # halo_every 4: plans for k = 0, 4, 8; eager, captured, replayed evaluations in between
        e, f = dom.step()
        torch.cuda.synchronize()
        e_full, f_full = full.energy_force(gpos.reshape(1, -1), boxt)
        f_full = f_full.reshape(N, 3)
        worst = max(worst, float((f - f_full[own]).abs().max() / f_full.abs().max()),
                    abs(float(e[0]) - float(e_full[0])) / abs(float(e_full[0])))
        gpos += ((torch.rand(N, 3, generator=gen, dtype=torch.float64) - 0.5) * 0.04).to(dev, dtype)
        dom.pos.copy_(gpos[own])
    dom.check()
    es = [None] * world
    dist.all_gather_object(es, float(e[0]))
    dom.close()
    model.close()
    full.close()
    q.put((rank, worst, es))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("halo_every,use_graph", [(4, True), (1, False)])
def test_two_processes(halo_every, use_graph):
    """Two ranks on two GPUs over CUDA IPC: ghost sets re-chosen every fourth evaluation with the evaluations in
    between replayed as a CUDA graph, and re-chosen before every evaluation (each plan prepared one evaluation
    ahead) with plain launches."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, halo_every, use_graph)) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, worst, es in out:
        assert worst <= 3e-6, (rank, worst)
        assert es[0] == es[1]
