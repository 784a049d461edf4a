"""gloo tests (CPU, world size 2 and 3) of the slab-decomposition host logic: halo selection, the two
face messages, the reverse force messages and the energy all-reduce.  The per-rank evaluation is a small
pair potential written in torch so that nothing here needs a GPU; the decomposed result must equal the
single-domain one - the reference's domain-decomposition parity check (test/test-lammps-dd-parity)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from alphanesgpu_b200.slab import SlabDomain, slab_of

L, RC = 12.0, 2.5


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def toy_compute(pos_all, type_all, n_owned, plan_changed=True):
    """E = 1/2 sum over owned centres i and all atoms j of (1 + t_i t_j/4)(1 - r/RC)^2 inside RC, minimum image."""
    p = pos_all.clone().requires_grad_(True)
    d = p[:n_owned, None, :] - p[None, :, :]
    d = d - torch.round(d / L) * L
    r = torch.sqrt((d * d).sum(-1) + 1e-30)
    mask = (r < RC) & (r > 1e-9)
    w = 1.0 + 0.25 * type_all[:n_owned, None].double() * type_all[None, :].double()
    e = 0.5 * (torch.where(mask, w * (1.0 - r / RC) ** 2, torch.zeros_like(r))).sum()
    f = -torch.autograd.grad(e, p)[0]
    return e.detach().reshape(1), f


def _config(seed=7, n=400):
    r = np.random.default_rng(seed)
    pos = r.uniform(-3.0, L + 3.0, size=(n, 3))  # some atoms outside the primary cell on purpose
    types = r.integers(0, 2, size=n).astype(np.int32)
    return torch.as_tensor(pos), torch.as_tensor(types)


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pos, types = _config()
    dom = SlabDomain(toy_compute, [L, 0, 0, L, 0, L], RC, rank, world)
    idx = dom.set_owned_from_global(pos, types)
    assert dom.types.tolist() == sorted(dom.types.tolist())  # species-sorted
    e, f = dom.step()
    e2, f2 = dom.step(rebuild=False)  # a second evaluation reuses the halo plan: only positions travel
    assert torch.equal(e, e2) and torch.equal(f, f2)
    q.put((rank, idx.numpy(), float(e), f.numpy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_slab_decomposition_matches_single_domain(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    pos, types = _config()
    e_ref, f_ref = toy_compute(pos, types, pos.shape[0])
    f = np.zeros((pos.shape[0], 3))
    seen = np.zeros(pos.shape[0], int)
    for rank, idx, e, fr in got:
        assert abs(e - float(e_ref)) <= 1e-12 * abs(float(e_ref))  # every rank holds the total
        f[idx] = fr
        seen[idx] += 1
    assert np.all(seen == 1)  # every atom is owned exactly once
    assert np.abs(f - f_ref.numpy()).max() <= 1e-12 * np.abs(f_ref.numpy()).max()


def test_slab_of_wraps_any_image():
    z = torch.tensor([-0.1, 0.0, 3.9, 4.0, 11.99, 12.0, 25.0])
    assert slab_of(z, 12.0, 3).tolist() == [2, 0, 0, 1, 2, 0, 0]


def test_slab_too_thin_is_rejected():
    with pytest.raises(ValueError):
        SlabDomain(toy_compute, [4.0, 0, 0, 4.0, 0, 4.0], 2.5, 0, 2)
