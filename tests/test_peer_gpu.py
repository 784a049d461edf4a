"""stafb_allreduce_adam: gradient averaging + Adam as one kernel over NVLink peer memory.

world 1 (any GPU box): the fused kernel equals stafb_adam_step_dev on the same gradient.
world 2 (needs two GPUs, skipped otherwise): two processes, one GPU each; every step of the fused exchange is
compared with all_reduce(grad) + Adam on a twin model, and the replicas of theta must stay bit-identical
across the ranks.  NVLS is switched off for the NCCL twin, as on any test that could lose a rank.
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


def _setup(dev, seeds):
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", seeds)
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape, dtype=np.float32)
    el, fl = synth.labels(len(seeds), shape.N)
    mk = lambda: StafModel(shape, CFG, theta, emb, 2, dtype=torch.float32, device=dev)
    d = [torch.as_tensor(a.astype(np.float32)).to(dev) for a in (pos, box, el, fl)]
    return mk, d


def test_world_one_equals_adam_step():
    from alphanesgpu_b200.dist import PeerExchange
    dev = torch.device("cuda:0")
    mk, d = _setup(dev, [2000, 2001, 2002, 2003])
    a, b = mk(), mk()
    px = PeerExchange(a)
    for k in range(4):
        sl = slice(2 * (k & 1), 2 * (k & 1) + 2)
        a.use_grad(px.grad(k & 1))
        a.loss_and_grad(*(t[sl] for t in d))
        b.grad.copy_(px.grad(k & 1))  # the same gradient for both updates (float atomics are not reproducible)
        px.allreduce_adam(a, k & 1, 1e-3)
        b.adam_update_dev(1e-3)
    torch.cuda.synchronize()
    assert px.status() == 0
    # same gradient, same formula, two kernels: equal up to the compiler's choice of fused multiply-adds
    # (an ulp or two of parameters of magnitude ~1)
    assert float((a.theta - b.theta).abs().max()) <= 5e-7
    assert int(a.step_d[0]) == 4
    px.close()
    a.close()
    b.close()


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from alphanesgpu_b200.dist import PeerExchange
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    mk, d = _setup(dev, [2100 + 4 * rank + i for i in range(4)])  # every rank its own frames
    a, b = mk(), mk()
    px = PeerExchange(a)
    worst = 0.0
    for k in range(6):
        sl = slice(2 * (k & 1), 2 * (k & 1) + 2)
        a.use_grad(px.grad(k & 1))
        a.loss_and_grad(*(t[sl] for t in d))
        b.grad.copy_(px.grad(k & 1))  # twin: the same local gradient, summed by NCCL, then the plain Adam kernel
        px.allreduce_adam(a, k & 1, 1e-3)
        dist.all_reduce(b.grad)
        b.adam_update_dev(1e-3, grad_scale=1.0 / world)
        torch.cuda.synchronize()
        worst = max(worst, float((a.theta - b.theta).abs().max()))
        b.theta.copy_(a.theta)
    status = px.status()
    mine = a.theta.clone()
    other = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(other, mine)
    same = all(torch.equal(o, mine) for o in other)
    q.put((rank, status, worst, same))
    px.close()
    a.close()
    b.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_world_two_matches_allreduce_then_adam():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, status, worst, same in got:
        assert status == 0, (rank, status)
        assert worst <= 5e-7, (rank, worst)  # same sums (a + b in either order), two kernels
        assert same, rank  # rank-ordered sums: the replicas do not drift


def _late_peer_worker(rank, world, port, q):
    """The wait bound is set to zero and rank 1 arrives late: rank 0's kernel must give up, record the status
    and leave theta untouched, and the context must stay usable (no trap, no hang)."""
    import time
    import torch.distributed as dist
    from alphanesgpu_b200.dist import PeerExchange
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", STAFB_PEER_WAIT_MS="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    mk, d = _setup(dev, [2200 + 4 * rank + i for i in range(4)])
    a = mk()
    px = PeerExchange(a)
    before = a.theta.clone()
    a.use_grad(px.grad(0))
    a.loss_and_grad(*(t[0:2] for t in d))
    torch.cuda.synchronize()
    dist.barrier()
    if rank == 1:
        time.sleep(0.5)  # rank 0 launches first and finds nothing from its peer
    px.allreduce_adam(a, 0, 1e-3)
    torch.cuda.synchronize()
    status = px.status()
    untouched = bool(torch.equal(a.theta, before))
    if rank == 0:  # the launch that gave up changed nothing at all: moments and step count included
        untouched = untouched and int(a.step_d[0]) == 0 and float(a.adam_m.abs().max()) == 0.0 \
            and float(a.adam_v.abs().max()) == 0.0
    e, f = a.energy_force(d[0][0:2], d[1][0:2])  # the context still works
    usable = bool(torch.isfinite(e).all())
    q.put((rank, status, untouched, usable))
    px.close()
    a.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_late_peer_gives_a_status_not_a_hang():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_late_peer_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict((r[0], r[1:]) for r in (q.get(timeout=240) for _ in range(2)))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    status, untouched, usable = got[0]
    assert status == 9 and untouched and usable  # STAFB_ERR_PEER_TIMEOUT on the rank that waited
    assert got[1][2]


def test_eight_emulated_ranks_on_one_gpu():
    """The kernel's indexing for a full node: eight ranks emulated on one GPU.  Their kernels run one after the
    other, so all of them store to their peers first and wait afterwards (no kernel may wait for another on the same
    GPU); what is checked is that each rank finds the right eight gradients, sums them in rank order and that all
    replicas end up bit-identical."""
    import ctypes as C
    from alphanesgpu_b200 import _lib
    from alphanesgpu_b200.dist import _DevArray
    from alphanesgpu_b200.ops import Context
    L = _lib.lib()
    dev = torch.device("cuda:0")
    ctx = Context(CFG["Rc"], CFG["nr"], CFG["na"], 96, CFG["Rs"], CFG["Ra"], 1, torch.float32, dev)
    W, n, lr = 8, 3001, 1e-3
    hs = (C.c_void_p * W)()
    for r in range(W):
        h = C.c_void_p()
        _lib.check(L.stafb_peer_create(ctx.h, r, W, n, C.byref(h)), "stafb_peer_create")
        hs[r] = h
    gen = torch.Generator(device="cpu").manual_seed(5)
    grads = [torch.randn(n, generator=gen).to(dev) for _ in range(W)]
    theta0 = torch.randn(n, generator=gen).to(dev)
    state = []
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    for r in range(W):
        _lib.check(L.stafb_peer_connect_local(hs[r], hs), "stafb_peer_connect_local")
        for par in (0, 1):
            g = torch.as_tensor(_DevArray(L.stafb_peer_grad(hs[r], par), n, torch.float32), device=dev)
            g.copy_(grads[r] if par == 0 else -grads[r])
        state.append(dict(theta=theta0.clone(), m=torch.zeros(n, device=dev), v=torch.zeros(n, device=dev),
                          step=torch.zeros(2, dtype=torch.int32, device=dev)))
    torch.cuda.synchronize()
    p = lambda t: C.c_void_p(t.data_ptr())
    for phase in (1, 2):  # every rank stores to its peers, then every rank waits and updates
        for r in range(W):
            s = state[r]
            _lib.check(L.stafb_allreduce_adam_phase(ctx.h, hs[r], stream, 0, p(s["theta"]), p(s["m"]), p(s["v"]), lr,
                                                    0.9, 0.999, 1e-7, p(s["step"]), phase), "stafb_allreduce_adam_phase")
    torch.cuda.synchronize()
    g = torch.zeros(n, device=dev)
    for r in range(W):
        g = g + grads[r]  # rank order, float32
    g = g / W
    m, v = 0.1 * g, 0.001 * g * g
    lr_t = lr * np.sqrt(1 - 0.999) / (1 - 0.9)
    want = theta0 - lr_t * m / (torch.sqrt(v) + 1e-7)
    for r in range(W):
        assert L.stafb_peer_status(hs[r]) == 0
        assert int(state[r]["step"][0]) == 1
        assert torch.equal(state[r]["theta"], state[0]["theta"]), r
    assert torch.allclose(state[0]["theta"], want, rtol=2e-6, atol=2e-7)
    for r in range(W):
        L.stafb_peer_destroy(hs[r])
    ctx.close()


def test_a_launch_that_gives_up_changes_nothing():
    """Peers that store nothing and a zero bound: every block of the launch gives up together (the decision is
    taken once per launch), so theta, both moments and the step counter are bit-identical to before, the status
    says STAFB_ERR_PEER_TIMEOUT and the next launch - with the peers' gradients in place - applies its update in
    full."""
    import ctypes as C
    from alphanesgpu_b200 import _lib
    from alphanesgpu_b200.dist import _DevArray
    from alphanesgpu_b200.ops import Context
    L = _lib.lib()
    dev = torch.device("cuda:0")
    ctx = Context(CFG["Rc"], CFG["nr"], CFG["na"], 96, CFG["Rs"], CFG["Ra"], 1, torch.float32, dev)
    W, n, lr = 4, 70001, 1e-3  # 274 blocks: more than one per SM
    hs = (C.c_void_p * W)()
    for r in range(W):
        h = C.c_void_p()
        _lib.check(L.stafb_peer_create(ctx.h, r, W, n, C.byref(h)), "stafb_peer_create")
        hs[r] = h
    gen = torch.Generator(device="cpu").manual_seed(11)
    grads = [torch.randn(n, generator=gen).to(dev) for _ in range(W)]
    for r in range(W):
        _lib.check(L.stafb_peer_connect_local(hs[r], hs), "stafb_peer_connect_local")
        _lib.check(L.stafb_peer_set_wait_ms(hs[r], 0), "stafb_peer_set_wait_ms")
        g = torch.as_tensor(_DevArray(L.stafb_peer_grad(hs[r], 0), n, torch.float32), device=dev)
        g.copy_(grads[r])
    theta0 = torch.randn(n, generator=gen).to(dev)
    m0, v0 = torch.rand(n, generator=gen).to(dev), torch.rand(n, generator=gen).to(dev)
    theta, m, v = theta0.clone(), m0.clone(), v0.clone()
    step = torch.zeros(2, dtype=torch.int32, device=dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())
    call = lambda: _lib.check(L.stafb_allreduce_adam(ctx.h, hs[0], stream, 0, p(theta), p(m), p(v), lr, 0.9, 0.999,
                                                     1e-7, p(step)), "stafb_allreduce_adam")
    call()  # no peer has published anything
    torch.cuda.synchronize()
    assert L.stafb_peer_status(hs[0]) == 9
    assert torch.equal(theta, theta0) and torch.equal(m, m0) and torch.equal(v, v0)
    assert step.tolist() == [0, 0]
    zeros = [torch.zeros(2, dtype=torch.int32, device=dev) for _ in range(W)]
    for r in range(1, W):  # now the peers store their gradients of step 1 (phase 1 touches nothing else)
        _lib.check(L.stafb_allreduce_adam_phase(ctx.h, hs[r], stream, 0, p(theta0), p(m0), p(v0), lr, 0.9, 0.999, 1e-7,
                                                p(zeros[r]), 1), "stafb_allreduce_adam_phase")
    call()  # the same step again, now with every peer's gradient in place
    torch.cuda.synchronize()
    assert step.tolist() == [1, 0]
    g = torch.zeros(n, device=dev)
    for r in range(W):
        g = g + grads[r]
    g = g / W
    mm, vv = 0.9 * m0 + 0.1 * g, 0.999 * v0 + 0.001 * g * g
    want = theta0 - (lr * np.sqrt(1 - 0.999) / (1 - 0.9)) * mm / (torch.sqrt(vv) + 1e-7)
    assert torch.allclose(theta, want, rtol=2e-6, atol=2e-7)
    for r in range(W):
        L.stafb_peer_destroy(hs[r])
    ctx.close()
