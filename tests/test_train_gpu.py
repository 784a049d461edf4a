"""GPU test of the training driver: its pipelined loop must produce, step by step, the losses of the same
sequence driven through the synchronous entry points, and write the reference's log files."""
import numpy as np
import pytest

from alphanesgpu_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_driver_matches_a_hand_written_loop(tmp_path):
    from alphanesgpu_b200 import train as T
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", list(range(1000, 1008)))
    el, fl = synth.labels(8, 96, seed=11)
    cfg = T.load_config(dict(buffer_stream_dim_tr=4, batch_size=2, number_of_epochs=2, displ_freq=3, Seed=5,
                             lr_dense_net="cosann 0.002 1 2.0 0.9 0.0", Radial_Buffer=60, Max_Angular_Neigh=60))
    data = dict(pos=pos, box=box, energy=el, force=fl, tipos=np.array(tipos))
    msgs = []
    res = T.train(cfg, str(tmp_path), data=data, log=msgs.append)
    rows = res["rows"]
    assert [r[0] for r in rows] == list(range(1, 9))          # 2 epochs x 2 buffers x 2 batches
    lines = open(tmp_path / "lcurve_notmean").read().split("\n")
    assert len([l for l in lines if l]) == 8 and len(open(tmp_path / "lr_step.dat").read().split()) == 8
    assert any("Time to elaborate 3 batch of 2 frames" in m for m in msgs)
    # the same sequence with the synchronous calls
    shape = res["shape"]
    theta, emb = T.init_params(shape, cfg, 5)
    m = StafModel(shape, res["geo"], theta, emb, 2, dtype=torch.float32, device="cuda:0")
    lr_of = T.build_learning_rate(cfg["lr_dense_net"], 2, 2, 4)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    step = 0
    for ep in range(2):
        for b in range(2):
            for k in range(2):
                sl = slice(4 * b + 2 * k, 4 * b + 2 * k + 2)
                l = m.loss_and_grad_host(f32(pos[sl]), f32(box[sl]), f32(el[sl]), f32(fl[sl]))
                m.adam_update_dev(lr_of(step))
                r = rows[step]
                assert r[5] == pytest.approx(lr_of(step))
                assert np.allclose([r[1], r[2], r[4], r[3]], l, rtol=2e-5), (step, r, l)
                step += 1
    torch.cuda.synchronize()
    assert np.allclose(res["theta"], m.theta.cpu().numpy(), rtol=1e-4, atol=1e-6)
    assert rows[-1][1] < rows[0][1]   # the loss went down
    m.close()


def test_driver_trains_on_energy_force_and_virial(tmp_path):
    """type_of_training: energy+force+virial (staf_train.py:291-294): the driver's rows against the same sequence
    of stafb_train_step_virial + Adam by hand; log columns step Loss_E Loss_F Loss_V Loss_Bound."""
    from alphanesgpu_b200 import train as T
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", list(range(1000, 1008)))
    el, fl = synth.labels(8, 96, seed=11)
    vl = np.random.default_rng(3).normal(0.0, 1.5, (8, 9))
    cfg = T.load_config(dict(buffer_stream_dim_tr=4, batch_size=2, number_of_epochs=2, displ_freq=3, Seed=5,
                             type_of_training="energy+force+virial", loss_virial_prefactor=0.5,
                             lr_dense_net="expdec 0.002 0.0000001"))
    data = dict(pos=pos, box=box, energy=el, force=fl, virial=vl, tipos=np.array(tipos))
    res = T.train(cfg, str(tmp_path), data=data, log=lambda *_: None)
    rows = res["rows"]
    assert [r[0] for r in rows] == list(range(1, 9))
    lines = [l for l in open(tmp_path / "lcurve_notmean").read().split("\n") if l]
    assert len(lines) == 8 and all(len(l.split()) == 5 for l in lines)
    shape = res["shape"]
    theta, emb = T.init_params(shape, cfg, 5)
    m = StafModel(shape, res["geo"], theta, emb, 2, dtype=torch.float32, device="cuda:0")
    lr_of = T.build_learning_rate(cfg["lr_dense_net"], 2, 2, 4)
    dv = lambda a: torch.as_tensor(np.ascontiguousarray(a, np.float32)).cuda()
    step = 0
    for ep in range(2):
        for b in range(2):
            for k in range(2):
                sl = slice(4 * b + 2 * k, 4 * b + 2 * k + 2)
                m.loss_and_grad_virial(dv(pos[sl]), dv(box[sl]), dv(el[sl]), dv(fl[sl]), dv(vl[sl]), pv=0.5)
                l = m.losses5.cpu().numpy().copy()
                m.adam_update_dev(lr_of(step))
                r = rows[step]
                assert np.allclose([r[1], r[2], r[4], r[3], r[6]], l, rtol=2e-5), (step, r, l)
                step += 1
    m.close()
    with pytest.raises(ValueError):
        T.train(cfg, str(tmp_path), data=dict(pos=pos, box=box, energy=el, force=fl, tipos=np.array(tipos)),
                log=lambda *_: None)


# ---- loss-curve parity of the data-parallel arm, the reference's none-vs-horovod check
# (test/test-training-pipeline/compare_distribute_lcurve.py; recorded bar
# test/test-training-pipeline/parity_distribute/float/summary.txt:1-12: 125 steps, rtol 1e-4, atol 1e-5)
RTOL, ATOL, STEPS = 1e-4, 1e-5, 125


def _parity_data(n_frames, seed0):
    pos, box, tipos = synth.water_frames("water96", list(range(seed0, seed0 + n_frames)))
    el, fl = synth.labels(n_frames, 96, seed=17)
    return dict(pos=pos, box=box, energy=el, force=fl, tipos=np.array(tipos))


def _curve(rows):
    return np.array([[r[2], r[3], r[4]] for r in rows])  # loss_e, loss_f, loss_bound per step


@pytest.mark.parametrize("precision", ["float", "double"])
def test_loss_curve_plain_adam_vs_exchange_kernel_on_one_rank(tmp_path, precision):
    """distribute none against the exchange arm with one rank (the reference runs `mpirun -np 1` for it): 125
    steps of the driver, Loss_E / Loss_F / Loss_Bound of every step."""
    from alphanesgpu_b200 import train as T
    data = _parity_data(50, 4000)
    base = dict(buffer_stream_dim_tr=10, batch_size=2, number_of_epochs=5, displ_freq=10, Seed=7, precision=precision,
                lr_dense_net="expdec 0.001 0.0000001")
    runs = {}
    for mode in ("allreduce", "peer_always"):
        d = tmp_path / mode
        d.mkdir()
        cfg = T.load_config(dict(base, grad_exchange=mode))
        runs[mode] = T.train(cfg, str(d), data=data, log=lambda *_: None)
        assert len(runs[mode]["rows"]) == STEPS
    assert runs["peer_always"]["exchange_fallbacks"] == []
    a, b = _curve(runs["allreduce"]["rows"]), _curve(runs["peer_always"]["rows"])
    assert np.allclose(b, a, rtol=RTOL, atol=ATOL), np.abs(a - b).max(0)
    assert np.allclose(runs["peer_always"]["theta"], runs["allreduce"]["theta"], rtol=1e-3, atol=1e-5)


@pytest.mark.parametrize("precision", ["float", "double"])
def test_loss_curve_one_rank_vs_two_emulated_ranks(tmp_path, precision):
    """One rank with batch 4 against two ranks with batch 2 each (the two halves of every global batch),
    gradients averaged by the exchange kernel, learning rate not scaled: the mean of the two ranks' losses
    follows the single-rank curve for 125 steps and the two replicas stay bit-identical.  The ranks are two
    models on ONE GPU connected inside the process; their kernels run one after the other, so both ranks
    store to each other before either waits (kernels on one GPU must never wait for each other)."""
    import ctypes as C
    from alphanesgpu_b200 import _lib, train as T
    from alphanesgpu_b200.dist import _DevArray
    from alphanesgpu_b200.model import StafModel, _p
    L = _lib.lib()
    data = _parity_data(100, 4100)
    cfg = T.load_config(dict(buffer_stream_dim_tr=20, batch_size=4, number_of_epochs=5, displ_freq=10, Seed=9,
                             precision=precision, lr_dense_net="expdec 0.001 0.0000001"))
    one = T.train(cfg, str(tmp_path), data=data, log=lambda *_: None)
    assert len(one["rows"]) == STEPS
    # ---- two emulated ranks
    double = precision == "double"
    np_dt, t_dt = (np.float64, torch.float64) if double else (np.float32, torch.float32)
    shape, geo = one["shape"], one["geo"]
    theta, emb = T.init_params(shape, cfg, 9)
    dev = torch.device("cuda:0")
    W = 2
    ms = [StafModel(shape, geo, theta, emb, 2, dtype=t_dt, device=dev) for _ in range(W)]
    hs = (C.c_void_p * W)()
    for r in range(W):
        h = C.c_void_p()
        _lib.check(L.stafb_peer_create(ms[r].ctx.h, r, W, shape.n_params, C.byref(h)), "stafb_peer_create")
        hs[r] = h
    grads = []
    for r in range(W):
        _lib.check(L.stafb_peer_connect_local(hs[r], hs), "stafb_peer_connect_local")
        grads.append([torch.as_tensor(_DevArray(L.stafb_peer_grad(hs[r], par), shape.n_params, t_dt), device=dev)
                      for par in (0, 1)])
        ms[r].step_d = torch.zeros(2, dtype=torch.int32, device=dev)
    lr_of = T.build_learning_rate(cfg["lr_dense_net"], 5, 5, 20)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    dv = lambda a: torch.as_tensor(np.ascontiguousarray(a, np_dt)).to(dev)
    curve = []
    step = 0
    for ep in range(5):
        for b in range(5):
            for k in range(5):
                g0 = 20 * b + 4 * k  # first frame of the global batch
                par = step & 1
                losses = []
                for r in range(W):
                    sl = slice(g0 + 2 * r, g0 + 2 * r + 2)
                    ms[r].use_grad(grads[r][par])
                    ms[r].loss_and_grad(dv(data["pos"][sl]), dv(data["box"][sl]), dv(data["energy"][sl]),
                                        dv(data["force"][sl]))
                    losses.append(ms[r].losses.cpu().numpy().copy())
                for phase in (1, 2):  # both ranks store to each other, then both wait and update
                    for r in range(W):
                        _lib.check(L.stafb_allreduce_adam_phase(ms[r].ctx.h, hs[r], stream, par, _p(ms[r].theta),
                                                                _p(ms[r].adam_m), _p(ms[r].adam_v), lr_of(step), 0.9,
                                                                0.999, 1e-7, _p(ms[r].step_d), phase),
                                   "stafb_allreduce_adam_phase")
                l = np.mean(losses, axis=0)  # (loss, loss_e, loss_bound, loss_f)
                curve.append([l[1], l[3], l[2]])
                step += 1
    torch.cuda.synchronize()
    assert all(L.stafb_peer_status(hs[r]) == 0 for r in range(W))
    assert torch.equal(ms[0].theta, ms[1].theta)  # rank-ordered sums: the replicas cannot drift
    a, b = _curve(one["rows"]), np.array(curve)
    assert np.allclose(b, a, rtol=RTOL, atol=ATOL), np.abs(a - b).max(0)
    for r in range(W):
        L.stafb_peer_destroy(hs[r])
        ms[r].close()
