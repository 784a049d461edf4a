"""GPU parity of the fused energy/force/training path (C ABI: stafb_energy_force, stafb_train_step,
stafb_adam_step) against the CPU oracle's full step on the same seeded inputs."""
import numpy as np
import pytest

from alphanesgpu_b200 import synth
from conftest import CFG, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = {np.float32: 1e-5, np.float64: 1e-11}


def _tdt(dtype):
    return torch.float32 if dtype == np.float32 else torch.float64


def _case(name, seeds, frame0):
    if name == "frame0":
        return frame0["pos"], frame0["box"], frame0["shape"], frame0["theta"], frame0["emb"]
    pos, box, tipos = synth.water_frames(name, seeds)
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape)
    return pos, box, shape, theta, emb


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("name,seeds", [("water96", [1000, 1001]), ("water768", [1100, 1101, 1102, 1103]),
                                        ("frame0", None)])
def test_energy_force(oracle, frame0, name, seeds, dtype):
    from alphanesgpu_b200.model import StafModel
    pos, box, shape, theta, emb = _case(name, seeds, frame0)
    nf = pos.shape[0]
    ref = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, dtype,
                                   per_atom_energy=False)
    assert ref["status"] == 0
    m = StafModel(shape, CFG, theta, emb, nf, dtype=_tdt(dtype))
    e, f = m.energy_force(pos.astype(dtype), box.astype(dtype))
    assert rel_err(e.cpu().numpy(), ref["energy"]) <= TOL[dtype]
    assert rel_err(f.cpu().numpy(), ref["force"]) <= TOL[dtype]
    if name == "frame0" and dtype == np.float32:
        # the reference's recorded values for this frame and model
        # (test/test-lammps-STAF-inference-STAF-comp/results/frames.csv:2)
        assert abs(float(e[0]) - (-102.25880432)) < 1.2e-4
        assert abs(float(torch.sqrt((f.double() ** 2).mean())) - 0.6993059698907058) < 5e-6
    m.close()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def _push_over_bound(shape, theta):
    """Two exponents beyond alpha_bound = 5 (on channels whose squared embedding is not zero), so that the bound
    term and its gradient are exercised."""
    theta = theta.copy()
    theta[shape.offsets(0)["a2"] + 1] = 5.5
    theta[shape.offsets(1)["a3"] + 4] = 6.0
    return theta


def _check_train_step(oracle, m, shape, pos, box, el, fl, theta, emb, dtype, loss, kw, host_path=True):
    """Energy, forces, the four losses and the gradient per parameter family (alpha2b, alpha3b, mu, Dense
    weights+biases of every species) against the oracle: the reference's own gradient regression, restated
    (test/test-regression/regression-grad-param/run_grad_param_regression.py:80-253)."""
    ref = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, dtype, with_grad=True,
                                   e_label=el, f_label=fl, loss_kind=0 if loss == "huber" else 1, **kw)
    assert ref["status"] == 0
    d = lambda a: torch.as_tensor(a.astype(dtype)).cuda()
    e, f = m.loss_and_grad(d(pos), d(box), d(el), d(fl), want_outputs=True)
    m.ctx.raise_on_status("train_step")
    tol = TOL[dtype]
    assert rel_err(e.cpu().numpy(), ref["energy"]) <= tol
    assert rel_err(f.cpu().numpy(), ref["force"]) <= tol
    losses = m.losses.cpu().numpy()
    assert np.allclose(losses, ref["losses"], rtol=tol * 10, atol=0)
    g, gr = m.grad.cpu().numpy().astype(np.float64), ref["grad"].astype(np.float64)
    for t in range(shape.nt):
        o = shape.offsets(t)
        for lo, hi in ((o["a2"], o["a3"]), (o["a3"], o["mu"]), (o["mu"], o["w"]), (o["w"], o["a2"] + o["size"])):
            assert rel_err(g[lo:hi], gr[lo:hi]) <= tol, (t, lo, hi)
    if host_path:  # host-buffer entry point gives the same numbers
        lh = m.loss_and_grad_host(pos, box, el, fl).copy()
        assert np.allclose(lh, losses, rtol=1e-6 if dtype == np.float32 else 1e-12)
        assert rel_err(m.grad.cpu().numpy(), g) <= (5e-6 if dtype == np.float32 else 1e-12)  # float atomics: order varies


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_train_step_on_the_reference_model_shape(oracle, frame0, dtype):
    """The reference's real frame with its exported model (Fr = 20, Fa = 40, MLP 60-140-140-1 per species): the
    training gradient per parameter family.  At this size the Dense layers no longer fit in shared memory all at
    once, so the MLP kernels run in their other staging modes, and every species-pair class has more active
    channels than one pass of the sweeps takes."""
    from alphanesgpu_b200.model import StafModel
    pos, box, shape, theta, emb = _case("frame0", None, frame0)
    theta = _push_over_bound(shape, theta)
    el, fl = synth.labels(1, shape.N)
    kw = dict(pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0)
    m = StafModel(shape, CFG, theta, emb, 1, dtype=_tdt(dtype), loss="huber", **kw)
    cfg = m.mlp_config()
    assert cfg["stage"] == (1 if dtype == np.float32 else 0), cfg  # layer-at-a-time in fp32, global reads in fp64
    assert cfg["mma"] == 0, cfg  # the tensor-core arm is opt-in
    assert max(shape.Fa) // shape.C > 8  # more active angular channels per class than one chunk of the sweeps
    _check_train_step(oracle, m, shape, pos, box, el, fl, theta, emb, dtype, "huber", kw)
    m.close()


@pytest.mark.parametrize("stage", [0, 1, 2])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_train_step_in_every_mlp_staging_mode(oracle, frame0, monkeypatch, dtype, stage):
    """The three ways the MLP kernels hold their Dense layers (all in shared memory, one layer at a time, read
    from global memory), each forced on the small model and checked against the oracle."""
    from alphanesgpu_b200.model import StafModel
    monkeypatch.setenv("STAFB_MLP_STAGE", str(stage))
    pos, box, shape, theta, emb = _case("water96", [1000, 1001], frame0)
    theta = _push_over_bound(shape, theta)
    el, fl = synth.labels(2, shape.N)
    kw = dict(pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0)
    m = StafModel(shape, CFG, theta, emb, 2, dtype=_tdt(dtype), loss="huber", **kw)
    assert m.mlp_config()["stage"] == stage
    _check_train_step(oracle, m, shape, pos, box, el, fl, theta, emb, dtype, "huber", kw, host_path=False)
    m.close()


@pytest.mark.parametrize("warps", [1, 2, 4, 8])
def test_train_step_with_the_tensor_core_mlp(oracle, frame0, monkeypatch, warps):
    """The tensor-core arm of the MLP kernels (fp32, STAFB_MLP_MMA=1) with 1, 2, 4 and 8 warps sharing a 16-atom
    tile; two frames of 96 atoms leave partly filled tiles."""
    from alphanesgpu_b200.model import StafModel
    monkeypatch.setenv("STAFB_MLP_MMA", "1")
    monkeypatch.setenv("STAFB_MLP_MMA_NW", str(warps))
    pos, box, shape, theta, emb = _case("water96", [1000, 1001], frame0)
    theta = _push_over_bound(shape, theta)
    el, fl = synth.labels(2, shape.N)
    kw = dict(pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0)
    m = StafModel(shape, CFG, theta, emb, 2, dtype=torch.float32, loss="huber", **kw)
    cfg = m.mlp_config()
    assert (cfg["mma"], cfg["mma_warps"]) == (1, warps), cfg
    _check_train_step(oracle, m, shape, pos, box, el, fl, theta, emb, np.float32, "huber", kw, host_path=False)
    m.close()


def test_the_tensor_core_mlp_on_the_reference_model_shape(oracle, frame0, monkeypatch):
    """60-140-140-1: 18 output tiles per layer, so the wide form of the product (five tiles per warp) runs."""
    from alphanesgpu_b200.model import StafModel
    monkeypatch.setenv("STAFB_MLP_MMA", "1")
    pos, box, shape, theta, emb = _case("frame0", None, frame0)
    el, fl = synth.labels(1, shape.N)
    kw = dict(pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0)
    m = StafModel(shape, CFG, theta, emb, 1, dtype=torch.float32, loss="huber", **kw)
    assert m.mlp_config()["mma"] == 1
    _check_train_step(oracle, m, shape, pos, box, el, fl, theta, emb, np.float32, "huber", kw, host_path=False)
    m.close()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("name,seeds,loss", [("water96", [1000, 1001], "huber"), ("water96", [1000, 1001], "mse"),
                                             ("water768", [1100, 1101], "huber"), ("frame0", None, "huber")])
def test_train_step_with_the_virial_loss(oracle, frame0, name, seeds, loss, dtype):
    """Energy + force + virial training evaluation (full_train_e_f_v, staf_model.py:313-384): energies, forces,
    virials, the five losses and the gradient per parameter family against the oracle, whose virial-loss gradient
    is pinned by finite differences in tests/test_oracle.py."""
    from alphanesgpu_b200.model import StafModel
    pos, box, shape, theta, emb = _case(name, seeds, frame0)
    theta = _push_over_bound(shape, theta)
    nf = pos.shape[0]
    el, fl = synth.labels(nf, shape.N)
    vl = np.random.default_rng(23).normal(0.0, 2.0, (nf, 9))  # both branches of the Huber loss
    kw = dict(pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0)
    ref = oracle.energy_force_virial_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, dtype,
                                          with_grad=True, e_label=el, f_label=fl, v_label=vl, pv=0.6,
                                          loss_kind=0 if loss == "huber" else 1, **kw)
    assert ref["status"] == 0 and ref["losses"][4] > 0
    m = StafModel(shape, CFG, theta, emb, nf, dtype=_tdt(dtype), loss=loss, **kw)
    d = lambda a: torch.as_tensor(a.astype(dtype)).cuda()
    e, f, w = m.loss_and_grad_virial(d(pos), d(box), d(el), d(fl), d(vl), pv=0.6, want_outputs=True)
    m.ctx.raise_on_status("train_step_virial")
    tol = TOL[dtype]
    assert rel_err(e.cpu().numpy(), ref["energy"]) <= tol
    assert rel_err(f.cpu().numpy(), ref["force"]) <= tol
    assert rel_err(w.cpu().numpy(), ref["virial"]) <= 10 * tol
    assert np.allclose(m.losses5.cpu().numpy(), ref["losses"], rtol=tol * 20, atol=0)
    g, gr = m.grad.cpu().numpy().astype(np.float64), ref["grad"].astype(np.float64)
    for t in range(shape.nt):
        o = shape.offsets(t)
        for lo, hi in ((o["a2"], o["a3"]), (o["a3"], o["mu"]), (o["mu"], o["w"]), (o["w"], o["a2"] + o["size"])):
            assert rel_err(g[lo:hi], gr[lo:hi]) <= 2 * tol, (t, lo, hi)
    # the pipelined host-buffer form, on a stream that can be captured: plain launches, capture, graph replay on
    # each of the two slots
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for k in range(7):
            m.grad.zero_()
            m.loss_and_grad_virial_host_begin(pos, box, el, fl, vl, k & 1, pv=0.6)
            lh = m.loss_and_grad_virial_host_end(k & 1)
            assert np.allclose(lh, ref["losses"], rtol=tol * 20, atol=0), (k, lh)
            assert rel_err(m.grad.cpu().numpy(), ref["grad"]) <= 2 * tol, k
    torch.cuda.synchronize()
    # the plain evaluation afterwards is not affected by the virial state
    m.loss_and_grad(d(pos), d(box), d(el), d(fl))
    plain = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, dtype, with_grad=True,
                                     e_label=el, f_label=fl, loss_kind=0 if loss == "huber" else 1, **kw)
    assert np.allclose(m.losses.cpu().numpy(), plain["losses"], rtol=tol * 10, atol=0)
    assert rel_err(m.grad.cpu().numpy(), plain["grad"]) <= tol
    m.close()


def test_train_step_batch_of_eight(oracle, frame0):
    """Eight 768-atom frames per step, the per-GPU batch of the data-parallel configuration."""
    from alphanesgpu_b200.model import StafModel
    pos, box, shape, theta, emb = _case("water768", list(range(1200, 1208)), frame0)
    theta = _push_over_bound(shape, theta)
    el, fl = synth.labels(8, shape.N)
    kw = dict(pe=1.0, pf=1.0, pb=1.0, alpha_bound=5.0)
    m = StafModel(shape, CFG, theta, emb, 8, dtype=torch.float32, loss="huber", **kw)
    _check_train_step(oracle, m, shape, pos, box, el, fl, theta, emb, np.float32, "huber", kw)
    m.close()


@pytest.mark.parametrize("name", ["water24576", "water6144"])
def test_energy_force_of_the_large_boxes(oracle, frame0, name):
    """The large inference box (8192 O + 16384 H, L = 62.7 A; 13 x 13 x 13 cells, the multi-kernel cell-list
    path) and a 6144-atom box (the size of a slab domain): energy and every force component against the oracle."""
    from alphanesgpu_b200.model import StafModel
    pos, box, shape, theta, emb = _case(name, [1400], frame0)
    ref = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, np.float32,
                                   per_atom_energy=False)
    assert ref["status"] == 0
    m = StafModel(shape, CFG, theta, emb, 1, dtype=torch.float32)
    e, f = m.energy_force(pos.astype(np.float32), box.astype(np.float32))
    assert rel_err(e.cpu().numpy(), ref["energy"]) <= 1e-5
    assert rel_err(f.cpu().numpy(), ref["force"]) <= 1e-5
    m.close()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("name,seeds,loss", [("water96", [1000, 1001], "huber"), ("water96", [1000, 1001], "mse"),
                                             ("water768", [1100, 1101, 1102, 1103], "huber")])
def test_train_step_losses_and_gradient(oracle, frame0, name, seeds, loss, dtype):
    from alphanesgpu_b200.model import StafModel
    pos, box, shape, theta, emb = _case(name, seeds, frame0)
    theta = _push_over_bound(shape, theta)
    nf = pos.shape[0]
    el, fl = synth.labels(nf, shape.N)
    kw = dict(pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0)
    ref = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, dtype, with_grad=True,
                                   e_label=el, f_label=fl, loss_kind=0 if loss == "huber" else 1, **kw)
    m = StafModel(shape, CFG, theta, emb, nf, dtype=_tdt(dtype), loss=loss, **kw)
    d = lambda a: torch.as_tensor(a.astype(dtype)).cuda()
    e, f = m.loss_and_grad(d(pos), d(box), d(el), d(fl), want_outputs=True)
    m.ctx.raise_on_status("train_step")
    tol = TOL[dtype]
    assert rel_err(e.cpu().numpy(), ref["energy"]) <= tol
    assert rel_err(f.cpu().numpy(), ref["force"]) <= tol
    losses = m.losses.cpu().numpy()
    assert np.allclose(losses, ref["losses"], rtol=tol * 10, atol=0)
    g, gr = m.grad.cpu().numpy().astype(np.float64), ref["grad"].astype(np.float64)
    # per parameter family, as the reference's own gradient regression does
    # (test/test-regression/regression-grad-param/run_grad_param_regression.py:80-253)
    for t in range(shape.nt):
        o = shape.offsets(t)
        for lo, hi in ((o["a2"], o["a3"]), (o["a3"], o["mu"]), (o["mu"], o["w"]), (o["w"], o["a2"] + o["size"])):
            assert rel_err(g[lo:hi], gr[lo:hi]) <= tol, (t, lo, hi)
    # host-buffer entry point gives the same numbers
    lh = m.loss_and_grad_host(pos, box, el, fl).copy()
    assert np.allclose(lh, losses, rtol=1e-6 if dtype == np.float32 else 1e-12)
    assert rel_err(m.grad.cpu().numpy(), g) <= (5e-6 if dtype == np.float32 else 1e-12)  # float atomics: order varies
    m.close()


def test_adam_matches_reference_formula():
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", [1000])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape)
    m = StafModel(shape, CFG, theta, emb, 1, dtype=torch.float64)
    rng = np.random.default_rng(3)
    th, mm, vv = theta.copy(), np.zeros_like(theta), np.zeros_like(theta)
    for step in range(1, 4):
        g = rng.normal(size=theta.shape)
        m.grad.copy_(torch.as_tensor(g).cuda())
        m.adam_update(1e-3)
        mm = 0.9 * mm + 0.1 * g
        vv = 0.999 * vv + 0.001 * g * g
        lr_t = 1e-3 * np.sqrt(1 - 0.999 ** step) / (1 - 0.9 ** step)
        th = th - lr_t * mm / (np.sqrt(vv) + 1e-7)
        assert np.allclose(m.theta.cpu().numpy(), th, rtol=1e-13, atol=1e-15)
    m.close()


def test_training_reduces_the_loss():
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", [1000, 1001])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape)
    el, fl = synth.labels(2, shape.N)
    m = StafModel(shape, CFG, theta, emb, 2, dtype=torch.float32)
    first = last = None
    for it in range(30):
        l = m.loss_and_grad_host(pos, box, el * 0.01, fl * 0.05)[0]
        first = l if first is None else first
        last = l
        m.adam_update(2e-3)
    assert np.isfinite(last) and last < first
    m.close()


@pytest.mark.parametrize("dtype,tol", [(np.float32, 2e-5), (np.float64, 1e-10)])
def test_energy_force_virial_matches_the_virial_ops(oracle, dtype, tol):
    """stafb_energy_force_virial = sum over central species of ComputeForceRadialVirial + ComputeForceTriplVirial
    (oracle op chain in double, pinned by the strain finite-difference test in tests/test_oracle.py)."""
    from alphanesgpu_b200.model import StafModel
    from conftest import oracle_force_and_virial
    pos, box, tipos = synth.water_frames("water96", [1000, 1001])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape)
    E, F, W = oracle_force_and_virial(oracle, shape, theta, emb, pos, box)
    tdt = torch.float32 if dtype == np.float32 else torch.float64
    m = StafModel(shape, CFG, theta, emb, 2, dtype=tdt, device="cuda:0")
    e, f, w = m.energy_force_virial(torch.as_tensor(pos.astype(dtype)).cuda(), torch.as_tensor(box.astype(dtype)).cuda())
    assert rel_err(e.cpu().numpy(), E) <= tol
    assert rel_err(f.cpu().numpy(), F) <= tol
    assert rel_err(w.cpu().numpy(), W) <= tol
    m.close()


def test_pipelined_host_steps_equal_the_synchronous_call():
    """stafb_train_step_host_begin/_end: two steps in flight give the losses and the gradient of the one-call form."""
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", [1000, 1001, 1002, 1003])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape, dtype=np.float32)
    el, fl = synth.labels(4, shape.N)
    m = StafModel(shape, CFG, theta, emb, 2, dtype=torch.float32, device="cuda:0")
    f32 = lambda a: a.astype(np.float32)
    ref, grads = [], []
    for h in range(2):
        sl = slice(2 * h, 2 * h + 2)
        ref.append(m.loss_and_grad_host(f32(pos[sl]), f32(box[sl]), f32(el[sl]), f32(fl[sl])).copy())
        grads.append(m.grad.clone())
    for h in range(2):
        sl = slice(2 * h, 2 * h + 2)
        m.loss_and_grad_host_begin(f32(pos[sl]), f32(box[sl]), f32(el[sl]), f32(fl[sl]), h)
    g_last = m.grad.clone()  # stream order: the second step's gradient
    got = [m.loss_and_grad_host_end(0), m.loss_and_grad_host_end(1)]
    torch.cuda.synchronize()
    for h in range(2):
        assert np.allclose(got[h], ref[h], rtol=1e-6, atol=0)
    assert rel_err(g_last.cpu().numpy(), grads[1].cpu().numpy()) <= 1e-6
    with pytest.raises(Exception):
        m.loss_and_grad_host_end(0)  # nothing in flight in that slot
    m.close()


@pytest.mark.gpu
def test_pipelined_host_steps_replayed_as_graphs():
    """Many begin/end rounds on both slots: plain launches, then capture, then graph replay (neighbour rows on the
    model's side stream) all give the losses and the gradient of the one-call form for the batch of that round."""
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", list(range(1100, 1108)))
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape, dtype=np.float32)
    el, fl = synth.labels(8, shape.N)
    m = StafModel(shape, CFG, theta, emb, 2, dtype=torch.float32, device="cuda:0")
    f32 = lambda a: a.astype(np.float32)
    batch = lambda h: tuple(f32(a[2 * h:2 * h + 2]) for a in (pos, box, el, fl))
    ref, grads = [], []
    for h in range(4):
        ref.append(m.loss_and_grad_host(*batch(h)).copy())
        grads.append(m.grad.clone())
    for k in range(12):
        h = (k * 3) % 4  # the batch changes on every use of a slot; the call signature does not
        m.loss_and_grad_host_begin(*batch(h), k & 1)
        g = m.grad.clone()
        got = m.loss_and_grad_host_end(k & 1)
        assert np.allclose(got, ref[h], rtol=1e-6, atol=0), k
        assert rel_err(g.cpu().numpy(), grads[h].cpu().numpy()) <= 1e-6, k
    m.close()


@pytest.mark.gpu
def test_prefetched_rows_on_a_side_stream():
    """stafb_descriptors_prefetch on another stream + stafb_train_step_prefetched == stafb_train_step."""
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", [1200, 1201, 1202, 1203])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape, dtype=np.float64)
    el, fl = synth.labels(4, shape.N)
    dev = torch.device("cuda:0")
    m = StafModel(shape, CFG, theta, emb, 2, dtype=torch.float64, device=dev)
    d = [torch.as_tensor(a).to(dev) for a in (pos, box, el, fl)]
    ref = []
    for h in range(2):
        m.loss_and_grad(*(a[2 * h:2 * h + 2] for a in d))
        ref.append((m.losses.clone(), m.grad.clone()))
    side = torch.cuda.Stream(device=dev)
    main = torch.cuda.current_stream(dev)
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    side.wait_stream(main)
    with torch.cuda.stream(side):  # both batches' rows before either step runs
        for h in range(2):
            m.prefetch_rows(d[0][2 * h:2 * h + 2], d[1][2 * h:2 * h + 2], h)
            ready[h].record(side)
    for h in (1, 0):
        main.wait_event(ready[h])
        m.loss_and_grad_prefetched(h, 2, d[2][2 * h:2 * h + 2], d[3][2 * h:2 * h + 2])
        torch.cuda.synchronize()
        assert torch.allclose(m.losses[:4], ref[h][0][:4], rtol=1e-12, atol=0)
        assert rel_err(m.grad.cpu().numpy(), ref[h][1].cpu().numpy()) <= 1e-11
    m.ctx.raise_on_status("prefetched step")
    m.close()
