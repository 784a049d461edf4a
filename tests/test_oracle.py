"""CPU tests that pin the oracle: against the reference's own CPU code (golden vectors made by
tests/golden/make_fixtures.py), against the reference's recorded known answers, and against finite
differences in double precision."""
import os

import numpy as np
import pytest

from alphanesgpu_b200 import params, synth
from conftest import CFG, GOLDEN, oracle_force_and_virial, rel_err, tie_groups_equal


@pytest.mark.parametrize("key,tag", [(k, t) for k in ("frame0", "water96_s1000", "water768_s1100")
                                     for t in ("f32", "f64")])
def test_neighbour_list_matches_reference_cpu_list(oracle, frame0, key, tag):
    g = np.load(os.path.join(GOLDEN, "ref_nl.npz"))
    dt = np.float32 if tag == "f32" else np.float64
    if key == "frame0":
        pos, box = frame0["pos"][0], frame0["box"][0]
    else:
        name, seed = key.split("_s")
        p, b, _ = synth.water_frames(name, [int(seed)])
        pos, box = p[0], b[0]
    r = oracle.neighbour_list(4.5, 60, pos, box, dt)
    assert r["status"] == 0
    assert np.array_equal(r["ncell"], g["%s_%s_ncell" % (key, tag)])
    assert np.array_equal(r["howmany"], g["%s_%s_howmany" % (key, tag)])
    assert np.array_equal(r["d2"], g["%s_%s_d2" % (key, tag)])  # bit-exact squared distances
    tie_groups_equal(r["with_"], g["%s_%s_with" % (key, tag)].astype(np.int32), r["d2"], r["howmany"])


def test_frame0_neighbour_statistics(oracle, frame0):
    # README.md:38 of the reference: 38.2 +- 0.8 neighbours inside 4.5 A
    r = oracle.neighbour_list(4.5, 60, frame0["pos"][0], frame0["box"][0], np.float32)
    assert abs(r["howmany"].mean() - 38.2) < 0.8


@pytest.mark.parametrize("tag,tol", [("f32", 2e-6), ("f64", 1e-13)])
def test_mlp_matches_reference_native_evaluator(oracle, frame0, tag, tol):
    g = np.load(os.path.join(GOLDEN, "ref_mlp.npz"))
    dt = np.float32 if tag == "f32" else np.float64
    shape = frame0["shape"]
    etot = 0.0
    for k in (0, 1):
        o = shape.offsets(k)
        F = shape.Fr[k] + shape.Fa[k]
        mu = frame0["theta"][o["mu"]:o["mu"] + F].astype(dt)
        w = frame0["theta"][o["w"]:o["w"] + shape.mlp_size(k)].astype(dt)
        e, nd = oracle.mlp_eval(shape.widths, g["af%d" % k].astype(dt), mu, w)
        etot += 0.5 * e.astype(np.float64).sum()
        assert rel_err(nd, g["%s_d%d" % (tag, k)]) < tol
    assert abs(etot - float(g["%s_energy" % tag])) < max(tol * 50, 1e-12) * abs(etot)


def test_known_answer_frame0_energy_and_force(oracle, frame0):
    # test/test-lammps-STAF-inference-STAF-comp/results/frames.csv:2 of the reference:
    # E = -102.25880432 (TF float) / -102.25872 (libstaf), rms|F| = 0.6993059698907058
    r = oracle.energy_force_grad(frame0["cfg"], frame0["shape"].desc(), frame0["pos"], frame0["box"],
                                 frame0["shape"].type_map, frame0["theta"], frame0["emb"], np.float32,
                                 per_atom_energy=False)
    assert r["status"] == 0
    assert abs(float(r["energy"][0]) - (-102.25880432)) < 1.2e-4  # the reference's own TF-vs-libstaf spread
    F = r["force"].astype(np.float64)
    assert abs(np.sqrt((F ** 2).mean()) - 0.6993059698907058) < 5e-6
    assert np.abs(F.reshape(-1, 3).sum(0)).max() < 1e-3


def _small_case(dtype, nf=2):
    pos, box, tipos = synth.water_frames("water96", [1000 + i for i in range(nf)])
    shape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(shape, dtype=dtype)
    el, fl = synth.labels(nf, shape.N, dtype=dtype)
    return pos.astype(dtype), box.astype(dtype), shape, theta, emb, el, fl


def test_structural_invariants(oracle):
    pos, box, shape, theta, emb, el, fl = _small_case(np.float64)
    d = oracle.descriptors(CFG["Rc"], CFG["Rs"], CFG["Ra"], 60, 1770, pos, box, np.float64)
    assert d["status"] == 0
    n = d["intmap2b"][..., 0]
    for b in range(pos.shape[0]):
        for i in range(shape.N):
            row = d["nbr_d2"][b, i, :n[b, i]]
            assert np.all(np.diff(row) >= 0)
            m = d["numtriplet"][b, i]
            assert m == n[b, i]  # Ra == Rc
            ids = d["intmap2b"][b, i, 1:1 + m]
            jj, kk = np.triu_indices(m, 1)
            T = len(jj)
            assert np.array_equal(d["intmap3b"][b, i, :2 * T].reshape(-1, 2), np.stack([ids[jj], ids[kk]], 1))
            assert np.all(d["intmap3b"][b, i, 2 * T:] == 0)
            assert np.all(d["angdescr"][b, i, T:] == 0)
    r = oracle.energy_force_grad(CFG, shape.desc(), pos, box, shape.type_map, theta, emb, np.float64)
    assert np.abs(r["force"].reshape(pos.shape[0], -1, 3).sum(1)).max() < 1e-12


def test_forces_are_minus_energy_gradient_fd(oracle):
    pos, box, shape, theta, emb, el, fl = _small_case(np.float64, nf=1)
    sd = shape.desc()

    def E(p):
        return float(oracle.energy_force_grad(CFG, sd, p, box, shape.type_map, theta, emb, np.float64,
                                              per_atom_energy=False)["energy"][0])
    F = oracle.energy_force_grad(CFG, sd, pos, box, shape.type_map, theta, emb, np.float64,
                                 per_atom_energy=False)["force"][0]
    rng = np.random.default_rng(5)
    h = 1e-5
    for idx in rng.choice(pos.shape[1], 12, replace=False):
        pp, pm = pos.copy(), pos.copy()
        pp[0, idx] += h
        pm[0, idx] -= h
        fd = -(E(pp) - E(pm)) / (2 * h)
        assert abs(fd - F[idx]) < 1e-7 * max(1.0, abs(F[idx])), (idx, fd, F[idx])


@pytest.mark.parametrize("loss_kind", [0, 1])
def test_parameter_gradients_fd(oracle, loss_kind):
    pos, box, shape, theta, emb, el, fl = _small_case(np.float64, nf=2)
    sd = shape.desc()
    # push a few alphas over the bound so that the bound term is exercised
    theta = theta.copy()
    theta[shape.offsets(0)["a2"] + 1] = 5.5
    theta[shape.offsets(1)["a3"] + 4] = 6.0
    kw = dict(with_grad=True, e_label=el, f_label=fl, pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0, loss_kind=loss_kind)
    r = oracle.energy_force_grad(CFG, sd, pos, box, shape.type_map, theta, emb, np.float64, **kw)
    g = r["grad"]
    rng = np.random.default_rng(7)
    picks = []
    for t in range(shape.nt):
        o = shape.offsets(t)
        for lo, hi in ((o["a2"], o["a3"]), (o["a3"], o["mu"]), (o["mu"], o["w"]), (o["w"], o["a2"] + o["size"])):
            picks += list(rng.integers(lo, hi, 4))
    h = 1e-6
    for i in picks:
        tp, tm = theta.copy(), theta.copy()
        tp[i] += h
        tm[i] -= h
        lp = oracle.energy_force_grad(CFG, sd, pos, box, shape.type_map, tp, emb, np.float64, **kw)["losses"][0]
        lm = oracle.energy_force_grad(CFG, sd, pos, box, shape.type_map, tm, emb, np.float64, **kw)["losses"][0]
        fd = (lp - lm) / (2 * h)
        assert abs(fd - g[i]) < 2e-6 * max(abs(g).max(), 1e-3), (i, fd, g[i])


@pytest.mark.parametrize("loss_kind", [0, 1])
def test_parameter_gradients_with_the_virial_loss_fd(oracle, loss_kind):
    """The energy + force + virial loss of full_train_e_f_v (staf_model.py:313-384): its gradient against central
    differences of the total loss in double precision, all parameter families; without virial labels the
    evaluation equals the energy + force one."""
    pos, box, shape, theta, emb, el, fl = _small_case(np.float64, nf=2)
    sd = shape.desc()
    theta = theta.copy()
    theta[shape.offsets(0)["a2"] + 1] = 5.5
    rng = np.random.default_rng(17)
    vl = rng.normal(0.0, 2.0, (2, 9))  # spread over both Huber branches
    kw = dict(with_grad=True, e_label=el, f_label=fl, v_label=vl, pe=0.7, pf=1.3, pv=0.6, pb=0.9, alpha_bound=5.0,
              loss_kind=loss_kind)
    r = oracle.energy_force_virial_grad(CFG, sd, pos, box, shape.type_map, theta, emb, np.float64, **kw)
    assert r["status"] == 0
    ls = r["losses"]
    assert abs(ls[0] - (0.7 * ls[1] + 0.9 * ls[2] + 1.3 * ls[3] + 0.6 * ls[4])) <= 1e-12 * abs(ls[0])
    assert ls[4] > 0
    plain = oracle.energy_force_grad(CFG, sd, pos, box, shape.type_map, theta, emb, np.float64, with_grad=True,
                                     e_label=el, f_label=fl, pe=0.7, pf=1.3, pb=0.9, alpha_bound=5.0,
                                     loss_kind=loss_kind)
    assert np.allclose(plain["losses"][1:4], ls[1:4], rtol=1e-13)
    assert np.abs(r["grad"] - plain["grad"]).max() > 1e-6  # the virial term does contribute
    g = r["grad"]
    picks = []
    for t in range(shape.nt):
        o = shape.offsets(t)
        for lo, hi in ((o["a2"], o["a3"]), (o["a3"], o["mu"]), (o["mu"], o["w"]), (o["w"], o["a2"] + o["size"])):
            picks += list(rng.integers(lo, hi, 3))
    h = 1e-6
    for i in picks:
        tp, tm = theta.copy(), theta.copy()
        tp[i] += h
        tm[i] -= h
        lp = oracle.energy_force_virial_grad(CFG, sd, pos, box, shape.type_map, tp, emb, np.float64, **kw)["losses"][0]
        lm = oracle.energy_force_virial_grad(CFG, sd, pos, box, shape.type_map, tm, emb, np.float64, **kw)["losses"][0]
        fd = (lp - lm) / (2 * h)
        assert abs(fd - g[i]) < 2e-6 * max(abs(g).max(), 1e-3), (i, fd, g[i])


def test_mlp_backward_fd(oracle):
    rng = np.random.default_rng(11)
    widths, F, n = [9, 6, 1], 7, 5
    nw = F * 9 + 9 + 9 * 6 + 6 + 6 + 1
    af = np.exp(rng.normal(size=(n, F)))
    mu, w = rng.normal(size=F), rng.normal(size=nw) * 0.5
    ebar, u = rng.normal(size=n), rng.normal(size=(n, F))

    def S(af_, mu_, w_):
        e, nd = oracle.mlp_eval(widths, af_, mu_, w_)
        return float((ebar * e).sum() + (u * nd).sum())
    e, nd, gw, gmu, gaf = oracle.mlp_eval(widths, af, mu, w, ebar, u)
    h = 1e-6
    for i in rng.choice(nw, 12, replace=False):
        wp, wm = w.copy(), w.copy()
        wp[i] += h
        wm[i] -= h
        assert abs((S(af, mu, wp) - S(af, mu, wm)) / (2 * h) - gw[i]) < 1e-6 * max(1, abs(gw).max())
    for i in range(F):
        mp, mm = mu.copy(), mu.copy()
        mp[i] += h
        mm[i] -= h
        assert abs((S(af, mp, w) - S(af, mm, w)) / (2 * h) - gmu[i]) < 1e-6 * max(1, abs(gmu).max())
    for a, i in [(0, 0), (2, 3), (4, 6)]:
        ap, am = af.copy(), af.copy()
        ap[a, i] += h * af[a, i]
        am[a, i] -= h * af[a, i]
        fd = (S(ap, mu, w) - S(am, mu, w)) / (2 * h * af[a, i])
        assert abs(fd - gaf[a, i]) < 1e-5 * max(1, abs(gaf).max())


def test_float_oracle_tracks_double_oracle(oracle, frame0):
    # the reference records max|dE| 6.5e-5 and max|dF| 4.3e-5 between its float and double builds on
    # its 10 frames (test/test-inference-pipeline/comparison_summary.txt:6-7) and gates at 1e-3
    # (analyze_compatibility.py:273-291); this frame must land at the recorded level
    out = {}
    for dt in (np.float32, np.float64):
        out[dt] = oracle.energy_force_grad(frame0["cfg"], frame0["shape"].desc(), frame0["pos"], frame0["box"],
                                           frame0["shape"].type_map, frame0["theta"], frame0["emb"], dt,
                                           per_atom_energy=False)
    assert abs(float(out[np.float32]["energy"][0]) - float(out[np.float64]["energy"][0])) < 1e-4
    assert np.abs(out[np.float32]["force"].astype(np.float64) - out[np.float64]["force"]).max() < 1e-4


def test_status_codes(oracle):
    pos, box, tipos = synth.water_frames("water96", [1000])
    # radial overflow: the reference exits the process here (descriptor_builder/reforce.cc:324-340)
    r = oracle.neighbour_list(4.5, 20, pos[0], box[0], np.float64)
    assert r["status"] == 1
    bad = box[0].copy()
    bad[3] = 0.0
    assert oracle.neighbour_list(4.5, 60, pos[0], bad, np.float64)["status"] == 4


def test_model_dir_writer_round_trips(tmp_path):
    """save_model_dir writes what load_model_dir (and staf_load) read."""
    from alphanesgpu_b200 import params, synth
    shape = synth.baseline_shape([5, 10])
    theta, emb = synth.init_params(shape)
    params.save_model_dir(str(tmp_path), CFG, shape, theta, emb)
    cfg2, shape2, theta2, emb2 = params.load_model_dir(str(tmp_path))
    assert cfg2 == CFG and shape2.tipos == [5, 10] and shape2.widths == shape.widths
    assert shape2.Fr == shape.Fr and shape2.Fa == shape.Fa
    assert np.array_equal(theta2, theta) and np.array_equal(emb2, emb)


def test_virial_is_minus_strain_derivative_of_the_energy_fd(oracle):
    """Pins the ...Virial force ops: W_ab = -dE/d(eps_ab) for a homogeneous strain r -> (1 + eps) r of positions
    and box (upper-triangular eps keeps the box upper-triangular), and W is symmetric."""
    pos, box, shape, theta, emb, el, fl = _small_case(np.float64, nf=1)
    sd = shape.desc()
    E0, F, W = oracle_force_and_virial(oracle, shape, theta, emb, pos, box)
    full = oracle.energy_force_grad(CFG, sd, pos, box, shape.type_map, theta, emb, np.float64, per_atom_energy=False)
    assert abs(E0[0] - full["energy"][0]) < 1e-12 * abs(E0[0])
    assert rel_err(F, full["force"]) < 1e-12
    W = W[0].reshape(3, 3)
    assert np.abs(W - W.T).max() < 1e-9 * np.abs(W).max()

    def E(eps):
        M = np.eye(3) + eps
        p = (pos.reshape(-1, 3) @ M.T).reshape(1, -1)
        b = box[0]
        H = np.array([[b[0], b[1], b[2]], [0, b[3], b[4]], [0, 0, b[5]]])
        H2 = M @ H
        b2 = np.array([[H2[0, 0], H2[0, 1], H2[0, 2], H2[1, 1], H2[1, 2], H2[2, 2]]])
        return float(oracle.energy_force_grad(CFG, sd, p, b2, shape.type_map, theta, emb, np.float64,
                                              per_atom_energy=False)["energy"][0])
    h = 1e-6
    for a in range(3):
        for c in range(a, 3):
            eps = np.zeros((3, 3))
            eps[a, c] = h
            fd = (E(eps) - E(-eps)) / (2 * h)
            assert abs(-fd - W[a, c]) < 2e-6 * np.abs(W).max(), (a, c, fd, W[a, c])
