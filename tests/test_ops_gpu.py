"""GPU parity of every reference operator, called through the C ABI, against the CPU oracle.

Tolerances are the ones the task states: integer tensors bit-exact (permutations allowed only inside
groups of bit-equal dist2), reals max|x-ref|/max|ref| <= 1e-5 in fp32 and <= 1e-11 in fp64.
"""
import numpy as np
import pytest

from alphanesgpu_b200 import synth
from conftest import CFG, rel_err, tie_groups_equal

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = {np.float32: 1e-5, np.float64: 1e-11}
CASES = [("water96", [1000, 1001]), ("water768", [1100, 1101]), ("frame0", None)]


def _inputs(case, frame0, dtype):
    name, seeds = case
    if name == "frame0":
        pos, box, shape = frame0["pos"], frame0["box"], frame0["shape"]
        theta, emb = frame0["theta"], frame0["emb"]
    else:
        pos, box, tipos = synth.water_frames(name, seeds)
        shape = synth.baseline_shape(tipos)
        theta, emb = synth.init_params(shape)
    return pos.astype(dtype), box.astype(dtype), shape, theta.astype(dtype), emb.astype(dtype)


@pytest.fixture(scope="module")
def ops():
    from alphanesgpu_b200 import ops as o
    return o


def _ctx(ops, dtype, N, nf):
    return ops.construct_descriptors_light(CFG["Rc"], CFG["nr"], CFG["na"], N, None, CFG["Rs"], CFG["Ra"], nf,
                                           dtype=torch.float32 if dtype == np.float32 else torch.float64)


def _t(a):
    return torch.as_tensor(a).cuda()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_compute_descriptors_light(ops, oracle, frame0, case, dtype):
    pos, box, shape, theta, emb = _inputs(case, frame0, dtype)
    nf, N = pos.shape[0], shape.N
    _ctx(ops, dtype, N, nf)
    ref = oracle.descriptors(CFG["Rc"], CFG["Rs"], CFG["Ra"], CFG["nr"], CFG["na"], pos, box, dtype)
    assert ref["status"] == 0
    out = ops.compute_descriptors_light(_t(pos), _t(box))
    names = ["raddescr", "angdescr", "des3bsupp", "intmap2b", "intmap3b", "der2b", "der3b", "der3bsupp", "numtriplet"]
    got = {n: t.cpu().numpy() for n, t in zip(names, out)}
    assert np.array_equal(got["numtriplet"], ref["numtriplet"])
    assert np.array_equal(got["intmap2b"][..., 0], ref["intmap2b"][..., 0])
    groups = 0
    for b in range(nf):
        groups += tie_groups_equal(got["intmap2b"][b, :, 1:], ref["intmap2b"][b, :, 1:], ref["nbr_d2"][b],
                                   ref["intmap2b"][b, :, 0])
    # with the deterministic slot order both sides resolve ties the same way
    assert np.array_equal(got["intmap2b"], ref["intmap2b"])
    assert np.array_equal(got["intmap3b"], ref["intmap3b"])
    for n in ("raddescr", "angdescr", "des3bsupp", "der2b", "der3b", "der3bsupp"):
        assert rel_err(got[n], ref[n]) <= TOL[dtype], n
    print("tie groups:", groups)


def _species_slices(d, shape, t):
    s, Nl = shape.shift(t), shape.tipos[t]
    return {k: np.ascontiguousarray(v[:, s:s + Nl]) for k, v in d.items() if isinstance(v, np.ndarray) and v.ndim >= 2}


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_all_operators(ops, oracle, frame0, case, dtype):
    pos, box, shape, theta, emb = _inputs(case, frame0, dtype)
    nf, N, nt, C = pos.shape[0], shape.N, shape.nt, shape.C
    _ctx(ops, dtype, N, nf)
    tol = TOL[dtype]
    ref = oracle.descriptors(CFG["Rc"], CFG["Rs"], CFG["Ra"], CFG["nr"], CFG["na"], pos, box, dtype)
    tm = shape.type_map
    rng = np.random.default_rng(99)
    for t in range(nt):
        d = _species_slices(ref, shape, t)
        o = shape.offsets(t)
        Fr, Fa, Nl, sh = shape.Fr[t], shape.Fa[t], shape.tipos[t], shape.shift(t)
        a2 = theta[o["a2"]:o["a2"] + nt * Fr].reshape(nt, Fr)
        a3 = theta[o["a3"]:o["a3"] + C * 3 * Fa].reshape(C, 3 * Fa)
        e2 = emb[o["emb"]:o["emb"] + nt * Fr].reshape(nt, Fr)
        e3 = emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + C * Fa].reshape(C, Fa)
        g = {k: _t(v) for k, v in d.items()}
        ta2, ta3, te2, te3, ttm = _t(a2), _t(a3), _t(e2), _t(e3), _t(tm)
        # forward fingerprints
        af2 = ops.compute_sort_proj(g["raddescr"], g["intmap2b"], ta2, te2, ttm).cpu().numpy()
        r2 = oracle.af_radial(d["raddescr"], d["intmap2b"], a2, e2, tm)
        assert rel_err(af2, r2) <= tol
        af3 = ops.compute_sort_proj3body(g["angdescr"], g["des3bsupp"], g["intmap3b"], g["intmap2b"], ta3, te3, ttm,
                                         g["numtriplet"]).cpu().numpy()
        r3 = oracle.af_angular(d["angdescr"], d["des3bsupp"], d["intmap3b"], a3, e3, tm, d["numtriplet"])
        assert rel_err(af3, r3) <= tol
        # forces
        nd2 = rng.normal(size=(nf, Nl, Fr)).astype(dtype)
        nd3 = rng.normal(size=(nf, Nl, Fa)).astype(dtype)
        tipos = np.array(shape.tipos, np.int32)
        f2 = ops.compute_force_radial(_t(nd2), g["der2b"], g["intmap2b"], g["raddescr"], ta2, te2, ttm, tipos,
                                      t).cpu().numpy()
        assert rel_err(f2, oracle.force_radial(nd2, d["der2b"], d["intmap2b"], d["raddescr"], a2, e2, tm, sh)) <= tol
        f3 = ops.compute_force_tripl(_t(nd3), g["des3bsupp"], g["angdescr"], g["der3bsupp"], g["der3b"],
                                     g["intmap2b"], g["intmap3b"], ta3, te3, ttm, tipos, t,
                                     g["numtriplet"]).cpu().numpy()
        assert rel_err(f3, oracle.force_tripl(nd3, d["des3bsupp"], d["angdescr"], d["der3bsupp"], d["der3b"],
                                              d["intmap3b"], a3, e3, tm, d["numtriplet"], sh)) <= tol
        # gradients of the fingerprints
        pg2 = rng.normal(size=(nf, Nl, Fr)).astype(dtype)
        pg3 = rng.normal(size=(nf, Nl, Fa)).astype(dtype)
        ga, ge = ops.compute_two_body_par_grad(_t(pg2), g["raddescr"], g["intmap2b"], ta2, te2, ttm)
        ra, re = oracle.grad_af_radial(pg2, d["raddescr"], d["intmap2b"], a2, e2, tm)
        assert rel_err(ga.cpu().numpy(), ra) <= tol and rel_err(ge.cpu().numpy(), re) <= tol
        ga, ge = ops.compute_sort_proj3body_grad(_t(pg3), g["angdescr"], g["des3bsupp"], g["intmap3b"], g["intmap2b"],
                                                 ta3, te3, ttm, g["numtriplet"])
        ra, re = oracle.grad_af_angular(pg3, d["angdescr"], d["des3bsupp"], d["intmap3b"], a3, e3, tm,
                                        d["numtriplet"])
        assert rel_err(ga.cpu().numpy(), ra) <= tol
        assert np.all(ge.cpu().numpy() == 0)  # the reference never accumulates this output
        # backward of the forces
        pF = rng.normal(size=(nf, 3 * N)).astype(dtype)
        gn, ga, ge = ops.compute_force_radial_grad(_t(pF), _t(nd2), g["der2b"], g["intmap2b"], g["raddescr"], ta2,
                                                   te2, ttm, tipos, t)
        rn, ra, re = oracle.grad_force_radial(pF, nd2, d["der2b"], d["intmap2b"], d["raddescr"], a2, e2, tm, sh)
        assert rel_err(gn.cpu().numpy(), rn) <= tol
        assert rel_err(ga.cpu().numpy(), ra) <= tol and rel_err(ge.cpu().numpy(), re) <= tol
        gn, ga, gck = ops.compute_force_tripl_grad(_t(pF), _t(nd3), g["des3bsupp"], g["angdescr"], g["der3bsupp"],
                                                   g["der3b"], g["intmap2b"], g["intmap3b"], ta3, te3, ttm, tipos, t,
                                                   g["numtriplet"])
        rn, ra, rck = oracle.grad_force_tripl(pF, nd3, d["des3bsupp"], d["angdescr"], d["der3bsupp"], d["der3b"],
                                              d["intmap3b"], a3, e3, tm, d["numtriplet"], sh)
        assert rel_err(gn.cpu().numpy(), rn) <= tol
        assert rel_err(ga.cpu().numpy(), ra) <= tol
        assert np.all(gck.cpu().numpy() == 0)
        # ...Virial and ...VirialGrad variants (STAF/src/force/*/reforce.cc:133-146 / 159-176,
        # STAF/src/grad_force/*/reforce.cc:160-176 / 186-206)
        tpos, tbox = _t(pos), _t(box)
        pW = rng.normal(size=(nf, 9)).astype(dtype)
        f2v, w2 = ops.compute_force_radial_virial(_t(nd2), g["der2b"], g["intmap2b"], g["raddescr"], ta2, te2, ttm,
                                                  tipos, t, tpos, tbox)
        rf, rw = oracle.force_radial(nd2, d["der2b"], d["intmap2b"], d["raddescr"], a2, e2, tm, sh, pos, box)
        assert rel_err(f2v.cpu().numpy(), rf) <= tol and rel_err(w2.cpu().numpy(), rw) <= 10 * tol
        f3v, w3 = ops.compute_force_tripl_virial(_t(nd3), g["des3bsupp"], g["angdescr"], g["der3bsupp"], g["der3b"],
                                                 g["intmap2b"], g["intmap3b"], ta3, te3, ttm, tipos, t,
                                                 g["numtriplet"], tpos, tbox)
        rf, rw = oracle.force_tripl(nd3, d["des3bsupp"], d["angdescr"], d["der3bsupp"], d["der3b"], d["intmap3b"],
                                    a3, e3, tm, d["numtriplet"], sh, pos, box)
        assert rel_err(f3v.cpu().numpy(), rf) <= tol and rel_err(w3.cpu().numpy(), rw) <= 10 * tol
        gn, ga, ge = ops.compute_force_radial_virial_grad(_t(pF), _t(pW), _t(nd2), g["der2b"], g["intmap2b"],
                                                          g["raddescr"], ta2, te2, ttm, tipos, t, tpos, tbox)
        rn, ra, re = oracle.grad_force_radial(pF, nd2, d["der2b"], d["intmap2b"], d["raddescr"], a2, e2, tm, sh,
                                              pos, box, pW)
        assert rel_err(gn.cpu().numpy(), rn) <= tol
        assert rel_err(ga.cpu().numpy(), ra) <= tol and rel_err(ge.cpu().numpy(), re) <= tol
        gn, ga, gck = ops.compute_force_tripl_virial_grad(_t(pF), _t(pW), _t(nd3), g["des3bsupp"], g["angdescr"],
                                                          g["der3bsupp"], g["der3b"], g["intmap2b"], g["intmap3b"],
                                                          ta3, te3, ttm, tipos, t, g["numtriplet"], tpos, tbox)
        rn, ra, rck = oracle.grad_force_tripl(pF, nd3, d["des3bsupp"], d["angdescr"], d["der3bsupp"], d["der3b"],
                                              d["intmap3b"], a3, e3, tm, d["numtriplet"], sh, pos, box, pW)
        assert rel_err(gn.cpu().numpy(), rn) <= tol
        assert rel_err(ga.cpu().numpy(), ra) <= tol
        assert np.all(gck.cpu().numpy() == 0)


def test_overflow_is_a_status_not_an_exit(ops):
    pos, box, tipos = synth.water_frames("water96", [1000])
    ctx = ops.construct_descriptors_light(4.5, 20, 190, 96, None, 2.25, 4.5, 1, dtype=torch.float32)
    with pytest.raises(ops.StafbError) as ei:
        ops.compute_descriptors_light(_t(pos.astype(np.float32)), _t(box.astype(np.float32)))
    assert ei.value.status == 1
    bad = box.copy()
    bad[0, 3] = 0.0
    ctx = ops.construct_descriptors_light(4.5, 60, 1770, 96, None, 2.25, 4.5, 1, dtype=torch.float32)
    with pytest.raises(ops.StafbError) as ei:
        ops.compute_descriptors_light(_t(pos.astype(np.float32)), _t(bad.astype(np.float32)))
    assert ei.value.status == 4
    # the context stays usable after an error
    out = ops.compute_descriptors_light(_t(pos.astype(np.float32)), _t(box.astype(np.float32)))
    assert int(out[3][0, :, 0].max()) <= 60


def test_descriptor_integer_outputs_are_deterministic(ops):
    pos, box, tipos = synth.water_frames("water768", [1100, 1101, 1102, 1103])
    _ctx(ops, np.float32, 768, 4)
    p, b = _t(pos.astype(np.float32)), _t(box.astype(np.float32))
    a = ops.compute_descriptors_light(p, b)
    for _ in range(3):
        c = ops.compute_descriptors_light(p, b)
        assert torch.equal(a[3], c[3]) and torch.equal(a[4], c[4]) and torch.equal(a[8], c[8])
        assert torch.equal(a[0], c[0]) and torch.equal(a[1], c[1])
