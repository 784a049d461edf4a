"""GPU test of the libstaf C API (include/staf.h) on the reference's real frame and exported model."""
import ctypes as C

import numpy as np
import pytest

from conftest import rel_err

pytestmark = pytest.mark.gpu


class StafOptions(C.Structure):
    _fields_ = [("mlp_backend", C.c_int), ("device_id", C.c_int), ("precision", C.c_int), ("reserved", C.c_int)]


@pytest.fixture(scope="module")
def lib():
    from alphanesgpu_b200 import _lib
    L = _lib.lib()
    L.staf_load.restype = C.c_void_p
    L.staf_load.argtypes = [C.c_char_p, C.POINTER(StafOptions)]
    L.staf_compute.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 5 + [C.c_int] + [C.c_void_p] * 3
    L.staf_free.argtypes = [C.c_void_p]
    return L


def _compute(lib, m, x, box, types):
    n = len(types)
    e = C.c_double()
    f = np.zeros(3 * n)
    vir = np.zeros(6)
    x = np.ascontiguousarray(x, np.float64)
    box = np.ascontiguousarray(box, np.float64)
    types = np.ascontiguousarray(types, np.int32)
    rc = lib.staf_compute(m, n, 0, x.ctypes.data, box.ctypes.data, types.ctypes.data, None, None, 0, C.byref(e),
                          f.ctypes.data, vir.ctypes.data)
    return rc, e.value, f, vir


@pytest.mark.parametrize("precision,tol", [(0, 1e-5), (1, 1e-11)])
def test_staf_compute_frame0(lib, oracle, frame0, precision, tol):
    opt = StafOptions()
    lib.staf_options_default(C.byref(opt))
    assert (opt.mlp_backend, opt.device_id, opt.precision) == (0, 0, 0)
    opt.precision = precision
    m = lib.staf_load(frame0["dir"].encode(), C.byref(opt))
    assert m
    shape = frame0["shape"]
    dt = np.float32 if precision == 0 else np.float64
    ref = oracle.energy_force_grad(frame0["cfg"], shape.desc(), frame0["pos"], frame0["box"], shape.type_map,
                                   frame0["theta"], frame0["emb"], dt, per_atom_energy=False)
    # caller order: interleave the species so that the type-sorted remap is exercised
    N = shape.N
    perm = np.random.default_rng(1).permutation(N)
    x = frame0["pos"].reshape(N, 3)[perm].ravel()
    types = shape.type_map[perm]
    rc, e, f, vir = _compute(lib, m, x, frame0["box"][0], types)
    assert rc == 0
    assert abs(e - float(ref["energy"][0])) <= tol * abs(float(ref["energy"][0])) * 10
    fref = ref["force"].reshape(N, 3)[perm].ravel()
    assert rel_err(f, fref) <= tol
    if precision == 0:
        # recorded by the reference for this frame: E = -102.25880432 (TF) / -102.25872 (libstaf)
        # (test/test-lammps-STAF-inference-STAF-comp/results/frames.csv:2)
        assert abs(e - (-102.25880432)) < 1.2e-4
    # the same species array again (the cached slot map and, from the third call on, the replayed graph), moved
    # atoms; then the same atoms in another caller order with the same species counts (the map is re-made)
    for k in range(3):
        rc, e_k, f_k, _ = _compute(lib, m, x, frame0["box"][0], types)
        assert rc == 0 and abs(e_k - e) <= tol * abs(e) and rel_err(f_k, fref) <= tol, k  # forces: atomic sums
    perm2 = np.random.default_rng(2).permutation(N)
    rc, e_p, f_p, _ = _compute(lib, m, frame0["pos"].reshape(N, 3)[perm2].ravel(), frame0["box"][0],
                               shape.type_map[perm2])
    assert rc == 0 and abs(e_p - e) <= tol * abs(e) * 10
    assert rel_err(f_p, ref["force"].reshape(N, 3)[perm2].ravel()) <= tol
    # a second call with fewer atoms of another composition reuses the handle
    sub = np.concatenate([np.arange(0, 200), np.arange(256, 256 + 400)])
    rc2, e2, f2, _ = _compute(lib, m, frame0["pos"].reshape(N, 3)[sub].ravel(), frame0["box"][0],
                              shape.type_map[sub])
    assert rc2 == 0 and np.isfinite(e2)
    lib.staf_free(m)


def test_staf_compute_error_codes(lib, frame0):
    m = lib.staf_load(frame0["dir"].encode(), None)
    assert m
    N = frame0["shape"].N
    x, box, types = frame0["pos"][0], frame0["box"][0], frame0["shape"].type_map
    assert _compute(lib, m, x[:0], box, types[:0])[0] == -3
    bad = box.copy()
    bad[3] = 0.0
    assert _compute(lib, m, x, bad, types)[0] == -7
    t2 = types.copy()
    t2[5] = 7
    assert _compute(lib, m, x, box, t2)[0] == -8
    how = np.ones(N, np.int32)
    bad_with = np.full(N, N + 5, np.int32)
    e = C.c_double()
    f = np.zeros(3 * N)
    xx = np.ascontiguousarray(x, np.float64)
    assert lib.staf_compute(m, N, 0, xx.ctypes.data, box.ctypes.data, types.ctypes.data, how.ctypes.data,
                            bad_with.ctypes.data, 1, C.byref(e), f.ctypes.data, None) == -9
    # a compressed box saturates the radial buffer: an error code, not an exit
    small = box * 0.6
    assert _compute(lib, m, x * 0.6, small, types)[0] == -11
    # the handle is still usable
    assert _compute(lib, m, x, box, types)[0] == 0
    lib.staf_free(m)
    assert lib.staf_load(b"/nonexistent/model/dir", None) is None


def _wrapped(frame0):
    """frame 0 wrapped into the (cubic) box: positions [N,3], L, species."""
    N = frame0["shape"].N
    L = float(frame0["box"][0][0])
    x = frame0["pos"].reshape(N, 3)
    return x - np.floor(x / L) * L, L, frame0["shape"].type_map.astype(np.int32)


def _call(lib, m, fn, nlocal, nghost, x, box, types, how=None, wth=None, maxneigh=0):
    nall = nlocal + nghost
    e = C.c_double()
    f = np.zeros(3 * nall)
    vir = np.zeros(6)
    x = np.ascontiguousarray(x, np.float64)
    box = np.ascontiguousarray(box, np.float64)
    types = np.ascontiguousarray(types, np.int32)
    if fn == "list":
        rc = lib.staf_compute(m, nlocal, nghost, x.ctypes.data, box.ctypes.data, types.ctypes.data, how.ctypes.data,
                              wth.ctypes.data, maxneigh, C.byref(e), f.ctypes.data, vir.ctypes.data)
    else:
        rc = lib.staf_compute_domain(m, nlocal, nghost, x.ctypes.data, box.ctypes.data, types.ctypes.data,
                                     C.byref(e), f.ctypes.data, vir.ctypes.data)
    return rc, e.value, f.reshape(nall, 3), vir


# fp32: the two paths round the pair vectors differently (Cartesian differences of coordinates up to L + Rc
# against minimum-image differences of fractional coordinates), which moves forces by ~2e-5 relative; the bar
# there is the reference's own domain-decomposition bar of 1e-4 (test/test-lammps-dd-parity/run_dd_parity.sh:14-15)
@pytest.mark.parametrize("precision,tol", [(0, 1e-4), (1, 1e-10)])
def test_staf_compute_caller_list_with_ghost_images(lib, frame0, precision, tol):
    """The LAMMPS contract (lammps/USER-STAF/pair_staf.cpp:180-256 of the reference): owned atoms + ghost
    images, rows cutoff-filtered and distance-sorted by the caller, no wrap inside the library, ghost forces
    folded back by the caller.  Must reproduce the library's own minimum-image result."""
    lib.staf_compute_domain.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 6
    opt = StafOptions()
    lib.staf_options_default(C.byref(opt))
    opt.precision = precision
    m = lib.staf_load(frame0["dir"].encode(), C.byref(opt))
    xw, L, types = _wrapped(frame0)
    N = len(types)
    box = frame0["box"][0]
    rc0, e0, f0, v0 = _compute(lib, m, xw.ravel(), box, types)
    assert rc0 == 0
    Rc = frame0["cfg"]["Rc"]
    # ghost shell: every periodic image that lies within Rc of the box
    gx, gowner = [], []
    for sx in (-1, 0, 1):
        for sy in (-1, 0, 1):
            for sz in (-1, 0, 1):
                if (sx, sy, sz) == (0, 0, 0):
                    continue
                img = xw + np.array([sx, sy, sz]) * L
                keep = np.all((img > -Rc) & (img < L + Rc), axis=1)
                gx.append(img[keep])
                gowner.append(np.nonzero(keep)[0])
    gx, gowner = np.concatenate(gx), np.concatenate(gowner)
    xall = np.concatenate([xw, gx])
    tall = np.concatenate([types, types[gowner]])
    nghost = len(gowner)
    maxneigh = 64
    how = np.zeros(N, np.int32)
    wth = np.zeros((N, maxneigh), np.int32)
    for i in range(N):
        d2 = ((xall - xw[i]) ** 2).sum(1)
        d2[i] = np.inf
        idx = np.nonzero(d2 < Rc * Rc)[0]
        idx = idx[np.argsort(d2[idx], kind="stable")]
        how[i] = len(idx)
        wth[i, :len(idx)] = idx
    assert how.max() <= 60
    rc, e, f, v = _call(lib, m, "list", N, nghost, xall.ravel(), box, tall, how, wth, maxneigh)
    assert rc == 0
    folded = f[:N].copy()
    np.add.at(folded, gowner, f[N:])
    assert abs(e - e0) <= 10 * tol * abs(e0)
    assert rel_err(folded, f0.reshape(N, 3)) <= tol
    assert rel_err(v[:3], v0[:3]) <= 20 * tol and np.all(v[3:] == 0)
    lib.staf_free(m)


@pytest.mark.parametrize("nslab", [2, 4])
@pytest.mark.parametrize("precision,tol", [(0, 1e-4), (1, 1e-10)])
def test_staf_compute_domain_slab_parity(lib, frame0, nslab, precision, tol):
    """Domain-decomposition parity, the reference's test/test-lammps-dd-parity (1 vs 2 vs 4 ranks: max|dE|,
    max|dF| <= 1e-4) restated without LAMMPS: z-slabs with one-cutoff halos, ghost forces folded back."""
    lib.staf_compute_domain.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 6
    opt = StafOptions()
    lib.staf_options_default(C.byref(opt))
    opt.precision = precision
    m = lib.staf_load(frame0["dir"].encode(), C.byref(opt))
    xw, L, types = _wrapped(frame0)
    N = len(types)
    box = frame0["box"][0]
    rc0, e0, f0, v0 = _compute(lib, m, xw.ravel(), box, types)
    assert rc0 == 0
    Rc = frame0["cfg"]["Rc"]
    w = L / nslab
    etot, ftot, vtot = 0.0, np.zeros((N, 3)), np.zeros(6)
    for r in range(nslab):
        z = xw[:, 2]
        owned = np.nonzero((z >= r * w) & (z < (r + 1) * w))[0]
        dz = (z - (r + 0.5) * w + 0.5 * L) % L - 0.5 * L  # periodic distance to the slab centre
        ghost = np.nonzero((np.abs(dz) < 0.5 * w + Rc) & ~((z >= r * w) & (z < (r + 1) * w)))[0]
        if nslab == 2:
            ghost = np.unique(ghost)
        ids = np.concatenate([owned, ghost])
        rc, e, f, v = _call(lib, m, "domain", len(owned), len(ghost), xw[ids].ravel(), box, types[ids])
        assert rc == 0
        etot += e
        np.add.at(ftot, ids, f)
        vtot += v
    assert abs(etot - e0) <= 10 * tol * abs(e0)
    assert rel_err(ftot, f0.reshape(N, 3)) <= tol
    assert rel_err(vtot[:3], v0[:3]) <= 20 * tol
    lib.staf_free(m)


class StafMlpEval(C.Structure):
    _fields_ = [("n_type", C.c_int), ("n_atoms", C.c_void_p), ("n_af", C.c_void_p), ("af_f32", C.c_void_p),
                ("af_f64", C.c_void_p), ("energy_f32", C.c_void_p), ("energy_f64", C.c_void_p),
                ("dE_daf_f32", C.c_void_p), ("dE_daf_f64", C.c_void_p)]


@pytest.mark.parametrize("precision,tag,tol", [(0, "f32", 5e-6), (1, "f64", 1e-12)])
def test_staf_mlp_eval_matches_the_reference_native_evaluator(lib, frame0, precision, tag, tol):
    """include/staf_mlp.h (the reference's libstaf/include/staf_mlp.h:17-42) on the fingerprints and outputs
    recorded from the reference's own native Dense evaluator (tests/golden/ref_mlp.npz, made by
    tests/golden/make_ref_fixtures.py from libstaf/src/mlp/staf_mlp_ort.cc)."""
    import os
    from conftest import GOLDEN
    g = np.load(os.path.join(GOLDEN, "ref_mlp.npz"))
    dt = np.float32 if precision == 0 else np.float64
    lib.staf_mlp_create.restype = C.c_void_p
    lib.staf_mlp_create.argtypes = [C.c_int, C.c_char_p, C.c_int, C.c_int]
    lib.staf_mlp_eval.argtypes = [C.c_void_p, C.POINTER(StafMlpEval)]
    lib.staf_mlp_destroy.argtypes = [C.c_void_p]
    for fn in (lib.staf_mlp_ntypes, lib.staf_mlp_precision):
        fn.argtypes = [C.c_void_p]
    lib.staf_mlp_n_af.argtypes = [C.c_void_p, C.c_int]
    h = lib.staf_mlp_create(2, frame0["dir"].encode(), precision, 0)
    assert h
    assert lib.staf_mlp_ntypes(h) == 2 and lib.staf_mlp_precision(h) == precision
    afs = [np.ascontiguousarray(g["af%d" % k], dt) for k in (0, 1)]
    assert [lib.staf_mlp_n_af(h, k) for k in (0, 1)] == [a.shape[1] for a in afs]
    for rep in range(2):
        n_atoms = np.array([a.shape[0] for a in afs], np.int32)
        n_af = np.array([a.shape[1] for a in afs], np.int32)
        packed = np.concatenate([a.ravel() for a in afs])
        energy = np.zeros(1, dt)
        dE = np.zeros_like(packed)
        io = StafMlpEval(2, n_atoms.ctypes.data, n_af.ctypes.data, None, None, None, None, None, None)
        if precision == 0:
            io.af_f32, io.energy_f32, io.dE_daf_f32 = packed.ctypes.data, energy.ctypes.data, dE.ctypes.data
        else:
            io.af_f64, io.energy_f64, io.dE_daf_f64 = packed.ctypes.data, energy.ctypes.data, dE.ctypes.data
        assert lib.staf_mlp_eval(h, C.byref(io)) == 0
        ref_d = np.concatenate([g["%s_d%d" % (tag, k)].ravel()[:a.size] for k, a in enumerate(afs)])
        ref_e = float(g["%s_energy" % tag])
        if rep == 0:
            assert rel_err(dE, ref_d) <= tol
            assert abs(float(energy[0]) - ref_e) <= 50 * tol * abs(ref_e)
            full = dE.copy()
            afs = [a[:3] for a in afs]  # next: fewer atoms of each type (the model's counts change)
        else:
            # the first 3 atoms of each type: the same rows of the full result
            n0 = g["af0"].shape[0] * g["af0"].shape[1]
            want = np.concatenate([full[:3 * afs[0].shape[1]], full[n0:n0 + 3 * afs[1].shape[1]]])
            assert rel_err(dE, want) <= tol
    bad = StafMlpEval(3, None, None, None, None, None, None, None, None)
    assert lib.staf_mlp_eval(h, C.byref(bad)) != 0
    lib.staf_mlp_destroy(h)
