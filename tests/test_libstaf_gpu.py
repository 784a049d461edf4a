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
    how = np.zeros(N, np.int32)
    e = C.c_double()
    f = np.zeros(3 * N)
    xx = np.ascontiguousarray(x, np.float64)
    assert lib.staf_compute(m, N, 0, xx.ctypes.data, box.ctypes.data, types.ctypes.data, how.ctypes.data,
                            how.ctypes.data, 1, C.byref(e), f.ctypes.data, None) == -10
    # a compressed box saturates the radial buffer: an error code, not an exit
    small = box * 0.6
    assert _compute(lib, m, x * 0.6, small, types)[0] == -11
    # the handle is still usable
    assert _compute(lib, m, x, box, types)[0] == 0
    lib.staf_free(m)
    assert lib.staf_load(b"/nonexistent/model/dir", None) is None
