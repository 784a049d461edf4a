"""ctypes/numpy front end of the CPU oracle (test infrastructure).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference arm may
import this module.  It loads oracle/_build/libstaf_oracle.so (the CPU restatement of
the reference's kernel math, see staf_oracle.hpp) and, when present, the pieces of the
reference's own CPU code built into oracle/_ref/.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None
MAX_TYPES, MAX_DENSE = 4, 6


def reference_dir():
    """Root of the reference tree if one can be found: $STAF_REFERENCE_DIR, else a folder named `reference`
    beside the repository; None otherwise (the prebuilt oracle/_ref files are then used as they are)."""
    cands = [os.environ.get("STAF_REFERENCE_DIR"),
             os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.isdir(os.path.join(c, "STAF", "src")):
            return c
    return None


def build(quiet=True):
    """Compile the oracle (and oracle/_ref when the reference tree is present)."""
    ref = reference_dir()
    out = subprocess.run(["make", "-C", _HERE] + (["REF=" + ref] if ref else []), capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + out.stdout + out.stderr)
    if not quiet:
        print(out.stdout)


def lib():
    global _LIB
    if _LIB is None:
        path = os.path.join(_HERE, "_build", "libstaf_oracle.so")
        if not os.path.exists(path):
            build()
        _LIB = C.CDLL(path)
    return _LIB


def _sfx(dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError(dtype)


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dtype):
    return np.ascontiguousarray(a, dtype=dtype)


def shape_desc(nt, tipos, Fr, Fa, widths):
    d = np.zeros(20, np.int32)
    d[0] = nt
    d[1:1 + nt] = tipos
    d[5:5 + nt] = Fr
    d[9:9 + nt] = Fa
    d[13] = len(widths)
    d[14:14 + len(widths)] = widths
    return d


def n_params(sd):
    return lib().stafo_n_params(_p(sd))


def n_emb(sd):
    return lib().stafo_n_emb(_p(sd))


def offsets(sd, t):
    o = np.zeros(6, np.int32)
    lib().stafo_offsets(_p(sd), int(t), _p(o))
    return dict(a2=int(o[0]), a3=int(o[1]), mu=int(o[2]), w=int(o[3]), emb=int(o[4]), size=int(o[5]))


def set_threads(n):
    lib().stafo_set_threads(int(n))


def max_threads():
    return lib().stafo_max_threads()


def fill_repulsion(Rc, Rs, Ra, dtype):
    out = np.zeros(5, dtype)
    getattr(lib(), "stafo_fill_repulsion_" + _sfx(dtype))(C.c_double(Rc), C.c_double(Rs), C.c_double(Ra), _p(out))
    return out


def neighbour_list(Rc, nr, pos, box, dtype):
    pos = _c(pos, dtype).reshape(-1, 3)
    box = _c(box, dtype)
    N = pos.shape[0]
    frac = np.zeros((N, 3), dtype)
    wth = np.zeros((N, nr), np.int32)
    how = np.zeros(N, np.int32)
    d2 = np.zeros((N, nr), dtype)
    nc = np.zeros(3, np.int32)
    st = getattr(lib(), "stafo_neighbour_list_" + _sfx(dtype))(
        C.c_double(Rc), nr, N, _p(pos), _p(box), _p(frac), _p(wth), _p(how), _p(d2), _p(nc))
    return dict(status=st, frac=frac, with_=wth, howmany=how, d2=d2, ncell=nc)


def descriptors(Rc, Rs, Ra, nr, na, pos, box, dtype):
    pos = _c(pos, dtype)
    box = _c(box, dtype)
    nf = box.shape[0]
    N = pos.shape[1] // 3
    o = dict(
        raddescr=np.zeros((nf, N, nr), dtype), angdescr=np.zeros((nf, N, na), dtype),
        des3bsupp=np.zeros((nf, N, nr), dtype), intmap2b=np.zeros((nf, N, nr + 1), np.int32),
        intmap3b=np.zeros((nf, N, na * 2), np.int32), der2b=np.zeros((nf, N, 3, nr), dtype),
        der3b=np.zeros((nf, N, 3, na * 2), dtype), der3bsupp=np.zeros((nf, N, 3, nr), dtype),
        numtriplet=np.zeros((nf, N), np.int32), nbr_d2=np.zeros((nf, N, nr), dtype))
    st = getattr(lib(), "stafo_descriptors_" + _sfx(dtype))(
        C.c_double(Rc), C.c_double(Rs), C.c_double(Ra), nr, na, nf, N, _p(pos), _p(box), _p(o["raddescr"]),
        _p(o["angdescr"]), _p(o["des3bsupp"]), _p(o["intmap2b"]), _p(o["intmap3b"]), _p(o["der2b"]), _p(o["der3b"]),
        _p(o["der3bsupp"]), _p(o["numtriplet"]), _p(o["nbr_d2"]))
    o["status"] = st
    return o


def af_radial(raddescr, intmap2b, alpha2b, e2, type_map):
    dt = raddescr.dtype
    nf, Nl, nr = raddescr.shape
    Fr = alpha2b.shape[1]
    out = np.zeros((nf, Nl, Fr), dt)
    getattr(lib(), "stafo_af_radial_" + _sfx(dt))(nf, Nl, nr, Fr, _p(_c(raddescr, dt)), _p(_c(intmap2b, np.int32)),
                                                  _p(_c(alpha2b, dt)), _p(_c(e2, dt)), _p(_c(type_map, np.int32)),
                                                  _p(out))
    return out


def af_angular(angdescr, des3bsupp, intmap3b, alpha3b, e3, type_map, numtriplet):
    dt = angdescr.dtype
    nf, Nl, na = angdescr.shape
    nr = des3bsupp.shape[2]
    Fa = alpha3b.shape[1] // 3
    out = np.zeros((nf, Nl, Fa), dt)
    getattr(lib(), "stafo_af_angular_" + _sfx(dt))(
        nf, Nl, nr, na, Fa, _p(_c(angdescr, dt)), _p(_c(des3bsupp, dt)), _p(_c(intmap3b, np.int32)),
        _p(_c(alpha3b, dt)), _p(_c(e3, dt)), _p(_c(type_map, np.int32)), _p(_c(numtriplet, np.int32)), _p(out))
    return out


def _vir_in(pos, box, dt):
    if pos is None:
        return None, None
    return _c(pos, dt), _c(box, dt)


def force_radial(netderiv, der2b, intmap2b, raddescr, alpha2b, e2, type_map, shift, pos=None, box=None):
    """ComputeForceRadial; with pos[nf,3N] and box[nf,6] the ...Virial variant: returns (force, virial[nf,9])."""
    dt = raddescr.dtype
    nf, Nl, nr = raddescr.shape
    Fr = alpha2b.shape[1]
    N = len(type_map)
    out = np.zeros((nf, 3 * N), dt)
    p_, b_ = _vir_in(pos, box, dt)
    vir = None if pos is None else np.zeros((nf, 9), dt)
    getattr(lib(), "stafo_force_radial_" + _sfx(dt))(
        nf, Nl, N, nr, Fr, int(shift), _p(_c(netderiv, dt)), _p(_c(der2b, dt)), _p(_c(intmap2b, np.int32)),
        _p(_c(raddescr, dt)), _p(_c(alpha2b, dt)), _p(_c(e2, dt)), _p(_c(type_map, np.int32)), _p(out),
        _p(p_), _p(b_), _p(vir))
    return out if pos is None else (out, vir)


def force_tripl(netderiv, des3bsupp, angdescr, der3bsupp, der3b, intmap3b, alpha3b, e3, type_map, numtriplet, shift,
                pos=None, box=None):
    """ComputeForceTripl; with pos and box the ...Virial variant: returns (force, virial[nf,9])."""
    dt = angdescr.dtype
    nf, Nl, na = angdescr.shape
    nr = des3bsupp.shape[2]
    Fa = alpha3b.shape[1] // 3
    N = len(type_map)
    out = np.zeros((nf, 3 * N), dt)
    p_, b_ = _vir_in(pos, box, dt)
    vir = None if pos is None else np.zeros((nf, 9), dt)
    getattr(lib(), "stafo_force_tripl_" + _sfx(dt))(
        nf, Nl, N, nr, na, Fa, int(shift), _p(_c(netderiv, dt)), _p(_c(des3bsupp, dt)), _p(_c(angdescr, dt)),
        _p(_c(der3bsupp, dt)), _p(_c(der3b, dt)), _p(_c(intmap3b, np.int32)), _p(_c(alpha3b, dt)), _p(_c(e3, dt)),
        _p(_c(type_map, np.int32)), _p(_c(numtriplet, np.int32)), _p(out), _p(p_), _p(b_), _p(vir))
    return out if pos is None else (out, vir)


def grad_af_radial(prevgrad, raddescr, intmap2b, alpha2b, e2, type_map):
    dt = raddescr.dtype
    nf, Nl, nr = raddescr.shape
    nt, Fr = alpha2b.shape
    ga, ge = np.zeros((nt, Fr), dt), np.zeros((nt, Fr), dt)
    getattr(lib(), "stafo_grad_af_radial_" + _sfx(dt))(
        nf, Nl, nr, Fr, nt, _p(_c(prevgrad, dt)), _p(_c(raddescr, dt)), _p(_c(intmap2b, np.int32)),
        _p(_c(alpha2b, dt)), _p(_c(e2, dt)), _p(_c(type_map, np.int32)), _p(ga), _p(ge))
    return ga, ge


def grad_af_angular(prevgrad, angdescr, des3bsupp, intmap3b, alpha3b, e3, type_map, numtriplet):
    dt = angdescr.dtype
    nf, Nl, na = angdescr.shape
    nr = des3bsupp.shape[2]
    Cc = alpha3b.shape[0]
    Fa = alpha3b.shape[1] // 3
    ga, ge = np.zeros((Cc, 3 * Fa), dt), np.zeros((Cc, Fa), dt)
    getattr(lib(), "stafo_grad_af_angular_" + _sfx(dt))(
        nf, Nl, nr, na, Fa, Cc, _p(_c(prevgrad, dt)), _p(_c(angdescr, dt)), _p(_c(des3bsupp, dt)),
        _p(_c(intmap3b, np.int32)), _p(_c(alpha3b, dt)), _p(_c(e3, dt)), _p(_c(type_map, np.int32)),
        _p(_c(numtriplet, np.int32)), _p(ga), _p(ge))
    return ga, ge


def grad_force_radial(prevgrad, netderiv, der2b, intmap2b, raddescr, alpha2b, e2, type_map, shift, pos=None,
                      box=None, prevgrad_virial=None):
    """ComputeForceRadialGrad; with pos, box and prevgrad_virial[nf,9] the ...VirialGrad variant."""
    dt = raddescr.dtype
    p_, b_ = _vir_in(pos, box, dt)
    w_ = None if prevgrad_virial is None else _c(prevgrad_virial, dt)
    nf, Nl, nr = raddescr.shape
    nt, Fr = alpha2b.shape
    N = len(type_map)
    gn, ga, ge = np.zeros((nf, Nl, Fr), dt), np.zeros((nt, Fr), dt), np.zeros((nt, Fr), dt)
    getattr(lib(), "stafo_grad_force_radial_" + _sfx(dt))(
        nf, Nl, N, nr, Fr, nt, int(shift), _p(_c(prevgrad, dt)), _p(_c(netderiv, dt)), _p(_c(der2b, dt)),
        _p(_c(intmap2b, np.int32)), _p(_c(raddescr, dt)), _p(_c(alpha2b, dt)), _p(_c(e2, dt)),
        _p(_c(type_map, np.int32)), _p(gn), _p(ga), _p(ge), _p(p_), _p(b_), _p(w_))
    return gn, ga, ge


def grad_force_tripl(prevgrad, netderiv, des3bsupp, angdescr, der3bsupp, der3b, intmap3b, alpha3b, e3, type_map,
                     numtriplet, shift, pos=None, box=None, prevgrad_virial=None):
    """ComputeForceTriplGrad; with pos, box and prevgrad_virial[nf,9] the ...VirialGrad variant."""
    dt = angdescr.dtype
    p_, b_ = _vir_in(pos, box, dt)
    w_ = None if prevgrad_virial is None else _c(prevgrad_virial, dt)
    nf, Nl, na = angdescr.shape
    nr = des3bsupp.shape[2]
    Cc = alpha3b.shape[0]
    Fa = alpha3b.shape[1] // 3
    N = len(type_map)
    gn, ga, gc = np.zeros((nf, Nl, Fa), dt), np.zeros((Cc, 3 * Fa), dt), np.zeros((Cc, Fa), dt)
    getattr(lib(), "stafo_grad_force_tripl_" + _sfx(dt))(
        nf, Nl, N, nr, na, Fa, Cc, int(shift), _p(_c(prevgrad, dt)), _p(_c(netderiv, dt)), _p(_c(des3bsupp, dt)),
        _p(_c(angdescr, dt)), _p(_c(der3bsupp, dt)), _p(_c(der3b, dt)), _p(_c(intmap3b, np.int32)),
        _p(_c(alpha3b, dt)), _p(_c(e3, dt)), _p(_c(type_map, np.int32)), _p(_c(numtriplet, np.int32)), _p(gn), _p(ga),
        _p(gc), _p(p_), _p(b_), _p(w_))
    return gn, ga, gc


def mlp_eval(widths, af, mu, w, ebar=None, u=None):
    """Forward + d(sum e)/dAF; with ebar/u also the backward (g_w, g_mu, g_af)."""
    dt = af.dtype
    n, F = af.shape
    widths = np.asarray(widths, np.int32)
    e = np.zeros(n, dt)
    nd = np.zeros((n, F), dt)
    af, mu, w = _c(af, dt), _c(mu, dt), _c(w, dt)
    fn = getattr(lib(), "stafo_mlp_eval_" + _sfx(dt))
    if ebar is None and u is None:
        fn(F, len(widths), _p(widths), n, _p(af), _p(mu), _p(w), _p(e), _p(nd), None, None, None, None, None)
        return e, nd
    ebar = np.zeros(n, dt) if ebar is None else _c(ebar, dt)
    u = np.zeros((n, F), dt) if u is None else _c(u, dt)
    gw, gmu, gaf = np.zeros_like(w), np.zeros(F, dt), np.zeros((n, F), dt)
    fn(F, len(widths), _p(widths), n, _p(af), _p(mu), _p(w), _p(e), _p(nd), _p(ebar), _p(u), _p(gw), _p(gmu), _p(gaf))
    return e, nd, gw, gmu, gaf


def energy_force_grad(cfg, sd, pos, box, type_map, theta, emb, dtype, per_atom_energy=True, with_grad=False,
                      e_label=None, f_label=None, pe=1.0, pf=1.0, pb=1.0, alpha_bound=5.0, loss_kind=0):
    """cfg = dict(Rc, Rs, Ra, nr, na).  Returns dict(status, energy, force[, losses, grad])."""
    pos = _c(pos, dtype)
    box = _c(box, dtype)
    nf = box.shape[0]
    N = pos.shape[1] // 3
    theta, emb = _c(theta, dtype), _c(emb, dtype)
    energy = np.zeros(nf, dtype)
    force = np.zeros((nf, 3 * N), dtype)
    losses = np.zeros(4, np.float64)
    grad = np.zeros_like(theta) if with_grad else None
    el = _c(e_label, dtype) if with_grad else None
    fl = _c(f_label, dtype) if with_grad else None
    st = getattr(lib(), "stafo_energy_force_grad_" + _sfx(dtype))(
        C.c_double(cfg["Rc"]), C.c_double(cfg["Rs"]), C.c_double(cfg["Ra"]), cfg["nr"], cfg["na"], _p(sd), nf,
        _p(pos), _p(box), _p(_c(type_map, np.int32)), _p(theta), _p(emb), int(per_atom_energy), _p(energy), _p(force),
        int(with_grad), _p(el), _p(fl), C.c_double(pe), C.c_double(pf), C.c_double(pb), C.c_double(alpha_bound),
        int(loss_kind), _p(losses), _p(grad))
    out = dict(status=st, energy=energy, force=force)
    if with_grad:
        out["losses"] = losses
        out["grad"] = grad
    return out


def energy_force_virial_grad(cfg, sd, pos, box, type_map, theta, emb, dtype, per_atom_energy=True, with_grad=False,
                             e_label=None, f_label=None, v_label=None, pe=1.0, pf=1.0, pv=1.0, pb=1.0,
                             alpha_bound=5.0, loss_kind=0):
    """energy_force_grad with the virial [nf,9] and, with_grad, the virial term of the loss
    (STAF/staf_models/staf_model.py:313-384): losses = (loss, loss_e, loss_bound, loss_f, loss_v)."""
    pos = _c(pos, dtype)
    box = _c(box, dtype)
    nf = box.shape[0]
    N = pos.shape[1] // 3
    theta, emb = _c(theta, dtype), _c(emb, dtype)
    energy = np.zeros(nf, dtype)
    force = np.zeros((nf, 3 * N), dtype)
    virial = np.zeros((nf, 9), dtype)
    losses = np.zeros(5, np.float64)
    grad = np.zeros_like(theta) if with_grad else None
    el = _c(e_label, dtype) if with_grad else None
    fl = _c(f_label, dtype) if with_grad else None
    vl = _c(v_label, dtype) if with_grad else None
    st = getattr(lib(), "stafo_energy_force_virial_grad_" + _sfx(dtype))(
        C.c_double(cfg["Rc"]), C.c_double(cfg["Rs"]), C.c_double(cfg["Ra"]), cfg["nr"], cfg["na"], _p(sd), nf,
        _p(pos), _p(box), _p(_c(type_map, np.int32)), _p(theta), _p(emb), int(per_atom_energy), _p(energy), _p(force),
        _p(virial), int(with_grad), _p(el), _p(fl), _p(vl), C.c_double(pe), C.c_double(pf), C.c_double(pv),
        C.c_double(pb), C.c_double(alpha_bound), int(loss_kind), _p(losses), _p(grad))
    out = dict(status=st, energy=energy, force=force, virial=virial)
    if with_grad:
        out["losses"] = losses
        out["grad"] = grad
    return out


# --------------------------------------------------------------------------
# The reference's own CPU code, compiled into oracle/_ref (may be absent).
def ref_available():
    return all(os.path.exists(os.path.join(_HERE, "_ref", n))
               for n in ("libref_nl_f32.so", "libref_nl_f64.so", "libref_mlp.so"))


def ref_neighbour_list(Rc, nr, pos, box, dtype):
    """Reference CPU cell list (STAF/src/descriptor_builder/cell_list.cu.cc:1080)."""
    L = C.CDLL(os.path.join(_HERE, "_ref", "libref_nl_%s.so" % _sfx(dtype)))
    assert L.ref_real_bytes() == np.dtype(dtype).itemsize
    pos = _c(pos, dtype).reshape(-1, 3)
    box = _c(box, dtype)
    N = pos.shape[0]
    wth = np.zeros((N, nr), np.int32)
    how = np.zeros(N, np.int32)
    d2 = np.zeros((N, nr), dtype)
    nc = np.zeros(3, np.int32)
    over = L.ref_neighbour_list(C.c_double(Rc), nr, N, _p(pos), _p(box), _p(wth), _p(how), _p(d2), _p(nc))
    return dict(overflow=over, with_=wth, howmany=how, d2=d2, ncell=nc)


def ref_mlp_eval(model_dir, af_per_type, dtype):
    """Reference native MLP (libstaf/src/mlp/staf_mlp_ort.cc:196-242): returns (0.5*sum e, dE/dAF per type)."""
    L = C.CDLL(os.path.join(_HERE, "_ref", "libref_mlp.so"))
    prec = 0 if np.dtype(dtype) == np.float32 else 1
    n_atoms = np.array([a.shape[0] for a in af_per_type], np.int32)
    n_af = np.array([a.shape[1] for a in af_per_type], np.int32)
    packed = np.concatenate([_c(a, dtype).ravel() for a in af_per_type])
    energy = np.zeros(1, dtype)
    dE = np.zeros_like(packed)
    rc = L.ref_mlp_eval(model_dir.encode(), prec, len(af_per_type), _p(n_atoms), _p(n_af), _p(packed), _p(energy),
                        _p(dE))
    if rc != 0:
        raise RuntimeError("ref_mlp_eval rc=%d" % rc)
    outs, o = [], 0
    for a in af_per_type:
        outs.append(dE[o:o + a.size].reshape(a.shape))
        o += a.size
    return energy[0], outs
