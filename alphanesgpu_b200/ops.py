"""The reference's operator surface on torch CUDA tensors.

Function names, argument order and tensor shapes are those of the TensorFlow custom ops of
the reference (REGISTER_OP in STAF/src/*/reforce.cc, called from STAF/source_routine/*.py);
each function forwards to the C ABI entry point of the same operator in include/stafb.h.
torch is used for device memory and streams only.

Like the reference, the geometry configuration is process state set by
construct_descriptors_light(); unlike the reference it is kept per (device, dtype) and
nothing here ever exits the process - saturated buffers raise StafbError.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import StafbError, check  # noqa: F401

_CTX = {}
_LAST = {}


class Context:
    """Owns one stafb_ctx (cutoffs, buffer sizes, per-device scratch)."""

    def __init__(self, radial_cutoff, radial_buffer, angular_buffer, numpar, rs, ra, max_batch, dtype, device=None):
        self.dtype = torch.float32 if dtype in (torch.float32, np.float32, "float", "float32") else torch.float64
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.Rc, self.Rs, self.Ra = float(radial_cutoff), float(rs), float(ra)
        self.nr, self.na, self.n_max, self.max_batch = int(radial_buffer), int(angular_buffer), int(numpar), int(max_batch)
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(_lib.lib().stafb_create(C.byref(h), 0 if self.dtype == torch.float32 else 1, self.Rc, self.Rs,
                                          self.Ra, self.nr, self.na, self.n_max, self.max_batch), "stafb_create")
        self.h = h

    def close(self):
        if getattr(self, "h", None):
            _lib.lib().stafb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def stream(self):
        return C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def status(self):
        return _lib.lib().stafb_status(self.h, self.stream())

    def raise_on_status(self, where):
        check(self.status(), where)

    def core_coefficients(self):
        out = np.zeros(5)
        _lib.lib().stafb_core_coefficients(self.h, out.ctypes.data_as(C.c_void_p))
        return out


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _ctx_for(t):
    key = (t.device.index if t.device.index is not None else torch.cuda.current_device(), t.dtype)
    if key not in _CTX:
        raise RuntimeError("STAF: operator called before construct_descriptors_light for %s" % (key,))
    return _CTX[key]


def _real(ctx, *ts):
    out = []
    for t in ts:
        if t.dtype != ctx.dtype or not t.is_cuda:
            raise TypeError("expected a CUDA tensor of dtype %s" % ctx.dtype)
        out.append(t.contiguous())
    return out


def _int(*ts):
    return [t.to(torch.int32).contiguous() for t in ts]


def construct_descriptors_light(radial_cutoff, radial_buffer, angular_buffer, numpar, boxer, rs, ra, max_batch,
                                dtype=torch.float32, device=None):
    """Op ConstructDescriptorsLight (descriptor_builder/reforce.cc:182-238): stores the geometry
    configuration and allocates the device scratch.  `boxer` is ignored, as in the reference."""
    ctx = Context(radial_cutoff, radial_buffer, angular_buffer, numpar, rs, ra, max_batch, dtype, device)
    key = (ctx.device.index, ctx.dtype)
    old = _CTX.pop(key, None)
    if old is not None:
        old.close()
    _CTX[key] = ctx
    return ctx


def compute_descriptors_light(positions, boxer, with_angular=True, ctx=None):
    """Op ComputeDescriptorsLight -> (raddescr, angdescr, des3bsupp, intmap2b, intmap3b, der2b, der3b,
    der3bsupp, numtriplet).  Raises StafbError where the reference prints and exits."""
    ctx = ctx or _ctx_for(positions)
    positions, boxer = _real(ctx, positions, boxer)
    nf, N = boxer.shape[0], positions.shape[1] // 3
    nr, na = ctx.nr, ctx.na
    dev, dt = positions.device, ctx.dtype
    e = lambda *s, d=dt: torch.empty(*s, dtype=d, device=dev)
    raddescr, des3bsupp = e(nf, N, nr), e(nf, N, nr)
    der2b, der3bsupp = e(nf, N, 3, nr), e(nf, N, 3, nr)
    intmap2b, numtriplet = e(nf, N, nr + 1, d=torch.int32), e(nf, N, d=torch.int32)
    if with_angular:
        angdescr, intmap3b, der3b = e(nf, N, na), e(nf, N, 2 * na, d=torch.int32), e(nf, N, 3, 2 * na)
    else:
        angdescr = intmap3b = der3b = None
    check(_lib.lib().stafb_compute_descriptors_light(
        ctx.h, ctx.stream(), _p(positions), _p(boxer), nf, N, _p(raddescr), _p(angdescr), _p(des3bsupp),
        _p(intmap2b), _p(intmap3b), _p(der2b), _p(der3b), _p(der3bsupp), _p(numtriplet)), "ComputeDescriptorsLight")
    ctx.raise_on_status("ComputeDescriptorsLight")
    return raddescr, angdescr, des3bsupp, intmap2b, intmap3b, der2b, der3b, der3bsupp, numtriplet


def compute_sort_proj(radial_descriptor, interaction_map_rad, alpha2b_parameters, type_emb2b_parameters, type_map):
    """Op ComputeSortProj -> two_body_afs[nf,Nl,Fr]."""
    ctx = _ctx_for(radial_descriptor)
    rd, a2, e2 = _real(ctx, radial_descriptor, alpha2b_parameters, type_emb2b_parameters)
    im2, tm = _int(interaction_map_rad, type_map)
    nf, Nl, nr = rd.shape
    nt, Fr = a2.shape
    assert nr == ctx.nr
    out = torch.empty(nf, Nl, Fr, dtype=ctx.dtype, device=rd.device)
    check(_lib.lib().stafb_compute_sort_proj(ctx.h, ctx.stream(), _p(rd), _p(im2), _p(a2), _p(e2), _p(tm), nf, Nl, nt,
                                             Fr, _p(out)), "ComputeSortProj")
    return out


def compute_sort_proj3body(angular_descriptor, radial_descriptor, interaction_map_angular, interaction_map_rad,
                           alpha3b_parameters, type_emb3b_parameters, type_map, num_triplet):
    """Op ComputeSortProj3body -> three_body_afs[nf,Nl,Fa]."""
    ctx = _ctx_for(angular_descriptor)
    ad, rd, a3, e3 = _real(ctx, angular_descriptor, radial_descriptor, alpha3b_parameters, type_emb3b_parameters)
    im3, im2, tm, ntr = _int(interaction_map_angular, interaction_map_rad, type_map, num_triplet)
    nf, Nl, na = ad.shape
    Fa = a3.shape[1] // 3
    nt = _nt_from_classes(a3.shape[0])
    assert na == ctx.na and rd.shape[2] == ctx.nr
    out = torch.empty(nf, Nl, Fa, dtype=ctx.dtype, device=ad.device)
    check(_lib.lib().stafb_compute_sort_proj3body(ctx.h, ctx.stream(), _p(ad), _p(rd), _p(im3), _p(im2), _p(a3),
                                                  _p(e3), _p(tm), _p(ntr), nf, Nl, nt, Fa, _p(out)),
          "ComputeSortProj3body")
    return out


def _nt_from_classes(C_):
    nt = int(round((np.sqrt(8 * C_ + 1) - 1) / 2))
    assert nt * (nt + 1) // 2 == C_
    return nt


def init_force_radial(buffdim):
    return _lib.lib().stafb_init_force_radial(int(buffdim))


def init_force_tripl(buffdim):
    return _lib.lib().stafb_init_force_tripl(int(buffdim))


def init_grad_force_radial(buffdim):
    return _lib.lib().stafb_init_grad_force_radial(int(buffdim))


def init_grad_force_tripl(buffdim):
    return _lib.lib().stafb_init_grad_force_tripl(int(buffdim))


def _dev_int(x, device):
    if torch.is_tensor(x):
        return x.to(device=device, dtype=torch.int32).reshape(-1).contiguous()
    return torch.tensor(np.atleast_1d(x), dtype=torch.int32, device=device)


def compute_force_radial(netderiv, descriptor_derivative_rad, interaction_map_rad, radial_descriptor,
                         alpha2b_parameters, type_emb2b_parameters, type_map, tipos, actual_type):
    """Op ComputeForceRadial -> force[nf,3N]."""
    ctx = _ctx_for(netderiv)
    nd, dd, rd, a2, e2 = _real(ctx, netderiv, descriptor_derivative_rad, radial_descriptor, alpha2b_parameters,
                               type_emb2b_parameters)
    im2, tm = _int(interaction_map_rad, type_map)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fr = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    out = torch.empty(nf, 3 * N, dtype=ctx.dtype, device=nd.device)
    check(_lib.lib().stafb_compute_force_radial(ctx.h, ctx.stream(), _p(nd), _p(dd), _p(im2), _p(rd), _p(a2), _p(e2),
                                                _p(tm), _p(tp), _p(at), nf, Nl, N, nt, Fr, _p(out)),
          "ComputeForceRadial")
    return out


def compute_force_tripl(netderiv, radial_descriptor, angular_descriptor, descriptor_derivative_rad,
                        descriptor_derivative_ang, interaction_map_rad, interaction_map_ang, alpha3b_parameters,
                        type_emb3b_parameters, type_map, tipos, actual_type, num_triplets):
    """Op ComputeForceTripl -> force[nf,3N]."""
    ctx = _ctx_for(netderiv)
    nd, rd, ad, ddr, dda, a3, e3 = _real(ctx, netderiv, radial_descriptor, angular_descriptor,
                                         descriptor_derivative_rad, descriptor_derivative_ang, alpha3b_parameters,
                                         type_emb3b_parameters)
    im2, im3, tm, ntr = _int(interaction_map_rad, interaction_map_ang, type_map, num_triplets)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fa = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    out = torch.empty(nf, 3 * N, dtype=ctx.dtype, device=nd.device)
    check(_lib.lib().stafb_compute_force_tripl(ctx.h, ctx.stream(), _p(nd), _p(rd), _p(ad), _p(ddr), _p(dda), _p(im2),
                                               _p(im3), _p(a3), _p(e3), _p(tm), _p(tp), _p(at), _p(ntr), nf, Nl, N,
                                               nt, Fa, _p(out)), "ComputeForceTripl")
    return out


def compute_two_body_par_grad(prev_grad, radial_descriptor, interaction_map_rad, alpha2b_parameters,
                              type_emb2b_parameters, type_map):
    """Op ComputeTwoBodyParGrad -> (nextgrad_alpha2b[nt,Fr], nextgrad_emb2b[nt,Fr])."""
    ctx = _ctx_for(prev_grad)
    pg, rd, a2, e2 = _real(ctx, prev_grad, radial_descriptor, alpha2b_parameters, type_emb2b_parameters)
    im2, tm = _int(interaction_map_rad, type_map)
    nf, Nl, Fr = pg.shape
    nt = a2.shape[0]
    ga, ge = torch.empty_like(a2), torch.empty_like(a2)
    check(_lib.lib().stafb_compute_two_body_par_grad(ctx.h, ctx.stream(), _p(pg), _p(rd), _p(im2), _p(a2), _p(e2),
                                                     _p(tm), nf, Nl, nt, Fr, _p(ga), _p(ge)), "ComputeTwoBodyParGrad")
    return ga, ge


def compute_sort_proj3body_grad(previous_gradient, angular_desciptors, radial_descriptors, intmap3b, intmap2b,
                                alpha3b, type_emb3b, type_map, num_triplets):
    """Op ComputeSortProj3bodyGrad -> (alphagrad3body[C,3Fa], nextgrad_emb3b[C,Fa] == 0)."""
    ctx = _ctx_for(previous_gradient)
    pg, ad, rd, a3, e3 = _real(ctx, previous_gradient, angular_desciptors, radial_descriptors, alpha3b, type_emb3b)
    im3, im2, tm, ntr = _int(intmap3b, intmap2b, type_map, num_triplets)
    nf, Nl, Fa = pg.shape
    nt = _nt_from_classes(a3.shape[0])
    ga = torch.empty_like(a3)
    ge = torch.empty(a3.shape[0], Fa, dtype=ctx.dtype, device=pg.device)
    check(_lib.lib().stafb_compute_sort_proj3body_grad(ctx.h, ctx.stream(), _p(pg), _p(ad), _p(rd), _p(im3), _p(im2),
                                                       _p(a3), _p(e3), _p(tm), _p(ntr), nf, Nl, nt, Fa, _p(ga),
                                                       _p(ge)), "ComputeSortProj3bodyGrad")
    return ga, ge


def compute_force_radial_grad(prevgrad, netderiv, descriptor_derivative_rad, interaction_map_rad, radial_descriptor,
                              alpha2b_parameters, type_emb2b_parameters, type_map, tipos, actual_type):
    """Op ComputeForceRadialGrad -> (gradnet[nf,Nl,Fr], grad_alpha2b[nt,Fr], grad_emb2b[nt,Fr])."""
    ctx = _ctx_for(prevgrad)
    pg, nd, dd, rd, a2, e2 = _real(ctx, prevgrad, netderiv, descriptor_derivative_rad, radial_descriptor,
                                   alpha2b_parameters, type_emb2b_parameters)
    im2, tm = _int(interaction_map_rad, type_map)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fr = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    gn, ga, ge = torch.empty_like(nd), torch.empty_like(a2), torch.empty_like(a2)
    check(_lib.lib().stafb_compute_force_radial_grad(ctx.h, ctx.stream(), _p(pg), _p(nd), _p(dd), _p(im2), _p(rd),
                                                     _p(a2), _p(e2), _p(tm), _p(tp), _p(at), nf, Nl, N, nt, Fr,
                                                     _p(gn), _p(ga), _p(ge)), "ComputeForceRadialGrad")
    return gn, ga, ge


def compute_force_tripl_grad(prevgrad, netderiv, radial_descriptor, angular_descriptor, descriptor_derivative_rad,
                             descriptor_derivative_ang, interaction_map_rad, interaction_map_ang, alpha3b_parameters,
                             type_emb3b_parameters, type_map, tipos, actual_type, num_triplets):
    """Op ComputeForceTriplGrad -> (gradnet[nf,Nl,Fa], gradalpha[C,3Fa], gradck[C,Fa] == 0)."""
    ctx = _ctx_for(prevgrad)
    pg, nd, rd, ad, ddr, dda, a3, e3 = _real(ctx, prevgrad, netderiv, radial_descriptor, angular_descriptor,
                                             descriptor_derivative_rad, descriptor_derivative_ang,
                                             alpha3b_parameters, type_emb3b_parameters)
    im2, im3, tm, ntr = _int(interaction_map_rad, interaction_map_ang, type_map, num_triplets)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fa = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    gn, ga = torch.empty_like(nd), torch.empty_like(a3)
    gck = torch.empty(a3.shape[0], Fa, dtype=ctx.dtype, device=nd.device)
    check(_lib.lib().stafb_compute_force_tripl_grad(ctx.h, ctx.stream(), _p(pg), _p(nd), _p(rd), _p(ad), _p(ddr),
                                                    _p(dda), _p(im2), _p(im3), _p(a3), _p(e3), _p(tm), _p(tp), _p(at),
                                                    _p(ntr), nf, Nl, N, nt, Fa, _p(gn), _p(ga), _p(gck)),
          "ComputeForceTriplGrad")
    return gn, ga, gck


def compute_force_radial_virial(netderiv, descriptor_derivative_rad, interaction_map_rad, radial_descriptor,
                                alpha2b_parameters, type_emb2b_parameters, type_map, tipos, actual_type, pos, box):
    """Op ComputeForceRadialVirial -> (force[nf,3N], virial[nf,9])."""
    ctx = _ctx_for(netderiv)
    nd, dd, rd, a2, e2, ps, bx = _real(ctx, netderiv, descriptor_derivative_rad, radial_descriptor,
                                       alpha2b_parameters, type_emb2b_parameters, pos, box)
    im2, tm = _int(interaction_map_rad, type_map)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fr = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    out = torch.empty(nf, 3 * N, dtype=ctx.dtype, device=nd.device)
    vir = torch.empty(nf, 9, dtype=ctx.dtype, device=nd.device)
    check(_lib.lib().stafb_compute_force_radial_virial(ctx.h, ctx.stream(), _p(nd), _p(dd), _p(im2), _p(rd), _p(a2),
                                                       _p(e2), _p(tm), _p(tp), _p(at), _p(ps), _p(bx), nf, Nl, N, nt,
                                                       Fr, _p(out), _p(vir)), "ComputeForceRadialVirial")
    return out, vir


def compute_force_tripl_virial(netderiv, radial_descriptor, angular_descriptor, descriptor_derivative_rad,
                               descriptor_derivative_ang, interaction_map_rad, interaction_map_ang,
                               alpha3b_parameters, type_emb3b_parameters, type_map, tipos, actual_type, num_triplets,
                               pos, box):
    """Op ComputeForceTriplVirial -> (force[nf,3N], virial[nf,9])."""
    ctx = _ctx_for(netderiv)
    nd, rd, ad, ddr, dda, a3, e3, ps, bx = _real(ctx, netderiv, radial_descriptor, angular_descriptor,
                                                 descriptor_derivative_rad, descriptor_derivative_ang,
                                                 alpha3b_parameters, type_emb3b_parameters, pos, box)
    im2, im3, tm, ntr = _int(interaction_map_rad, interaction_map_ang, type_map, num_triplets)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fa = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    out = torch.empty(nf, 3 * N, dtype=ctx.dtype, device=nd.device)
    vir = torch.empty(nf, 9, dtype=ctx.dtype, device=nd.device)
    check(_lib.lib().stafb_compute_force_tripl_virial(ctx.h, ctx.stream(), _p(nd), _p(rd), _p(ad), _p(ddr), _p(dda),
                                                      _p(im2), _p(im3), _p(a3), _p(e3), _p(tm), _p(tp), _p(at),
                                                      _p(ntr), _p(ps), _p(bx), nf, Nl, N, nt, Fa, _p(out), _p(vir)),
          "ComputeForceTriplVirial")
    return out, vir


def compute_force_radial_virial_grad(prevgrad, prevgrad_virial, netderiv, descriptor_derivative_rad,
                                     interaction_map_rad, radial_descriptor, alpha2b_parameters,
                                     type_emb2b_parameters, type_map, tipos, actual_type, pos, box):
    """Op ComputeForceRadialVirialGrad -> (gradnet[nf,Nl,Fr], grad_alpha2b[nt,Fr], grad_emb2b[nt,Fr])."""
    ctx = _ctx_for(prevgrad)
    pg, pv, nd, dd, rd, a2, e2, ps, bx = _real(ctx, prevgrad, prevgrad_virial, netderiv, descriptor_derivative_rad,
                                               radial_descriptor, alpha2b_parameters, type_emb2b_parameters, pos, box)
    im2, tm = _int(interaction_map_rad, type_map)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fr = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    gn, ga, ge = torch.empty_like(nd), torch.empty_like(a2), torch.empty_like(a2)
    check(_lib.lib().stafb_compute_force_radial_virial_grad(ctx.h, ctx.stream(), _p(pg), _p(pv), _p(nd), _p(dd),
                                                            _p(im2), _p(rd), _p(a2), _p(e2), _p(tm), _p(tp), _p(at),
                                                            _p(ps), _p(bx), nf, Nl, N, nt, Fr, _p(gn), _p(ga),
                                                            _p(ge)), "ComputeForceRadialVirialGrad")
    return gn, ga, ge


def compute_force_tripl_virial_grad(prevgrad, prevgrad_virial, netderiv, radial_descriptor, angular_descriptor,
                                    descriptor_derivative_rad, descriptor_derivative_ang, interaction_map_rad,
                                    interaction_map_ang, alpha3b_parameters, type_emb3b_parameters, type_map, tipos,
                                    actual_type, num_triplets, pos, box):
    """Op ComputeForceTriplVirialGrad -> (gradnet[nf,Nl,Fa], gradalpha[C,3Fa], gradck[C,Fa] == 0)."""
    ctx = _ctx_for(prevgrad)
    pg, pv, nd, rd, ad, ddr, dda, a3, e3, ps, bx = _real(ctx, prevgrad, prevgrad_virial, netderiv, radial_descriptor,
                                                         angular_descriptor, descriptor_derivative_rad,
                                                         descriptor_derivative_ang, alpha3b_parameters,
                                                         type_emb3b_parameters, pos, box)
    im2, im3, tm, ntr = _int(interaction_map_rad, interaction_map_ang, type_map, num_triplets)
    tp, at = _dev_int(tipos, nd.device), _dev_int(actual_type, nd.device)
    nf, Nl, Fa = nd.shape
    N, nt = tm.shape[0], tp.shape[0]
    gn, ga = torch.empty_like(nd), torch.empty_like(a3)
    gck = torch.empty(a3.shape[0], Fa, dtype=ctx.dtype, device=nd.device)
    check(_lib.lib().stafb_compute_force_tripl_virial_grad(ctx.h, ctx.stream(), _p(pg), _p(pv), _p(nd), _p(rd),
                                                           _p(ad), _p(ddr), _p(dda), _p(im2), _p(im3), _p(a3),
                                                           _p(e3), _p(tm), _p(tp), _p(at), _p(ntr), _p(ps), _p(bx),
                                                           nf, Nl, N, nt, Fa, _p(gn), _p(ga), _p(gck)),
          "ComputeForceTriplVirialGrad")
    return gn, ga, gck
