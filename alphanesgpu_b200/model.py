"""Host-side driver of the fused path: the model the reference builds in
STAF/staf_models/staf_model.py (per-species fingerprints -> log-normalisation -> MLP ->
energy; forces through d(sum e)/dAF; Huber/MSE loss; Adam), with every device step done by
the C ABI (include/stafb.h).  torch supplies device buffers, streams and, for data-parallel
training, the NCCL all-reduce of the flat gradient.
"""
import ctypes as C

import numpy as np
import torch

from . import _lib
from ._lib import check
from .ops import Context
from .params import ModelShape


def _p(t):
    return None if t is None else C.c_void_p(t.data_ptr())


class StafModel:
    """One potential: geometry config + parameter layout + device buffers."""

    def __init__(self, shape: ModelShape, cfg, theta, emb, max_batch, dtype=torch.float32, device=None,
                 pe=1.0, pf=1.0, pb=1.0, alpha_bound=5.0, loss="huber", n_max=None):
        """n_max: atoms per frame the scratch is sized for (default shape.N); larger values leave room for
        ghost atoms (energy_force_domain) and for set_counts()."""
        self.shape = shape
        self.cfg = dict(cfg)
        self.dtype = dtype
        self.n_max = int(n_max) if n_max else shape.N
        self.n_centres = shape.N
        self.ctx = Context(cfg["Rc"], cfg["nr"], cfg["na"], self.n_max, cfg["Rs"], cfg["Ra"], max_batch, dtype, device)
        self.device = self.ctx.device
        self.max_batch = int(max_batch)
        h = C.c_void_p()
        sd = shape.desc()
        with torch.cuda.device(self.device):
            check(_lib.lib().stafb_model_create(self.ctx.h, sd.ctypes.data_as(C.c_void_p), C.byref(h)),
                  "stafb_model_create")
        self.h = h
        assert _lib.lib().stafb_model_n_params(h) == shape.n_params
        assert _lib.lib().stafb_model_n_emb(h) == shape.n_emb
        self.theta = torch.as_tensor(np.asarray(theta), dtype=dtype).to(self.device).contiguous()
        self.emb = torch.as_tensor(np.asarray(emb), dtype=dtype).to(self.device).contiguous()
        self.grad = torch.zeros_like(self.theta)
        self.adam_m = torch.zeros_like(self.theta)
        self.adam_v = torch.zeros_like(self.theta)
        self.losses = torch.zeros(4, dtype=torch.float64, device=self.device)
        self.losses_h = np.zeros(4, np.float64)
        self.step = 0
        self.pe, self.pf, self.pb, self.alpha_bound = float(pe), float(pf), float(pb), float(alpha_bound)
        self.loss_kind = 0 if loss == "huber" else 1

    def close(self):
        if getattr(self, "h", None):
            _lib.lib().stafb_model_destroy(self.h)
            self.h = None
        self.ctx.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _dev(self, a):
        if torch.is_tensor(a):
            return a.to(device=self.device, dtype=self.dtype).contiguous()
        return torch.as_tensor(np.asarray(a), dtype=self.dtype).to(self.device).contiguous()

    def energy_force(self, pos, box, per_atom_energy=False, check_status=True):
        """Energies [nf] and forces [nf,3N] (inference convention 0.5*sum e_i unless per_atom_energy)."""
        pos, box = self._dev(pos), self._dev(box)
        nf = box.shape[0]
        energy = torch.empty(nf, dtype=self.dtype, device=self.device)
        force = torch.empty(nf, 3 * self.shape.N, dtype=self.dtype, device=self.device)
        check(_lib.lib().stafb_energy_force(self.ctx.h, self.h, self.ctx.stream(), _p(pos), _p(box), nf,
                                            _p(self.theta), _p(self.emb), int(per_atom_energy), _p(energy),
                                            _p(force)), "stafb_energy_force")
        if check_status:
            self.ctx.raise_on_status("stafb_energy_force")
        return energy, force

    def energy_force_virial(self, pos, box, per_atom_energy=False):
        """energy_force plus the 3x3 virial W_ab = -sum g_a r_b per frame ([nf,9], row-major)."""
        pos, box = self._dev(pos), self._dev(box)
        nf = box.shape[0]
        energy = torch.empty(nf, dtype=self.dtype, device=self.device)
        force = torch.empty(nf, 3 * self.n_centres, dtype=self.dtype, device=self.device)
        virial = torch.empty(nf, 9, dtype=self.dtype, device=self.device)
        check(_lib.lib().stafb_energy_force_virial(self.ctx.h, self.h, self.ctx.stream(), _p(pos), _p(box), nf,
                                                   _p(self.theta), _p(self.emb), int(per_atom_energy), _p(energy),
                                                   _p(force), _p(virial)), "stafb_energy_force_virial")
        self.ctx.raise_on_status("stafb_energy_force_virial")
        return energy, force, virial

    def set_counts(self, tipos):
        """New numbers of (owned) atoms per species; the sum must stay within n_max."""
        t = np.ascontiguousarray(tipos, np.int32)
        check(_lib.lib().stafb_model_set_counts(self.h, t.ctypes.data_as(C.c_void_p)), "stafb_model_set_counts")
        self.n_centres = int(t.sum())

    def energy_force_domain(self, pos_all, box, type_map, howmany=None, with_=None, virial=False,
                            check_status=True, out=None):
        """One frame of nall atoms whose first n_centres (species-sorted) are owned and the rest are ghosts:
        energy 0.5*sum over the owned atoms, forces [nall,3] for all.  type_map: int32 [nall] on the device.
        howmany/with_ (int32 device tensors [n_centres], [n_centres, nr]): caller-built, distance-sorted rows
        taken without any periodic wrap; otherwise the list is built with the minimum image of box[6].
        out=(energy[1], force[>=nall,3]): device tensors to fill instead of fresh ones (fixed addresses, for a
        captured graph)."""
        pos_all = self._dev(pos_all)
        box = None if box is None else self._dev(box)
        nall = pos_all.numel() // 3
        if out is not None:
            energy, force = out
            assert energy.dtype == self.dtype and force.dtype == self.dtype and force.numel() >= 3 * nall
        else:
            energy = torch.empty(1, dtype=self.dtype, device=self.device)
            force = torch.empty(nall, 3, dtype=self.dtype, device=self.device)
        vir = torch.empty(9, dtype=self.dtype, device=self.device) if virial else None
        check(_lib.lib().stafb_energy_force_domain(self.ctx.h, self.h, self.ctx.stream(), _p(pos_all), _p(box), nall,
                                                   _p(type_map), _p(howmany), _p(with_), _p(self.theta),
                                                   _p(self.emb), _p(energy), _p(force), _p(vir)),
              "stafb_energy_force_domain")
        if check_status:
            self.ctx.raise_on_status("stafb_energy_force_domain")
        return (energy, force, vir) if virial else (energy, force)

    def loss_and_grad(self, pos, box, e_label, f_label, want_outputs=False):
        """One training evaluation on device tensors: fills self.losses (loss, loss_e, loss_bound, loss_f)
        and self.grad; asynchronous on the current stream."""
        nf = box.shape[0]
        energy = force = None
        if want_outputs:
            energy = torch.empty(nf, dtype=self.dtype, device=self.device)
            force = torch.empty(nf, 3 * self.shape.N, dtype=self.dtype, device=self.device)
        check(_lib.lib().stafb_train_step(self.ctx.h, self.h, self.ctx.stream(), _p(pos), _p(box), nf, _p(self.theta),
                                          _p(self.emb), _p(e_label), _p(f_label), self.pe, self.pf, self.pb,
                                          self.alpha_bound, self.loss_kind, _p(self.losses), _p(self.grad),
                                          _p(energy), _p(force)), "stafb_train_step")
        return energy, force

    def loss_and_grad_virial(self, pos, box, e_label, f_label, v_label, pv=1.0, want_outputs=False):
        """Energy + force + virial training evaluation (full_train_e_f_v, STAF/staf_models/staf_model.py:313-384):
        v_label [nf,9] total virials; fills self.losses5 (loss, loss_e, loss_bound, loss_f, loss_v) and self.grad.
        Returns (energy, force, virial) when want_outputs."""
        nf = box.shape[0]
        if not hasattr(self, "losses5"):
            self.losses5 = torch.zeros(5, dtype=torch.float64, device=self.device)
        energy = force = virial = None
        if want_outputs:
            energy = torch.empty(nf, dtype=self.dtype, device=self.device)
            force = torch.empty(nf, 3 * self.shape.N, dtype=self.dtype, device=self.device)
            virial = torch.empty(nf, 9, dtype=self.dtype, device=self.device)
        check(_lib.lib().stafb_train_step_virial(self.ctx.h, self.h, self.ctx.stream(), _p(pos), _p(box), nf,
                                                 _p(self.theta), _p(self.emb), _p(e_label), _p(f_label), _p(v_label),
                                                 self.pe, self.pf, float(pv), self.pb, self.alpha_bound,
                                                 self.loss_kind, _p(self.losses5), _p(self.grad), _p(energy),
                                                 _p(force), _p(virial)), "stafb_train_step_virial")
        return energy, force, virial

    def use_grad(self, tensor):
        """Makes the following evaluations accumulate their gradient into `tensor` (n_params elements on this
        device, e.g. a PeerExchange buffer) instead of the model's own; returns the previous buffer."""
        assert tensor.numel() == self.theta.numel() and tensor.dtype == self.dtype and tensor.is_cuda
        old, self.grad = self.grad, tensor
        return old

    def prefetch_rows(self, pos, box, slot):
        """Builds the neighbour rows of a batch (device tensors) into row set `slot` (0 or 1) on the current
        stream.  They depend on no trainable parameter, so this may run on a side stream while the previous
        step is still in flight; loss_and_grad_prefetched(slot, ...) must be ordered after it."""
        check(_lib.lib().stafb_descriptors_prefetch(self.ctx.h, self.h, self.ctx.stream(), _p(pos), _p(box),
                                                    box.shape[0], int(slot)), "stafb_descriptors_prefetch")

    def loss_and_grad_prefetched(self, slot, nf, e_label, f_label):
        """loss_and_grad on the rows that prefetch_rows left in `slot`."""
        check(_lib.lib().stafb_train_step_prefetched(self.ctx.h, self.h, self.ctx.stream(), int(slot), int(nf),
                                                     _p(self.theta), _p(self.emb), _p(e_label), _p(f_label), self.pe,
                                                     self.pf, self.pb, self.alpha_bound, self.loss_kind,
                                                     _p(self.losses), _p(self.grad), None, None),
              "stafb_train_step_prefetched")

    def loss_and_grad_host(self, pos, box, e_label, f_label):
        """Same with HOST numpy inputs: host->device copies, the step and the device->host read of the
        losses all happen inside the call (it returns after the stream has drained)."""
        dt = np.float32 if self.dtype == torch.float32 else np.float64
        pos, box = np.ascontiguousarray(pos, dt), np.ascontiguousarray(box, dt)
        e_label, f_label = np.ascontiguousarray(e_label, dt), np.ascontiguousarray(f_label, dt)
        nf = box.shape[0]
        vp = lambda a: a.ctypes.data_as(C.c_void_p)
        check(_lib.lib().stafb_train_step_host(self.ctx.h, self.h, self.ctx.stream(), vp(pos), vp(box), nf,
                                               _p(self.theta), _p(self.emb), vp(e_label), vp(f_label), self.pe,
                                               self.pf, self.pb, self.alpha_bound, self.loss_kind,
                                               vp(self.losses_h), _p(self.grad)), "stafb_train_step_host")
        return self.losses_h

    def loss_and_grad_host_begin(self, pos, box, e_label, f_label, slot):
        """Pipelined loss_and_grad_host: stages the HOST inputs, enqueues copies + step and returns at once.
        Collect with loss_and_grad_host_end(slot); two slots (0, 1) let step k+1 be prepared while step k runs."""
        dt = np.float32 if self.dtype == torch.float32 else np.float64
        pos, box = np.ascontiguousarray(pos, dt), np.ascontiguousarray(box, dt)
        e_label, f_label = np.ascontiguousarray(e_label, dt), np.ascontiguousarray(f_label, dt)
        vp = lambda a: a.ctypes.data_as(C.c_void_p)
        check(_lib.lib().stafb_train_step_host_begin(self.ctx.h, self.h, self.ctx.stream(), vp(pos), vp(box),
                                                     box.shape[0], _p(self.theta), _p(self.emb), vp(e_label),
                                                     vp(f_label), self.pe, self.pf, self.pb, self.alpha_bound,
                                                     self.loss_kind, _p(self.grad), int(slot)),
              "stafb_train_step_host_begin")

    def loss_and_grad_host_end(self, slot):
        """Waits for the step begun in `slot`; returns its losses (loss, loss_e, loss_bound, loss_f)."""
        out = np.zeros(4, np.float64)
        check(_lib.lib().stafb_train_step_host_end(self.ctx.h, self.h, int(slot), out.ctypes.data_as(C.c_void_p)),
              "stafb_train_step_host_end")
        return out

    def loss_and_grad_virial_host_begin(self, pos, box, e_label, f_label, v_label, slot, pv=1.0):
        """Pipelined energy + force + virial evaluation with HOST numpy inputs (v_label [nf,9]); collect with
        loss_and_grad_virial_host_end(slot)."""
        dt = np.float32 if self.dtype == torch.float32 else np.float64
        pos, box = np.ascontiguousarray(pos, dt), np.ascontiguousarray(box, dt)
        e_label, f_label = np.ascontiguousarray(e_label, dt), np.ascontiguousarray(f_label, dt)
        v_label = np.ascontiguousarray(v_label, dt).reshape(box.shape[0], 9)
        vp = lambda a: a.ctypes.data_as(C.c_void_p)
        check(_lib.lib().stafb_train_step_virial_host_begin(self.ctx.h, self.h, self.ctx.stream(), vp(pos), vp(box),
                                                            box.shape[0], _p(self.theta), _p(self.emb), vp(e_label),
                                                            vp(f_label), vp(v_label), self.pe, self.pf, float(pv),
                                                            self.pb, self.alpha_bound, self.loss_kind, _p(self.grad),
                                                            int(slot)),
              "stafb_train_step_virial_host_begin")

    def loss_and_grad_virial_host_end(self, slot):
        """Waits for the step begun in `slot`; returns (loss, loss_e, loss_bound, loss_f, loss_v)."""
        out = np.zeros(5, np.float64)
        check(_lib.lib().stafb_train_step_virial_host_end(self.ctx.h, self.h, int(slot),
                                                          out.ctypes.data_as(C.c_void_p)),
              "stafb_train_step_virial_host_end")
        return out

    def adam_update(self, lr, beta1=0.9, beta2=0.999, eps=1e-7, grad_scale=1.0):
        """Keras Adam (epsilon default 1e-7: STAF/optimizer_learning_rate_utility.py:64-68)."""
        self.step += 1
        check(_lib.lib().stafb_adam_step(self.ctx.h, self.ctx.stream(), _p(self.theta), _p(self.grad),
                                         _p(self.adam_m), _p(self.adam_v), self.theta.numel(), float(lr),
                                         float(beta1), float(beta2), float(eps), self.step, float(grad_scale)),
              "stafb_adam_step")

    # order of the phase marks of a training evaluation / of an inference evaluation
    PHASES = ["descriptors", "af_fwd", "mlp_fwd", "force", "force_grad", "loss", "mlp_bwd"]
    PHASES_INFERENCE = ["descriptors", "af_fwd", "mlp_fwd", "force", "loss"]

    def adam_update_dev(self, lr, beta1=0.9, beta2=0.999, eps=1e-7, grad_scale=1.0):
        """Adam with the step counter on the device (safe to capture in a CUDA graph and replay)."""
        if not hasattr(self, "step_d"):
            self.step_d = torch.zeros(2, dtype=torch.int32, device=self.device)  # step, block counter
        check(_lib.lib().stafb_adam_step_dev(self.ctx.h, self.ctx.stream(), _p(self.theta), _p(self.grad),
                                             _p(self.adam_m), _p(self.adam_v), self.theta.numel(), float(lr),
                                             float(beta1), float(beta2), float(eps), _p(self.step_d),
                                             float(grad_scale)), "stafb_adam_step_dev")

    def set_phase_timing(self, on):
        check(_lib.lib().stafb_set_phase_timing(self.ctx.h, int(on)), "stafb_set_phase_timing")

    def phase_times_ms(self):
        buf = np.zeros(16, np.float32)
        n = _lib.lib().stafb_get_phase_times(self.ctx.h, buf.ctypes.data_as(C.c_void_p), 16)
        names = self.PHASES if n > len(self.PHASES_INFERENCE) else self.PHASES_INFERENCE
        return dict(zip(names[:n], buf[:n].tolist()))

    def mlp_config(self):
        """(staging mode, atoms per thread group, forward smem bytes, backward smem bytes) of the MLP kernels."""
        out = np.zeros(4, np.int32)
        _lib.lib().stafb_model_mlp_config(self.h, out.ctypes.data_as(C.c_void_p))
        mma = np.zeros(4, np.int32)
        _lib.lib().stafb_model_mlp_mma_config(self.h, mma.ctypes.data_as(C.c_void_p))
        return dict(stage=int(out[0]), apt=int(out[1]), fwd_smem=int(out[2]), bwd_smem=int(out[3]),
                    mma=int(mma[0]), mma_warps=int(mma[1]), mma_staged=int(mma[2]), mma_bwd_smem=int(mma[3]))

    def launches(self):
        return _lib.lib().stafb_last_launch_count(self.ctx.h)
