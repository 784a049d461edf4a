"""Slab-decomposed energy/force evaluation of one large periodic system on several GPUs.

What LAMMPS does around `pair_style staf` in the reference (lammps/USER-STAF/pair_staf.cpp:129-145,
180-256: owned atoms + ghost atoms within one cutoff, forces on ghosts returned and summed onto their
owners by reverse_comm), restated without LAMMPS for ONE box of GPUs: the periodic box is cut into
`world` slabs along one axis, every rank owns the atoms of one slab, receives the atoms of its two
neighbour slabs that lie within one cutoff of its faces (one message per face), evaluates its owned
centres over owned + ghost atoms, and sends the ghost forces back (one message per face).  The only
collective is the all-reduce of the scalar energy.  torch.distributed is the transport: NCCL on GPUs
(device tensors, NVLink), gloo in the CPU tests.

As in LAMMPS, WHICH atoms are ghosts is decided only every `halo_every` evaluations, with the halo widened by
a skin so that the set stays valid while atoms move; in between, only the positions of that fixed set
travel (one message per face and direction, no counts, no host synchronisation).

Ghosts keep their original (unshifted) coordinates: the evaluation applies the minimum-image
convention of the global box, so any periodic image will do, and every physical atom appears at most
once per rank as long as the slab is at least one cutoff wide (two cutoffs when world == 2, where the
lower and the upper neighbour are the same rank).
"""
import numpy as np
import torch
import torch.distributed as dist


def slab_of(z, L, world):
    """Slab index of coordinates z (any image) for a box length L cut into `world` equal slabs."""
    zw = z - torch.floor(z / L) * L
    return torch.clamp((zw * (world / L)).to(torch.int64), max=world - 1)


class SlabDomain:
    """One rank's share of a slab decomposition.

    compute(pos_all[nall,3], type_all[nall] int32, n_owned, plan_changed) -> (energy tensor [1], force[nall,3])
    evaluates the owned centres (the first n_owned atoms, species-sorted) over all atoms; energy is the owned
    atoms' share.  plan_changed tells it that the atom counts or species may differ from the previous call.
    """

    def __init__(self, compute, box6, cutoff, rank, world, axis=2, group=None, nt=2, skin=0.0, halo_every=1):
        self.compute, self.rank, self.world, self.axis, self.group = compute, int(rank), int(world), int(axis), group
        self.box6 = [float(v) for v in box6]
        self.L = self.box6[(0, 3, 5)[axis]]
        self.rc = float(cutoff)
        self.reach = float(cutoff) + float(skin)  # halo width
        self.halo_every = max(1, int(halo_every))
        self.nt = int(nt)
        w = self.L / self.world
        need = self.reach if self.world > 2 else 2.0 * self.reach
        if self.world > 1 and w < need:
            raise ValueError("slab width %.3f is below %.3f: an atom would be a ghost twice" % (w, need))
        self.lo = (self.rank - 1) % self.world
        self.hi = (self.rank + 1) % self.world
        self.pos = self.types = self.counts = None
        self._plan = None
        self._nstep = 0

    # -- ownership ------------------------------------------------------------------------------
    def set_owned_from_global(self, pos_all, types_all):
        """Takes this rank's atoms out of a global configuration (every rank passes the same arrays),
        species-sorted as the kernels require.  Returns their global indices."""
        pos_all = torch.as_tensor(pos_all).reshape(-1, 3)
        types_all = torch.as_tensor(types_all).to(torch.int32)
        mine = slab_of(pos_all[:, self.axis], self.L, self.world) == self.rank
        idx = torch.nonzero(mine).squeeze(1)
        order = torch.argsort(types_all[idx].to(torch.int64), stable=True)
        idx = idx[order]
        self.pos = pos_all[idx].contiguous()
        self.types = types_all[idx].contiguous()
        self.counts = torch.bincount(self.types.to(torch.int64), minlength=self.nt).tolist()
        self._plan = None
        return idx

    # -- messages -------------------------------------------------------------------------------
    def _swap(self, out_lo, out_hi, in_lo, in_hi):
        """One message to and one from each face neighbour.  What goes out through my lower face arrives
        through my lower neighbour's UPPER face, so the receives are posted upper-first: with world == 2
        both neighbours are the same rank and messages between two ranks match in posting order."""
        g = self.group
        ops = [dist.P2POp(dist.isend, out_lo, self.lo, g), dist.P2POp(dist.isend, out_hi, self.hi, g),
               dist.P2POp(dist.irecv, in_hi, self.hi, g), dist.P2POp(dist.irecv, in_lo, self.lo, g)]
        for r in dist.batch_isend_irecv(ops):
            r.wait()

    def _make_plan(self):
        """Chooses the atoms that leave through each face (within `reach` of it), learns how many arrive,
        exchanges their species and lays out the owned + ghost buffers."""
        pos, types, dev = self.pos, self.types, self.pos.device
        n_own = pos.shape[0]
        w = self.L / self.world
        z = pos[:, self.axis]
        zw = z - torch.floor(z / self.L) * self.L - self.rank * w  # height above the slab's lower face
        i_lo = torch.nonzero(zw < self.reach).squeeze(1)
        i_hi = torch.nonzero(zw >= w - self.reach).squeeze(1)
        n_out = torch.tensor([i_lo.shape[0], i_hi.shape[0]], dtype=torch.int64, device=dev)
        n_in = torch.zeros_like(n_out)
        self._swap(n_out[0:1], n_out[1:2], n_in[0:1], n_in[1:2])
        n_lo, n_hi = (int(v) for v in n_in.tolist())
        t_lo = torch.empty(n_lo, dtype=torch.int32, device=dev)
        t_hi = torch.empty(n_hi, dtype=torch.int32, device=dev)
        self._swap(types[i_lo].contiguous(), types[i_hi].contiguous(), t_lo, t_hi)
        nall = n_own + n_lo + n_hi
        pos_all = torch.empty((nall, 3), dtype=pos.dtype, device=dev)
        self._plan = dict(i_lo=i_lo, i_hi=i_hi, n_lo=n_lo, n_hi=n_hi, pos_all=pos_all,
                          type_all=torch.cat([types, t_lo, t_hi]).contiguous(),
                          got_lo=torch.empty((i_lo.shape[0], 3), dtype=pos.dtype, device=dev),
                          got_hi=torch.empty((i_hi.shape[0], 3), dtype=pos.dtype, device=dev))

    # -- one evaluation ---------------------------------------------------------------------------
    def step(self, rebuild=None):
        """Energy of the whole system (tensor [1], identical on every rank) and forces on the owned atoms."""
        pos, types = self.pos, self.types
        n_own = pos.shape[0]
        if rebuild is None:
            rebuild = self._plan is None or self._nstep % self.halo_every == 0
        self._nstep += 1
        if self.world == 1:
            e, f = self.compute(pos, types, n_own, rebuild)
            return e, f[:n_own]
        if rebuild:
            self._make_plan()
        P = self._plan
        n_lo, n_hi, pos_all = P["n_lo"], P["n_hi"], P["pos_all"]
        pos_all[:n_own].copy_(pos)
        self._swap(pos[P["i_lo"]], pos[P["i_hi"]], pos_all[n_own:n_own + n_lo], pos_all[n_own + n_lo:])
        e, f = self.compute(pos_all, P["type_all"], n_own, rebuild)
        # ghost forces go back through the face they came in by
        self._swap(f[n_own:n_own + n_lo], f[n_own + n_lo:], P["got_lo"], P["got_hi"])
        f_own = f[:n_own]
        f_own.index_add_(0, P["i_lo"], P["got_lo"])
        f_own.index_add_(0, P["i_hi"], P["got_hi"])
        dist.all_reduce(e, group=self.group)
        return e, f_own


def model_compute(model, box6):
    """compute() for SlabDomain on top of StafModel.energy_force_domain (device tensors).  The device status
    word (saturated neighbour buffers ...) is read whenever the halo plan changes, not on every call."""
    box = torch.as_tensor(np.asarray(box6, np.float64)).to(device=model.device, dtype=model.dtype)
    nt = model.shape.nt

    def compute(pos_all, type_all, n_owned, plan_changed):
        if plan_changed:
            model.set_counts(torch.bincount(type_all[:n_owned].to(torch.int64), minlength=nt).tolist())
        return model.energy_force_domain(pos_all, box, type_all, check_status=plan_changed)
    return compute
