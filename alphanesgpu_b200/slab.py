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
            # no ghosts to re-choose: the counts (and the device status word) are looked at on the first call only
            first = self._plan is None
            self._plan = self._plan or {}
            e, f = self.compute(pos, types, n_own, first)
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


class PeerSlabDomain(SlabDomain):
    """The same decomposition with all traffic carried by the ranks' own kernels over NVLink peer memory
    (stafb_halo_*): positions stored straight into the neighbours' atom arrays, ghost forces stored back, energies
    summed in rank order; the ghost sets, too, are chosen on the device and agreed through mailboxes in the peers'
    memory, with one host synchronisation (six integers) per re-choice and no message library anywhere.  An
    evaluation is push, bounded wait, the model's energy/force kernels, return, collect - issued eagerly, or
    (use_graph) captured once per plan and replayed, which pays when plans live long.

    self.pos is a view of the owned rows of the shared atom array: write new positions into it in place.
    One node only (CUDA IPC); every rank constructs it collectively with the same capacities.  local=True: the
    ranks are objects of ONE process (several ranks emulated on one GPU in the tests) - connect them with
    connect_local() and drive them with plan_local() and the phase_*() calls, every phase for all ranks before the
    next, because kernels on one GPU must never wait for one another."""

    def __init__(self, model, box6, cutoff, rank, world, cap_atoms, cap_face, axis=2, group=None, skin=0.0,
                 halo_every=1, local=False, use_graph=False):
        import ctypes as C
        from . import _lib
        super().__init__(None, box6, cutoff, rank, world, axis=axis, group=group, nt=model.shape.nt, skin=skin,
                         halo_every=halo_every)
        if world < 2:
            raise ValueError("PeerSlabDomain needs at least two ranks; use SlabDomain for one")
        self.model, self.cap_atoms, self.cap_face = model, int(cap_atoms), int(cap_face)
        self.box = torch.as_tensor(np.asarray(box6, np.float64)).to(device=model.device, dtype=model.dtype)
        self._lib = _lib
        h = C.c_void_p()
        self._local = bool(local)
        L = _lib.lib()
        make = lambda: _lib.check(L.stafb_halo_create(model.ctx.h, self.rank, self.world, self.cap_atoms,
                                                      self.cap_face, C.byref(h)), "stafb_halo_create") or h
        if local:
            self.h = make()
        else:
            from .dist import connect_collectively
            # raises RuntimeError on every rank alike when peer memory is not available somewhere
            self.h = connect_collectively(make, L.stafb_halo_handle, L.stafb_halo_connect, L.stafb_halo_destroy,
                                          self.world, model.device, group, "stafb_halo")
        from .dist import _DevArray
        ptr = _lib.lib().stafb_halo_positions(self.h)
        self.pos_all = torch.as_tensor(_DevArray(ptr, 3 * self.cap_atoms, model.dtype),
                                       device=model.device).view(self.cap_atoms, 3)
        # species of owned + ghost atoms: two arrays, because a plan may be prepared while the one before is in use
        self._types_all = [torch.zeros(self.cap_atoms, dtype=torch.int32, device=model.device) for _ in range(2)]
        self._types_sel = 0
        self._pending = False
        self.force = torch.zeros(self.cap_atoms, 3, dtype=model.dtype, device=model.device)
        self.e_own = torch.zeros(1, dtype=model.dtype, device=model.device)
        self.e_total = torch.zeros(1, dtype=model.dtype, device=model.device)
        self._graph = None
        self.use_graph = bool(use_graph) and not local

    @staticmethod
    def connect_local(domains):
        """Ranks of one process: maps every rank's block into the others without IPC."""
        import ctypes as C
        arr = (C.c_void_p * len(domains))(*[d.h for d in domains])
        for d in domains:
            d._lib.check(d._lib.lib().stafb_halo_connect_local(d.h, arr), "stafb_halo_connect_local")

    def set_owned_from_global(self, pos_all, types_all):
        idx = super().set_owned_from_global(pos_all, types_all)
        n = self.pos.shape[0]
        if n > self.cap_atoms:
            raise ValueError("%d owned atoms exceed cap_atoms %d" % (n, self.cap_atoms))
        self.pos_all[:n].copy_(self.pos)
        self.pos = self.pos_all[:n]
        self.model.set_counts(self.counts)
        return idx

    # -- plans ------------------------------------------------------------------------------------
    def _plan_launch(self, which):
        from .model import _p
        L, st = self._lib.lib(), self.model.ctx.stream()
        if which == 0:
            self._lib.check(L.stafb_halo_plan_select(self.h, st, self.pos.shape[0], _p(self.types), self.axis, self.L,
                                                     self.reach), "stafb_halo_plan_select")
        elif which == 1:
            self._lib.check(L.stafb_halo_plan_layout(self.h, st, _p(self._types_all[self._types_sel ^ 1])),
                            "stafb_halo_plan_layout")
        else:
            self._lib.check(L.stafb_halo_plan_done(self.h, st), "stafb_halo_plan_done")

    def _plan_finish(self):
        import ctypes as C
        out = (C.c_int * 4)()
        self._lib.check(self._lib.lib().stafb_halo_plan_finish(self.h, self.model.ctx.stream(), out),
                        "stafb_halo_plan_finish")
        n_lo, n_hi = int(out[0]), int(out[1])
        nall = self.pos.shape[0] + n_lo + n_hi
        self._types_sel ^= 1
        self._pending = False
        self._plan = dict(n_lo=n_lo, n_hi=n_hi, n_send_lo=int(out[2]), n_send_hi=int(out[3]), nall=nall,
                          type_all=self._types_all[self._types_sel][:nall])
        self._graph = None
        self._fresh = True

    def _make_plan(self):
        for which in range(3):
            self._plan_launch(which)
        self._plan_finish()

    @staticmethod
    def plan_local(domains):
        """Ranks of one process: each plan launch for all ranks before the next."""
        for which in range(3):
            for d in domains:
                d._plan_launch(which)
        for d in domains:
            d._plan_finish()

    def _faces(self):
        w = self.L / self.world
        z = self.pos[:, self.axis]
        zw = z - torch.floor(z / self.L) * self.L - self.rank * w
        return torch.nonzero(zw < self.reach).squeeze(1), torch.nonzero(zw >= w - self.reach).squeeze(1)

    @staticmethod
    def plan_local_explicit(domains):
        """The same plan made on the host and installed with stafb_halo_set_plan - the entry point for a caller
        that has its own ghost lists (an MD code's communication lists)."""
        from .model import _p
        torch.cuda.synchronize()
        faces = [d._faces() for d in domains]
        n_lo = [faces[d.lo][1].shape[0] for d in domains]  # what arrives from lo left through lo's upper face
        for d in domains:
            lo, hi = domains[d.lo], domains[d.hi]
            t_lo = lo.types[faces[d.lo][1]]
            t_hi = hi.types[faces[d.hi][0]]
            n_own = d.pos.shape[0]
            nall = n_own + t_lo.shape[0] + t_hi.shape[0]
            d._types_sel ^= 1
            d._types_all[d._types_sel][:nall] = torch.cat([d.types, t_lo, t_hi])
            s_lo = faces[d.rank][0].to(torch.int32).contiguous()
            s_hi = faces[d.rank][1].to(torch.int32).contiguous()
            dst_lo = lo.pos.shape[0] + n_lo[d.lo]  # lo's "ghosts from hi" rows
            dst_hi = hi.pos.shape[0]               # hi's "ghosts from lo" rows
            d._lib.check(d._lib.lib().stafb_halo_set_plan(
                d.h, d.model.ctx.stream(), n_own, t_lo.shape[0], t_hi.shape[0], _p(s_lo), s_lo.shape[0], int(dst_lo),
                _p(s_hi), s_hi.shape[0], int(dst_hi)), "stafb_halo_set_plan")
            d._plan = dict(n_lo=t_lo.shape[0], n_hi=t_hi.shape[0], n_send_lo=s_lo.shape[0], n_send_hi=s_hi.shape[0],
                           nall=nall, type_all=d._types_all[d._types_sel][:nall])
            d._graph, d._fresh = None, True
        torch.cuda.synchronize()

    # -- one evaluation, in the four phases that may be issued rank by rank ---------------------------
    def phase_push(self):
        self._lib.check(self._lib.lib().stafb_halo_push_positions(self.h, self.model.ctx.stream()), "stafb_halo_push")

    def phase_wait(self):
        self._lib.check(self._lib.lib().stafb_halo_wait_positions(self.h, self.model.ctx.stream()), "stafb_halo_wait")

    def phase_eval_return(self):
        from .model import _p
        P = self._plan
        self.model.energy_force_domain(self.pos_all[:P["nall"]], self.box, P["type_all"], check_status=False,
                                       out=(self.e_own, self.force))
        self._lib.check(self._lib.lib().stafb_halo_return_forces(self.h, self.model.ctx.stream(), _p(self.force),
                                                                 _p(self.e_own)), "stafb_halo_return_forces")

    def phase_collect(self):
        from .model import _p
        self._lib.check(self._lib.lib().stafb_halo_collect(self.h, self.model.ctx.stream(), _p(self.force),
                                                           _p(self.e_total)), "stafb_halo_collect")

    def _sequence(self):
        self.phase_push()
        self.phase_wait()
        self.phase_eval_return()
        self.phase_collect()

    def step(self, rebuild=None):
        """Energy of the whole system (tensor [1], bit-identical on every rank) and forces on the owned atoms;
        both are views of buffers the next step overwrites.  Asynchronous except when the ghost sets are re-chosen."""
        # The ghost sets of evaluations r, r+1, ... (r a multiple of halo_every) are chosen from the positions of
        # evaluation r-1: the three plan launches go ahead of that evaluation's own launches, and the host picks the
        # result up while the GPU is busy with it - no idle GPU at a re-plan.  (The skin covers the one evaluation
        # of extra drift.)  The very first plan, and one the caller asks for, is made on the spot.
        if rebuild is None:
            rebuild = self._plan is None
            early = not rebuild and (self._nstep + 1) % self.halo_every == 0
        else:
            early = False
        self._nstep += 1
        if rebuild:
            if self._pending:
                self._plan_finish()  # a prepared plan must be consumed before the next is started
            self._make_plan()
        if early:
            for which in range(3):
                self._plan_launch(which)
            self._pending = True
        if early:
            self._sequence()  # under the plan still in force
            self._plan_finish()
        elif not self.use_graph or self._fresh:
            self._sequence()  # a plan's first evaluation always runs eagerly (allocations on first use)
            self._fresh = False
        else:
            if self._graph is None:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, capture_error_mode="thread_local"):
                    self._sequence()
                self._graph = g
            self._graph.replay()
        return self.e_total, self.force[:self.pos.shape[0]]

    def check(self):
        """Reads the device status words of the model (a saturated neighbour buffer ...) and of the exchange; waits
        for the device.  step() itself never looks at them: call this at the points where a wait does not hurt."""
        self.model.ctx.raise_on_status("stafb_energy_force_domain")
        st = self._lib.lib().stafb_halo_status(self.h)
        if st:
            raise self._lib.StafbError(st, "stafb_halo")

    def set_wait_ms(self, ms):
        self._lib.check(self._lib.lib().stafb_halo_set_wait_ms(self.h, int(ms)), "stafb_halo_set_wait_ms")

    def close(self):
        """Collective: no rank unmaps while another may still store into its block."""
        if self.h is not None:
            torch.cuda.synchronize()
            if not self._local:
                dist.barrier(group=self.group)
            self._graph = None
            self.pos = self.pos_all = None
            self._lib.lib().stafb_halo_destroy(self.h)
            self.h = None
