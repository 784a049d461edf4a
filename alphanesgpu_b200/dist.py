"""Data-parallel training plumbing: frames are sharded across ranks, every rank evaluates its own
frames, the flat gradient is summed with ONE all-reduce per step and divided by the world size
before Adam (what hvd.DistributedOptimizer does variable by variable in the reference:
STAF/staf_train.py:484-487).  The learning rate is NOT scaled by the world size
(STAF/staf_train.py:458-463; README.md:95-105 of the reference records that scaling it stalls
force training).  torch.distributed is the transport (NCCL on GPUs, gloo in the CPU tests).
"""
import numpy as np
import torch
import torch.distributed as dist


def shard_indices(n_frames, rank, world):
    """Frame indices of this rank: idx[rank::world], truncated so that every rank gets the same count
    (STAF/staf_train.py:131-146).  Equal counts make the mean of per-rank gradients equal to the
    gradient of the global batch."""
    per = n_frames // world
    return np.arange(n_frames)[rank::world][:per]


def broadcast_params_(theta, src=0, group=None):
    """hvd.broadcast_variables equivalent (STAF/staf_train.py:616-618): rank `src` wins."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.broadcast(theta, src=src, group=group)
    return theta


def allreduce_sum_(flat_grad, group=None):
    """One collective for the whole flat gradient (alpha2b, alpha3b, mu, MLP weights of all species)."""
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat_grad, op=dist.ReduceOp.SUM, group=group)
    return flat_grad


def world_size(group=None):
    return dist.get_world_size(group) if dist.is_initialized() else 1


def dp_train_step(model, pos, box, e_label, f_label, lr, group=None, **adam):
    """One data-parallel step on device tensors of this rank's frames."""
    model.loss_and_grad(pos, box, e_label, f_label)
    allreduce_sum_(model.grad, group)
    model.adam_update_dev(lr, grad_scale=1.0 / world_size(group), **adam)


class HostWatchdog:
    """Host-side failure detection for the data-parallel loop: every rank publishes a heartbeat
    counter in the rendezvous store before it enters the step's collective; a rank that sees a peer
    more than `patience` steps behind, or missing after `timeout_s`, raises instead of hanging in the
    all-reduce.  Nothing here touches the GPU."""

    def __init__(self, store, rank, world, timeout_s=5.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, float(timeout_s)

    def beat(self, step):
        self.store.set("hb_%d" % self.rank, str(step))

    def check(self, step):
        import time
        t0 = time.time()
        while True:
            behind = []
            for r in range(self.world):
                try:
                    v = int(self.store.get("hb_%d" % r))
                except Exception:
                    v = -1
                if v < step:
                    behind.append(r)
            if not behind:
                return
            if time.time() - t0 > self.timeout_s:
                raise RuntimeError("ranks %s did not reach step %d within %.1f s" % (behind, step, self.timeout_s))
            time.sleep(0.01)


def connect_collectively(create, get_handle, connect, destroy, world, device, group, what):
    """Creates this rank's peer-memory block (create() -> handle), exchanges the CUDA IPC handles and maps the
    peers' blocks.  A failure on any rank (no peer access between two GPUs, out of memory) reaches every rank:
    all of them go through the same collectives, release what they made and raise RuntimeError together, so the
    caller can fall back to a message-based path on all ranks alike."""
    import ctypes as C
    from . import _lib
    h, err, mine = None, None, b""
    try:
        h = create()
        buf = C.create_string_buffer(64)
        _lib.check(get_handle(h, buf), what + "_handle")
        mine = bytes(buf.raw)
    except Exception as exc:  # noqa: BLE001 - whatever it is, the other ranks must learn of it
        err = exc
    handles = [None] * world
    dist.all_gather_object(handles, mine, group=group)
    if err is None and all(len(x) == 64 for x in handles):
        try:
            _lib.check(connect(h, b"".join(handles)), what + "_connect")
        except Exception as exc:  # noqa: BLE001
            err = exc
    elif err is None:
        err = RuntimeError("a peer rank could not create its block")
    ok = torch.tensor([0.0 if err is not None else 1.0], device=device)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    if float(ok) == 0.0:
        if h is not None:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            dist.barrier(group=group)  # nobody unmaps while another rank may still be mapping
            destroy(h)
        else:
            dist.barrier(group=group)
        raise RuntimeError("%s: peer memory is not available on every rank (%s)" % (what, err))
    dist.barrier(group=group)
    return h


class _DevArray:
    """Minimal __cuda_array_interface__ carrier, so that torch can wrap memory the library allocated."""

    def __init__(self, ptr, n, dtype):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": "<f4" if dtype == torch.float32 else "<f8",
                                         "data": (int(ptr), False), "version": 2}


class PeerExchange:
    """Gradient averaging + Adam as one kernel per rank over NVLink peer memory (stafb_allreduce_adam) for the
    ranks of one node: the replacement of all_reduce(grad) + Adam in the data-parallel step.

    Every rank calls the constructor collectively (the CUDA IPC handles travel through
    torch.distributed.all_gather_object), then alternates parity 0 / 1 from step to step:

        model.use_grad(px.grad(k & 1)); model.loss_and_grad(...); px.allreduce_adam(model, k & 1, lr)

    The kernel's wait for the peers is bounded; status() returns STAFB_ERR_PEER_TIMEOUT after a miss."""

    def __init__(self, model, group=None):
        import ctypes as C
        from . import _lib
        self.model, self.group = model, group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = world_size(group)
        self.n = model.theta.numel()
        h = C.c_void_p()
        self.h = None
        if self.world == 1:
            _lib.check(_lib.lib().stafb_peer_create(model.ctx.h, self.rank, self.world, self.n, C.byref(h)),
                       "stafb_peer_create")
            self.h = h
        else:
            # every rank goes through the same collectives whatever fails locally (no peer access between two
            # GPUs, no memory ...), and all ranks raise together
            self.h = connect_collectively(
                lambda: _lib.check(_lib.lib().stafb_peer_create(model.ctx.h, self.rank, self.world, self.n,
                                                                C.byref(h)), "stafb_peer_create") or h,
                _lib.lib().stafb_peer_handle, _lib.lib().stafb_peer_connect, _lib.lib().stafb_peer_destroy,
                self.world, model.device, group, "stafb_peer")
        self._grads = []
        for par in (0, 1):
            ptr = _lib.lib().stafb_peer_grad(self.h, par)
            self._grads.append(torch.as_tensor(_DevArray(ptr, self.n, model.dtype), device=model.device))

    def grad(self, parity):
        """Gradient buffer of this rank for steps of the given parity (a torch view of library memory)."""
        return self._grads[parity & 1]

    def allreduce_adam(self, model, parity, lr, beta1=0.9, beta2=0.999, eps=1e-7):
        from . import _lib
        from .model import _p
        if not hasattr(model, "step_d"):
            model.step_d = torch.zeros(2, dtype=torch.int32, device=model.device)
        _lib.check(_lib.lib().stafb_allreduce_adam(model.ctx.h, self.h, model.ctx.stream(), int(parity) & 1,
                                                   _p(model.theta), _p(model.adam_m), _p(model.adam_v), float(lr),
                                                   float(beta1), float(beta2), float(eps), _p(model.step_d)),
                   "stafb_allreduce_adam")

    def status(self):
        """First status the exchange kernels recorded (0, or STAFB_ERR_PEER_TIMEOUT); waits for the device."""
        from . import _lib
        return _lib.lib().stafb_peer_status(self.h)

    def set_wait_ms(self, ms):
        """Bound of the kernel's wait for the peers' gradients, in milliseconds of SM clock."""
        from . import _lib
        _lib.check(_lib.lib().stafb_peer_set_wait_ms(self.h, int(ms)), "stafb_peer_set_wait_ms")

    def close(self):
        """Collective: every rank must have finished its last step before any rank unmaps the buffers."""
        from . import _lib
        if self.h is not None:
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)
            self._grads = []
            _lib.lib().stafb_peer_destroy(self.h)
            self.h = None
