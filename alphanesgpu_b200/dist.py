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
