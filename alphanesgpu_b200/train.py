"""Minimal training driver with the reference's step semantics (STAF/staf_train.py, energy+force and
energy+force+virial).

    python -m alphanesgpu_b200.train input.yaml            # one GPU
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m alphanesgpu_b200.train input.yaml

What is kept from the reference: the YAML keys it reads for this path (precision, dataset_folder with
train/{pos,box,energy,force}.npy + type.dat, buffer_stream_dim_tr, batch_size, number_of_epochs, Rc/Rs/
Rc_Angular/Radial_Buffer/Max_Angular_Neigh, map_rad_afs/map_ang_afs, number_of_decoding_nodes, alpha_bound,
loss_*_prefactor, loss_method, lr_dense_net, optimizer_net, displ_freq, Seed, distribute); buffers of
`buffer_stream_dim_tr` frames cut into batches of `batch_size` (staf_train.py:689-729); one Adam update per
batch with a per-step learning rate from `expdec` or `cosann` (optimizer_learning_rate_utility.py:9-60; as in
the reference only the net optimizer is applied and it updates every trained parameter, staf_model.py:253);
frame buffers sharded idx[rank::world] and the learning rate NOT scaled by the world size
(staf_train.py:131-146,458-463); `lcurve_notmean`-style rows "step loss_e loss_f loss_bound" and `lr_step.dat`.
type_of_training: energy+force+virial (staf_train.py:291-294,372-382: train/virial.npy with 9 values per frame,
loss_virial_prefactor, rows "step loss_e loss_f loss_v loss_bound") runs the virial form of the step per batch.
What is not: restart modes, validation passes, SavedModel export.
Every device step is the C ABI (pipelined stafb_train_step_host_begin/_end, with the virial
stafb_train_step_virial_host_begin/_end; then stafb_adam_step_dev or the peer exchange).
"""
import math
import os
import sys
import time

import numpy as np


# ---------------------------------------------------------------- learning-rate schedules
def expdec(initial_lr, final_lr, total_steps):
    """Keras ExponentialDecay(initial, decay_steps=1, rate=(final/initial)**(1/total), staircase=False)."""
    rate = (final_lr / initial_lr) ** (1.0 / max(1, total_steps))
    return lambda step: initial_lr * rate ** step


def cosann(initial_lr, first_decay_steps, t_mul=2.0, m_mul=1.0, alpha=0.0):
    """Keras CosineDecayRestarts (SGDR) with the reference's argument order."""
    def lr(step):
        frac = step / float(first_decay_steps)
        if t_mul == 1.0:
            i = math.floor(frac)
            frac -= i
        else:
            i = math.floor(math.log(1.0 - frac * (1.0 - t_mul)) / math.log(t_mul))
            frac = (frac - (1.0 - t_mul ** i) / (1.0 - t_mul)) / t_mul ** i
        m = m_mul ** i
        return initial_lr * ((1.0 - alpha) * m * 0.5 * (1.0 + math.cos(math.pi * frac)) + alpha)
    return lr


def build_learning_rate(param, n_epochs, batches_per_buffer, buffer_dim):
    """param: the YAML string, e.g. "expdec 0.001 0.0000001" or "cosann 0.001 3000 1.4 0.9 1e-7"
    (optimizer_learning_rate_utility.py:9-60: expdec decays over n_epochs*buffer_dim steps; cosann's first period
    is first_decay_step*batches_per_buffer*buffer_dim steps)."""
    p = str(param).split()
    f = lambda i, d: float(p[i]) if len(p) > i else d
    if p[0] == "expdec":
        return expdec(f(1, 1e-3), f(2, 1e-7), n_epochs * buffer_dim)
    if p[0] == "cosann":
        return cosann(f(1, 1e-2), int(f(2, 2.0) * batches_per_buffer * buffer_dim), f(3, 2.0), f(4, 1.0), f(5, 0.0))
    raise ValueError("learning rate can be expdec or cosann")


# ---------------------------------------------------------------- configuration
DEFAULTS = dict(precision="float", distribute="none", buffer_stream_dim_tr=4, batch_size=4, number_of_epochs=1,
                Rc=4.5, Rs=2.25, Rc_Angular=4.5, Radial_Buffer=60, Max_Angular_Neigh=60, alpha_bound=5.0,
                loss_energy_prefactor=1.0, loss_force_prefactor=1.0, loss_bound_prefactor=1.0,
                loss_virial_prefactor=1.0, loss_method="huber",
                lr_dense_net="expdec 0.001 0.0000001", optimizer_net="adam", displ_freq=10, Seed=0,
                type_of_training="energy+force", model_name="model_log", number_of_decoding_nodes="64 32",
                map_rad_afs={0: [5, 5], 1: [5, 5]}, map_ang_afs={0: [5, 5, 5], 1: [5, 5, 5]})


def load_config(path_or_dict):
    import yaml
    cfg = dict(DEFAULTS)
    if isinstance(path_or_dict, dict):
        cfg.update(path_or_dict)
    else:
        with open(path_or_dict) as f:
            cfg.update(yaml.safe_load(f) or {})
    if cfg["type_of_training"] not in ("energy+force", "energy+force+virial"):
        raise ValueError("type_of_training can be energy+force or energy+force+virial in this driver")
    return cfg


def model_shape_from_config(cfg, tipos):
    """Fr / Fa per central species from the channel maps (map_rad_afs: species -> counts per partner species,
    map_ang_afs: species -> counts per species-pair class), MLP widths from number_of_decoding_nodes + [1]."""
    from .params import ModelShape
    nt = len(tipos)
    Fr = [int(sum(cfg["map_rad_afs"][t])) for t in range(nt)]
    Fa = [int(sum(cfg["map_ang_afs"][t])) for t in range(nt)]
    widths = [int(w) for w in str(cfg["number_of_decoding_nodes"]).split()] + [1]
    return ModelShape(nt=nt, tipos=[int(t) for t in tipos], Fr=Fr, Fa=Fa, widths=widths)


def init_params(shape, cfg, seed, dtype=np.float64):
    """Initial parameters in the flat layout of include/stafb.h: alpha ~ U(-b, b) for the radial and the first
    two angular exponents, the third angular exponent ~ U(-10, 0), mu ~ U(-b, b)
    (STAF/init_params/init_AFs_param.py:55-71), Glorot-uniform Dense kernels with zero biases (Keras default);
    embeddings are the 0/1 masks of the channel maps, squared."""
    rng = np.random.default_rng(seed)
    nt, C = shape.nt, shape.C
    theta = np.zeros(shape.n_params)
    emb = np.zeros(shape.n_emb)
    b = 1.0
    for t in range(nt):
        o = shape.offsets(t)
        Fr, Fa = shape.Fr[t], shape.Fa[t]
        theta[o["a2"]:o["a2"] + nt * Fr] = rng.uniform(-b, b, nt * Fr)
        a3 = np.zeros((C * Fa, 3))
        a3[:, :2] = rng.uniform(-b, b, (C * Fa, 2))
        a3[:, 2] = rng.uniform(-10.0, 0.0, C * Fa)
        theta[o["a3"]:o["a3"] + C * 3 * Fa] = a3.reshape(C, 3 * Fa).ravel()
        theta[o["mu"]:o["mu"] + Fr + Fa] = rng.uniform(-b, b, Fr + Fa)
        w, n_in = o["w"], Fr + Fa
        for width in shape.widths:
            lim = math.sqrt(6.0 / (n_in + width))
            theta[w:w + n_in * width] = rng.uniform(-lim, lim, n_in * width)
            w += n_in * width + width
            n_in = width
        e2 = np.zeros((nt, Fr))
        c0 = 0
        for q, cnt in enumerate(cfg["map_rad_afs"][t]):
            e2[q, c0:c0 + cnt] = 1.0
            c0 += cnt
        e3 = np.zeros((C, Fa))
        c0 = 0
        for s, cnt in enumerate(cfg["map_ang_afs"][t]):
            e3[s, c0:c0 + cnt] = 1.0
            c0 += cnt
        emb[o["emb"]:o["emb"] + nt * Fr] = e2.ravel()
        emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + C * Fa] = e3.ravel()
    return theta.astype(dtype), emb.astype(dtype)


def buffer_indices(n_frames, buffer_dim, rank=0, world=1):
    """Frame indices per buffer (rows), sharded like STAF/staf_train.py:131-146: buffers idx[rank::world]."""
    nbuf = n_frames // buffer_dim
    idx = np.arange(nbuf * buffer_dim).reshape(nbuf, buffer_dim)
    return idx[rank::world][: nbuf // world] if world > 1 else idx


# ---------------------------------------------------------------- the loop
def train(cfg, out_dir=".", data=None, max_steps=None, log=print):
    """Runs the training loop.  data = dict(pos[nfr,3N], box[nfr,6], energy[nfr], force[nfr,3N], tipos) overrides
    dataset_folder.  Returns the list of per-step losses rows (step, loss, loss_e, loss_f, loss_bound, lr)."""
    import torch
    import torch.distributed as dist
    from . import dist as dp
    from .model import StafModel

    cfg = load_config(cfg)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    own_pg = False
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
        own_pg = True
    if data is None:
        root = cfg["dataset_folder"]
        ld = lambda n: np.load(os.path.join(root, "train", n), mmap_mode="r")
        data = dict(pos=ld("pos.npy"), box=ld("box.npy"), energy=ld("energy.npy"), force=ld("force.npy"),
                    tipos=np.loadtxt(os.path.join(root, "type.dat"), dtype=int).reshape(-1))
        if cfg["type_of_training"] == "energy+force+virial":
            data["virial"] = ld("virial.npy")
    with_virial = cfg["type_of_training"] == "energy+force+virial"
    if with_virial:
        if "virial" not in data:
            raise ValueError("type_of_training=energy+force+virial requires virial labels (train/virial.npy)")
        if int(np.prod(data["virial"].shape[1:])) != 9:
            raise ValueError("virial labels must have 9 values per frame (full tensor, total eV)")
    pv = float(cfg["loss_virial_prefactor"])
    double = str(cfg["precision"]).lower() in ("double", "float64", "fp64")
    np_dt, t_dt = (np.float64, torch.float64) if double else (np.float32, torch.float32)
    shape = model_shape_from_config(cfg, data["tipos"])
    N = shape.N
    theta, emb = init_params(shape, cfg, int(cfg["Seed"]))
    M = int(cfg["Max_Angular_Neigh"])
    geo = dict(Rc=float(cfg["Rc"]), Rs=float(cfg["Rs"]), Ra=float(cfg["Rc_Angular"]), nr=int(cfg["Radial_Buffer"]),
               na=M * (M - 1) // 2)  # angular buffer = M(M-1)/2 (STAF/staf_train.py:231-232)
    bs, bdim, ne = int(cfg["batch_size"]), int(cfg["buffer_stream_dim_tr"]), int(cfg["number_of_epochs"])
    nb = bdim // bs
    model = StafModel(shape, geo, theta, emb, bs, dtype=t_dt, device=dev, pe=float(cfg["loss_energy_prefactor"]),
                      pf=float(cfg["loss_force_prefactor"]), pb=float(cfg["loss_bound_prefactor"]),
                      alpha_bound=float(cfg["alpha_bound"]), loss="huber" if cfg["loss_method"] == "huber" else "mse")
    dp.broadcast_params_(model.theta)  # rank 0's initial parameters win (hvd.broadcast_variables)
    opt = str(cfg["optimizer_net"]).split()
    if opt[0] != "adam":
        raise ValueError("optimizer can only be adam in this driver")
    eps = float(opt[1]) if len(opt) > 1 else 1e-7
    lr_of = build_learning_rate(cfg["lr_dense_net"], ne, nb, bdim)
    bufs = buffer_indices(data["pos"].shape[0], bdim, rank, world)
    if bufs.shape[0] == 0:
        raise ValueError("no training buffer for rank %d (world %d)" % (rank, world))
    chief = rank == 0
    lcurve = open(os.path.join(out_dir, "lcurve_notmean"), "w") if chief else None
    lrfile = open(os.path.join(out_dir, "lr_step.dat"), "w") if chief else None
    rows, step, pending = [], 0, None
    displ = int(cfg["displ_freq"])
    t0 = time.time()
    # Several ranks on one node: gradient averaging + Adam as one peer-memory kernel (grad_exchange: peer, the
    # default); grad_exchange: allreduce keeps the NCCL all-reduce followed by the Adam kernel (needed across nodes).
    # grad_exchange: peer_always takes the exchange kernel also on a single rank (what `mpirun -np 1` with
    # distribute: horovod is in the reference's none-vs-horovod loss-curve check,
    # test/test-training-pipeline/compare_distribute_lcurve.py).
    px = None
    mode = str(cfg.get("grad_exchange", "peer")).lower()
    if (world > 1 and mode == "peer") or mode == "peer_always":
        px = dp.PeerExchange(model)
        # Horovod simply waits for a slow rank; the kernel's wait has to be bounded, so the bound is generous here
        # (ranks read different memory-mapped buffers and may be seconds apart) - the short default is for tests.
        px.set_wait_ms(int(cfg.get("peer_wait_ms", 60000)))
    own_grad = model.grad
    fallbacks = []

    def check_exchange(where):
        """Collective.  If any rank's exchange kernel gave up on a late peer, the replicas may differ from that step
        on: rank 0's parameters, moments and step count are re-broadcast and training continues on the NCCL
        all-reduce arm."""
        nonlocal px
        if px is None:
            return
        bad = torch.tensor([float(px.status())], device=dev)
        if world > 1:
            dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if float(bad) == 0.0:
            return
        log("gradient exchange: status %d at %s - re-broadcasting the parameters, continuing with all-reduce"
            % (int(bad), where))
        fallbacks.append((where, int(bad)))
        stream.synchronize()
        px.close()
        px = None
        model.use_grad(own_grad)
        for t in (model.theta, model.adam_m, model.adam_v, model.step_d):
            dp.broadcast_params_(t)
    # a stream of its own: the library replays each step as CUDA graphs, which the legacy default stream cannot capture
    stream = torch.cuda.Stream(device=dev)
    stream.wait_stream(torch.cuda.current_stream(dev))
    torch.cuda.set_stream(stream)

    def collect(p):
        st, slot, lr = p
        if with_virial:
            l = model.loss_and_grad_virial_host_end(slot)
        else:
            l = model.loss_and_grad_host_end(slot)
        if st % displ == 0:
            check_exchange("step %d" % st)
        if with_virial:  # columns of the reference: step Loss_E Loss_F Loss_V Loss_Bound (staf_train.py:625,742-745)
            rows.append((st, l[0], l[1], l[3], l[2], lr, l[4]))
            if chief:
                lcurve.write("%d %.9g %.9g %.9g %.9g\n" % (st, l[1], l[3], l[4], l[2]))
                lrfile.write("%.9g\n" % lr)
            return
        rows.append((st, l[0], l[1], l[3], l[2], lr))
        if chief:
            lcurve.write("%d %.9g %.9g %.9g\n" % (st, l[1], l[3], l[2]))
            lrfile.write("%.9g\n" % lr)

    done = False
    for ep in range(ne):
        for el in bufs:
            el = np.sort(el)
            pos = np.asarray(data["pos"][el], np_dt)
            box = np.asarray(data["box"][el], np_dt)
            en = np.asarray(data["energy"][el], np_dt).reshape(-1)
            fo = np.asarray(data["force"][el], np_dt).reshape(len(el), -1)
            vi = np.asarray(data["virial"][el], np_dt).reshape(len(el), 9) if with_virial else None
            if world > 1:
                dist.barrier()  # the ranks read different buffers: start the buffer's steps together
            for k in range(nb):
                sl = slice(k * bs, (k + 1) * bs)
                lr = lr_of(step)
                step += 1
                if px is not None:
                    model.use_grad(px.grad(step & 1))
                if with_virial:
                    model.loss_and_grad_virial_host_begin(pos[sl].reshape(bs, 3 * N), box[sl], en[sl], fo[sl], vi[sl],
                                                          step & 1, pv=pv)
                else:
                    model.loss_and_grad_host_begin(pos[sl].reshape(bs, 3 * N), box[sl], en[sl], fo[sl], step & 1)
                if px is not None:
                    px.allreduce_adam(model, step & 1, lr, eps=eps)
                else:
                    dp.allreduce_sum_(model.grad)
                    model.adam_update_dev(lr, eps=eps, grad_scale=1.0 / world)
                if pending is not None:
                    collect(pending)
                pending = (step, step & 1, lr)
                if chief and step % displ == 0:
                    log("Epoch %d step %d. Time to elaborate %d batch of %d frames is %.4f"
                        % (ep, step, displ, bs, time.time() - t0))
                    t0 = time.time()
                if max_steps is not None and step >= max_steps:
                    done = True
                    break
            if done:
                break
        if done:
            break
    if pending is not None:
        collect(pending)
    if chief:
        lcurve.close()
        lrfile.close()
    stream.synchronize()
    torch.cuda.set_stream(torch.cuda.default_stream(dev))
    check_exchange("the last step")
    if px is not None:
        px.close()
    result = dict(rows=rows, theta=model.theta.detach().cpu().numpy().copy(), shape=shape, geo=geo,
                  exchange_fallbacks=fallbacks)
    model.close()
    if own_pg:
        dist.destroy_process_group()
    return result


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python -m alphanesgpu_b200.train input.yaml [output_dir]")
    train(sys.argv[1], sys.argv[2] if len(sys.argv) > 2 else ".")
