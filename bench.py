#!/usr/bin/env python
"""Benchmark of the STAF hot path on B200: 768-atom water energy+force training step, fp32.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference] [--workload md]

One "step" = one training evaluation of a batch of B frames (neighbour list, descriptors, fingerprints, MLP,
forces, loss, backward to alpha/mu/MLP weights) followed by the Adam update; with N > 1 (launched by
torch.distributed.run, one rank per GPU) every rank works on its own frames and the flat gradient is averaged
once per step (learning rate not scaled by N).  Prints one JSON line (rank 0).

`value`       frames/s with the inputs resident in HBM, the step replayed from CUDA graphs, L2 flushed between
              steps, CUDA-event time summed over exactly K steps, max over ranks.  The K-step block is then
              repeated until a quarter of a second of device time is covered: `repeat` has median and spread.
`e2e`         frames/s through the host-buffer entry points of the C ABI (stafb_train_step_host_begin/_end +
              Adam): host->device reads of positions/box/labels and the device->host write of the losses are
              inside the timed region (wall clock, synchronised both sides).
`roofline`    the dominant kernel of the step, timed live with CUDA events on the launching stream.
`roofline_operator_boundary`  the operator path on materialised tensors (descriptor fill and the four angular
              operators), each against its algorithmic bytes.
`fp32_pipe`, `fp64`, `real_model`, `batch8`, `md`  sub-records: FMA-pipe fraction from a counted flop figure, the
              same step in float64, the reference's real frame with its exported 60-140-140-1 model, eight
              frames per GPU, and the 24,576-atom inference box (atom-steps/s).
`cpu_baseline` the CPU oracle (a restatement of the reference's kernel math; the reference's own ops are GPU-only)
              on a bounded sample at one thread and at all host threads, plus the two pieces of the reference's
              own CPU code that compile stand-alone (neighbour list, native MLP) on their stages.
`--impl reference` times that same CPU restatement as the reference arm.
"""
import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(Rc=4.5, Rs=2.25, Ra=4.5, nr=60, na=1770)
METRIC = "768-atom water E+F train frames/s"
MD_METRIC = "24576-atom water E+F atom-steps/s (slab-decomposed inference)"
PUBLISHED_V100_FRAMES_PER_S = 10.9  # reference README.md:42-45 (V100, fp32, batch 4)
# Counted floating-point operations of the three sweeps per (triplet, active channel), multiply-add = 2, one per
# exponential (alphanesgpu_b200/csrc/sweep.cuh): fingerprints + d(AF)/d(alpha) 21, forces 2 x 15 (ordered pairs),
# backward of the forces 44; per triplet (geometry, cotangent projections, force assembly): 9 + 2 x 21 + 44.
FLOPS_PER_TRIPLET_CHANNEL = 21 + 30 + 44
FLOPS_PER_TRIPLET = 9 + 42 + 44
# dram__bytes_read.sum + dram__bytes_write.sum per launch at batch 4 (one ncu capture; None: not captured)
TRAFFIC_NCU_B4 = {"af_fwd": 6.852e6, "force": 7.196e6, "force_grad": 7.232e6, "mlp_fwd": 0.397e6, "mlp_bwd": 3.863e6}


def make_batches(rank, n_batches, B, dtype, seed0=1100):
    from alphanesgpu_b200 import synth
    seeds = [seed0 + 64 * rank + i for i in range(n_batches * B)]
    pos, box, tipos = synth.water_frames("water768", seeds)
    shape = synth.baseline_shape(tipos)
    N = shape.N
    el, fl = synth.labels(n_batches * B, N, seed=3000 + rank)
    rs = lambda a, *s: np.ascontiguousarray(a.reshape(n_batches, B, *s).astype(dtype))
    return shape, rs(pos, 3 * N), rs(box, 6), rs(el), rs(fl, 3 * N)


def real_model_batches(n_batches, B, dtype):
    """The reference's real 768-atom frame (test/test-inference-pipeline/frames/pos_0) copied n_batches*B times with
    a small seeded jitter, and its exported model (test/test-lammps-smoke/model_onnx_grad_float: Fr 20, Fa 40,
    MLP 60-140-140-1), both from the fixtures under tests/golden/ref_frame0."""
    from alphanesgpu_b200 import params, synth
    d = os.path.join(ROOT, "tests", "golden", "ref_frame0")
    cfg, shape, theta, emb = params.load_model_dir(d, np.float64)
    pos0 = np.load(os.path.join(d, "pos_0.npy")).reshape(1, -1)
    box0 = np.load(os.path.join(d, "box_0.npy")).reshape(1, 6)
    rng = np.random.default_rng(77)
    n = n_batches * B
    pos = pos0 + rng.normal(0.0, 0.02, size=(n, pos0.shape[1]))
    box = np.repeat(box0, n, axis=0)
    el, fl = synth.labels(n, shape.N, seed=3100)
    rs = lambda a, *s: np.ascontiguousarray(a.reshape(n_batches, B, *s).astype(dtype))
    return shape, theta, emb, rs(pos, 3 * shape.N), rs(box, 6), rs(el), rs(fl, 3 * shape.N)


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                sm = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(
                    nv, "nvmlDeviceGetCurrentClocksEventReasons") else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.rows.append((sm, rs))
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        if self._t:
            self._stop.set()
            self._t.join()
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not self.nv or not self.rows:
            return out
        nv = self.nv
        out["sm_mhz"] = float(np.median([r[0] for r in self.rows]))
        try:
            out["sm_max_mhz"] = float(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
        except Exception:
            pass
        names = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        seen = 0
        for _, rs in self.rows:
            seen |= rs
        out["reasons"] = [n for bit, n in names.items() if seen & bit]
        out["samples"] = len(self.rows)
        return out


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_port_frames_per_s(B, n_steps, threads):
    """Times the CPU oracle's full training evaluation (no optimizer) on n_steps batches of B frames."""
    from oracle import oracle
    from alphanesgpu_b200 import synth
    oracle.set_threads(int(threads))
    shape, pos, box, el, fl = make_batches(0, n_steps, B, np.float32)
    theta, emb = synth.init_params(shape, dtype=np.float32)
    sd = shape.desc()
    oracle.energy_force_grad(CFG, sd, pos[0, :1], box[0, :1], shape.type_map, theta, emb, np.float32, with_grad=True,
                             e_label=el[0, :1], f_label=fl[0, :1])  # warm-up (one frame)
    t0 = time.perf_counter()
    for i in range(n_steps):
        r = oracle.energy_force_grad(CFG, sd, pos[i], box[i], shape.type_map, theta, emb, np.float32, with_grad=True,
                                     e_label=el[i], f_label=fl[i])
        assert r["status"] == 0
    dt = time.perf_counter() - t0
    return B * n_steps / dt, dt


def cpu_reference_pieces(B):
    """The two pieces of the reference's own CPU code that compile stand-alone (oracle/_ref), timed on their
    stages of one batch: the distance-ordered neighbour list (STAF/src/descriptor_builder/cell_list.cu.cc) and
    the native MLP evaluator (libstaf/src/mlp/staf_mlp_ort.cc:196-242, real exported weights)."""
    from oracle import oracle
    out = {}
    if not oracle.ref_available():
        return {"unavailable": "oracle/_ref was not built (needs the reference tree at build time)"}
    try:
        shape, pos, box, el, fl = make_batches(0, 1, B, np.float32)
        t0 = time.perf_counter()
        for b in range(B):
            oracle.ref_neighbour_list(CFG["Rc"], CFG["nr"], pos[0, b:b + 1], box[0, b:b + 1], np.float32)
        dt = time.perf_counter() - t0
        out["neighbour_list"] = {"frames_per_s": B / dt, "threads": 1, "sample": "%d frames of 768 atoms" % B}
    except Exception as exc:  # the fixture-level pins live in tests/; a timing that cannot run is only reported
        out["neighbour_list"] = {"unavailable": str(exc)[:200]}
    try:
        d = os.path.join(ROOT, "tests", "golden", "ref_frame0")
        rng = np.random.default_rng(5)
        afs = [rng.uniform(0.05, 3.0, size=(256 * B, 60)), rng.uniform(0.05, 3.0, size=(512 * B, 60))]
        t0 = time.perf_counter()
        oracle.ref_mlp_eval(d, afs, np.float32)
        dt = time.perf_counter() - t0
        out["native_mlp"] = {"atoms_per_s": 768 * B / dt, "frames_per_s": B / dt, "threads": 1,
                             "sample": "%d atoms, 60-140-140-1" % (768 * B)}
    except Exception as exc:
        out["native_mlp"] = {"unavailable": str(exc)[:200]}
    return out


def cpu_baseline_record(B):
    """Bounded sample: one batch at one thread, six batches at all host threads."""
    ncpu = os.cpu_count() or 1
    f1, t1 = cpu_port_frames_per_s(B, 1, 1)
    fa, ta = cpu_port_frames_per_s(B, 6, ncpu)
    return {"value": fa, "unit": "frames/s", "cores": ncpu, "kind": "port",
            "sample": "6 batches of %d frames at %d threads (%.1f s); 1 batch at 1 thread (%.1f s)" % (B, ncpu, ta, t1),
            "one_thread": {"value": f1, "unit": "frames/s", "cores": 1},
            "reference_cpu_pieces": cpu_reference_pieces(B)}


def run_reference(args):
    """Reference arm: the reference's hot path on the host cores.  Its own ops are GPU-only TensorFlow kernels
    (TensorFlow cannot be installed here), so the timed code is the CPU restatement in oracle/, OpenMP over atoms,
    on every host thread whatever OMP_NUM_THREADS the launcher exported."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B = args.batch
    ncpu = os.cpu_count() or 1
    # bounded sample: each "step" is one batch; cap the total so that the run ends within minutes
    steps = max(1, min(args.steps, 12))
    warm = max(1, min(args.warmup, 1))
    for _ in range(warm):
        cpu_port_frames_per_s(B, 1, ncpu)
    fps, dt = cpu_port_frames_per_s(B, steps, ncpu)
    line = {
        "impl": "reference", "metric": METRIC, "value": fps, "unit": "frames/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "water768 E+F training evaluation, batch %d, fp32" % B,
                   "note": "CPU restatement of the reference kernels (oracle/), OpenMP over atoms on %d threads; "
                           "no optimizer step; a bounded sample of %d batches" % (ncpu, steps)},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": ncpu, "kind": "port",
                         "sample": "%d batches of %d frames" % (steps, B)},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------ GPU arm
class Stepper:
    """The training step of one model as replayed CUDA graphs: per distinct batch one graph for the neighbour
    records (they depend on positions only, so they are built on a second stream while the previous step is still
    running) and one for the rest of the step including the optimiser.  exchange: None (local Adam), "peer" (the
    fused peer-memory average + Adam kernel inside the step graph) or "nccl" (all-reduce between two graphs)."""

    def __init__(self, torch, dist, model, data, lr, world, exchange=None, px=None):
        self.torch, self.dist, self.model, self.lr, self.world = torch, dist, model, lr, world
        self.d_pos, self.d_box, self.d_el, self.d_fl = data
        self.NB, self.B = self.d_pos.shape[0], self.d_pos.shape[1]
        assert self.NB % 2 == 0  # batch i always uses record set i & 1
        self.exchange, self.px = exchange, px
        dev = model.device
        self.main = torch.cuda.current_stream(dev)
        self.side = torch.cuda.Stream(device=dev)
        self.rows_stream = torch.cuda.Stream(device=dev)
        self.own_grad = model.grad
        for i in range(2):  # allocate both record sets and set the kernels' attributes outside any capture
            model.prefetch_rows(self.d_pos[i], self.d_box[i], i)
            model.loss_and_grad_prefetched(i, self.B, self.d_el[i], self.d_fl[i])
        model.adam_update_dev(lr)
        torch.cuda.synchronize()
        self.graphs = self._build()
        self.ready = [torch.cuda.Event(), torch.cuda.Event()]
        self.go = torch.cuda.Event()
        with torch.cuda.stream(self.rows_stream):  # records of the very first step
            self.graphs[0][0].replay()
            self.ready[0].record(self.rows_stream)
        self.counter = 0

    def _build(self):
        torch, model, px = self.torch, self.model, self.px
        graphs = []
        self.side.wait_stream(self.main)
        with torch.cuda.stream(self.side):
            for i in range(self.NB):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=self.side):
                    model.prefetch_rows(self.d_pos[i], self.d_box[i], i & 1)
                g1 = torch.cuda.CUDAGraph()
                model.use_grad(px.grad(i & 1) if self.exchange == "peer" else self.own_grad)
                with torch.cuda.graph(g1, stream=self.side):
                    model.loss_and_grad_prefetched(i & 1, self.B, self.d_el[i], self.d_fl[i])
                    if self.exchange is None:
                        model.adam_update_dev(self.lr)
                    elif self.exchange == "peer":
                        px.allreduce_adam(model, i & 1, self.lr)
                g2 = None
                if self.exchange == "nccl":
                    g2 = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g2, stream=self.side):
                        model.adam_update_dev(self.lr, grad_scale=1.0 / self.world)
                graphs.append((gr, g1, g2))
        self.main.wait_stream(self.side)
        torch.cuda.synchronize()
        return graphs

    def step(self):
        """One training step.  Every step also builds the records of the NEXT one; it returns only after those are
        complete on the device timeline of the main stream, so that a CUDA-event interval around the call contains
        all the work of exactly one step."""
        k = self.counter
        self.counter += 1
        i, s = k % self.NB, k & 1
        self.go.record(self.main)
        self.rows_stream.wait_event(self.go)  # the next records start inside this step, not during the flush before it
        with self.torch.cuda.stream(self.rows_stream):
            self.graphs[(k + 1) % self.NB][0].replay()
            self.ready[s ^ 1].record(self.rows_stream)
        self.main.wait_event(self.ready[s])
        self.graphs[i][1].replay()
        if self.exchange == "nccl":
            self.dist.all_reduce(self.model.grad)
            self.graphs[i][2].replay()
        self.main.wait_event(self.ready[s ^ 1])

    def time_steps(self, K, flush, barrier):
        """Device milliseconds of each of K steps, L2 flushed before every step."""
        torch = self.torch
        ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
        ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
        barrier()
        for k in range(K):
            flush.zero_()
            ev0[k].record()
            self.step()
            ev1[k].record()
        barrier()
        return np.array([a.elapsed_time(b) for a, b in zip(ev0, ev1)])


def time_blocks(stepper, K, W, flush, barrier, reduce_max, min_total_ms=250.0, max_blocks=400):
    """W warm-up steps, then blocks of exactly K steps until min_total_ms of device time (max over ranks) is
    covered.  Returns the per-block totals (ms, max over ranks) and the per-step times of the first block."""
    for _ in range(W):
        stepper.step()
        flush.zero_()
    totals, first = [], None
    while len(totals) < max_blocks:
        per_step = stepper.time_steps(K, flush, barrier)
        if first is None:
            first = per_step
        totals.append(reduce_max(float(per_step.sum())))
        if sum(totals) >= min_total_ms:
            break
    return np.array(totals), first


def operator_boundary(torch, model, ctx, shape, d_pos, d_box, B, N, peak, flush):
    """The operator path on materialised tensors (what the TensorFlow graph of the reference moves through HBM):
    the angular descriptor fill and the four angular operators of one central species at a time, each timed with
    CUDA events and set against its algorithmic bytes (per atom: T(7s+8) + 4m s for the force operators, T(s+8) +
    m s for the fingerprint operators, s = 4).  Also the sum over the operator chain of one training evaluation."""
    from alphanesgpu_b200 import ops
    out = []
    nr_, na_ = CFG["nr"], CFG["na"]
    isz = 4
    dev = d_pos.device
    te = lambda *sh, d=torch.float32: torch.empty(*sh, dtype=d, device=dev)
    o_ang, o_im3, o_d3b = te(B, N, na_), te(B, N, 2 * na_, d=torch.int32), te(B, N, 3, 2 * na_)
    o_rad, o_d3s, o_d2b, o_d3bs = te(B, N, nr_), te(B, N, nr_), te(B, N, 3, nr_), te(B, N, 3, nr_)
    o_im2, o_ntr = te(B, N, nr_ + 1, d=torch.int32), te(B, N, d=torch.int32)
    from alphanesgpu_b200 import _lib
    vp = lambda t: None if t is None else C.c_void_p(t.data_ptr())

    def desc_call(angular):
        a = (o_ang, o_im3, o_d3b) if angular else (None, None, None)
        rc = _lib.lib().stafb_compute_descriptors_light(ctx.h, ctx.stream(), vp(d_pos), vp(d_box), B, N, vp(o_rad),
                                                        vp(a[0]), vp(o_d3s), vp(o_im2), vp(a[1]), vp(o_d2b), vp(a[2]),
                                                        vp(o_d3bs), vp(o_ntr))
        assert rc == 0, rc

    def timed(fn, reps=10):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        fn()
        tot = 0.0
        for _ in range(reps):
            flush.zero_()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        return tot / reps

    t_no, t_with = timed(lambda: desc_call(False)), timed(lambda: desc_call(True))
    ctx.raise_on_status("operator-boundary descriptors")
    ang_bytes = B * N * na_ * (isz + 8 + 6 * isz)
    ang_ms = max(t_with - t_no, 1e-6)

    def entry(kernel, ms, nbytes):
        gbs = nbytes / (ms * 1e-3) / 1e9
        return {"bound": "hbm", "kernel": kernel, "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak,
                "traffic": None, "ms_per_launch": ms, "algorithmic_bytes_per_launch": nbytes}
    out.append(entry("k_angular (ComputeDescriptorsLight angular tensors)", ang_ms, ang_bytes))
    # the four angular operators on the tensors just written, central species by central species
    m_i = o_ntr.to(torch.float64)
    n_i = o_im2[..., 0].to(torch.float64)
    tm = torch.as_tensor(shape.type_map.astype(np.int32)).to(dev)
    tipos = torch.as_tensor(np.asarray(shape.tipos, np.int32)).to(dev)
    theta, emb = model.theta, model.emb
    total_ms = {"force": 0.0, "force_grad": 0.0, "af": 0.0, "af_grad": 0.0}
    total_bytes = {"force": 0.0, "force_grad": 0.0, "af": 0.0, "af_grad": 0.0}
    prev = torch.randn(B, 3 * N, device=dev)
    for t in range(shape.nt):
        s0, Nl = shape.shift(t), shape.tipos[t]
        sl = slice(s0, s0 + Nl)
        cut = lambda x: x[:, sl].contiguous()
        ang, d3s, im3, im2, d3b, d3bs, ntr = (cut(x) for x in (o_ang, o_d3s, o_im3, o_im2, o_d3b, o_d3bs, o_ntr))
        o = shape.offsets(t)
        Fr, Fa, nt, Cc = shape.Fr[t], shape.Fa[t], shape.nt, shape.C
        a3 = theta[o["a3"]:o["a3"] + Cc * 3 * Fa].reshape(Cc, 3 * Fa).contiguous()
        e3 = emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + Cc * Fa].reshape(Cc, Fa).contiguous()
        nd = torch.randn(B, Nl, Fa, device=dev)
        at = torch.tensor([t], dtype=torch.int32, device=dev)
        T_t = float((m_i[:, sl] * (m_i[:, sl] - 1) / 2).sum())
        M_t = float(m_i[:, sl].sum())
        A_t = float(B * Nl)
        b_force = T_t * (7 * isz + 8) + 4 * M_t * isz + A_t * Fa * isz
        b_fgrad = b_force + 3 * isz * (A_t + M_t) + A_t * Fa * isz
        b_af = T_t * (isz + 8) + M_t * isz + A_t * Fa * isz
        calls = {
            "force": lambda: ops.compute_force_tripl(nd, d3s, ang, d3bs, d3b, im2, im3, a3, e3, tm, tipos, at, ntr),
            "force_grad": lambda: ops.compute_force_tripl_grad(prev, nd, d3s, ang, d3bs, d3b, im2, im3, a3, e3, tm,
                                                               tipos, at, ntr),
            "af": lambda: ops.compute_sort_proj3body(ang, d3s, im3, im2, a3, e3, tm, ntr),
            "af_grad": lambda: ops.compute_sort_proj3body_grad(nd, ang, d3s, im3, im2, a3, e3, tm, ntr),
        }
        for name, nb in (("force", b_force), ("force_grad", b_fgrad), ("af", b_af), ("af_grad", b_af)):
            total_ms[name] += timed(calls[name], reps=5)
            total_bytes[name] += nb
    names = {"force": "k_force_ang (ComputeForceTripl)", "force_grad": "k_grad_force_ang (ComputeForceTriplGrad)",
             "af": "k_af_ang (ComputeSortProj3body)", "af_grad": "k_grad_af_ang (ComputeSortProj3bodyGrad)"}
    for k in ("force", "force_grad", "af", "af_grad"):
        e = entry(names[k] + ", all central species", total_ms[k], total_bytes[k])
        e["note"] = "includes the output allocation and zero-fill of the Python operator wrapper"
        out.append(e)
    chain_ms = t_with + sum(total_ms.values())
    return out, {"ms": chain_ms, "frames_per_s": B / (chain_ms * 1e-3),
                 "what": "descriptors with angular tensors + the four angular operators (the radial operators and "
                         "the MLP are not included), batch %d" % B}


def md_record(torch, dist, args, rank, world, local, dev, K):
    """Energy+forces of one 24,576-atom water box (8192 O + 16384 H, L = 62.7 A), neighbour list rebuilt every call,
    atoms cut into `world` slabs along z with one-cutoff halos (alphanesgpu_b200/slab.py)."""
    import tempfile
    from alphanesgpu_b200 import params, synth, _lib
    from alphanesgpu_b200.model import StafModel
    from alphanesgpu_b200.params import ModelShape
    from alphanesgpu_b200.slab import PeerSlabDomain, SlabDomain, model_compute, slab_of

    W = 3
    pos, box, tipos = synth.water_frames("water24576", [1400])
    gshape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(gshape, dtype=np.float32)
    N = gshape.N
    types = gshape.type_map.astype(np.int32)
    gpos = torch.as_tensor(pos.reshape(N, 3).astype(np.float32)).to(dev)
    gtypes = torch.as_tensor(types).to(dev)
    SKIN, HALO_EVERY = 1.0, 10  # ghost sets are re-chosen every 10 evaluations with a 1 A skin, as an MD code does
    if world == 1:
        dom = SlabDomain(None, box[0], CFG["Rc"], rank, world, nt=gshape.nt, skin=SKIN, halo_every=HALO_EVERY)
        own_idx = dom.set_owned_from_global(gpos, gtypes)
        n_own = dom.pos.shape[0]
        shape = ModelShape(nt=gshape.nt, tipos=list(dom.counts), Fr=gshape.Fr, Fa=gshape.Fa, widths=gshape.widths)
        model = StafModel(shape, CFG, theta, emb, 1, dtype=torch.float32, device=dev, n_max=n_own + 1024)
        dom.compute = model_compute(model, box[0])
    else:
        # positions, ghost forces and energies travel by the ranks' own stores over NVLink (stafb_halo_*); every
        # rank sizes its block alike (the peers address it by the common layout)
        L = float(box[0][5])
        n_mine = int((slab_of(gpos[:, 2], L, world) == rank).sum())
        halo = 2.0 * (CFG["Rc"] + SKIN) / (L / world)
        caps = torch.tensor([int(n_mine * (1.0 + halo) * 1.25) + 1024, int(n_mine * halo * 0.75) + 1024], device=dev)
        dist.all_reduce(caps, op=dist.ReduceOp.MAX)
        cap, cap_face = (int(v) for v in caps.tolist())
        shape = ModelShape(nt=gshape.nt, tipos=[1] * gshape.nt, Fr=gshape.Fr, Fa=gshape.Fa, widths=gshape.widths)
        model = StafModel(shape, CFG, theta, emb, 1, dtype=torch.float32, device=dev, n_max=cap)
        transport = "peer"
        try:
            dom = PeerSlabDomain(model, box[0], CFG["Rc"], rank, world, cap_atoms=cap, cap_face=cap_face, skin=SKIN,
                                 halo_every=HALO_EVERY)
        except RuntimeError as exc:  # raised on every rank alike (e.g. no peer access between these GPUs)
            sys.stderr.write("rank %d: halo exchange over peer memory unavailable (%s); using messages\n" % (rank, exc))
            transport = "messages"
            dom = SlabDomain(model_compute(model, box[0]), box[0], CFG["Rc"], rank, world, nt=gshape.nt, skin=SKIN,
                             halo_every=HALO_EVERY)
        own_idx = dom.set_owned_from_global(gpos, gtypes)
        n_own = dom.pos.shape[0]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(W):
        e, f = dom.step()
    dd_err = None
    if world > 1:
        # decomposition parity (the reference's test/test-lammps-dd-parity): every rank also evaluates the whole
        # box on its own GPU once and compares its owned forces and the total energy
        full = StafModel(gshape, CFG, theta, emb, 1, dtype=torch.float32, device=dev)
        e_full, f_full = full.energy_force(gpos.reshape(1, -1), torch.as_tensor(box.astype(np.float32)).to(dev))
        f_ref = f_full.reshape(N, 3)[own_idx]
        err = torch.stack([(f - f_ref).abs().max() / f_full.abs().max(), ((e - e_full).abs() / e_full.abs()).max()])
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        dd_err = {"force_rel": float(err[0]), "energy_rel": float(err[1])}
        full.close()
        del full, e_full, f_full
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    sampler = ClockSampler(local)
    ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    barrier()
    sampler.start()
    for k in range(K):
        flush.zero_()
        ev0[k].record()
        e, f = dom.step()
        ev1[k].record()
    barrier()
    clocks = sampler.stop()
    total_ms = float(sum(a.elapsed_time(b) for a, b in zip(ev0, ev1)))
    peer = world > 1 and transport == "peer"
    launches = model.launches() + (4 if peer else 0)  # push, wait, return, collect of the halo exchange
    if peer:
        dom.check()
    else:
        model.ctx.raise_on_status("md timed region")
    # end to end: owned positions start in (pinned) host memory and owned forces end there, every step
    pin_x = dom.pos.cpu().pin_memory()
    pin_f = torch.empty_like(pin_x)
    lib = _lib.lib()
    if world == 1:
        # through the libstaf C API (host double arrays in and out), the call LAMMPS makes
        class StafOptions(C.Structure):
            _fields_ = [("mlp_backend", C.c_int), ("device_id", C.c_int), ("precision", C.c_int), ("reserved", C.c_int)]
        tmp = tempfile.mkdtemp(prefix="stafb_md_")
        params.save_model_dir(tmp, CFG, gshape, theta.astype(np.float64), emb.astype(np.float64))
        lib.staf_load.restype = C.c_void_p
        lib.staf_load.argtypes = [C.c_char_p, C.c_void_p]
        lib.staf_compute.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 5 + [C.c_int] + [C.c_void_p] * 3
        lib.staf_free.argtypes = [C.c_void_p]
        opt = StafOptions(0, local, 0, 0)
        h = lib.staf_load(tmp.encode(), C.byref(opt))
        assert h
        x64 = np.ascontiguousarray(pos[0], np.float64)
        b64 = np.ascontiguousarray(box[0], np.float64)
        f64 = np.zeros(3 * N)
        e64 = C.c_double()
        vir = np.zeros(6)

        def e2e_step():
            rc = lib.staf_compute(h, N, 0, x64.ctypes.data, b64.ctypes.data, types.ctypes.data, None, None, 0,
                                  C.byref(e64), f64.ctypes.data, vir.ctypes.data)
            assert rc == 0, rc
        # the caller's double arrays travel as they are (the library converts and permutes on the device); the
        # species array is uploaded only when it changes
        h2d, d2h = 8 * (3 * N + 6), 8 * (3 * N + 1 + 9)
    else:
        def e2e_step():
            dom.pos.copy_(pin_x, non_blocking=True)
            e_, f_ = dom.step()
            pin_f.copy_(f_, non_blocking=True)
            torch.cuda.synchronize()
        h2d, d2h = 4 * 3 * n_own, 4 * 3 * n_own
    Ke = max(5, min(K, 100))
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(Ke):
        e2e_step()
    barrier()
    t = torch.tensor([total_ms, (time.perf_counter() - t0) * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms = float(t[0]), float(t[1])
    if world == 1:
        e_check = float(e64.value)
        assert abs(e_check - float(e)) <= 1e-4 * abs(float(e)), (e_check, float(e))
        lib.staf_free(h)
    # phases of one evaluation on this rank
    model.set_phase_timing(True)
    acc = {}
    for k in range(5):
        flush.zero_()
        dom.step(rebuild=False)
        for name, ms in model.phase_times_ms().items():
            acc[name] = acc.get(name, 0.0) + ms / 5
    model.set_phase_timing(False)
    rec = None
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline and args.workload == "md":
            from oracle import oracle
            oracle.set_threads(os.cpu_count() or 1)
            t0 = time.perf_counter()
            r = oracle.energy_force_grad(CFG, gshape.desc(), pos, box, gshape.type_map, theta, emb, np.float32,
                                         per_atom_energy=False)
            dt = time.perf_counter() - t0
            assert r["status"] == 0
            assert abs(float(r["energy"][0]) - float(e)) <= 2e-5 * abs(float(e)), (r["energy"], float(e))
            cpu = {"value": N / dt, "unit": "atom-steps/s", "cores": oracle.max_threads(), "kind": "port",
                   "sample": "1 evaluation of the 24576-atom box (%.1f s); energy agrees with the GPU" % dt}
        rec = {
            "metric": MD_METRIC, "value": N * K / (total_ms * 1e-3), "unit": "atom-steps/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "water24576 energy+forces, list rebuilt every call, fp32",
                       "decomposition": "%d z-slab(s), %.1f A halos (cutoff + %.1f A skin, ghost sets re-chosen every "
                                        "%d evaluations), owned atoms on rank 0: %d" % (world, dom.reach, SKIN,
                                                                                         HALO_EVERY, n_own),
                       "l2": "flushed between steps (256 MiB write); per-step CUDA events summed",
                       "model": "2 species, Fr=10, Fa=15, MLP 25-64-32-1 tanh"},
            "e2e": {"value": N * Ke / (e2e_ms * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": Ke,
                    "path": "staf_compute (libstaf C API, host double arrays)" if world == 1 else
                            "slab driver: pinned host -> device, halo exchange (%s), forces -> pinned host" % transport},
            "gpu_launches": launches * K, "launches_per_step": launches, "clocks": clocks, "phase_ms": acc,
            "energy": float(e), "dd_parity": dd_err, "cpu_baseline": cpu,
        }
    messages_ms = None
    if world > 1 and not peer and rec is not None:
        rec["transport"] = {"halo": "torch.distributed messages (peer memory was not available)"}
    if peer:
        # the same decomposition with torch.distributed messages (NCCL send/recv per face, all-reduce of the
        # energy) instead of the peer stores, for comparison
        dom.check()
        msg = SlabDomain(model_compute(model, box[0]), box[0], CFG["Rc"], rank, world, nt=gshape.nt, skin=SKIN,
                         halo_every=HALO_EVERY)
        msg.set_owned_from_global(gpos, gtypes)
        for _ in range(W):
            msg.step()
        Km = max(5, min(K, 50))
        a = [torch.cuda.Event(enable_timing=True) for _ in range(Km)]
        b = [torch.cuda.Event(enable_timing=True) for _ in range(Km)]
        barrier()
        for k in range(Km):
            flush.zero_()
            a[k].record()
            msg.step()
            b[k].record()
        barrier()
        t = torch.tensor([sum(x.elapsed_time(y) for x, y in zip(a, b)) / Km], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        messages_ms = float(t[0])
        if rec is not None:
            rec["transport"] = {"halo": "peer stores over NVLink; ghost sets chosen on the device, one host sync per re-choice",
                                "ms_per_step_with_nccl_messages": messages_ms}
        dom.close()
    model.close()
    del flush
    return rec


def run_ours(args):
    import torch
    import torch.distributed as dist
    from alphanesgpu_b200 import _lib, ops, synth
    from alphanesgpu_b200.model import StafModel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def reduce_max(x):
        if world == 1:
            return float(x)
        t = torch.tensor([float(x)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    if args.workload == "md":
        rec = md_record(torch, dist, args, rank, world, local, dev, args.steps if args.steps != 2000 else 50)
        if rank == 0:
            print(json.dumps(rec))
        if world > 1:
            dist.destroy_process_group()
        return

    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    dtype = np.float32
    NB = 8  # distinct batches cycled through
    shape, pos, box, el, fl = make_batches(rank, NB, B, dtype)
    N = shape.N
    theta, emb = synth.init_params(shape, dtype=dtype)
    model = StafModel(shape, CFG, theta, emb, B, dtype=torch.float32, device=dev)
    lr = 1e-3
    to_dev = lambda arrs: tuple(torch.as_tensor(a).to(dev) for a in arrs)
    data = to_dev((pos, box, el, fl))
    d_pos, d_box, d_el, d_fl = data
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    for w in range(3):  # plain launches first: one-time kernel attributes, status check
        model.loss_and_grad(d_pos[w], d_box[w], d_el[w], d_fl[w])
        model.adam_update_dev(lr)
    model.ctx.raise_on_status("bench warm-up")
    launches_per_step = model.launches() + 1  # + Adam (or the exchange kernel)
    torch.cuda.synchronize()

    def sync_replicas(mdl):
        """Rank 0's parameters, moments and step count to every rank (the warm-up steps above were local)."""
        if world > 1:
            for t_ in (mdl.theta, mdl.adam_m, mdl.adam_v, mdl.step_d):
                dist.broadcast(t_, 0)
    sync_replicas(model)

    # ---- several GPUs: gradient averaging + Adam as ONE kernel per rank over NVLink peer memory
    # (stafb_allreduce_adam) instead of an NCCL all-reduce between two graphs; --allreduce nccl keeps the latter
    px, exchange = None, None
    if world > 1:
        exchange = "nccl"
        if args.allreduce == "peer":
            from alphanesgpu_b200.dist import PeerExchange
            ok = torch.ones(1, device=dev)
            try:
                px = PeerExchange(model)
            except Exception as exc:  # e.g. no peer access between these GPUs: every rank falls back to NCCL
                sys.stderr.write("rank %d: peer exchange unavailable (%s)\n" % (rank, exc))
                ok.zero_()
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if float(ok) == 0.0:
                if px is not None:
                    px.close()
                px = None
            else:
                exchange = "peer"
    own_grad = model.grad
    stepper = Stepper(torch, dist, model, data, lr, world, exchange, px)
    sync_replicas(model)  # the stepper's set-up ran one local update
    for w in range(W):
        stepper.step()
        flush.zero_()
    torch.cuda.synchronize()
    if px is not None:
        # a peer that did not arrive within the kernel's bound leaves a status; then every rank goes back to NCCL
        bad = reduce_max(px.status())
        if bad != 0.0:
            sys.stderr.write("rank %d: peer exchange status %d, falling back to NCCL\n" % (rank, int(bad)))
            px.close()
            px, exchange = None, "nccl"
            model.use_grad(own_grad)
            sync_replicas(model)
            stepper = Stepper(torch, dist, model, data, lr, world, exchange, None)

    # ---- timed region: exactly K steps, L2 flushed between steps, device time per step summed; then the same
    # block again until a quarter of a second is covered
    sampler = ClockSampler(local)
    sampler.start()
    totals, per_step = time_blocks(stepper, K, W, flush, barrier, reduce_max)
    clocks = sampler.stop()
    total_ms = float(totals[0])
    value = world * B * K / (total_ms * 1e-3)
    per_block_ms_step = totals / K
    repeat = {"blocks": int(len(totals)), "steps_per_block": K,
              "ms_per_step_median": float(np.median(per_block_ms_step)), "ms_per_step_min": float(per_block_ms_step.min()),
              "ms_per_step_max": float(per_block_ms_step.max()),
              "value_median": world * B / (float(np.median(per_block_ms_step)) * 1e-3)}
    # ---- same, back to back without flushing (working set stays in L2)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for k in range(K):
        stepper.step()
    b.record()
    barrier()
    warm_ms = reduce_max(a.elapsed_time(b))
    model.ctx.raise_on_status("bench timed region")
    value_warm = world * B * K / (warm_ms * 1e-3)

    # ---- several GPUs: cost of the exchange (the same step with a local Adam instead), spread over the ranks,
    # and the replicas' parameters compared
    multi = None
    if world > 1:
        mine = float(per_step.sum()) / K
        allms = [torch.zeros(1, dtype=torch.float64, device=dev) for _ in range(world)]
        dist.all_gather(allms, torch.tensor([mine], dtype=torch.float64, device=dev))
        allms = [float(x) for x in allms]
        chk = model.theta.double().sum().reshape(1)
        chks = [torch.zeros_like(chk) for _ in range(world)]
        dist.all_gather(chks, chk)
        theta0 = model.theta.clone()
        others = [torch.empty_like(theta0) for _ in range(world)]
        dist.all_gather(others, theta0)
        identical = all(bool(torch.equal(o, theta0)) for o in others)
        # local-Adam twin of the step on a scratch copy of the optimiser state
        saved = [t_.clone() for t_ in (model.theta, model.adam_m, model.adam_v, model.step_d)]
        model.use_grad(own_grad)
        local_stepper = Stepper(torch, dist, model, data, lr, world, None, None)
        ltot, _ = time_blocks(local_stepper, K, W, flush, barrier, reduce_max, min_total_ms=100.0)
        for t_, s_ in zip((model.theta, model.adam_m, model.adam_v, model.step_d), saved):
            t_.copy_(s_)
        local_ms = float(np.median(ltot)) / K
        multi = {"exchange": {"peer": "stafb_allreduce_adam (peer memory, inside the step graph)",
                              "nccl": "NCCL all-reduce between the step graph and the Adam graph"}[exchange],
                 "exchange_us": 1e3 * (float(np.median(per_block_ms_step)) - local_ms),
                 "ms_per_step_without_exchange": local_ms,
                 "ms_per_step_by_rank": allms, "replicas_bit_identical": identical,
                 "theta_checksum_spread": float(max(float(c) for c in chks) - min(float(c) for c in chks))}
        del local_stepper

    # ---- end to end through host buffers: every step reads its inputs from the slot's pinned block and writes
    # its losses to host memory.  The two-slot begin/end form of the C ABI lets the host stage step k+1 while the
    # GPU runs step k; the losses of step k are read one iteration later, all inside the timed region.
    Ke = max(10, min(K, 500))
    if px is not None:
        model.use_grad(px.grad(0))
    for k in range(3):
        model.loss_and_grad_host(pos[k % NB], box[k % NB], el[k % NB], fl[k % NB])
    barrier()
    side = torch.cuda.Stream(device=dev)

    def e2e_loop(n):
        # on a stream of its own: the library replays the step as CUDA graphs, which the legacy default stream
        # cannot capture
        with torch.cuda.stream(side):
            for k in range(n):
                i = k % NB
                if px is not None:
                    model.use_grad(px.grad(k & 1))
                model.loss_and_grad_host_begin(pos[i], box[i], el[i], fl[i], k & 1)
                if px is not None:
                    px.allreduce_adam(model, k & 1, lr)
                else:
                    if world > 1:
                        dist.all_reduce(model.grad)
                    model.adam_update_dev(lr, grad_scale=1.0 / world)
                if k > 0:
                    model.loss_and_grad_host_end((k - 1) & 1)
            return model.loss_and_grad_host_end((n - 1) & 1)

    e2e_loop(6)  # plain launches, capture, first replays
    barrier()
    t0 = time.perf_counter()
    e2e_losses = e2e_loop(Ke)
    barrier()
    e2e_s = reduce_max(time.perf_counter() - t0)
    assert np.all(np.isfinite(e2e_losses))
    # the synchronous call (stage, run, wait, read back in one call) for comparison
    barrier()
    model.use_grad(own_grad)
    t1 = time.perf_counter()
    for k in range(min(Ke, 100)):
        i = k % NB
        model.loss_and_grad_host(pos[i], box[i], el[i], fl[i])
        if world > 1:
            dist.all_reduce(model.grad)
        model.adam_update_dev(lr, grad_scale=1.0 / world)
    barrier()
    e2e_sync_s = (time.perf_counter() - t1) / min(Ke, 100)
    e2e_value = world * B * Ke / e2e_s
    isz = np.dtype(dtype).itemsize
    h2d = isz * (B * 3 * N * 2 + B * 6 + B)
    d2h = 8 * 4 + 4
    # a late peer in the end-to-end loop: decided by all ranks together (a rank that left alone would hang the rest)
    exchange_status = int(reduce_max(px.status())) if px is not None else 0

    # ---- per-phase device times (eager launches, CUDA events between phases, L2 flushed)
    def phase_times(mdl, dd, Kp=30):
        mdl.set_phase_timing(True)
        acc = {}
        nb = dd[0].shape[0]
        for k in range(Kp):
            flush.zero_()
            mdl.loss_and_grad(dd[0][k % nb], dd[1][k % nb], dd[2][k % nb], dd[3][k % nb])
            for name, ms in mdl.phase_times_ms().items():
                acc[name] = acc.get(name, 0.0) + ms / Kp
        mdl.set_phase_timing(False)
        return acc
    acc = phase_times(model, data)
    dom = max((n for n in acc if n not in ("descriptors", "loss")), key=lambda n: acc[n])
    # algorithmic bytes of one launch of the dominant sweep kernel: the neighbour records it reads (two 16-byte
    # entries and the index per neighbour, the 48-byte header), its per-atom channel row in and out, and the
    # gathered force cotangents / scattered forces
    ctx = ops.construct_descriptors_light(CFG["Rc"], CFG["nr"], CFG["na"], N, None, CFG["Rs"], CFG["Ra"], B,
                                          dtype=torch.float32, device=dev)
    outs = ops.compute_descriptors_light(d_pos[0], d_box[0], with_angular=False, ctx=ctx)
    n_i = outs[3][..., 0].to(torch.float64)
    m_i = outs[8].to(torch.float64)
    trip = float((m_i * (m_i - 1) / 2).sum())
    mean_neigh = float(n_i.mean())
    F = shape.Fr[0] + shape.Fa[0]
    nact = shape.Fa[0] / shape.C  # active angular channels per species-pair class
    row_bytes = float((n_i * 36 + 48).sum())
    chan = B * N * F * isz
    nv_bytes = B * N * (shape.nt * shape.Fr[0] + shape.C * 3 * shape.Fa[0]) * isz
    gather = float(((n_i + 1) * 3 * isz).sum())
    alg = {"af_fwd": row_bytes + chan + nv_bytes, "force": row_bytes + chan + gather,
           "force_grad": row_bytes + 2 * chan + gather, "mlp_fwd": 3 * chan, "mlp_bwd": 4 * chan + nv_bytes}[dom]
    # DRAM traffic per launch of each kernel (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of
    # this workload at batch 4, summarised in profiles/step_kernels_water768_b4_fp32.md); it scales with the atoms
    traffic = TRAFFIC_NCU_B4.get(dom)
    if traffic is not None:
        traffic *= B / 4.0
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = alg / (acc[dom] * 1e-3) / 1e9
    kname = {"af_fwd": "k_sweep<fingerprints + d(AF)/d(alpha)>", "force": "k_sweep<force>",
             "force_grad": "k_sweep<force backward>", "mlp_fwd": "k_mlp_fwd", "mlp_bwd": "k_mlp_bwd"}[dom]
    roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": "measured" if peaks else "fallback",
                "ms_per_launch": acc[dom], "algorithmic_bytes_per_launch": alg,
                "note": "the triplet geometry is rebuilt on chip from 36-byte neighbour entries, so this kernel is "
                        "bound by instruction issue (FP32 / SFU pipes), not by HBM: see fp32_pipe; triplet-channel "
                        "evaluations per launch = %.3g" % (trip * nact)}

    # ---- the operator boundary on materialised tensors
    roofline_ops, opchain = operator_boundary(torch, model, ctx, shape, d_pos[0], d_box[0], B, N, peak, flush)

    # ---- FP32 pipe: measured FMA peak of this GPU against the counted flops of the three sweeps
    pk32, pk64 = C.c_double(), C.c_double()
    _lib.lib().stafb_measure_fma_peak(0, model.ctx.stream(), C.byref(pk32))
    _lib.lib().stafb_measure_fma_peak(1, model.ctx.stream(), C.byref(pk64))
    step_flops = trip * (FLOPS_PER_TRIPLET + nact * FLOPS_PER_TRIPLET_CHANNEL)
    sweep_ms = acc.get("af_fwd", 0) + acc.get("force", 0) + acc.get("force_grad", 0)
    ms_step_med = float(np.median(per_block_ms_step))
    fp32_pipe = {"fma_peak_tflops_measured": pk32.value, "fp64_fma_peak_tflops_measured": pk64.value,
                 "counted_flops_per_triplet": FLOPS_PER_TRIPLET + nact * FLOPS_PER_TRIPLET_CHANNEL,
                 "counted_flops_per_step": step_flops,
                 "achieved_tflops": step_flops / (ms_step_med * 1e-3) / 1e12,
                 "frac_of_fma_peak": step_flops / (ms_step_med * 1e-3) / 1e12 / pk32.value,
                 "sweeps_only": {"ms": sweep_ms, "achieved_tflops": step_flops / (sweep_ms * 1e-3) / 1e12,
                                 "frac_of_fma_peak": step_flops / (sweep_ms * 1e-3) / 1e12 / pk32.value},
                 "note": "flops counted in the source of the sweeps (multiply-add = 2, exponential = 1); the MLP "
                         "kernels, the neighbour list and the loss are not counted"}

    # ---- sub-records on one more model each (single-rank form of the step; at N > 1 every rank runs them
    # concurrently and the slowest rank counts)
    def sub_record(mdl, dd, Bsub, label, Ksub):
        st = Stepper(torch, dist, mdl, dd, lr, world, None, None)
        tot, _ = time_blocks(st, Ksub, 3, flush, barrier, reduce_max, min_total_ms=100.0)
        ms = float(np.median(tot)) / Ksub
        ph = phase_times(mdl, dd, Kp=10)
        mdl.ctx.raise_on_status(label)
        return {"value": Bsub / (ms * 1e-3), "unit": "frames/s per GPU", "ms_per_step": ms, "steps": Ksub,
                "blocks": int(len(tot)), "phase_ms": ph}

    Ksub = max(10, min(K, 200))
    # energy + force + virial training evaluation beside the energy + force one, both as plain launches with the
    # L2 flushed (the extra work: the virial in the force sweep, nine more loss terms, three more FMAs per neighbour
    # in the backward sweep's prologue)
    def eager_ms(fn, Kp=30):
        a_ = [torch.cuda.Event(enable_timing=True) for _ in range(Kp)]
        b_ = [torch.cuda.Event(enable_timing=True) for _ in range(Kp)]
        for k in range(3):
            fn(k)
        torch.cuda.synchronize()
        for k in range(Kp):
            flush.zero_()
            a_[k].record()
            fn(k)
            b_[k].record()
        torch.cuda.synchronize()
        return float(np.median([x.elapsed_time(y) for x, y in zip(a_, b_)]))
    vlab = torch.zeros(B, 9, dtype=torch.float32, device=dev)
    ms_plain = eager_ms(lambda k: model.loss_and_grad(d_pos[k % NB], d_box[k % NB], d_el[k % NB], d_fl[k % NB]))
    ms_vir = eager_ms(lambda k: model.loss_and_grad_virial(d_pos[k % NB], d_box[k % NB], d_el[k % NB], d_fl[k % NB],
                                                           vlab, pv=1.0))
    model.ctx.raise_on_status("virial training leg")
    virial_rec = {"ms_per_evaluation": ms_vir, "ms_per_evaluation_energy_force_only": ms_plain,
                  "ratio": ms_vir / ms_plain, "what": "stafb_train_step_virial vs stafb_train_step, plain launches "
                  "(neighbour records in line, no optimiser), batch %d" % B}
    # the same step in float64: time ratio and FP64-pipe fraction of the sweeps
    model64 = StafModel(shape, CFG, theta.astype(np.float64), emb.astype(np.float64), B, dtype=torch.float64, device=dev)
    d64 = to_dev(tuple(a.astype(np.float64) for a in (pos, box, el, fl)))
    fp64 = sub_record(model64, d64, B, "fp64 leg", Ksub)
    sw64 = fp64["phase_ms"].get("af_fwd", 0) + fp64["phase_ms"].get("force", 0) + fp64["phase_ms"].get("force_grad", 0)
    fp64.update({"time_ratio_fp64_over_fp32": fp64["ms_per_step"] / ms_step_med,
                 "fp64_pipe": {"achieved_tflops": step_flops / (fp64["ms_per_step"] * 1e-3) / 1e12,
                               "frac_of_fma_peak": step_flops / (fp64["ms_per_step"] * 1e-3) / 1e12 / pk64.value,
                               "sweeps_only_frac_of_fma_peak": step_flops / (sw64 * 1e-3) / 1e12 / pk64.value},
                 "note": "graph-replayed like the fp32 step; exponentials are full-precision exp, not counted as "
                         "more than one flop"})
    model64.close()
    del d64
    # eight frames per GPU (the data-parallel configuration's batch)
    shape8, *h8 = make_batches(rank, 4, 8, dtype, seed0=1200)
    model8 = StafModel(shape8, CFG, theta, emb, 8, dtype=torch.float32, device=dev)
    d8 = to_dev(tuple(h8))
    batch8 = sub_record(model8, d8, 8, "batch 8", Ksub)
    if world > 1:
        # with the exchange: the figure whose ratio to N x the line above is the scaling efficiency at batch 8
        px8 = None
        if exchange == "peer":
            from alphanesgpu_b200.dist import PeerExchange
            px8 = PeerExchange(model8)
        st8 = Stepper(torch, dist, model8, d8, lr, world, exchange, px8)
        sync_replicas(model8)
        tot8, _ = time_blocks(st8, Ksub, 3, flush, barrier, reduce_max, min_total_ms=100.0)
        ms8 = float(np.median(tot8)) / Ksub
        batch8["with_exchange"] = {"value": world * 8 / (ms8 * 1e-3), "unit": "frames/s (all GPUs)",
                                   "ms_per_step": ms8, "efficiency_vs_no_exchange": batch8["ms_per_step"] / ms8}
        if px8 is not None:
            st8_bad = int(reduce_max(px8.status()))
            if st8_bad:
                batch8["with_exchange"]["invalid"] = "the peer exchange recorded status %d" % st8_bad
            px8.close()
        del st8
    model8.close()
    del d8
    # the reference's real frame with its exported model
    rshape, rtheta, remb, *hr = real_model_batches(NB, B, dtype)
    modelr = StafModel(rshape, CFG, rtheta, remb, B, dtype=torch.float32, device=dev)
    dr = to_dev(tuple(hr))
    real = sub_record(modelr, dr, B, "real model", max(10, Ksub // 2))
    outs_r = ops.compute_descriptors_light(dr[0][0], dr[1][0], with_angular=False, ctx=ctx)
    mr = outs_r[8].to(torch.float64)
    real.update({"mean_neighbours": float(outs_r[3][..., 0].to(torch.float64).mean()),
                 "triplets_per_atom": float((mr * (mr - 1) / 2).mean()),
                 "model": "Fr=20, Fa=40 (13-14 active channels per class), MLP 60-140-140-1", "mlp": modelr.mlp_config(),
                 "frames": "the reference's frame pos_0, %d jittered copies (sigma 0.02 A)" % (NB * B)})
    modelr.close()
    del dr
    ctx.close()
    model.close()
    if px is not None:
        px.close()
    del stepper, data, d_pos, d_box, d_el, d_fl
    torch.cuda.empty_cache()
    # the 24,576-atom inference box, bounded to a few seconds
    md = md_record(torch, dist, args, rank, world, local, dev, 20)
    if md is not None:
        md = {k: md[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "scaling", "config", "e2e",
                                 "launches_per_step", "phase_ms", "dd_parity", "transport") if k in md}

    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            cpu = cpu_baseline_record(B)
        line = {
            "metric": METRIC, "value": value, "unit": "frames/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / PUBLISHED_V100_FRAMES_PER_S, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "water768 E+F training step (eval + Adam), batch %d per GPU, fp32" % B,
                       "frames": "seeded synthetic water, 256 O + 512 H, L=19.6 A, %d distinct batches, %.1f "
                                 "neighbours per atom" % (NB, mean_neigh),
                       "model": "2 species, Fr=10, Fa=15, MLP 25-64-32-1 tanh", "parallelism": "dp%d" % world,
                       "l2": "flushed between steps (256 MiB write); per-step CUDA events summed",
                       "launch": "two CUDA graphs per step: neighbour records of the NEXT batch on a second stream, "
                                 "the rest of the step on the main stream; each timed interval contains both"
                                 + ("" if world == 1 else ("; gradient averaging + Adam as one peer-memory kernel in the step graph"
                                                            if exchange == "peer" else
                                                            "; NCCL all-reduce between the step graph and the Adam graph")),
                       "vs_baseline_note": "published number is the reference on a V100 (README.md:42-45)"},
            "repeat": repeat, "value_l2_warm": value_warm, "ms_per_step_min": float(per_step.min()),
            "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": Ke, "path": "stafb_train_step_host_begin/_end (two pinned slots) + "
                            + ("stafb_allreduce_adam" if exchange == "peer" else "stafb_adam_step_dev"),
                    "synchronous_call_value": world * B / e2e_sync_s},
            "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
            "clocks": clocks, "roofline": roofline, "roofline_operator_boundary": roofline_ops,
            "operator_chain": opchain, "fp32_pipe": fp32_pipe, "fp64": fp64, "batch8": batch8, "real_model": real, "virial_training": virial_rec,
            "md": md, "multi_gpu": multi, "phase_ms": acc, "cpu_baseline": cpu,
        }
        if exchange_status:
            line["e2e"]["invalid"] = "the peer exchange recorded status %d during the end-to-end loop" % exchange_status
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--allreduce", default="peer", choices=["peer", "nccl"],
                    help="N > 1: gradient exchange by the fused peer-memory kernel or by an NCCL all-reduce")
    ap.add_argument("--workload", default="train", choices=["train", "md"],
                    help="train: the 768-atom training step (the headline metric, with the sub-records); md: only "
                         "the 24,576-atom inference box")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
