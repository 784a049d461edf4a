#!/usr/bin/env python
"""Benchmark of the STAF hot path on B200: 768-atom water energy+force training step, fp32.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

One "step" = one training evaluation of a batch of B frames (neighbour list, descriptors,
fingerprints, MLP, forces, loss, backward to alpha/mu/MLP weights) followed by the Adam update;
with N > 1 (launched by torch.distributed.run, one rank per GPU) every rank works on its own frames
and the flat gradient is summed with ONE NCCL all-reduce per step before Adam (learning rate not
scaled by N).  Prints one JSON line (rank 0).

`value`   frames/s with the inputs resident in HBM, the step replayed from a CUDA graph, L2 flushed
          between steps, CUDA-event time summed over exactly K steps, max over ranks.
`e2e`     frames/s through the host-buffer entry point of the C ABI (stafb_train_step_host + Adam):
          host->device copies of positions/box/labels and the device->host read of the losses are
          inside the timed region (wall clock, synchronised both sides).
`roofline` the dominant kernel of the step, timed live with CUDA events on the launching stream.
`cpu_baseline` the CPU oracle (a port of the reference's kernel math; the reference's own ops are
          GPU-only) on a bounded sample, all host threads.
`--impl reference` times that same CPU port as the reference arm.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(Rc=4.5, Rs=2.25, Ra=4.5, nr=60, na=1770)
METRIC = "768-atom water E+F train frames/s"
PUBLISHED_V100_FRAMES_PER_S = 10.9  # reference README.md:42-45 (V100, fp32, batch 4)


def make_batches(rank, n_batches, B, dtype):
    from alphanesgpu_b200 import synth
    seeds = [1100 + 64 * rank + i for i in range(n_batches * B)]
    pos, box, tipos = synth.water_frames("water768", seeds)
    shape = synth.baseline_shape(tipos)
    N = shape.N
    el, fl = synth.labels(n_batches * B, N, seed=3000 + rank)
    rs = lambda a, *s: np.ascontiguousarray(a.reshape(n_batches, B, *s).astype(dtype))
    return shape, rs(pos, 3 * N), rs(box, 6), rs(el), rs(fl, 3 * N)


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
            time.sleep(0.02)

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


def cpu_port_frames_per_s(B, n_steps, threads=None):
    """Times the CPU oracle's full training evaluation (no optimizer) on n_steps batches of B frames."""
    from oracle import oracle
    if threads:
        oracle.set_threads(threads)
    shape, pos, box, el, fl = make_batches(0, n_steps, B, np.float32)
    from alphanesgpu_b200 import synth
    theta, emb = synth.init_params(shape, dtype=np.float32)
    sd = shape.desc()
    oracle.energy_force_grad(CFG, sd, pos[0], box[0], shape.type_map, theta, emb, np.float32, with_grad=True,
                             e_label=el[0], f_label=fl[0])  # warm-up
    t0 = time.perf_counter()
    for i in range(n_steps):
        r = oracle.energy_force_grad(CFG, sd, pos[i], box[i], shape.type_map, theta, emb, np.float32, with_grad=True,
                                     e_label=el[i], f_label=fl[i])
        assert r["status"] == 0
    dt = time.perf_counter() - t0
    return B * n_steps / dt, dt, oracle.max_threads()


def run_reference(args):
    """Reference arm: the reference's hot path on the host cores.  Its own ops are GPU-only TensorFlow
    kernels (TensorFlow is not installable here), so the timed code is the CPU port in oracle/."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    B = args.batch
    # bounded sample: each "step" is one batch; cap the total so the run ends within minutes
    steps = max(1, min(args.steps, 12))
    warm = max(1, min(args.warmup, 1))
    for _ in range(warm):
        cpu_port_frames_per_s(B, 1)
    fps, dt, cores = cpu_port_frames_per_s(B, steps)
    line = {
        "impl": "reference", "metric": METRIC, "value": fps, "unit": "frames/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": 1e3 * dt / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "water768 E+F training evaluation, batch %d, fp32 (BASELINE configs[1])" % B,
                   "note": "CPU port of the reference kernels (oracle/), OpenMP over atoms; no optimizer step"},
        "cpu_baseline": {"value": fps, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": "%d batches of %d frames" % (steps, B)},
        "e2e": {"value": fps, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import torch.distributed as dist
    from alphanesgpu_b200 import ops, synth
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
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    dtype = np.float32
    NB = 8  # distinct batches cycled through
    shape, pos, box, el, fl = make_batches(rank, NB, B, dtype)
    N = shape.N
    theta, emb = synth.init_params(shape, dtype=dtype)
    model = StafModel(shape, CFG, theta, emb, B, dtype=torch.float32, device=dev)
    lr = 1e-3
    d_pos, d_box, d_el, d_fl = (torch.as_tensor(a).to(dev) for a in (pos, box, el, fl))

    def step_eager(i):
        model.loss_and_grad(d_pos[i], d_box[i], d_el[i], d_fl[i])
        if world > 1:
            dist.all_reduce(model.grad)
        model.adam_update_dev(lr, grad_scale=1.0 / world)

    for w in range(W):
        step_eager(w % NB)
    model.ctx.raise_on_status("bench warm-up")
    launches_per_step = model.launches() + 2  # + Adam and its step counter
    torch.cuda.synchronize()

    # ---- several GPUs: gradient averaging + Adam as ONE kernel per rank over NVLink peer memory
    # (stafb_allreduce_adam) instead of an NCCL all-reduce between two graphs; --allreduce nccl keeps the latter
    px = None
    if world > 1 and args.allreduce == "peer":
        from alphanesgpu_b200.dist import PeerExchange
        ok = torch.ones(1, device=dev)
        try:
            px = PeerExchange(model)
        except Exception as exc:  # e.g. no peer access between these GPUs: every rank falls back to NCCL
            sys.stderr.write("rank %d: peer exchange unavailable (%s)\n" % (rank, exc))
            ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0.0:
            px = None
    own_grad = model.grad

    # ---- CUDA graphs, two per distinct batch (pointers differ): the neighbour rows of a batch depend on its
    # positions only, so they are built on a second stream while the previous step is still running (and, on
    # several GPUs, during the gradient all-reduce and the Adam update); the rest of the step follows on the main
    # stream.  The NCCL all-reduce stays between two graphs (capturing it into the graph made a 2-rank run hang
    # on this pool, so it is not attempted).
    assert NB % 2 == 0  # batch i always uses row set i & 1
    main = torch.cuda.current_stream(dev)
    side = torch.cuda.Stream(device=dev)
    rows_stream = torch.cuda.Stream(device=dev)
    for i in range(2):  # allocate both row sets and set the kernels' attributes outside any capture
        model.prefetch_rows(d_pos[i], d_box[i], i)
        model.loss_and_grad_prefetched(i, B, d_el[i], d_fl[i])
    torch.cuda.synchronize()

    def build_graphs(px):
        graphs = []
        side.wait_stream(main)
        with torch.cuda.stream(side):
            for i in range(NB):
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=side):
                    model.prefetch_rows(d_pos[i], d_box[i], i & 1)
                g1 = torch.cuda.CUDAGraph()
                model.use_grad(px.grad(i & 1) if px is not None else own_grad)
                with torch.cuda.graph(g1, stream=side):
                    model.loss_and_grad_prefetched(i & 1, B, d_el[i], d_fl[i])
                    if world == 1:
                        model.adam_update_dev(lr)
                    elif px is not None:
                        px.allreduce_adam(model, i & 1, lr)
                g2 = None
                if world > 1 and px is None:
                    g2 = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g2, stream=side):
                        model.adam_update_dev(lr, grad_scale=1.0 / world)
                graphs.append((gr, g1, g2))
        main.wait_stream(side)
        torch.cuda.synchronize()
        return graphs

    graphs = build_graphs(px)

    ready = [torch.cuda.Event(), torch.cuda.Event()]
    go = torch.cuda.Event()
    with torch.cuda.stream(rows_stream):  # rows of the very first step
        graphs[0][0].replay()
        ready[0].record(rows_stream)
    counter = [0]

    def step_graph(_k=None):
        """One training step.  Steps are numbered by an internal counter, because every step also builds the rows
        of the NEXT one; it returns only after those rows are complete on the device timeline of the main stream,
        so that a CUDA-event interval around the call contains all the work of exactly one step."""
        k = counter[0]
        counter[0] += 1
        i, s = k % NB, k & 1
        go.record(main)
        rows_stream.wait_event(go)  # the next rows start inside this step, not during the cache flush before it
        with torch.cuda.stream(rows_stream):
            graphs[(k + 1) % NB][0].replay()
            ready[s ^ 1].record(rows_stream)
        main.wait_event(ready[s])
        graphs[i][1].replay()
        if world > 1 and px is None:
            dist.all_reduce(model.grad)
            graphs[i][2].replay()
        main.wait_event(ready[s ^ 1])

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for w in range(W):
        step_graph(w)
        flush.zero_()
    torch.cuda.synchronize()
    if px is not None:
        # a peer that did not arrive within the kernel's bound leaves a status; then every rank goes back to NCCL
        bad = torch.tensor([float(px.status())], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if float(bad) != 0.0:
            sys.stderr.write("rank %d: peer exchange status %d, falling back to NCCL\n" % (rank, int(bad)))
            px.close()
            px = None
            model.use_grad(own_grad)
            dist.broadcast(model.theta, 0)
            graphs = build_graphs(None)
            for w in range(W):
                step_graph(w)
                flush.zero_()
            torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- timed region: exactly K steps, L2 flushed between steps, device time per step summed
    sampler = ClockSampler(local)
    ev0 = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ev1 = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    barrier()
    sampler.start()
    for k in range(K):
        flush.zero_()
        ev0[k].record()
        step_graph(k)
        ev1[k].record()
    barrier()
    per_step = np.array([a.elapsed_time(b) for a, b in zip(ev0, ev1)])
    total_ms = float(per_step.sum())
    # ---- same, back to back without flushing (working set stays in L2)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for k in range(K):
        step_graph(k)
    b.record()
    barrier()
    warm_ms = a.elapsed_time(b)
    clocks = sampler.stop()
    model.ctx.raise_on_status("bench timed region")
    t = torch.tensor([total_ms, warm_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms, warm_ms = float(t[0]), float(t[1])
    value = world * B * K / (total_ms * 1e-3)
    value_warm = world * B * K / (warm_ms * 1e-3)

    # ---- end to end through host buffers: every step copies its inputs host->device (one pinned block) and
    # its losses device->host.  The two-slot begin/end form of the C ABI lets the host stage step k+1 while the
    # GPU runs step k; the losses of step k are read one iteration later, all inside the timed region.
    Ke = max(10, min(K, 500))
    for k in range(3):
        model.loss_and_grad_host(pos[k % NB], box[k % NB], el[k % NB], fl[k % NB])
    barrier()

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
                    losses = model.loss_and_grad_host_end((k - 1) & 1)
            return model.loss_and_grad_host_end((n - 1) & 1)

    e2e_loop(6)  # plain launches, capture, first replays
    barrier()
    t0 = time.perf_counter()
    e2e_losses = e2e_loop(Ke)
    barrier()
    e2e_s = time.perf_counter() - t0
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
    t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_value = world * B * Ke / float(t[0])
    isz = np.dtype(dtype).itemsize
    h2d = isz * (B * 3 * N * 2 + B * 6 + B)
    d2h = 8 * 4 + 4

    # ---- per-phase device times (eager launches, CUDA events between phases, L2 flushed)
    model.set_phase_timing(True)
    acc = {}
    Kp = 30
    for k in range(Kp):
        flush.zero_()
        model.loss_and_grad(d_pos[k % NB], d_box[k % NB], d_el[k % NB], d_fl[k % NB])
        for name, ms in model.phase_times_ms().items():
            acc[name] = acc.get(name, 0.0) + ms / Kp
    model.set_phase_timing(False)
    dom = max((n for n in acc if n not in ("descriptors", "loss")), key=lambda n: acc[n])
    # algorithmic bytes of one launch of the dominant sweep kernel: the compact neighbour rows it
    # reads (vector+norm 16 B, two scalar derivatives 8 B, descriptor 4 B, cutoff 4 B, index 4 B per
    # neighbour), its per-atom channel row in and out, and the gathered force cotangents
    ctx = ops.construct_descriptors_light(CFG["Rc"], CFG["nr"], CFG["na"], N, None, CFG["Rs"], CFG["Ra"], B,
                                          dtype=torch.float32, device=dev)
    outs = ops.compute_descriptors_light(d_pos[0], d_box[0], with_angular=False, ctx=ctx)
    n_i = outs[3][..., 0].to(torch.float64)
    m_i = outs[8].to(torch.float64)
    trip = float((m_i * (m_i - 1) / 2).sum())
    F = shape.Fr[0] + shape.Fa[0]
    row_bytes = float((n_i * (16 + 8 + 4 + 4 + 4) + 8).sum())
    chan = B * N * F * isz
    alg = {"af_fwd": row_bytes + chan, "force": row_bytes + chan + float(((n_i + 1) * 3 * isz).sum()),
           "force_grad": row_bytes + 2 * chan + float(((n_i + 1) * 3 * isz).sum()),
           "af_grad": row_bytes + chan, "mlp_fwd": 3 * chan, "mlp_bwd": 4 * chan}[dom]
    # DRAM traffic per launch of each sweep (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of
    # this workload at batch 4, profiles/k_sweep_water768_b4_fp32.md); it scales with the number of atoms
    traffic_ncu_b4 = {"af_fwd": 5.23e6, "force": 5.56e6, "force_grad": 5.58e6, "mlp_fwd": 0.40e6, "mlp_bwd": 3.85e6}
    traffic = traffic_ncu_b4.get(dom)
    if traffic is not None:
        traffic *= B / 4.0
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = alg / (acc[dom] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "k_sweep<%s>" % dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "traffic": traffic, "peak_source": "measured" if peaks else "fallback",
                "ms_per_launch": acc[dom], "algorithmic_bytes_per_launch": alg,
                "note": "geometry is rebuilt on chip, so this kernel is bound by the FP32/SFU pipes, not by HBM; "
                        "triplet-channel evaluations per launch = %.3g" % (trip * shape.Fa[0] / shape.C)}
    # the HBM-bound kernel of the operator boundary: the angular descriptor fill (write-once tensors), timed as
    # the difference between the operator with and without its three angular outputs (outputs preallocated,
    # no host synchronisation inside the timed region)
    import ctypes as C
    from alphanesgpu_b200 import _lib
    nr_, na_ = CFG["nr"], CFG["na"]
    te = lambda *sh, d=torch.float32: torch.empty(*sh, dtype=d, device=dev)
    o_rad, o_d3s, o_d2b, o_d3bs = te(B, N, nr_), te(B, N, nr_), te(B, N, 3, nr_), te(B, N, 3, nr_)
    o_im2, o_ntr = te(B, N, nr_ + 1, d=torch.int32), te(B, N, d=torch.int32)
    o_ang, o_im3, o_d3b = te(B, N, na_), te(B, N, 2 * na_, d=torch.int32), te(B, N, 3, 2 * na_)
    vp = lambda t: None if t is None else C.c_void_p(t.data_ptr())

    def desc_call(k, angular):
        a = (o_ang, o_im3, o_d3b) if angular else (None, None, None)
        rc = _lib.lib().stafb_compute_descriptors_light(ctx.h, ctx.stream(), vp(d_pos[k % NB]), vp(d_box[k % NB]), B, N,
                                                        vp(o_rad), vp(a[0]), vp(o_d3s), vp(o_im2), vp(a[1]), vp(o_d2b),
                                                        vp(a[2]), vp(o_d3bs), vp(o_ntr))
        assert rc == 0, rc
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    for k in range(3):
        desc_call(k, True)
    t_no, t_with = 0.0, 0.0
    for k in range(10):
        flush.zero_()
        e0.record()
        desc_call(k, False)
        e1.record()
        desc_call(k, True)
        e2.record()
        torch.cuda.synchronize()
        t_no += e0.elapsed_time(e1) / 10
        t_with += e1.elapsed_time(e2) / 10
    ctx.raise_on_status("operator-boundary descriptors")
    ang_bytes = B * N * CFG["na"] * (isz + 8 + 6 * isz)
    ang_ms = max(t_with - t_no, 1e-6)
    roofline_ops = {"bound": "hbm", "kernel": "k_angular (ComputeDescriptorsLight angular tensors)",
                    "achieved": ang_bytes / (ang_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": ang_bytes / (ang_ms * 1e-3) / 1e9 / peak, "traffic": None, "ms_per_launch": ang_ms,
                    "algorithmic_bytes_per_launch": ang_bytes}
    del o_ang, o_im3, o_d3b

    # ---- FP32 pipe: measured FMA peak of this GPU against the algorithmic flops of the step
    # (about 1.3 kFLOP per triplet for fingerprints + forces + both backward sweeps, 5 active channels per class)
    pk32, pk64 = C.c_double(), C.c_double()
    _lib.lib().stafb_measure_fma_peak(0, model.ctx.stream(), C.byref(pk32))
    _lib.lib().stafb_measure_fma_peak(1, model.ctx.stream(), C.byref(pk64))
    step_flops = trip * 1.3e3
    fp32_pipe = {"fma_peak_tflops_measured": pk32.value, "fp64_fma_peak_tflops_measured": pk64.value,
                 "algorithmic_flops_per_step": step_flops,
                 "achieved_tflops": step_flops / (total_ms / K * 1e-3) / 1e12,
                 "frac_of_fma_peak": step_flops / (total_ms / K * 1e-3) / 1e12 / pk32.value}

    # ---- the same step in float64 (BASELINE configs[2]): time ratio against fp32
    model64 = StafModel(shape, CFG, theta.astype(np.float64), emb.astype(np.float64), B, dtype=torch.float64, device=dev)
    d64 = [torch.as_tensor(a.astype(np.float64)).to(dev) for a in (pos, box, el, fl)]
    for k in range(3):
        model64.loss_and_grad(d64[0][k % NB], d64[1][k % NB], d64[2][k % NB], d64[3][k % NB])
        model64.adam_update_dev(lr)
    K64 = 30
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t64 = 0.0
    for k in range(K64):
        flush.zero_()
        e0.record()
        model64.loss_and_grad(d64[0][k % NB], d64[1][k % NB], d64[2][k % NB], d64[3][k % NB])
        model64.adam_update_dev(lr)
        e1.record()
        torch.cuda.synchronize()
        t64 += e0.elapsed_time(e1)
    model64.ctx.raise_on_status("fp64 leg")
    fp64 = {"value": B * K64 / (t64 * 1e-3), "unit": "frames/s", "ms_per_step": t64 / K64, "steps": K64,
            "time_ratio_fp64_over_fp32": (t64 / K64) / (total_ms / K),
            "note": "eager launches (no graph); fp32 figure is the graph-replayed step"}
    model64.close()

    line = None
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            fps, dt, cores = cpu_port_frames_per_s(B, 6)
            cpu = {"value": fps, "unit": "frames/s", "cores": cores, "kind": "port",
                   "sample": "6 batches of %d frames (%.1f s)" % (B, dt)}
        line = {
            "metric": METRIC, "value": value, "unit": "frames/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / PUBLISHED_V100_FRAMES_PER_S, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "water768 E+F training step (eval + Adam), batch %d per GPU, fp32 "
                                   "(BASELINE configs[1])" % B,
                       "frames": "seeded synthetic water, 256 O + 512 H, L=19.6 A, %d distinct batches" % NB,
                       "model": "2 species, Fr=10, Fa=15, MLP 25-64-32-1 tanh", "parallelism": "dp%d" % world,
                       "l2": "flushed between steps (256 MiB write); per-step CUDA events summed",
                       "launch": "two CUDA graphs per step: neighbour rows of the NEXT batch on a second stream, "
                                 "the rest of the step on the main stream; each timed interval contains both"
                                 + ("" if world == 1 else ("; gradient averaging + Adam as one peer-memory kernel in the step graph"
                                                            if px is not None else
                                                            "; NCCL all-reduce between the step graph and the Adam graph")),
                       "vs_baseline_note": "published number is the reference on a V100 (README.md:42-45)"},
            "value_l2_warm": value_warm, "ms_per_step_min": float(per_step.min()),
            "e2e": {"value": e2e_value, "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": Ke, "path": "stafb_train_step_host_begin/_end (two pinned slots) + "
                            + ("stafb_allreduce_adam" if px is not None else "stafb_adam_step_dev"),
                    "synchronous_call_value": world * B / e2e_sync_s},
            "gpu_launches": launches_per_step * K, "launches_per_step": launches_per_step,
            "clocks": clocks, "roofline": roofline, "roofline_operator_boundary": roofline_ops,
            "fp32_pipe": fp32_pipe, "fp64": fp64, "phase_ms": acc, "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    if px is not None:
        if px.status() != 0:
            raise SystemExit("peer exchange reported status %d" % px.status())
        px.close()
    model.close()
    if world > 1:
        dist.destroy_process_group()


MD_METRIC = "24576-atom water E+F atom-steps/s (slab-decomposed inference)"


def run_md(args):
    """BASELINE configs[4]: energy+forces of one 24,576-atom water box, neighbour list rebuilt every call,
    atoms cut into `world` slabs along z with one-cutoff halos (alphanesgpu_b200/slab.py)."""
    import tempfile
    import ctypes as C
    import torch
    import torch.distributed as dist
    from alphanesgpu_b200 import params, synth, _lib
    from alphanesgpu_b200.model import StafModel
    from alphanesgpu_b200.params import ModelShape
    from alphanesgpu_b200.slab import SlabDomain, model_compute

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    K, W = args.steps, max(args.warmup, 3)
    pos, box, tipos = synth.water_frames("water24576", [1400])
    gshape = synth.baseline_shape(tipos)
    theta, emb = synth.init_params(gshape, dtype=np.float32)
    N = gshape.N
    types = gshape.type_map.astype(np.int32)
    gpos = torch.as_tensor(pos.reshape(N, 3).astype(np.float32)).to(dev)
    gtypes = torch.as_tensor(types).to(dev)
    SKIN, HALO_EVERY = 1.0, 10  # ghost sets are re-chosen every 10 evaluations with a 1 A skin, as an MD code does
    dom = SlabDomain(None, box[0], CFG["Rc"], rank, world, nt=gshape.nt, skin=SKIN, halo_every=HALO_EVERY)
    own_idx = dom.set_owned_from_global(gpos, gtypes)
    n_own = dom.pos.shape[0]
    halo = 0 if world == 1 else 2.0 * dom.reach / (dom.L / world)
    cap = int(n_own * (1.0 + halo) * 1.25) + 1024
    shape = ModelShape(nt=gshape.nt, tipos=list(dom.counts), Fr=gshape.Fr, Fa=gshape.Fa, widths=gshape.widths)
    model = StafModel(shape, CFG, theta, emb, 1, dtype=torch.float32, device=dev, n_max=cap)
    dom.compute = model_compute(model, box[0])

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
    launches = model.launches()
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
        h2d, d2h = 4 * (3 * N + 6 + N), 4 * (3 * N + 1 + 9)
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
        dom.step()
        for name, ms in model.phase_times_ms().items():
            acc[name] = acc.get(name, 0.0) + ms / 5
    model.set_phase_timing(False)
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            from oracle import oracle
            t0 = time.perf_counter()
            r = oracle.energy_force_grad(CFG, gshape.desc(), pos, box, gshape.type_map, theta, emb, np.float32,
                                         per_atom_energy=False)
            dt = time.perf_counter() - t0
            assert r["status"] == 0
            assert abs(float(r["energy"][0]) - float(e)) <= 2e-5 * abs(float(e)), (r["energy"], float(e))
            cpu = {"value": N / dt, "unit": "atom-steps/s", "cores": oracle.max_threads(), "kind": "port",
                   "sample": "1 evaluation of the 24576-atom box (%.1f s); energy agrees with the GPU" % dt}
        line = {
            "metric": MD_METRIC, "value": N * K / (total_ms * 1e-3), "unit": "atom-steps/s", "n_gpus": world,
            "steps": K, "warmup": W, "ms_per_step": total_ms / K, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "water24576 energy+forces, list rebuilt every call, fp32 (BASELINE configs[4])",
                       "decomposition": "%d z-slab(s), %.1f A halos (cutoff + %.1f A skin, ghost sets re-chosen every "
                                        "%d evaluations), owned atoms on rank 0: %d" % (world, dom.reach, SKIN,
                                                                                         HALO_EVERY, n_own),
                       "l2": "flushed between steps (256 MiB write); per-step CUDA events summed",
                       "model": "2 species, Fr=10, Fa=15, MLP 25-64-32-1 tanh"},
            "e2e": {"value": N * Ke / (e2e_ms * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": Ke,
                    "path": "staf_compute (libstaf C API, host double arrays)" if world == 1 else
                            "slab driver: pinned host -> device, halo exchange, forces -> pinned host"},
            "gpu_launches": launches * K, "launches_per_step": launches, "clocks": clocks, "phase_ms": acc,
            "energy": float(e), "dd_parity": dd_err, "cpu_baseline": cpu,
        }
        print(json.dumps(line))
    model.close()
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
                    help="train: BASELINE configs[1]/[3] (the headline metric); md: BASELINE configs[4]")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "md":
        if args.steps == 2000:
            args.steps = 50
        run_md(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
