"""Generates tests/golden/* from a checkout of the reference (run once, where that checkout exists).

  python tests/golden/make_fixtures.py <path of the reference tree>

What it writes:
  ref_frame0/            the reference's real 768-atom water frame
                         (test/test-inference-pipeline/frames/{pos_0,box_0,type.dat}) and its exported
                         model in TF-free formats (test/test-lammps-smoke/model_onnx_grad_float:
                         type{k}_*.dat, mlp_type{k}.bin, staf_jmd.cfg) - data files, copied verbatim;
  ref_nl.npz             neighbour lists produced by the reference's own CPU cell list
                         (STAF/src/descriptor_builder/cell_list.cu.cc:1080, built into oracle/_ref) for
                         frame0 and for two seeded synthetic frames, float and double;
  ref_mlp.npz            energy and dE/dAF produced by the reference's own native MLP
                         (libstaf/src/mlp/staf_mlp_ort.cc:196-242, built into oracle/_ref) on seeded
                         AF inputs, float weights and a double re-export of the same weights.
Known answers that the reference records as text (energy and rms force of frame 0) are cited in the
tests themselves.
"""
import os
import shutil
import struct
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from alphanesgpu_b200 import params, synth  # noqa: E402
from oracle import oracle  # noqa: E402


def write_mlp_bin(path, mu, layers, dtype):
    prec = 1 if np.dtype(dtype) == np.float64 else 0
    with open(path, "wb") as f:
        f.write(b"STAFMLP1")
        f.write(struct.pack("<3i", prec, len(mu), len(layers)))
        f.write(np.asarray(mu, dtype).tobytes())
        for act, W, b in layers:
            f.write(struct.pack("<3i", act, W.shape[0], W.shape[1]))
            f.write(np.asarray(W, dtype).tobytes())
            f.write(np.asarray(b, dtype).tobytes())


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_fixtures.py <path of the reference tree>")
    ref = sys.argv[1]
    oracle.build()
    assert oracle.ref_available(), "oracle/_ref not built"
    out = os.path.join(HERE, "ref_frame0")
    os.makedirs(out, exist_ok=True)
    fr = os.path.join(ref, "test/test-inference-pipeline/frames")
    md = os.path.join(ref, "test/test-lammps-smoke/model_onnx_grad_float")
    np.save(os.path.join(out, "pos_0.npy"), np.loadtxt(os.path.join(fr, "pos_0")))
    np.save(os.path.join(out, "box_0.npy"), np.loadtxt(os.path.join(fr, "box_0")))
    for n in ["type.dat", "staf_jmd.cfg", "mlp_type0.bin", "mlp_type1.bin"] + [
            "type%d_%s.dat" % (k, s) for k in (0, 1)
            for s in ("alpha_2body", "alpha_3body", "alpha_mu", "type_emb_2b_sq", "type_emb_3b_sq")]:
        shutil.copy(os.path.join(md, n), os.path.join(out, n))

    # --- neighbour lists from the reference's CPU cell list
    nl = {}
    pos0 = np.load(os.path.join(out, "pos_0.npy"))
    box0 = np.load(os.path.join(out, "box_0.npy"))
    frames = {"frame0": (pos0, box0)}
    for name, seed in (("water96", 1000), ("water768", 1100)):
        p, b, _ = synth.water_frames(name, [seed])
        frames["%s_s%d" % (name, seed)] = (p[0], b[0])
    for key, (p, b) in frames.items():
        for dt, tag in ((np.float32, "f32"), (np.float64, "f64")):
            r = oracle.ref_neighbour_list(4.5, 60, p, b, dt)
            assert r["overflow"] == 0
            nl["%s_%s_with" % (key, tag)] = r["with_"].astype(np.int16)
            nl["%s_%s_howmany" % (key, tag)] = r["howmany"].astype(np.int16)
            nl["%s_%s_d2" % (key, tag)] = r["d2"]
            nl["%s_%s_ncell" % (key, tag)] = r["ncell"]
    np.savez_compressed(os.path.join(HERE, "ref_nl.npz"), **nl)

    # --- MLP from the reference's native evaluator
    rng = np.random.default_rng(4242)
    af = [np.exp(rng.normal(0.0, 1.0, size=(7, 60))), np.exp(rng.normal(0.0, 1.0, size=(5, 60)))]
    mlp = {}
    e, d = oracle.ref_mlp_eval(out, af, np.float32)
    mlp["af0"], mlp["af1"] = af
    mlp["f32_energy"], mlp["f32_d0"], mlp["f32_d1"] = e, d[0], d[1]
    with tempfile.TemporaryDirectory() as tmp:
        for k in (0, 1):
            m = params.read_mlp_bin(os.path.join(out, "mlp_type%d.bin" % k))
            write_mlp_bin(os.path.join(tmp, "mlp_type%d.bin" % k), m["mu"], m["layers"], np.float64)
        e, d = oracle.ref_mlp_eval(tmp, af, np.float64)
    mlp["f64_energy"], mlp["f64_d0"], mlp["f64_d1"] = e, d[0], d[1]
    np.savez_compressed(os.path.join(HERE, "ref_mlp.npz"), **mlp)
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
