"""Flat parameter layout of the per-species model and readers for the reference's
exported model directory (type{k}_alpha_2body.dat, ..., mlp_type{k}.bin).

Per central species t the trained block is
    alpha2b[nt, Fr_t] | alpha3b[C, 3*Fa_t] | mu[Fr_t+Fa_t] | W0[in,out] b0 | W1 b1 | ...
(weights row-major [in, out] as Keras; libstaf/src/mlp/staf_mlp_ort.cc:20-24), blocks
concatenated over t.  The squared type embeddings, which the reference never updates
(STAF/staf_models/staf_model.py:225-253), live in a second flat buffer
    e2[nt, Fr_t] | e3[C, Fa_t]   per species.
The same layout is used by the C ABI (include/stafb.h) and by the CPU oracle.
"""
import os
import struct
from dataclasses import dataclass, field
from typing import List

import numpy as np

MAX_TYPES, MAX_DENSE = 4, 6


@dataclass
class ModelShape:
    nt: int
    tipos: List[int]
    Fr: List[int]
    Fa: List[int]
    widths: List[int] = field(default_factory=lambda: [64, 32, 1])

    def __post_init__(self):
        if not (1 <= self.nt <= MAX_TYPES and 1 <= len(self.widths) <= MAX_DENSE and self.widths[-1] == 1):
            raise ValueError("unsupported model shape")

    @property
    def C(self):
        return self.nt * (self.nt + 1) // 2

    @property
    def N(self):
        return int(sum(self.tipos))

    def shift(self, t):
        return int(sum(self.tipos[:t]))

    def mlp_size(self, t):
        n_in, s = self.Fr[t] + self.Fa[t], 0
        for w in self.widths:
            s += n_in * w + w
            n_in = w
        return s

    def block_size(self, t):
        return self.nt * self.Fr[t] + self.C * 3 * self.Fa[t] + self.Fr[t] + self.Fa[t] + self.mlp_size(t)

    def offsets(self, t):
        b = sum(self.block_size(u) for u in range(t))
        a3 = b + self.nt * self.Fr[t]
        mu = a3 + self.C * 3 * self.Fa[t]
        w = mu + self.Fr[t] + self.Fa[t]
        e = sum(self.nt * self.Fr[u] + self.C * self.Fa[u] for u in range(t))
        return dict(a2=b, a3=a3, mu=mu, w=w, emb=e, size=self.block_size(t))

    @property
    def n_params(self):
        return sum(self.block_size(t) for t in range(self.nt))

    @property
    def n_emb(self):
        return sum(self.nt * self.Fr[t] + self.C * self.Fa[t] for t in range(self.nt))

    @property
    def type_map(self):
        return np.repeat(np.arange(self.nt, dtype=np.int32), self.tipos)

    def desc(self):
        """int32[20] descriptor passed through the C ABI: nt, tipos[4], Fr[4], Fa[4], n_dense, width[6]."""
        d = np.zeros(20, np.int32)
        d[0] = self.nt
        d[1:1 + self.nt] = self.tipos
        d[5:5 + self.nt] = self.Fr
        d[9:9 + self.nt] = self.Fa
        d[13] = len(self.widths)
        d[14:14 + len(self.widths)] = self.widths
        return d


def read_mlp_bin(path):
    """STAFMLP1 container (libstaf/src/mlp/staf_mlp_ort.cc:99-165):
    magic, int32 precision, n_af, n_layers; mu[n_af]; per layer int32 act, in, out; W[in*out]; b[out]."""
    with open(path, "rb") as f:
        raw = f.read()
    if raw[:8] != b"STAFMLP1":
        raise ValueError("bad magic in %s" % path)
    prec, n_af, n_layers = struct.unpack_from("<3i", raw, 8)
    dt = np.float64 if prec == 1 else np.float32
    isz = np.dtype(dt).itemsize
    off = 20
    mu = np.frombuffer(raw, dt, n_af, off).copy()
    off += n_af * isz
    layers = []
    for _ in range(n_layers):
        act, n_in, n_out = struct.unpack_from("<3i", raw, off)
        off += 12
        W = np.frombuffer(raw, dt, n_in * n_out, off).reshape(n_in, n_out).copy()
        off += n_in * n_out * isz
        b = np.frombuffer(raw, dt, n_out, off).copy()
        off += n_out * isz
        layers.append((act, W, b))
    return dict(precision=prec, n_af=n_af, mu=mu, layers=layers)


def read_jmd_cfg(path):
    """staf_jmd.cfg key = value lines (libstaf/vendor/jmd/nn_nn_mlp.cu:371-383)."""
    cfg = {}
    with open(path) as f:
        for line in f:
            if "=" in line:
                k, v = line.split("=", 1)
                cfg[k.strip()] = v.strip()
    return cfg


def load_model_dir(model_dir, dtype=np.float64):
    """Read a model directory exported by the reference (libstaf/include/staf.h:36 lists the
    files).  Returns (cfg dict, ModelShape, theta, emb)."""
    cfgp = os.path.join(model_dir, "staf_jmd.cfg")
    raw = read_jmd_cfg(cfgp) if os.path.exists(cfgp) else {}
    cfg = dict(Rc=float(raw.get("Cutoff", 4.5)), Ra=float(raw.get("Cutoff_Angular", 4.5)),
               Rs=float(raw.get("Hardcore_Cutoff", 2.25)), nr=int(raw.get("Buffer_radial_descriptors", 60)),
               na=int(raw.get("Buffer_angular_descriptors", 1770)))
    nt = int(raw.get("number_of_types", 2))
    tipos = np.loadtxt(os.path.join(model_dir, raw.get("file_of_tipos", "type.dat")), dtype=int).reshape(-1).tolist()
    C = nt * (nt + 1) // 2
    a2, a3, e2, e3, mus, nets = [], [], [], [], [], []
    for k in range(nt):
        a2.append(np.loadtxt(os.path.join(model_dir, "type%d_alpha_2body.dat" % k)).reshape(nt, -1))
        a3.append(np.loadtxt(os.path.join(model_dir, "type%d_alpha_3body.dat" % k)).reshape(C, -1))
        e2.append(np.loadtxt(os.path.join(model_dir, "type%d_type_emb_2b_sq.dat" % k)).reshape(nt, -1))
        e3.append(np.loadtxt(os.path.join(model_dir, "type%d_type_emb_3b_sq.dat" % k)).reshape(C, -1))
        mus.append(np.loadtxt(os.path.join(model_dir, "type%d_alpha_mu.dat" % k)).reshape(-1))
        nets.append(read_mlp_bin(os.path.join(model_dir, "mlp_type%d.bin" % k)))
    widths = [W.shape[1] for (_, W, _) in nets[0]["layers"]]
    shape = ModelShape(nt=nt, tipos=tipos, Fr=[a.shape[1] for a in a2], Fa=[a.shape[1] // 3 for a in a3],
                       widths=widths)
    theta = np.zeros(shape.n_params, np.float64)
    emb = np.zeros(shape.n_emb, np.float64)
    for k in range(nt):
        o = shape.offsets(k)
        Fr, Fa = shape.Fr[k], shape.Fa[k]
        theta[o["a2"]:o["a2"] + nt * Fr] = a2[k].ravel()
        theta[o["a3"]:o["a3"] + C * 3 * Fa] = a3[k].ravel()
        theta[o["mu"]:o["mu"] + Fr + Fa] = mus[k]
        w = o["w"]
        for (act, W, b) in nets[k]["layers"]:
            theta[w:w + W.size] = W.ravel()
            w += W.size
            theta[w:w + b.size] = b
            w += b.size
        emb[o["emb"]:o["emb"] + nt * Fr] = e2[k].ravel()
        emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + C * Fa] = e3[k].ravel()
    return cfg, shape, theta.astype(dtype), emb.astype(dtype)


def write_mlp_bin(path, mu, layers, precision=1):
    """Writes the STAFMLP1 container read_mlp_bin reads (format of STAF/save_models/export_mlp_onnx.py:106-126
    of the reference): layers = [(act, W[in,out], b[out])], act 1 = tanh, 0 = linear."""
    dt = np.float64 if precision == 1 else np.float32
    with open(path, "wb") as f:
        f.write(b"STAFMLP1")
        f.write(struct.pack("<3i", int(precision), len(mu), len(layers)))
        f.write(np.asarray(mu, dt).tobytes())
        for act, W, b in layers:
            f.write(struct.pack("<3i", int(act), W.shape[0], W.shape[1]))
            f.write(np.ascontiguousarray(W, dt).tobytes())
            f.write(np.asarray(b, dt).tobytes())


def save_model_dir(model_dir, cfg, shape, theta, emb, precision=1):
    """Writes a model directory in the layout staf_load / load_model_dir read: staf_jmd.cfg, type.dat,
    type{k}_alpha_{2body,3body,mu}.dat, type{k}_type_emb_{2b,3b}_sq.dat and mlp_type{k}.bin."""
    os.makedirs(model_dir, exist_ok=True)
    nt, C = shape.nt, shape.C
    theta = np.asarray(theta, np.float64)
    emb = np.asarray(emb, np.float64)
    with open(os.path.join(model_dir, "staf_jmd.cfg"), "w") as f:
        f.write("Buffer_radial_descriptors = %d\nBuffer_angular_descriptors = %d\n" % (cfg["nr"], cfg["na"]))
        f.write("Cutoff = %r\nCutoff_Angular = %r\nHardcore_Cutoff = %r\n" % (cfg["Rc"], cfg["Ra"], cfg["Rs"]))
        f.write("number_of_types = %d\nfile_of_tipos = type.dat\nnn_export_dir = .\n" % nt)
    np.savetxt(os.path.join(model_dir, "type.dat"), np.asarray(shape.tipos, int).reshape(1, -1), fmt="%d")
    for k in range(nt):
        o = shape.offsets(k)
        Fr, Fa = shape.Fr[k], shape.Fa[k]
        sv = lambda name, a: np.savetxt(os.path.join(model_dir, "type%d_%s.dat" % (k, name)), a, fmt="%.17g")
        sv("alpha_2body", theta[o["a2"]:o["a2"] + nt * Fr].reshape(nt, Fr))
        sv("alpha_3body", theta[o["a3"]:o["a3"] + C * 3 * Fa].reshape(C, 3 * Fa))
        mu = theta[o["mu"]:o["mu"] + Fr + Fa]
        sv("alpha_mu", mu)
        sv("type_emb_2b_sq", emb[o["emb"]:o["emb"] + nt * Fr].reshape(nt, Fr))
        sv("type_emb_3b_sq", emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + C * Fa].reshape(C, Fa))
        w, n_in, layers = o["w"], Fr + Fa, []
        for li, width in enumerate(shape.widths):
            W = theta[w:w + n_in * width].reshape(n_in, width)
            w += n_in * width
            b = theta[w:w + width]
            w += width
            layers.append((1 if li < len(shape.widths) - 1 else 0, W, b))
            n_in = width
        write_mlp_bin(os.path.join(model_dir, "mlp_type%d.bin" % k), mu, layers, precision)
