"""Seeded synthetic water frames and model parameters.

The reference's published numbers were measured on an MB-pol water data set that is
not distributed with it; these generators produce stand-in frames with the same
shapes and neighbour statistics (768 atoms, L about 19.6 A, about 38 neighbours inside
4.5 A) and parameter sets with the reference's tensor shapes
(STAF/init_params/init_AFs_param.py:14-37 for the 0/1 embedding masks).
"""
import numpy as np

from .params import ModelShape

R_OH = 0.9572
HOH_DEG = 104.52


def gen_water(nx, ny, nz, L, seed):
    """One water frame: nx*ny*nz molecules on a jittered lattice in a cubic box L.

    Returns (pos[3N] float64 Cartesian, unwrapped; box6 float64; tipos=[nO, nH]).
    Atom order is all O then all H (species-sorted, as the ops require).
    """
    rng = np.random.default_rng(seed)
    ix, iy, iz = np.meshgrid(np.arange(nx), np.arange(ny), np.arange(nz), indexing="ij")
    O = np.stack([(ix.ravel() + 0.5) * L / nx, (iy.ravel() + 0.5) * L / ny, (iz.ravel() + 0.5) * L / nz], axis=1)
    nO = O.shape[0]
    O = O + rng.normal(0.0, 0.1, size=(nO, 3))
    q = rng.normal(size=(nO, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    w, x, y, z = q.T
    R = np.stack([
        np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], axis=1),
        np.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], axis=1),
        np.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], axis=1)], axis=1)
    half = np.deg2rad(HOH_DEG) / 2
    h1 = R_OH * np.array([np.sin(half), 0.0, np.cos(half)])
    h2 = R_OH * np.array([-np.sin(half), 0.0, np.cos(half)])
    H1 = O + R @ h1
    H2 = O + R @ h2
    H = np.stack([H1, H2], axis=1).reshape(-1, 3)
    pos = np.concatenate([O, H], axis=0).reshape(-1)
    box = np.array([L, 0.0, 0.0, L, 0.0, L])
    return pos, box, [nO, 2 * nO]


WATER_CONFIGS = {
    # name: (nx, ny, nz, L)
    "water96": (4, 4, 2, 9.86),
    "water768": (8, 8, 4, 19.6),
    "water6144": (16, 16, 8, 39.2),
    "water24576": (16, 16, 32, 62.7),
}


def water_frames(name, seeds):
    nx, ny, nz, L = WATER_CONFIGS[name]
    P, B = [], []
    tipos = None
    for s in seeds:
        p, b, tipos = gen_water(nx, ny, nz, L, s)
        P.append(p)
        B.append(b)
    return np.stack(P), np.stack(B), tipos


def baseline_shape(tipos, n_rad=5, n_ang=5, widths=(64, 32, 1)):
    """2 species; n_rad radial AFs per partner species and n_ang angular AFs per
    species-pair class for each central species."""
    nt = len(tipos)
    C = nt * (nt + 1) // 2
    return ModelShape(nt=nt, tipos=list(tipos), Fr=[n_rad * nt] * nt, Fa=[n_ang * C] * nt, widths=list(widths))


def block_mask(rows, per_row):
    m = np.zeros((rows, rows * per_row))
    for r in range(rows):
        m[r, r * per_row:(r + 1) * per_row] = 1.0
    return m


def init_params(shape, seed_alpha=2000, seed_mu=2001, seed_mlp=2002, dtype=np.float64):
    """theta (trained, flat) and emb (squared 0/1 masks, flat) with seeded values:
    alpha ~ U(0.5, 2.0), mu ~ U(-1, 1), Glorot-uniform MLP weights, zero biases."""
    theta = np.zeros(shape.n_params, np.float64)
    emb = np.zeros(shape.n_emb, np.float64)
    ra, rm, rw = (np.random.default_rng(s) for s in (seed_alpha, seed_mu, seed_mlp))
    nt, C = shape.nt, shape.C
    for t in range(nt):
        o = shape.offsets(t)
        Fr, Fa = shape.Fr[t], shape.Fa[t]
        theta[o["a2"]:o["a2"] + nt * Fr] = ra.uniform(0.5, 2.0, nt * Fr)
        theta[o["a3"]:o["a3"] + C * 3 * Fa] = ra.uniform(0.5, 2.0, C * 3 * Fa)
        theta[o["mu"]:o["mu"] + Fr + Fa] = rm.uniform(-1.0, 1.0, Fr + Fa)
        w = o["w"]
        n_in = Fr + Fa
        for width in shape.widths:
            lim = np.sqrt(6.0 / (n_in + width))
            theta[w:w + n_in * width] = rw.uniform(-lim, lim, n_in * width)
            w += n_in * width + width
            n_in = width
        emb[o["emb"]:o["emb"] + nt * Fr] = block_mask(nt, Fr // nt).ravel()
        emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + C * Fa] = block_mask(C, Fa // C).ravel()
    return theta.astype(dtype), emb.astype(dtype)


def labels(nf, N, seed=3000, dtype=np.float64):
    r = np.random.default_rng(seed)
    return r.normal(size=nf).astype(dtype), r.normal(size=(nf, 3 * N)).astype(dtype)
