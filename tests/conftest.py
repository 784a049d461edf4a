import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def frame0():
    """The reference's real 768-atom water frame and exported model (tests/golden/ref_frame0)."""
    import numpy as np
    from alphanesgpu_b200 import params
    d = os.path.join(GOLDEN, "ref_frame0")
    cfg, shape, theta, emb = params.load_model_dir(d, np.float64)
    pos = np.load(os.path.join(d, "pos_0.npy")).reshape(1, -1)
    box = np.load(os.path.join(d, "box_0.npy")).reshape(1, 6)
    return dict(cfg=cfg, shape=shape, theta=theta, emb=emb, pos=pos, box=box, dir=d)


CFG = dict(Rc=4.5, Rs=2.25, Ra=4.5, nr=60, na=1770)


def rel_err(x, ref):
    import numpy as np
    x = np.asarray(x, np.float64)
    ref = np.asarray(ref, np.float64)
    den = np.abs(ref).max()
    return float(np.abs(x - ref).max() / (den if den > 0 else 1.0))


def tie_groups_equal(with_a, with_b, d2, howmany):
    """Neighbour rows equal except for permutations inside runs of bit-equal dist2
    (the reference's own order there depends on atomicAdd arrival:
    STAF/src/descriptor_builder/celle_gpu.cu.cc:197-200).  Returns the number of tie groups."""
    import numpy as np
    groups = 0
    for i in range(with_a.shape[0]):
        n = int(howmany[i])
        k = 0
        while k < n:
            e = k + 1
            while e < n and d2[i, e] == d2[i, k]:
                e += 1
            if e - k > 1:
                groups += 1
                assert sorted(with_a[i, k:e].tolist()) == sorted(with_b[i, k:e].tolist()), (i, k, e)
            else:
                assert with_a[i, k] == with_b[i, k], (i, k)
            k = e
    return groups


def oracle_force_and_virial(oracle, shape, theta, emb, pos, box):
    """Total force and virial of the op chain (descriptors -> AF -> MLP -> ...Virial force ops), double."""
    import numpy as np
    dt = np.float64
    nf, N, nt, C = pos.shape[0], shape.N, shape.nt, shape.C
    ref = oracle.descriptors(CFG["Rc"], CFG["Rs"], CFG["Ra"], CFG["nr"], CFG["na"], pos, box, dt)
    tm = shape.type_map
    F, W, E = np.zeros((nf, 3 * N)), np.zeros((nf, 9)), np.zeros(nf)
    for t in range(nt):
        s, Nl = shape.shift(t), shape.tipos[t]
        d = {k: np.ascontiguousarray(v[:, s:s + Nl]) for k, v in ref.items() if isinstance(v, np.ndarray) and v.ndim >= 2}
        o = shape.offsets(t)
        Fr, Fa = shape.Fr[t], shape.Fa[t]
        a2 = theta[o["a2"]:o["a2"] + nt * Fr].reshape(nt, Fr)
        a3 = theta[o["a3"]:o["a3"] + C * 3 * Fa].reshape(C, 3 * Fa)
        e2 = emb[o["emb"]:o["emb"] + nt * Fr].reshape(nt, Fr)
        e3 = emb[o["emb"] + nt * Fr:o["emb"] + nt * Fr + C * Fa].reshape(C, Fa)
        mu = theta[o["mu"]:o["mu"] + Fr + Fa]
        w = theta[o["w"]:o["a2"] + o["size"]]
        af2 = oracle.af_radial(d["raddescr"], d["intmap2b"], a2, e2, tm)
        af3 = oracle.af_angular(d["angdescr"], d["des3bsupp"], d["intmap3b"], a3, e3, tm, d["numtriplet"])
        af = np.concatenate([af2, af3], axis=2).reshape(nf * Nl, Fr + Fa)
        e, nd = oracle.mlp_eval(shape.widths, af, mu, w)
        nd = nd.reshape(nf, Nl, Fr + Fa)
        E += 0.5 * e.reshape(nf, Nl).sum(1)
        f2, w2 = oracle.force_radial(np.ascontiguousarray(nd[..., :Fr]), d["der2b"], d["intmap2b"], d["raddescr"], a2,
                                     e2, tm, s, pos, box)
        f3, w3 = oracle.force_tripl(np.ascontiguousarray(nd[..., Fr:]), d["des3bsupp"], d["angdescr"], d["der3bsupp"],
                                    d["der3b"], d["intmap3b"], a3, e3, tm, d["numtriplet"], s, pos, box)
        F += f2 + f3
        W += w2 + w3
    return E, F, W
