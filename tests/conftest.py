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
