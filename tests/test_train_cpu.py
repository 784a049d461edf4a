"""CPU checks of the training driver's host logic: learning-rate schedules against the closed forms of the
Keras schedules the reference uses (STAF/optimizer_learning_rate_utility.py:9-60), configuration -> model
shape, parameter initialisation ranges and buffer sharding."""
import math

import numpy as np
import pytest

from alphanesgpu_b200 import train as T


def test_expdec_reaches_the_final_rate_after_epochs_times_buffer_steps():
    lr = T.build_learning_rate("expdec 0.001 0.0000001", n_epochs=50, batches_per_buffer=1, buffer_dim=4)
    assert lr(0) == pytest.approx(1e-3)
    assert lr(200) == pytest.approx(1e-7, rel=1e-9)
    assert lr(100) == pytest.approx(1e-5, rel=1e-9)  # geometric


def test_cosann_restarts_with_longer_and_lower_periods():
    lr = T.build_learning_rate("cosann 0.01 2.5 2.0 0.9 0.0", n_epochs=1, batches_per_buffer=1, buffer_dim=4)
    first = int(2.5 * 1 * 4)
    assert lr(0) == pytest.approx(0.01)
    assert lr(first // 2) == pytest.approx(0.005)
    assert lr(first) == pytest.approx(0.009)               # restart, scaled by m_mul
    assert lr(first + first) == pytest.approx(0.0045)      # middle of the second period (twice as long)
    assert lr(3 * first) == pytest.approx(0.0081)          # second restart
    lr2 = T.cosann(0.01, 10, 1.0, 1.0, 0.1)
    assert lr2(10) == pytest.approx(0.01) and lr2(5) == pytest.approx(0.01 * (0.9 * 0.5 + 0.1))
    with pytest.raises(ValueError):
        T.build_learning_rate("linear 0.1", 1, 1, 1)


def test_config_to_shape_and_initial_parameters():
    cfg = T.load_config(dict(map_rad_afs={0: [10, 10], 1: [10, 10]}, map_ang_afs={0: [20, 20, 20], 1: [20, 20, 20]},
                             number_of_decoding_nodes="240 240"))
    shape = T.model_shape_from_config(cfg, [256, 512])
    assert shape.Fr == [20, 20] and shape.Fa == [60, 60] and shape.widths == [240, 240, 1] and shape.N == 768
    theta, emb = T.init_params(shape, cfg, seed=3)
    o = shape.offsets(1)
    a3 = theta[o["a3"]:o["a3"] + 3 * 3 * 60].reshape(3 * 60, 3)
    assert np.all(np.abs(a3[:, :2]) <= 1.0) and np.all((a3[:, 2] <= 0.0) & (a3[:, 2] >= -10.0))
    e2 = emb[o["emb"]:o["emb"] + 2 * 20].reshape(2, 20)
    assert e2[0, :10].all() and not e2[0, 10:].any() and e2[1, 10:].all()   # channel c listens to one partner species
    e3 = emb[o["emb"] + 40:o["emb"] + 40 + 3 * 60].reshape(3, 60)
    assert (e3.sum(0) == 1).all() and e3[2, 40:].all()
    # zero biases, Glorot-bounded kernels
    w = o["w"]
    lim = math.sqrt(6.0 / (80 + 240))
    assert np.abs(theta[w:w + 80 * 240]).max() <= lim and not theta[w + 80 * 240:w + 80 * 240 + 240].any()
    with pytest.raises(ValueError):
        T.load_config(dict(type_of_training="energy"))


def test_buffers_are_sharded_by_rank_with_equal_counts():
    all_ = T.buffer_indices(37, 4)
    assert all_.shape == (9, 4) and all_[-1, -1] == 35
    parts = [T.buffer_indices(37, 4, r, 2) for r in range(2)]
    assert [p.shape for p in parts] == [(4, 4), (4, 4)]
    assert parts[0][1, 0] == 8 and parts[1][0, 0] == 4   # buffers idx[rank::world]
    assert len(set(np.concatenate(parts).ravel().tolist())) == 32
