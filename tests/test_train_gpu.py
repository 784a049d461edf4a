"""GPU test of the training driver: its pipelined loop must produce, step by step, the losses of the same
sequence driven through the synchronous entry points, and write the reference's log files."""
import numpy as np
import pytest

from alphanesgpu_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_driver_matches_a_hand_written_loop(tmp_path):
    from alphanesgpu_b200 import train as T
    from alphanesgpu_b200.model import StafModel
    pos, box, tipos = synth.water_frames("water96", list(range(1000, 1008)))
    el, fl = synth.labels(8, 96, seed=11)
    cfg = T.load_config(dict(buffer_stream_dim_tr=4, batch_size=2, number_of_epochs=2, displ_freq=3, Seed=5,
                             lr_dense_net="cosann 0.002 1 2.0 0.9 0.0", Radial_Buffer=60, Max_Angular_Neigh=60))
    data = dict(pos=pos, box=box, energy=el, force=fl, tipos=np.array(tipos))
    msgs = []
    res = T.train(cfg, str(tmp_path), data=data, log=msgs.append)
    rows = res["rows"]
    assert [r[0] for r in rows] == list(range(1, 9))          # 2 epochs x 2 buffers x 2 batches
    lines = open(tmp_path / "lcurve_notmean").read().split("\n")
    assert len([l for l in lines if l]) == 8 and len(open(tmp_path / "lr_step.dat").read().split()) == 8
    assert any("Time to elaborate 3 batch of 2 frames" in m for m in msgs)
    # the same sequence with the synchronous calls
    shape = res["shape"]
    theta, emb = T.init_params(shape, cfg, 5)
    m = StafModel(shape, res["geo"], theta, emb, 2, dtype=torch.float32, device="cuda:0")
    lr_of = T.build_learning_rate(cfg["lr_dense_net"], 2, 2, 4)
    f32 = lambda a: np.ascontiguousarray(a, np.float32)
    step = 0
    for ep in range(2):
        for b in range(2):
            for k in range(2):
                sl = slice(4 * b + 2 * k, 4 * b + 2 * k + 2)
                l = m.loss_and_grad_host(f32(pos[sl]), f32(box[sl]), f32(el[sl]), f32(fl[sl]))
                m.adam_update_dev(lr_of(step))
                r = rows[step]
                assert r[5] == pytest.approx(lr_of(step))
                assert np.allclose([r[1], r[2], r[4], r[3]], l, rtol=2e-5), (step, r, l)
                step += 1
    torch.cuda.synchronize()
    assert np.allclose(res["theta"], m.theta.cpu().numpy(), rtol=1e-4, atol=1e-6)
    assert rows[-1][1] < rows[0][1]   # the loss went down
    m.close()
