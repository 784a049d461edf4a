"""GPU test of stafb_compute_descriptors_light_noalloc, the descriptor entry point for callers that
cannot allocate device memory (op callbacks running under a framework-owned allocator, plug-ins entered
while the allocator is locked, fixed-budget processes).  It must give the same tensors as the regular
entry point, which takes its scratch from cudaMalloc, on two calls in a row that share the built-in
scratch array - the second call uses a different, smaller system so that stale contents would show.
Collected last on purpose (file name), and written to pass both alone and after the other tests."""
import ctypes as C

import numpy as np
import pytest

from alphanesgpu_b200 import synth

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

RC, RS, RA, NR, NA = 4.5, 2.25, 4.5, 60, 1770


def _noalloc(L, pos, box, tdt, NR=NR, NA=NA):
    nf, N = box.shape[0], pos.shape[1] // 3
    dev = pos.device
    e = lambda *s, d=tdt: torch.full(s, -7, dtype=d, device=dev)  # poison: every element must be written
    out = [e(nf, N, NR), e(nf, N, NA), e(nf, N, NR), e(nf, N, NR + 1, d=torch.int32),
           e(nf, N, 2 * NA, d=torch.int32), e(nf, N, 3, NR), e(nf, N, 3, 2 * NA), e(nf, N, 3, NR),
           e(nf, N, d=torch.int32)]
    status = torch.full((1,), -1, dtype=torch.int32, device=dev)
    p = lambda t: C.c_void_p(t.data_ptr())
    fn = L.stafb_compute_descriptors_light_noalloc
    fn.argtypes = [C.c_int, C.c_double, C.c_double, C.c_double, C.c_int, C.c_int] + [C.c_void_p] * 3 + \
                  [C.c_int, C.c_int] + [C.c_void_p] * 10
    rc = fn(0 if tdt == torch.float32 else 1, RC, RS, RA, NR, NA,
            C.c_void_p(torch.cuda.current_stream().cuda_stream), p(pos), p(box), nf, N, *[p(t) for t in out],
            p(status))
    torch.cuda.synchronize()
    return rc, out, int(status.item())


@pytest.mark.parametrize("tdt", [torch.float32, torch.float64])
def test_noalloc_matches_regular_entry_point_twice_in_a_row(tdt):
    from alphanesgpu_b200 import _lib, ops
    L = _lib.lib()
    ndt = np.float32 if tdt == torch.float32 else np.float64
    cases = [synth.water_frames("water768", [1100]), synth.water_frames("water96", [1000, 1001, 1002])]
    for pos, box, tipos in cases:  # two calls in a row on the shared scratch
        dpos = torch.as_tensor(pos.astype(ndt)).cuda()
        dbox = torch.as_tensor(box.astype(ndt)).cuda()
        rc, got, status = _noalloc(L, dpos, dbox, tdt)
        assert rc == 0 and status == 0
        ops.construct_descriptors_light(RC, NR, NA, pos.shape[1] // 3, None, RS, RA, box.shape[0], dtype=tdt)
        ref = ops.compute_descriptors_light(dpos, dbox)
        for g, r in zip(got, ref):
            assert torch.equal(g, r)  # same kernels, same arithmetic: identical bits


def test_noalloc_rejects_sizes_beyond_the_builtin_scratch():
    from alphanesgpu_b200 import _lib
    L = _lib.lib()
    L.stafb_noalloc_scratch_bytes.restype = C.c_size_t
    assert 1 << 20 < L.stafb_noalloc_scratch_bytes() < 8 << 20
    pos, box, _ = synth.water_frames("water768", [1100, 1101])  # 1536 atoms > 1024
    dpos = torch.as_tensor(pos.astype(np.float32)).cuda()
    dbox = torch.as_tensor(box.astype(np.float32)).cuda()
    rc, _, _ = _noalloc(L, dpos, dbox, torch.float32)
    assert rc == 7  # STAFB_ERR_CAPACITY
    # a saturated radial buffer is reported through the status word, as with the regular entry point
    pos, box, _ = synth.water_frames("water96", [1000])
    dpos = torch.as_tensor((pos * 0.6).astype(np.float32)).cuda()
    dbox = torch.as_tensor((box * 0.6).astype(np.float32)).cuda()
    rc, _, status = _noalloc(L, dpos, dbox, torch.float32)
    assert rc == 0 and status == 1


def test_noalloc_at_the_edge_of_the_builtin_scratch():
    """The largest request the built-in scratch takes in every dimension at once: 16 frames x 64 atoms = 1024
    atoms, radial_buffer 64, float64 (the widest rows)."""
    from alphanesgpu_b200 import _lib, ops
    L = _lib.lib()
    nr, na = 64, 64 * 63 // 2
    pos, box, _ = synth.water_frames("water96", list(range(1300, 1316)))
    pos = np.ascontiguousarray(pos.reshape(16, 96, 3)[:, :64].reshape(16, -1))  # any 64 atoms of each frame
    dpos, dbox = torch.as_tensor(pos).cuda(), torch.as_tensor(box).cuda()
    rc, got, status = _noalloc(L, dpos, dbox, torch.float64, nr, na)
    assert rc == 0 and status == 0
    ops.construct_descriptors_light(RC, nr, na, 64, None, RS, RA, 16, dtype=torch.float64)
    ref = ops.compute_descriptors_light(dpos, dbox)
    for g, r in zip(got, ref):
        assert torch.equal(g, r)
    # one more frame, one more atom or a wider row is refused
    rc, _, _ = _noalloc(L, torch.cat([dpos, dpos[:1]]), torch.cat([dbox, dbox[:1]]), torch.float64, nr, na)
    assert rc == 7
    rc, _, _ = _noalloc(L, dpos, dbox, torch.float64, 65, 65 * 64 // 2)
    assert rc == 7
