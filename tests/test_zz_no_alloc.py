"""The allocation-free entry point (bfuse_softmax_layernorm_queue_noalloc) against the regular
registered work-queue path.

Some callers cannot allocate device memory at launch time -- their process has given all of it to a
pool, or they sit in a latency-critical loop where cudaMalloc / cudaFree would stall the device --
so the library offers this one launch whose queue counters live in a static device array.  The
test calls it through the C ABI twice in a row (the array is shared between calls and keeps what
the previous call left, so the second call proves the counters are cleared) and requires the
outputs to equal the registered path's bit for bit, the tolerance every fused-vs-unfused check in
this suite uses.  A third case has more queue tickets than resident CTAs, so the persistent part of the
queue (a CTA drawing several tickets) runs too, and device memory in use is compared before and after a
warm call: the entry point's purpose is that it allocates none.  Problems beyond the documented ticket
limit must be refused.
"""
import ctypes as C

import numpy as np
import pytest

import bfuse_project_b200 as bf
from bfuse_project_b200 import workloads as wl

pytestmark = pytest.mark.gpu


def _noalloc_fn():
    L = bf.lib()
    fn = L.bfuse_softmax_layernorm_queue_noalloc
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    fn.argtypes = [vp, vp, i, i, f, vp, vp, vp, vp, vp, i, i, f, vp]
    fn.restype = C.c_int
    return fn


def test_noalloc_matches_registered_work_queue_twice_in_a_row():
    import torch
    fn = _noalloc_fn()
    rt = bf.Runtime(0)
    try:
        for call, seed in enumerate((21, 22)):
            # second call: other data and a residual, ragged row counts
            rows = 12 * 128 + (5 if call else 0)
            rng = np.random.default_rng(seed)
            a = wl.softmax("softmax", rng, rows, 512, 0.125)
            b = wl.layernorm("layernorm", rng, 128 + (3 if call else 0), 768, 1e-5, residual=bool(call))
            spec = wl.PairSpec("noalloc", a, b, "f32", "hbm")
            pair = wl.DevicePair(rt, spec)
            pair.clear_outputs()
            rt.launch_fused(pair.fusion(bf.WORK_QUEUE, 1, 1))
            want = pair.read_outputs()

            pair.clear_outputs()
            torch.cuda.synchronize()
            ba, bb = pair.buffers
            rc = fn(ba[0].data_ptr(), ba[1].data_ptr(), a.shape[0], a.shape[1], a.fparam[0],
                    bb[0].data_ptr(), None if bb[1] is None else bb[1].data_ptr(), bb[2].data_ptr(), bb[3].data_ptr(),
                    bb[4].data_ptr(), b.shape[0], b.shape[1], b.fparam[0], None)
            assert rc == 0
            got = pair.read_outputs()
            for k in range(2):
                assert np.array_equal(got[k][0].view(np.uint8), want[k][0].view(np.uint8)), (call, k)
            assert np.abs(got[0][0].sum(1) - 1.0).max() < 1e-5
    finally:
        rt.close()


def test_noalloc_persistent_queue_and_no_device_allocation():
    """16384 softmax rows (2048 tickets, more than the resident grid) beside a LayerNorm: every CTA draws
    several tickets.  Same bits as the registered work-queue path, and a warm call leaves the amount of
    free device memory exactly where it was."""
    import torch
    fn = _noalloc_fn()
    rt = bf.Runtime(0)
    try:
        rng = np.random.default_rng(23)
        a = wl.softmax("softmax", rng, 16384, 512, 0.125)
        b = wl.layernorm("layernorm", rng, 2051, 768, 1e-5, residual=True)
        pair = wl.DevicePair(rt, wl.PairSpec("noalloc_persistent", a, b, "f32", "hbm"))
        fusion = pair.fusion(bf.WORK_QUEUE, 1, 1)
        info = rt.fusion_info(fusion)
        assert info["launched_ctas"] < info["GridDim"][0], "the case must have more tickets than launched CTAs"
        pair.clear_outputs()
        rt.launch_fused(fusion)
        want = pair.read_outputs()
        ba, bb = pair.buffers
        args = (ba[0].data_ptr(), ba[1].data_ptr(), a.shape[0], a.shape[1], a.fparam[0],
                bb[0].data_ptr(), bb[1].data_ptr(), bb[2].data_ptr(), bb[3].data_ptr(),
                bb[4].data_ptr(), b.shape[0], b.shape[1], b.fparam[0], None)
        pair.clear_outputs()
        assert fn(*args) == 0                      # may be this device's first call (one-time set-up)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        for _ in range(3):
            assert fn(*args) == 0                  # warm calls
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "a warm call changed the device memory in use"
        got = pair.read_outputs()
        for k in range(2):
            assert np.array_equal(got[k][0].view(np.uint8), want[k][0].view(np.uint8)), k
    finally:
        rt.close()


def test_noalloc_rejects_oversized_and_malformed_problems():
    import torch
    fn = _noalloc_fn()
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    # 8 rows per CTA at 512 columns: 9M rows would need more than 2^20 tickets
    assert fn(p, p, 9_000_000, 512, 1.0, p, None, p, p, p, 8, 768, 1e-5, None) == 2
    assert fn(p, p, 8, 30, 1.0, p, None, p, p, p, 8, 768, 1e-5, None) == 2       # cols not vectorisable
    assert fn(p, None, 8, 512, 1.0, p, None, p, p, p, 8, 768, 1e-5, None) == 1   # missing output
    assert fn(p + 4, p, 8, 512, 1.0, p, None, p, p, p, 8, 768, 1e-5, None) == 1  # misaligned input
    torch.cuda.synchronize()
