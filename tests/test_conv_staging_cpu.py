"""The staged im2col of the tensor-core conv body, replayed on the CPU: with the geometry the library
reports (bfuse_debug_conv_staging), a raw slot filled the way the TMA fills it (rows y0 + j * ey, columns
x_start + i, zeros outside the image) and the body's offset rule (pixel origin + per-k table entry, the
slot of a chunk of four k found by the body's comparisons) must deliver exactly the im2col element of
every (pixel, k) -- for every tile of the image, including tiles that start in the middle of an output
row, padded borders and strided one-row windows."""
import ctypes as C

import numpy as np
import pytest

import bfuse_project_b200 as bf

NAMES = ("slots", "cc", "rows", "pitch", "ex", "ey", "step_x", "step_y", "x_start", "x_off", "slot_bytes", "slot_pitch", "tile_px")


def staging(shape, bn):
    fn = bf.lib().bfuse_debug_conv_staging
    fn.argtypes = [C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.c_int]
    fn.restype = C.c_int
    out = (C.c_int * 13)()
    assert fn((C.c_int * 9)(*shape), bn, out, 13) == 0
    return dict(zip(NAMES, out))


CASES = [((1, 64, 56, 56, 128, 3, 3, 2, 1), 128), ((1, 64, 56, 56, 128, 1, 1, 2, 0), 128), ((1, 32, 56, 56, 128, 3, 3, 2, 1), 128),
         ((1, 32, 20, 20, 200, 3, 3, 1, 1), 128), ((1, 96, 31, 16, 40, 1, 1, 2, 0), 128), ((1, 32, 12, 12, 130, 5, 5, 3, 2), 128),
         ((1, 32, 28, 28, 128, 3, 3, 1, 1), 128), ((1, 32, 9, 24, 16, 1, 3, 2, 1), 128), ((1, 32, 16, 8, 16, 3, 1, 1, 1), 128),
         ((1, 8, 14, 12, 16, 2, 2, 2, 0), 128), ((1, 32, 5, 160, 16, 3, 3, 1, 1), 128), ((1, 32, 6, 200, 16, 3, 3, 2, 1), 128)]


@pytest.mark.parametrize("shape,bn", CASES)
def test_staged_operand_equals_im2col(shape, bn):
    n, ci, h, w, co, kh, kw, stride, pad = shape
    st = staging(shape, bn)
    assert st["slots"] == 3 and st["ex"] == 1 and st["pitch"] % 4 == 0 and st["x_start"] % 4 == 0 and st["cc"] % 4 == 0
    assert st["slot_bytes"] == st["cc"] * st["rows"] * st["pitch"] * 4 and st["slot_pitch"] % 128 == 0
    assert st["pitch"] * st["ex"] <= 256 and st["rows"] * st["ey"] <= 256
    oh, ow = (h + 2 * pad - kh) // stride + 1, (w + 2 * pad - kw) // stride + 1
    rng = np.random.default_rng(1)
    x = rng.standard_normal((ci, h, w)).astype(np.float32)
    K, khw, kslot = ci * kh * kw, kh * kw, st["cc"] * kh * kw
    plane = st["rows"] * st["pitch"]
    # the per-k table of the body: (channel within its slot, dy, dx) as an offset inside a slot
    k = np.arange(K)
    ch, t = k // khw, k % khw
    tab = (ch % st["cc"]) * plane + (t // kw) * st["pitch"] + t % kw
    # tiles of whole output rows wherever they fill at least three quarters of the 128 lanes
    tile = st["tile_px"]
    assert tile == ((bn // ow) * ow if ow <= bn and (bn // ow) * ow >= bn - bn // 4 else bn)
    for px0 in range(0, oh * ow, tile):
        oy0 = px0 // ow
        y0 = oy0 * stride - pad
        # every slot of the tile as the TMA delivers it
        slots = []
        for g in range((K - 1) // kslot + 1):
            raw = np.zeros((st["cc"], st["rows"], st["pitch"]), np.float32)
            for cl in range(st["cc"]):
                c = g * st["cc"] + cl
                for j in range(st["rows"]):
                    y = y0 + j * st["ey"]
                    for i in range(st["pitch"]):
                        xx = st["x_start"] + i * st["ex"]
                        if c < ci and 0 <= y < h and 0 <= xx < w:
                            raw[cl, j, i] = x[c, y, xx]
            slots.append(raw.reshape(-1))
        # which slot the body reads each chunk of four k from: K block kb starts `kin` values of k into ring
        # position `first`; chunk i reads the next slot from j1 on, the one after from j2 on
        slot_of = np.zeros(K, np.int64)
        kin, first = 0, 0
        for kb in range(K // 32):
            j1 = (kslot - kin) >> 2
            j2 = j1 + (kslot >> 2)
            for i in range(8):
                slot_of[kb * 32 + 4 * i: kb * 32 + 4 * i + 4] = first + (2 if i >= j2 else 1 if i >= j1 else 0)
            passed = int(kin + 32 >= kslot) + int(kin + 32 >= 2 * kslot)
            kin += 32 - passed * kslot
            first += passed
            assert 0 <= kin < kslot
        assert np.array_equal(slot_of, np.arange(K) // kslot)
        for pix in range(px0, min(px0 + tile, oh * ow)):
            oy, ox = divmod(pix, ow)
            pixoff = (oy - oy0) * st["step_y"] * st["pitch"] + ox * st["step_x"] + st["x_off"]
            assert 0 <= pixoff and pixoff + tab.max() < st["cc"] * plane
            got = np.array([slots[slot_of[kk]][pixoff + tab[kk]] for kk in range(K)])
            want = np.zeros(K, np.float32)
            for kk in range(K):
                c, dy, dx = kk // khw, (kk % khw) // kw, kk % kw
                yy, xx = oy * stride + dy - pad, ox * stride + dx - pad
                if 0 <= yy < h and 0 <= xx < w:
                    want[kk] = x[c, yy, xx]
            assert np.array_equal(got, want), (px0, pix)


def test_what_cannot_be_staged():
    assert staging((1, 256, 35, 35, 64, 1, 1, 1, 0), 128)["slots"] == 0      # 35 floats per row: no 16-byte multiple
    assert staging((1, 512, 7, 7, 512, 3, 3, 1, 1), 32)["slots"] == 0
    assert staging((1, 64, 56, 56, 128, 3, 3, 2, 1), 64)["slots"] == 0       # the tile is the 128 lanes of tensor memory
    assert staging((1, 12, 20, 20, 200, 3, 3, 1, 1), 128)["slots"] == 0      # K = 108: no whole number of K blocks
    assert staging((1, 64, 56, 56, 128, 3, 3, 2, 1), 128)["slots"] == 3
