"""Launch the reference fuser's generated kernels (compiled by baseline/Makefile into
baseline/_ref/*.cubin) on the GPU, for bench.py's "reference fuser output" baseline.

The kernels exist only at the reference suite's batch-1024 fp32 shapes
(tests/benchmark/config/kernels.yaml of the reference); launch dims are the fused dims its fuser
wrote to {b,h}fuse_kernels.yaml: bfuse grid = G1 + G2, block = 128; hfuse grid = max(G), block = 256.
Arguments are (A1, B1, out1, A2, B2, out2) as float32 device buffers.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# pair -> (kernel-1 shapes, kernel-2 shapes, unfused grids, our operator description)
#   dense:  A[M,K], B[N,K], out[M,N]           grid (M/32, N/64)
#   bgemm:  A[b,M,K], B[b,N,K], out[b,M,N]     grid (M/32, b*N/64)
#   conv:   data[n,ci,h,w], weight[co,ci,kh,kw], out[n,co,oh,ow]   grid (n*oh*ow/32, co/64)
PAIRS = {
    "dense1_0_dense2_0": dict(kind="dense", M=1024, N=768, K=768, grids=(384, 384)),
    "dense1_5_dense2_5": dict(kind="dense", M=1024, N=1024, K=4096, grids=(512, 512)),
    "dense1_6_dense2_6": dict(kind="dense", M=1024, N=14336, K=4096, grids=(7168, 7168)),
    "bgemm1_0_bgemm2_0": dict(kind="bgemm", b=1024, M=512, N=512, K=64, grids=(131072, 131072)),
    "conv2d1_3_conv2d2_5": dict(kind="conv", n=1024, ci=64, h=56, w=56, co=128, k=(3, 1), stride=2, pad=(1, 0),
                                grids=(50176, 50176)),
}


def shapes(name):
    p = PAIRS[name]
    if p["kind"] == "dense":
        s = [(p["M"], p["K"]), (p["N"], p["K"]), (p["M"], p["N"])]
        return s, s
    if p["kind"] == "bgemm":
        s = [(p["b"], p["M"], p["K"]), (p["b"], p["N"], p["K"]), (p["b"], p["M"], p["N"])]
        return s, s
    out = []
    for k, pad in zip(p["k"], p["pad"]):
        o = (p["h"] + 2 * pad - k) // p["stride"] + 1
        out.append([(p["n"], p["ci"], p["h"], p["w"]), (p["co"], p["ci"], k, k), (p["n"], p["co"], o, o)])
    return out[0], out[1]


def available():
    return [n for n in PAIRS if os.path.exists(os.path.join(HERE, "_ref", n + "_bfuse.cubin"))]


class RefKernel:
    def __init__(self, name, flavour):
        from cuda.bindings import driver
        self.drv = driver
        path = os.path.join(HERE, "_ref", "%s_%s.cubin" % (name, flavour))
        data = open(path, "rb").read()
        err, self.mod = driver.cuModuleLoadData(data)
        assert err == driver.CUresult.CUDA_SUCCESS, err
        err, self.fn = driver.cuModuleGetFunction(self.mod, ("%s_fused_%s" % (name, flavour)).encode())
        assert err == driver.CUresult.CUDA_SUCCESS, err
        g1, g2 = PAIRS[name]["grids"]
        self.grid = g1 + g2 if flavour == "bfuse" else max(g1, g2)
        self.block = 128 if flavour == "bfuse" else 256

    def launch(self, ptrs, stream):
        args = (ctypes.c_void_p * 6)(*ptrs)
        arg_ptrs = (ctypes.c_void_p * 6)(*[ctypes.addressof(args) + 8 * i for i in range(6)])
        (err,) = self.drv.cuLaunchKernel(self.fn, self.grid, 1, 1, self.block, 1, 1, 0, stream, ctypes.addressof(arg_ptrs), 0)
        assert err == self.drv.CUresult.CUDA_SUCCESS, err
