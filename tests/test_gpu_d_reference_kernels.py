"""Operator arithmetic against the reference's OWN kernels: the fused kernels its fuser generated
(tests/benchmark/cuda/*_bfuse.cu of the reference, compiled for sm_100a by baseline/Makefile into
baseline/_ref/*.cubin) are launched on the GPU on seeded inputs and this runtime's operators must
reproduce their outputs: the CUDA-core fp32 bodies within 1e-5 (same arithmetic, different
summation order), the tcgen05 tf32 bodies within 5e-3.  Skipped where the cubins were not built
(they need a reference checkout at build time)."""
import os
import sys

import numpy as np
import pytest

import bfuse_project_b200 as bf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import ref_fuser  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    r = bf.Runtime(0)
    yield r
    r.close()


def _close(got, ref, tol):
    rms = float(ref.double().pow(2).mean().sqrt())
    return float(((got - ref).abs() - tol * ref.abs()).max()) <= tol * rms


@pytest.mark.parametrize("name", ["dense1_0_dense2_0", "dense1_5_dense2_5"])
def test_dense_pairs_match_the_reference_fused_kernel(rt, name):
    import torch
    if name not in ref_fuser.available():
        pytest.skip("baseline/_ref cubins not built")
    torch.manual_seed(3)
    cfg = ref_fuser.PAIRS[name]
    sh1, sh2 = ref_fuser.shapes(name)
    bufs = [(torch.rand(*s, device="cuda") - 0.5) for s in sh1 + sh2]   # U(-0.5, 0.5) as the reference's rand_tensor
    ptrs = [b.data_ptr() for b in bufs]
    stream = torch.cuda.current_stream().cuda_stream
    ref_out = {}
    for flavour in ("bfuse", "hfuse"):
        bufs[2].zero_(), bufs[5].zero_()
        ref_fuser.RefKernel(name, flavour).launch(ptrs, stream)
        torch.cuda.synchronize()
        ref_out[flavour] = (bufs[2].clone(), bufs[5].clone())
    # the reference's two fusion flavours agree with each other bit for bit
    assert all(torch.equal(a, b) for a, b in zip(ref_out["bfuse"], ref_out["hfuse"]))
    for op, tol in ((bf.OP_GEMM_F32_SIMT, 1e-5), (bf.OP_GEMM_TF32, 5e-3)):
        shape = (1, cfg["M"], cfg["N"], cfg["K"]) + ((0, 0) if op == bf.OP_GEMM_TF32 else ())
        ks = [rt.register_kernel(rt.describe("g%d" % i, op, shape, [ptrs[3 * i], ptrs[3 * i + 1], None, ptrs[3 * i + 2]])) for i in range(2)]
        for pattern in (bf.ZIGZAG, bf.RANGE_SPLIT):
            bufs[2].zero_(), bufs[5].zero_()
            rt.launch_fused(rt.register_fusion(ks[0], ks[1], pattern, 1 if pattern == bf.ZIGZAG else 0, 1 if pattern == bf.ZIGZAG else 0), stream)
            torch.cuda.synchronize()
            assert rt.read_status() == 0
            assert _close(bufs[2], ref_out["bfuse"][0], tol) and _close(bufs[5], ref_out["bfuse"][1], tol), (op, pattern)
            # and the reference's own acceptance rule (check_matrix, eps 1e-3) holds for the fp32 bodies
            if op == bf.OP_GEMM_F32_SIMT:
                assert bf.check_matrix(bufs[2].cpu().numpy(), ref_out["bfuse"][0].cpu().numpy()) == 0


def test_conv_pair_matches_the_reference_fused_kernel(rt):
    import torch
    name = "conv2d1_3_conv2d2_5"
    if name not in ref_fuser.available():
        pytest.skip("baseline/_ref cubins not built")
    torch.manual_seed(4)
    cfg = ref_fuser.PAIRS[name]
    sh1, sh2 = ref_fuser.shapes(name)
    bufs = [(torch.rand(*s, device="cuda") - 0.5) for s in sh1 + sh2]
    ptrs = [b.data_ptr() for b in bufs]
    stream = torch.cuda.current_stream().cuda_stream
    ref_fuser.RefKernel(name, "bfuse").launch(ptrs, stream)
    torch.cuda.synchronize()
    ref_out = (bufs[2].clone(), bufs[5].clone())
    shapes = [(cfg["n"], cfg["ci"], cfg["h"], cfg["w"], cfg["co"], kk, kk, cfg["stride"], pp) for kk, pp in zip(cfg["k"], cfg["pad"])]
    ks = [rt.register_kernel(rt.describe("c%d" % i, bf.OP_CONV2D_TF32, shapes[i], [ptrs[3 * i], ptrs[3 * i + 1], ptrs[3 * i + 2]])) for i in range(2)]
    bufs[2].zero_(), bufs[5].zero_()
    rt.launch_fused(rt.register_fusion(ks[0], ks[1], bf.ZIGZAG, 1, 1), stream)
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert _close(bufs[2], ref_out[0], 5e-3) and _close(bufs[5], ref_out[1], 5e-3)
