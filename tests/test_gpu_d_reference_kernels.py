"""Operator arithmetic against the reference's OWN kernels: the fused kernels its fuser generated
(tests/benchmark/cuda/*_{b,h}fuse.cu of the reference, compiled for sm_100a by baseline/Makefile into
baseline/_ref/*.cubin) are launched on the GPU on seeded inputs and this runtime's operators must
reproduce their outputs -- all five pairs the reference's output exists for, both of its fusion
flavours: the CUDA-core fp32 bodies within 1e-5 (same arithmetic, different summation order), the
tcgen05 tf32 bodies within 5e-3, by the rule stated in tests/pair_oracle.py.  Skipped where the
cubins were not built (they need a reference checkout at build time)."""
import os
import sys

import pytest

import bfuse_project_b200 as bf
from pair_oracle import within

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))
import ref_fuser  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    r = bf.Runtime(0)
    yield r
    r.close()


def reference_outputs(name, seed):
    """Seeded U(-0.5, 0.5) inputs (the reference's rand_tensor) and the outputs of the reference's
    bfuse and hfuse kernels on them."""
    import torch
    if name not in ref_fuser.available():
        pytest.skip("baseline/_ref cubins not built")
    torch.manual_seed(seed)
    sh1, sh2 = ref_fuser.shapes(name)
    bufs = [(torch.rand(*s, device="cuda") - 0.5) for s in sh1 + sh2]
    ptrs = [b.data_ptr() for b in bufs]
    stream = torch.cuda.current_stream().cuda_stream
    out = {}
    for flavour in ("bfuse", "hfuse"):
        bufs[2].zero_(), bufs[5].zero_()
        ref_fuser.RefKernel(name, flavour).launch(ptrs, stream)
        torch.cuda.synchronize()
        out[flavour] = (bufs[2].clone(), bufs[5].clone())
    # the reference's two fusion flavours run the same two bodies: same bits
    assert all(torch.equal(a, b) for a, b in zip(out["bfuse"], out["hfuse"])), "reference bfuse != hfuse"
    del out["hfuse"]
    return bufs, ptrs, stream, out["bfuse"]


@pytest.mark.parametrize("name", ["dense1_0_dense2_0", "dense1_5_dense2_5", "dense1_6_dense2_6", "bgemm1_0_bgemm2_0"])
def test_gemm_pairs_match_the_reference_fused_kernels(rt, name):
    import torch
    bufs, ptrs, stream, ref = reference_outputs(name, 3)
    cfg = ref_fuser.PAIRS[name]
    batch = cfg.get("b", 1)
    for op, tol in ((bf.OP_GEMM_F32_SIMT, 1e-5), (bf.OP_GEMM_TF32, 5e-3)):
        shape = (batch, cfg["M"], cfg["N"], cfg["K"]) + ((0, 0) if op == bf.OP_GEMM_TF32 else ())
        ks = [rt.register_kernel(rt.describe("g%d" % i, op, shape, [ptrs[3 * i], ptrs[3 * i + 1], None, ptrs[3 * i + 2]])) for i in range(2)]
        for pattern in (bf.ZIGZAG, bf.RANGE_SPLIT):
            mn = 1 if pattern == bf.ZIGZAG else 0
            bufs[2].zero_(), bufs[5].zero_()
            f = rt.register_fusion(ks[0], ks[1], pattern, mn, mn)
            rt.launch_fused(f, stream)
            torch.cuda.synchronize()
            assert rt.read_status() == 0
            for got, want in ((bufs[2], ref[0]), (bufs[5], ref[1])):
                ok, worst = within(got, want, tol)
                assert ok, (name, op, bf.PATTERN_NAMES[pattern], worst)
            # and the reference's own acceptance rule (check_matrix, eps 1e-3) holds for the fp32 bodies
            if op == bf.OP_GEMM_F32_SIMT and bufs[2].numel() <= 1 << 24:
                assert bf.check_matrix(bufs[2].cpu().numpy(), ref[0].cpu().numpy()) == 0
            rt.unregister_fusion(f)
        for k in ks:
            rt.unregister_kernel(k)


def test_conv_pair_matches_the_reference_fused_kernels(rt):
    import torch
    name = "conv2d1_3_conv2d2_5"
    bufs, ptrs, stream, ref = reference_outputs(name, 4)
    cfg = ref_fuser.PAIRS[name]
    shapes = [(cfg["n"], cfg["ci"], cfg["h"], cfg["w"], cfg["co"], kk, kk, cfg["stride"], pp) for kk, pp in zip(cfg["k"], cfg["pad"])]
    for op, tol in ((bf.OP_CONV2D_F32_SIMT, 1e-5), (bf.OP_CONV2D_TF32, 5e-3)):
        ks = [rt.register_kernel(rt.describe("c%d" % i, op, shapes[i], [ptrs[3 * i], ptrs[3 * i + 1], ptrs[3 * i + 2]])) for i in range(2)]
        bufs[2].zero_(), bufs[5].zero_()
        rt.launch_fused(rt.register_fusion(ks[0], ks[1], bf.ZIGZAG, 1, 1), stream)
        torch.cuda.synchronize()
        assert rt.read_status() == 0
        for got, want in ((bufs[2], ref[0]), (bufs[5], ref[1])):
            ok, worst = within(got, want, tol)
            assert ok, (op, worst)
