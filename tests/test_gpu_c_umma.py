"""Parity of the tcgen05 GEMM bodies (tf32 and bf16) and of the pairs built on them."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
from bfuse_project_b200 import workloads as wl
from pair_oracle import check_against_oracle
from test_gpu_b_pairs import BLOCK_PATTERNS, check_retiled, run_and_check

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    r = bf.Runtime(0)
    yield r
    r.close()


def test_single_tf32_tile(rt):
    rng = np.random.default_rng(1)
    a = wl.gemm("g1", rng, bf.OP_GEMM_TF32, 1, 128, 64, 32, w_std=1.0, bn=64, split=1)       # one tile, one K block
    b = wl.gemm("g2", rng, bf.OP_GEMM_TF32, 1, 128, 128, 256, bias=True, w_std=1.0, bn=128, split=1)
    run_and_check(rt, wl.PairSpec("tile", a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1)])


def test_single_bf16_tile(rt):
    rng = np.random.default_rng(2)
    a = wl.gemm("g1", rng, bf.OP_GEMM_BF16, 1, 128, 32, 64, w_std=1.0, bn=64, split=1)
    b = wl.gemm("g2", rng, bf.OP_GEMM_BF16, 1, 256, 256, 512, w_std=0.05, bn=256, split=1)
    run_and_check(rt, wl.PairSpec("tile16", a, b, "bf16", "tensor"), [(bf.ZIGZAG, 1, 1)])


def test_ragged_umma_shapes(rt):
    rng = np.random.default_rng(3)
    # M, N not multiples of the tile; K not a multiple of the K block; batch > 1; causal with M != N
    a = wl.gemm("g1", rng, bf.OP_GEMM_TF32, 3, 200, 72, 40, bias=True, w_std=1.0, bn=32, split=1)
    b = wl.gemm("g2", rng, bf.OP_GEMM_TF32, 2, 130, 260, 100, causal=True, w_std=1.0, bn=64, split=1)
    run_and_check(rt, wl.PairSpec("ragged_tf32", a, b, "tf32", "hbm"), BLOCK_PATTERNS)
    c = wl.gemm("g3", rng, bf.OP_GEMM_BF16, 2, 100, 136, 72, w_std=0.1, bn=64, split=1)
    d = wl.gemm("g4", rng, bf.OP_GEMM_BF16, 1, 384, 96, 1000, w_std=0.05, bn=64, split=1)
    run_and_check(rt, wl.PairSpec("ragged_bf16", c, d, "bf16", "tensor"), BLOCK_PATTERNS)


def test_tall_tiles_share_the_w_tile(rt):
    """256-row tiles (two accumulators, one W tile per k-step): ragged M and N, bias, causal mask, both
    operand kinds, beside a 128-row partner; fused == unfused bit for bit, oracle within tolerance."""
    rng = np.random.default_rng(77)
    a = wl.gemm("t1", rng, bf.OP_GEMM_TF32, 2, 300, 520, 200, bias=True, w_std=1.0, bn=256, split=1, bm=256)
    b = wl.gemm("t2", rng, bf.OP_GEMM_TF32, 1, 512, 512, 96, causal=True, w_std=1.0, bn=128, split=1, bm=256)
    run_and_check(rt, wl.PairSpec("tall_tf32", a, b, "tf32", "hbm"), BLOCK_PATTERNS)
    c = wl.gemm("t3", rng, bf.OP_GEMM_BF16, 1, 640, 768, 1024, w_std=0.05, bn=256, split=1, bm=256)
    d = wl.gemm("t4", rng, bf.OP_GEMM_BF16, 1, 130, 136, 72, w_std=0.1, bn=64, split=1, bm=128)
    pair = run_and_check(rt, wl.PairSpec("tall_bf16", c, d, "bf16", "tensor"), BLOCK_PATTERNS)
    # two operators of 512 and 64 tensor-memory columns cannot share one CTA
    with pytest.raises(bf.BfuseError) as e:
        pair.fusion(bf.THREAD_SPLIT, 1, 1)
    assert e.value.code == 7


@pytest.mark.parametrize("kind", ["tf32", "bf16"])
def test_split_k_cluster_reduction(rt, kind):
    """k-slices of a tile reduced over distributed shared memory: every split width, ragged M / N,
    uneven k-slices, bias and causal mask; unsplit and split results agree within the oracle tolerance
    and fused == unfused bit for bit."""
    rng = np.random.default_rng(40)
    op = bf.OP_GEMM_TF32 if kind == "tf32" else bf.OP_GEMM_BF16
    bk = 32 if kind == "tf32" else 64
    std = 1.0 if kind == "tf32" else 0.05
    cases = {"tf32": ((2, 256, 256, 512, 4), (3, 128, 200, 264, 7), (4, 256, 128, 768, 24), (6, 128, 512, 768, 24),
                      (8, 256, 256, 520, 24), (8, 64, 130, 72, 19), (5, 32, 128, 32, 5)),
             "bf16": ((2, 256, 256, 512, 4), (3, 128, 200, 264, 7), (4, 256, 128, 768, 24), (5, 128, 512, 768, 24),
                      (4, 64, 130, 72, 19), (5, 64, 128, 64, 5))}[kind]
    for split, bn, M, N, kblocks in cases:
        K = kblocks * bk - (8 if kind == "tf32" and split == 3 else 0)
        a = wl.gemm("g1", rng, op, 1, M, N, K, bias=(kind == "tf32"), w_std=std, bn=bn, split=split)
        b = wl.gemm("g2", rng, op, 2 if split == 2 else 1, M, N, K, causal=(kind == "tf32" and split in (3, 4)),
                    w_std=std, bn=bn, split=split)
        run_and_check(rt, wl.PairSpec("split%d" % split, a, b, kind, "hbm"),
                      [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0), (bf.SM_STRIPED, 0, 0), (bf.PROPORTIONAL, 1, 0)])


def test_split_gemm_with_unsplit_partner_and_unsupported_patterns(rt):
    rng = np.random.default_rng(41)
    a = wl.gemm("g1", rng, bf.OP_GEMM_TF32, 1, 256, 256, 256, w_std=1.0, bn=256, split=4)
    b = wl.layernorm("ln", rng, 100, 768, 1e-5, residual=True)   # 25 CTAs: clusters of 4 get padding CTAs
    pair = run_and_check(rt, wl.PairSpec("split_ln", a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])
    assert rt.fusion_info(pair.fusion(bf.ZIGZAG, 1, 1))["retiled_unsplit"] == (False, False)
    for pat in (bf.THREAD_SPLIT, bf.WORK_QUEUE):   # no clusters there: the GEMM runs with one k-slice instead
        check_retiled(rt, pair, pat)
    c = wl.gemm("g3", rng, bf.OP_GEMM_TF32, 1, 256, 256, 256, w_std=1.0, bn=256, split=2)
    mixed = wl.DevicePair(rt, wl.PairSpec("mixed", a, c, "tf32", "hbm"))
    with pytest.raises(bf.BfuseError) as e:   # different cluster widths cannot share a launch
        mixed.fusion(bf.ZIGZAG, 1, 1)
    assert e.value.code == 7


def test_pipeline_depths(rt):
    rng = np.random.default_rng(4)
    for smem_stages in (1, 2, 3, 6):
        a = wl.gemm("g1", rng, bf.OP_GEMM_TF32, 1, 128, 64, 512, w_std=1.0, bn=64, split=1)
        a.smem = 2048 + smem_stages * (16384 + 64 * 128)
        b = wl.gemm("g2", rng, bf.OP_GEMM_BF16, 1, 128, 128, 1024, w_std=0.05, bn=128, split=1)
        b.smem = 2048 + smem_stages * (16384 + 128 * 128)
        run_and_check(rt, wl.PairSpec("stages%d" % smem_stages, a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.WORK_QUEUE, 1, 1)])


@pytest.mark.parametrize("name", ["cfg2_q_k_proj", "cfg3_qkt_res_layernorm", "cfg4b_k_v_proj"])
def test_tensor_core_pairs_small(rt, name):
    run_and_check(rt, wl.make_pair(name, seed=5, scale=0.25), BLOCK_PATTERNS)
    run_and_check(rt, wl.make_pair(name, seed=5, scale=0.25, split=1), BLOCK_PATTERNS)


@pytest.mark.parametrize("name", ["cfg2_q_k_proj", "cfg3_qkt_res_layernorm", "cfg4b_k_v_proj"])
def test_tensor_core_pairs_full_size(rt, name):
    run_and_check(rt, wl.make_pair(name, seed=6), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])


def test_tensor_core_matches_cuda_core_body(rt):
    # the tcgen05 body against the CUDA-core body on the same inputs (both on the GPU)
    tc = wl.make_pair("cfg2_q_k_proj", seed=7, scale=0.5)
    cc = wl.make_pair("cfg2_q_k_proj", seed=7, scale=0.5, tensor_cores=False)
    ptc, pcc = wl.DevicePair(rt, tc), wl.DevicePair(rt, cc)
    rt.launch_fused(ptc.fusion(bf.ZIGZAG, 1, 1))
    rt.launch_fused(pcc.fusion(bf.ZIGZAG, 1, 1))
    a, b = ptc.read_outputs(), pcc.read_outputs()
    for k in range(2):
        rms = np.sqrt(np.mean(b[k][0].astype(np.float64) ** 2))
        assert np.abs(a[k][0] - b[k][0]).max() <= 5e-3 * (np.abs(b[k][0]).max() + rms)


def test_gate_up_row_sample_full_size(rt):
    """Full-size gate || up (120 GFLOP, too large for the CPU oracle inside a test): a sample of
    output rows spanning all four M tiles is checked against the oracle across all 14336 columns."""
    import oracle
    spec = wl.make_pair("cfg4a_gate_up_proj", seed=8)
    pair = wl.DevicePair(rt, spec)
    rt.launch_fused(pair.fusion(bf.ZIGZAG, 1, 1))
    out = pair.read_outputs()
    assert rt.read_status() == 0
    rows = np.array([0, 1, 127, 128, 255, 300, 511])
    for k, ks in enumerate((spec.a, spec.b)):
        ref = oracle.gemm_nt_bf16(np.ascontiguousarray(ks.host[0][0][rows]), ks.host[1][0])
        g = oracle.bf16_to_f32(out[k][0][0][rows].reshape(-1)).astype(np.float64)
        r = oracle.bf16_to_f32(ref.reshape(-1)).astype(np.float64)
        rms = np.sqrt(np.mean(r * r))
        assert np.all(np.abs(g - r) <= 5e-3 * (np.abs(r) + rms))


def test_conv_tensor_core_pairs(rt):
    """Implicit-GEMM conv on tcgen05: the ResNet-18 branch pair (N = 1 and 3), both against the
    oracle and fused == unfused under every pattern."""
    run_and_check(rt, wl.make_pair("cfg5_conv_branches", seed=9, conv_batch=1), BLOCK_PATTERNS)
    run_and_check(rt, wl.make_pair("cfg5_conv_branches", seed=10, conv_batch=3), [(bf.ZIGZAG, 1, 1), (bf.WORK_QUEUE, 1, 1)])


def test_conv_staged_operand_mode(rt):
    """shape[11] = 1: input rows staged in shared memory by TMA (zero padding = the load's out-of-bounds fill,
    one-row windows with a stride load only the rows they use), the im2col rows written from there into TENSOR
    memory as the MMA's A operand, pixels in the accumulator's lanes.  Padded strided 3x3 whose K blocks straddle
    the raw slots, a 1x1 with stride, a 5x5 with stride 3 on an image smaller than a tile, a ragged second
    channel tile, a long K, and the ResNet branch pair; each against the oracle and fused == unfused under every
    pattern.  What the form cannot do is rejected: rows that are no 16-byte multiples, tiles other than 128
    pixels, a split K, a K that is no whole number of K blocks."""
    rng = np.random.default_rng(61)
    run_and_check(rt, wl.make_pair("cfg5_conv_branches", seed=13, conv_batch=3, conv_mode=1), BLOCK_PATTERNS)
    a = wl.conv2d("s3x3", rng, bf.OP_CONV2D_TF32, 2, 32, 20, 24, 136, 3, 2, 1, bn=128, mode=1)     # K = 288 in slots of 36: K blocks straddle slots
    b = wl.conv2d("s1x1", rng, bf.OP_CONV2D_TF32, 1, 96, 31, 16, 40, 1, 2, 0, bn=128, mode=1)      # one-row window: rows loaded with element stride 2
    pair = run_and_check(rt, wl.PairSpec("staged_a", a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.WORK_QUEUE, 1, 1), (bf.THREAD_SPLIT, 0, 0)])
    assert pair.spec.a.shape[11] == 1 and pair.spec.b.shape[11] == 1
    c = wl.conv2d("s5x5", rng, bf.OP_CONV2D_TF32, 1, 32, 20, 20, 130, 5, 3, 2, bn=128, mode=1)     # 5x5 stride 3 pad 2, K = 800, 49 pixels
    d = wl.conv2d("s3x3s1", rng, bf.OP_CONV2D_TF32, 2, 128, 28, 28, 128, 3, 1, 1, bn=128, mode=1)  # K = 1152, stride 1
    run_and_check(rt, wl.PairSpec("staged_5x5", c, d, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])
    g = wl.gemm("g", rng, bf.OP_GEMM_TF32, 1, 100, 64, 64, w_std=1.0, bn=64, split=1)
    run_and_check(rt, wl.PairSpec("staged_gemm", a, g, "tf32", "hbm"), BLOCK_PATTERNS)
    wide = wl.conv2d("swide", rng, bf.OP_CONV2D_TF32, 1, 32, 5, 160, 136, 3, 1, 1, bn=128, mode=1)       # rows of 160 pixels: tiles start inside a row
    run_and_check(rt, wl.PairSpec("staged_wide", wide, g, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])
    for bad in (wl.conv2d("o", rng, bf.OP_CONV2D_TF32, 1, 96, 17, 17, 96, 3, 2, 0, bn=128, mode=1),        # 17 floats per row
                wl.conv2d("o", rng, bf.OP_CONV2D_TF32, 1, 32, 20, 24, 136, 3, 2, 1, bn=64, mode=1),        # 64-pixel tiles
                wl.conv2d("o", rng, bf.OP_CONV2D_TF32, 1, 256, 16, 16, 256, 3, 1, 1, bn=128, split=4, mode=1),   # K split over a cluster
                wl.conv2d("o", rng, bf.OP_CONV2D_TF32, 1, 20, 20, 24, 136, 3, 2, 1, bn=128, mode=1)):      # K = 180
        with pytest.raises(bf.BfuseError) as err:
            wl.DevicePair(rt, wl.PairSpec("bad", bad, g, "tf32", "hbm"))
        assert err.value.code == 2


def test_conv_staged_ctas_that_walk_several_tiles(rt):
    """A staged conv registered on fewer CTAs than it has tiles: every CTA takes every grid-size-th tile with its
    rings, barrier phases and tensor memory kept across tiles.  3 x 3 (the four-channel walk), 1 x 1 with stride and
    5 x 5 (the table-driven repack), on grids of 5 and of 1 CTA, alone and fused: the same bits as one CTA per tile."""
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    for (ci, h, w, co, k, stride, pad) in ((32, 56, 56, 136, 3, 2, 1), (64, 31, 16, 40, 1, 2, 0), (32, 20, 20, 130, 5, 3, 2)):
        n = 6
        oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
        x = torch.randn(n, ci, h, w, device="cuda", generator=g)
        wt = torch.randn(co, ci, k, k, device="cuda", generator=g) * 0.05
        outs, kernels = [], []
        for grid in (None, (5, 1, 1), (1, 1, 1)):
            y = torch.zeros(n, co, oh, ow, device="cuda")
            d = rt.describe("c", bf.OP_CONV2D_TF32, (n, ci, h, w, co, k, k, stride, pad, 128, 1, 1), [x.data_ptr(), wt.data_ptr(), y.data_ptr()], grid=grid)
            kern = rt.register_kernel(d)
            rt.launch_kernel(kern)
            assert rt.read_status() == 0
            outs.append(y)
            kernels.append(kern)
        assert bool(outs[0].any())
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), (ci, k)
        # fused with itself on another grid, under a block-level pattern and the work queue
        for pattern in ((bf.ZIGZAG, 1, 1), (bf.WORK_QUEUE, 1, 1)):
            want = outs[0].clone()
            outs[1].zero_(), outs[2].zero_()
            rt.launch_fused(rt.register_fusion(kernels[1], kernels[2], *pattern))
            assert rt.read_status() == 0
            assert torch.equal(want, outs[1]) and torch.equal(want, outs[2]), (ci, k, pattern)
    with pytest.raises(bf.BfuseError) as err:   # more CTAs than tiles
        rt.register_kernel(rt.describe("c", bf.OP_CONV2D_TF32, (1, 32, 56, 56, 128, 3, 3, 2, 1, 128, 1, 1), [x.data_ptr(), wt.data_ptr(), outs[0].data_ptr()],
                                       grid=(8, 1, 1)))
    assert err.value.code == 2


def test_conv_tensor_core_ragged_shapes(rt):
    rng = np.random.default_rng(11)
    # co not a multiple of 128, pixels not a multiple of 128, K = ci*kh*kw not a multiple of the K block
    a = wl.conv2d("c1", rng, bf.OP_CONV2D_TF32, 2, 12, 20, 20, 200, 3, 1, 1)     # K = 108, 400 pixels, stride 1
    b = wl.conv2d("c2", rng, bf.OP_CONV2D_TF32, 1, 36, 30, 18, 40, 1, 2, 0)      # 1x1, K = 36, 15 x 9 = 135 ... must be %4
    b = wl.conv2d("c2", rng, bf.OP_CONV2D_TF32, 1, 36, 31, 16, 40, 1, 2, 0)      # 16 x 8 = 128 pixels exactly
    run_and_check(rt, wl.PairSpec("ragged_conv", a, b, "tf32", "hbm"), BLOCK_PATTERNS)
    c = wl.conv2d("c3", rng, bf.OP_CONV2D_TF32, 1, 8, 17, 17, 130, 5, 3, 2)      # 5x5 stride 3 pad 2: 6 x 6 = 36 pixels, K = 200
    d = wl.gemm("g", rng, bf.OP_GEMM_TF32, 1, 100, 64, 64, w_std=1.0, bn=64, split=1)
    run_and_check(rt, wl.PairSpec("conv_gemm", c, d, "tf32", "hbm"), BLOCK_PATTERNS)


def test_conv_long_k_and_odd_pixel_counts(rt):
    """Shapes of the deeper ResNet-18 / Inception-v3 layers: K = ci*kh*kw beyond 1024 (the offset
    table grows with K), output images whose pixel count is not a multiple of 4 (rows that the TMA
    cannot describe: the body stores them itself), channel counts that are no tile multiples."""
    rng = np.random.default_rng(33)
    a = wl.conv2d("deep3x3", rng, bf.OP_CONV2D_TF32, 1, 512, 7, 7, 512, 3, 1, 1)       # K = 4608, 7 x 7 = 49 pixels
    b = wl.conv2d("odd1x1", rng, bf.OP_CONV2D_TF32, 2, 256, 35, 35, 48, 1, 1, 0)       # 1225 pixels, 48 channels
    run_and_check(rt, wl.PairSpec("conv_deep_odd", a, b, "tf32", "hbm"), BLOCK_PATTERNS)
    c = wl.conv2d("mid3x3", rng, bf.OP_CONV2D_TF32, 1, 128, 28, 28, 128, 3, 1, 1)      # K = 1152, 784 pixels
    d = wl.conv2d("odd3x3s2", rng, bf.OP_CONV2D_TF32, 1, 96, 35, 35, 96, 3, 2, 0)      # 17 x 17 = 289 pixels, K = 864
    for bn in (0, 32, 128):
        c.shape, d.shape = c.shape[:9] + (bn,), d.shape[:9] + (bn,)
        run_and_check(rt, wl.PairSpec("conv_mid_odd_bn%d" % bn, c, d, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.WORK_QUEUE, 1, 1)])


def test_conv_split_k_over_a_cluster(rt):
    """K of a conv split over 2, 4 and 8 CTAs of a cluster (uneven last slice included), every pixel-tile
    width, odd pixel counts; the runtime's own choice for a deep layer on a small image is a split one;
    thread split and the work queue refuse the clustered operator."""
    rng = np.random.default_rng(55)
    for split, bn in ((2, 128), (4, 64), (8, 32), (3, 32)):
        # both operators of a launch need the same cluster width: K block counts (74 and 24) that every split here survives
        a = wl.conv2d("deep", rng, bf.OP_CONV2D_TF32, 1, 260, 14, 14, 256, 3, 1, 1, bn=bn, split=split)    # K = 2340 (74 blocks, uneven slices), 196 pixels
        b = wl.conv2d("odd", rng, bf.OP_CONV2D_TF32, 2, 768, 17, 17, 160, 1, 1, 0, bn=bn, split=split)      # K = 768 (24 blocks), 289 pixels
        pair = run_and_check(rt, wl.PairSpec("conv_split%d" % split, a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])
        assert pair.spec.a.launch[0][0] == split * -(-196 // bn)
    c = wl.conv2d("auto", rng, bf.OP_CONV2D_TF32, 1, 512, 7, 7, 512, 3, 1, 1)                              # K = 4608 on 8 tiles
    d = wl.conv2d("plain", rng, bf.OP_CONV2D_TF32, 1, 64, 56, 56, 128, 1, 2, 0)
    pair = run_and_check(rt, wl.PairSpec("conv_auto_split", c, d, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.SM_STRIPED, 0, 0)])
    assert pair.spec.a.launch[0][0] > 2                      # more CTAs along x than the 2 pixel tiles: K was split
    for pat in (bf.THREAD_SPLIT, bf.WORK_QUEUE):
        check_retiled(rt, pair, pat)


def test_conv_pixel_tile_widths(rt):
    """Every pixel-tile width of the tensor-core conv body (32, 64, 128 pixels; 4, 2, 1 gather threads
    per pixel) on a padded 3x3 stride-2 conv and a 1x1 conv whose pixel count is not a tile multiple."""
    rng = np.random.default_rng(21)
    for bn in (32, 64, 128):
        a = wl.conv2d("c3x3", rng, bf.OP_CONV2D_TF32, 2, 24, 30, 30, 136, 3, 2, 1, bn=bn)      # 15 x 15 = 225 ... not % 4
        a = wl.conv2d("c3x3", rng, bf.OP_CONV2D_TF32, 2, 24, 31, 31, 136, 3, 2, 1, bn=bn)      # 16 x 16 = 256 pixels, K = 216
        b = wl.conv2d("c1x1", rng, bf.OP_CONV2D_TF32, 1, 40, 20, 18, 64, 1, 1, 0, bn=bn)       # 360 pixels, K = 40
        pair = run_and_check(rt, wl.PairSpec("conv_bn%d" % bn, a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])
        assert pair.spec.a.launch[0][0] == -(-256 // bn) and pair.spec.b.launch[0][0] == -(-360 // bn)


def test_conv_tensor_core_matches_cuda_core_body(rt):
    tc = wl.make_pair("cfg5_conv_branches", seed=12, conv_batch=2)
    cc = wl.make_pair("cfg5_conv_branches", seed=12, conv_batch=2, tensor_cores=False)
    ptc, pcc = wl.DevicePair(rt, tc), wl.DevicePair(rt, cc)
    rt.launch_fused(ptc.fusion(bf.ZIGZAG, 1, 1))
    rt.launch_fused(pcc.fusion(bf.ZIGZAG, 1, 1))
    a, b = ptc.read_outputs(), pcc.read_outputs()
    for k in range(2):
        rms = np.sqrt(np.mean(b[k][0].astype(np.float64) ** 2))
        assert np.abs(a[k][0] - b[k][0]).max() <= 5e-3 * (np.abs(b[k][0]).max() + rms)


def test_clustered_pair_that_would_need_a_second_wave_gets_half_sm_rings(rt):
    """A conv split over clusters of 4 (100 CTAs) beside a 40-CTA conv whose ring was sized for a whole
    SM: 140 CTAs, but clusters of 4 at one CTA per SM do not fit 148 SMs, so the runtime halves the rings;
    the record reports what the occupancy calculator answered, and the results stay bit-identical to the unfused launches."""
    rng = np.random.default_rng(91)
    a = wl.conv2d("deep", rng, bf.OP_CONV2D_TF32, 1, 128, 28, 28, 128, 3, 1, 1)       # K = 1152: split 4, 25 x 4 CTAs
    b = wl.conv2d("wide", rng, bf.OP_CONV2D_TF32, 1, 256, 35, 35, 64, 1, 1, 0)        # 1225 pixels, K = 256: 39 CTAs, whole-SM ring
    pair = run_and_check(rt, wl.PairSpec("cluster_capacity", a, b, "tf32", "hbm"), [(bf.ZIGZAG, 1, 1)])
    assert pair.spec.a.launch[0][0] == 100 and pair.spec.b.launch[0][0] == 39
    info = rt.fusion_info(pair.fusion(bf.ZIGZAG, 1, 1))
    assert info["GridDim"][0] == 140 and info["smem_bytes"] <= 112 * 1024 + 1024
    # the occupancy calculator counts one CTA per SM for kernels that allocate tensor memory: whole clusters of 4 on 148 SMs
    assert 0 < info["resident_ctas"] <= rt.sm_count and info["resident_ctas"] % 4 == 0 and info["resident_ctas"] < info["GridDim"][0]
