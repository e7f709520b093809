"""The BASELINE configurations at their full sizes: the ResNet-18 branch pair over a batch of 256
images (bit-equality of the fused launch under every pattern, a sample of images against the oracle,
and the batch partition: shards by pointer offset reproduce the unsharded output bit for bit) and
the Llama gate || up pair (bit-equality of the fused launch under the block-level patterns)."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
from bfuse_project_b200 import partition
from bfuse_project_b200 import workloads as wl
from pair_oracle import assert_close

pytestmark = pytest.mark.gpu

PATTERNS = [(bf.ZIGZAG, 1, 1), (bf.PROPORTIONAL, 1, 0), (bf.RANGE_SPLIT, 0, 0), (bf.SM_STRIPED, 0, 0), (bf.WORK_QUEUE, 1, 1),
            (bf.THREAD_SPLIT, 0, 0)]


@pytest.fixture(scope="module")
def rt():
    r = bf.Runtime(0)
    yield r
    r.close()


@pytest.fixture(scope="module")
def batch256(rt):
    import torch
    b = wl.ConvBranchBatch(rt, torch, 0, 256, seed=17)
    k3, k1 = b.shard(0, 256)
    rt.launch_kernel(k3)
    rt.launch_kernel(k1)
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    b.want = (b.y3.clone(), b.y1.clone())       # the unfused launches over the whole batch
    yield b
    del b
    torch.cuda.empty_cache()


def test_conv_branches_batch_256_against_the_oracle(rt, batch256):
    """Images 0, 32, 64, ..., 224 and 255 of the unfused outputs against the CPU oracle (fp32 and
    tf32-truncated), all 128 channels and 784 pixels of each."""
    import oracle
    b = batch256
    w3, w1 = b.w3.cpu().numpy(), b.w1.cpu().numpy()
    for img in list(range(0, 256, 32)) + [255]:
        x = b.x[img:img + 1].cpu().numpy()
        for got, w, pad, what in ((b.want[0], w3, 1, "3x3"), (b.want[1], w1, 0, "1x1")):
            g = got[img:img + 1].cpu().numpy()
            assert_close(g, oracle.conv2d_nchw(x, w, 2, pad, tf32=True), 2e-4, "image %d %s (tf32-truncated oracle)" % (img, what))
            assert_close(g, oracle.conv2d_nchw(x, w, 2, pad), 5e-3, "image %d %s (fp32 oracle)" % (img, what))


@pytest.mark.parametrize("pattern,m,n", PATTERNS)
def test_conv_branches_batch_256_fused_equals_unfused(rt, batch256, pattern, m, n):
    import torch
    b = batch256
    k3, k1 = b.shard(0, 256)
    try:
        f = rt.register_fusion(k3, k1, pattern, m, n)
    except bf.BfuseError as e:
        if e.code not in (3, 7):
            raise
        pytest.skip("%s cannot host this pair: %s" % (bf.PATTERN_NAMES[pattern], e))
    assert rt.fusion_info(f)["retiled_unsplit"] == (False, False)
    b.clear_outputs()
    rt.launch_fused(f)
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert torch.equal(b.y3, b.want[0]) and torch.equal(b.y1, b.want[1]), bf.PATTERN_NAMES[pattern]
    rt.unregister_fusion(f)


def test_conv_branches_batch_256_staged_operand_equals_gathered_within_tolerance(rt, batch256):
    """The staged operand path (shape[11] = 1) at the full batch, where every SM holds two CTAs with three-slot raw
    rings: fused == unfused bit for bit, and the 3x3 output agrees with the gathered path's (same products, same
    summation order: equal bits)."""
    import torch
    b = batch256
    s = wl.ConvBranchBatch(rt, torch, 0, 256, seed=17, mode=1)
    assert torch.equal(s.x, b.x) and torch.equal(s.w3, b.w3)
    k3, k1 = s.shard(0, 256)
    rt.launch_kernel(k3)
    rt.launch_kernel(k1)
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert torch.equal(s.y3, b.want[0]) and torch.equal(s.y1, b.want[1])
    s.clear_outputs()
    rt.launch_fused(rt.register_fusion(k3, k1, bf.ZIGZAG, 1, 1))
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert torch.equal(s.y3, b.want[0]) and torch.equal(s.y1, b.want[1])
    del s
    torch.cuda.empty_cache()


@pytest.mark.parametrize("world", [2, 4, 8, 3])
def test_conv_branches_batch_shards_reproduce_the_whole_batch(rt, batch256, world):
    """The multi-GPU partition on one GPU: rank r's shard (partition.shard_batch) is the same batch at a
    pointer offset; the shards' outputs, written into their slices of the one output, equal the
    unsharded launch bit for bit (world 3: uneven shards of 86 + 85 + 85 images)."""
    import torch
    b = batch256
    b.clear_outputs()
    covered = 0
    for r in range(world):
        first, count = partition.shard_batch(256, world, r)
        assert first == covered
        covered += count
        k3, k1 = b.shard(first, count)
        rt.launch_fused(rt.register_fusion(k3, k1, bf.ZIGZAG, 1, 1))
    assert covered == 256
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert torch.equal(b.y3, b.want[0]) and torch.equal(b.y1, b.want[1])


def test_gate_up_full_size_fused_equals_unfused(rt):
    """Llama-3-8B gate || up at full size (2 x [512, 4096] x [4096, 14336], bf16): the fused launch under
    the block-level patterns writes the bits of the two unfused launches."""
    import torch
    spec = wl.make_pair("cfg4a_gate_up_proj", seed=18)
    pair = wl.DevicePair(rt, spec)
    rt.launch_kernel(pair.kernels[0])
    rt.launch_kernel(pair.kernels[1])
    torch.cuda.synchronize()
    want = [pair.buffers[k][3].clone() for k in range(2)]
    assert all(bool(w.any()) for w in want)
    for pattern, m, n in ((bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0), (bf.SM_STRIPED, 0, 0), (bf.PROPORTIONAL, 1, 0)):
        pair.clear_outputs()
        rt.launch_fused(pair.fusion(pattern, m, n))
        torch.cuda.synchronize()
        assert rt.read_status() == 0
        for k in range(2):
            assert torch.equal(pair.buffers[k][3], want[k]), (bf.PATTERN_NAMES[pattern], k)
