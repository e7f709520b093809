"""Parity of every fused pair on the GPU, through the C ABI: fused output == unfused output bit
for bit (the reference's own check, main_cc.py:82-122, at eps = 0), and both against the CPU
oracle within the tolerances in tests/pair_oracle.py."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
from bfuse_project_b200 import workloads as wl
from pair_oracle import check_against_oracle

pytestmark = pytest.mark.gpu

BLOCK_PATTERNS = [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0), (bf.SM_STRIPED, 0, 0), (bf.WORK_QUEUE, 1, 1),
                  (bf.THREAD_SPLIT, 0, 0)]


@pytest.fixture(scope="module")
def rt():
    r = bf.Runtime(0)
    yield r
    r.close()


def run_and_check(rt, spec, patterns, check_oracle=True):
    pair = wl.DevicePair(rt, spec)
    pair.clear_outputs()
    rt.launch_kernel(pair.kernels[0])
    rt.launch_kernel(pair.kernels[1])
    unfused = pair.read_outputs()
    assert rt.read_status() == 0
    if check_oracle:
        check_against_oracle(spec.a, unfused[0], spec.name + "/" + spec.a.name)
        check_against_oracle(spec.b, unfused[1], spec.name + "/" + spec.b.name)
    ran = []
    for pat, m, n in patterns:
        try:
            fusion = pair.fusion(pat, m, n)
        except bf.BfuseError as e:
            # skipped: a pattern that cannot host the pair (code 7), and a thread split whose two windows do not
            # fit one CTA's shared memory side by side (code 3)
            if e.code != 7 and not (e.code == 3 and pat == bf.THREAD_SPLIT):
                raise
            continue
        if any(rt.fusion_info(fusion)["retiled_unsplit"]):
            # an operator registered with several k-slices runs unsplit under this pattern: its sums differ in
            # the last bits from the k-split kernel launched alone, so the check is the fusion's own sequential mode
            check_retiled(rt, pair, pat)
            continue
        ran.append(pat)
        pair.clear_outputs()
        rt.launch_fused(fusion)
        fused = pair.read_outputs()
        assert rt.read_status() == 0
        for k in range(2):
            for u, f in zip(unfused[k], fused[k]):
                assert np.array_equal(u.view(np.uint8), f.view(np.uint8)), \
                    "%s: fused (%s) differs from unfused for kernel %d" % (spec.name, bf.PATTERN_NAMES[pat], k)
    assert ran, "no pattern could host this pair"
    # the parallel and sequential baselines run the same bodies
    pair.clear_outputs()
    rt.launch_parallel(pair.fusion(ran[0], *[(m, n) for p_, m, n in patterns if p_ == ran[0]][0]))
    par = pair.read_outputs()
    for k in range(2):
        assert np.array_equal(par[k][0].view(np.uint8), unfused[k][0].view(np.uint8))
    return pair


def check_retiled(rt, pair, pat):
    """Thread split / work queue with an operator that was registered with several k-slices: the fusion
    runs a one-k-slice re-tiling of it and says so; within the fusion fused == sequential bit for bit,
    and the result agrees with the oracle within tolerance."""
    fusion = pair.fusion(pat, 1, 1)
    assert any(rt.fusion_info(fusion)["retiled_unsplit"])
    pair.clear_outputs()
    rt.launch_sequential(fusion)
    seq = pair.read_outputs()
    pair.clear_outputs()
    rt.launch_fused(fusion)
    fused = pair.read_outputs()
    assert rt.read_status() == 0
    for k, ks in enumerate((pair.spec.a, pair.spec.b)):
        assert np.array_equal(seq[k][0].view(np.uint8), fused[k][0].view(np.uint8)), (bf.PATTERN_NAMES[pat], k)
        check_against_oracle(ks, fused[k], "%s/%s retiled" % (pair.spec.name, ks.name))


@pytest.mark.parametrize("name", ["cfg1_softmax_layernorm", "cfg4c_rmsnorm_rope"])
def test_memory_bound_pairs_small(rt, name):
    run_and_check(rt, wl.make_pair(name, seed=3, scale=0.25), BLOCK_PATTERNS)


@pytest.mark.parametrize("name", ["cfg1_softmax_layernorm", "cfg4c_rmsnorm_rope"])
def test_memory_bound_pairs_full_size(rt, name):
    run_and_check(rt, wl.make_pair(name, seed=4), [(bf.ZIGZAG, 1, 1), (bf.RANGE_SPLIT, 0, 0)])


def test_softmax_rows_sum_to_one_full_size(rt):
    # size-independent property at the full BASELINE size
    pair = wl.DevicePair(rt, wl.make_pair("cfg1_softmax_layernorm", seed=5))
    rt.launch_fused(pair.fusion(bf.ZIGZAG, 1, 1))
    out = pair.read_outputs()
    assert np.allclose(out[0][0].sum(1), 1.0, atol=1e-5)
    y = out[1][0].astype(np.float64)
    g, b = pair.spec.b.host[2].astype(np.float64), pair.spec.b.host[3].astype(np.float64)
    z = (y - b) / g  # undo the affine part: rows must be standardised
    assert np.allclose(z.mean(1), 0.0, atol=1e-4) and np.allclose(z.var(1), 1.0, atol=1e-3)


def test_ragged_rows_and_custom_tilings(rt):
    rng = np.random.default_rng(9)
    a = wl.softmax("softmax", rng, 1001, 256, 0.5)       # 1001 rows: last CTA partly empty
    a.block, a.grid = (64, 4, 1), (251, 1, 1)             # 64 threads per row, 4 rows per CTA
    b = wl.layernorm("layernorm", rng, 77, 2048, 1e-5, residual=True)
    b.block, b.grid = (128, 2, 1), (39, 1, 1)
    run_and_check(rt, wl.PairSpec("ragged", a, b, "f32", "hbm"), BLOCK_PATTERNS)
    c = wl.rmsnorm("rmsnorm", rng, 33, 1024, 1e-6)
    d = wl.rope("rope", rng, 19, 8, 64, 10000.0)
    run_and_check(rt, wl.PairSpec("ragged_bf16", c, d, "bf16", "hbm"), BLOCK_PATTERNS)


def test_simt_gemm_and_conv_pairs(rt):
    run_and_check(rt, wl.make_pair("cfg2_q_k_proj", seed=6, scale=0.25, tensor_cores=False), BLOCK_PATTERNS)
    run_and_check(rt, wl.make_pair("cfg3_qkt_res_layernorm", seed=7, scale=0.25, tensor_cores=False),
                  [(bf.ZIGZAG, 1, 1), (bf.THREAD_SPLIT, 0, 0), (bf.WORK_QUEUE, 2, 1)])
    run_and_check(rt, wl.make_pair("cfg5_conv_branches", seed=8, conv_batch=2, tensor_cores=False), BLOCK_PATTERNS)


def test_simt_gemm_ragged_shapes(rt):
    rng = np.random.default_rng(10)
    a = wl.gemm("g1", rng, bf.OP_GEMM_F32_SIMT, 2, 70, 90, 36, bias=True, w_std=1.0)
    b = wl.gemm("g2", rng, bf.OP_GEMM_F32_SIMT, 1, 130, 50, 20, causal=True, w_std=1.0)
    run_and_check(rt, wl.PairSpec("ragged_gemm", a, b, "f32", "hbm"), BLOCK_PATTERNS)


def test_host_buffer_entry_points(rt):
    spec = wl.make_pair("cfg1_softmax_layernorm", seed=11, scale=0.25)
    pair = wl.DevicePair(rt, spec)
    h1 = [None if a is None else a.copy() for a in spec.a.host]
    h2 = [None if a is None else a.copy() for a in spec.b.host]
    rt.run_fuse(pair.fusion(bf.ZIGZAG, 1, 1), h1, h2)
    check_against_oracle(spec.a, [h1[1]], "run_fuse softmax")
    check_against_oracle(spec.b, [h2[4]], "run_fuse layernorm")
    g1 = [None if a is None else a.copy() for a in spec.a.host]
    rt.run_kernel(pair.kernels[0], g1)
    assert np.array_equal(g1[1], h1[1])
    p1 = [None if a is None else a.copy() for a in spec.a.host]
    p2 = [None if a is None else a.copy() for a in spec.b.host]
    rt.run_parallel(pair.fusion(bf.ZIGZAG, 1, 1), p1, p2)
    assert np.array_equal(p1[1], h1[1]) and np.array_equal(p2[4], h2[4])
    assert bf.check_matrix(h1[1], g1[1]) == 0


def test_graph_replay_and_timing(rt):
    specs = [wl.make_pair("cfg4c_rmsnorm_rope", seed=s, scale=0.25) for s in (1, 2, 3)]
    pairs = [wl.DevicePair(rt, s) for s in specs]
    fus = [p.fusion(bf.ZIGZAG, 1, 1) for p in pairs]
    g = rt.graph_create(fus, bf.MODE_FUSED)
    for p in pairs:
        p.clear_outputs()
    rt.graph_launch(g)
    for p in pairs:
        out = p.read_outputs()
        check_against_oracle(p.spec.a, out[0], "graph rmsnorm")
        check_against_oracle(p.spec.b, out[1], "graph rope")
    mean, mn = rt.time(fus[0], bf.MODE_FUSED, warmup=3, iters=10)
    assert 0 < mn <= mean * 4 and mean < 1e5


def test_rejected_registrations(rt):
    import torch
    buf = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = buf.data_ptr()
    with pytest.raises(bf.BfuseError) as e:   # cols not divisible into 128-bit vectors
        rt.describe("bad", bf.OP_SOFTMAX_F32, (4, 30), [p, p], (1.0,))
    assert e.value.code == 2
    d = rt.describe("s", bf.OP_SOFTMAX_F32, (64, 512), [p, p], (1.0,))
    d.BlockDim = bf.Dim3(48, 1, 1)            # not a power of two / multiple of 32
    with pytest.raises(bf.BfuseError):
        rt.register_kernel(d)
    d = rt.describe("s", bf.OP_SOFTMAX_F32, (64, 512), [p, p], (1.0,))
    d.GridDim = bf.Dim3(2, 1, 1)              # grid does not cover the rows
    with pytest.raises(bf.BfuseError):
        rt.register_kernel(d)
    d = rt.describe("s", bf.OP_SOFTMAX_F32, (64, 512), [p, 0], (1.0,))   # missing output buffer
    with pytest.raises(bf.BfuseError):
        rt.register_kernel(d)
    d = rt.describe("s", bf.OP_SOFTMAX_F32, (64, 512), [p + 4, p], (1.0,))  # misaligned
    with pytest.raises(bf.BfuseError):
        rt.register_kernel(d)
    with pytest.raises(bf.BfuseError):
        rt.register_fusion(0, 10 ** 6, bf.ZIGZAG)
    ok = rt.register_kernel(rt.describe("s", bf.OP_SOFTMAX_F32, (64, 512), [p, p], (1.0,)))
    with pytest.raises(bf.BfuseError):
        rt.register_fusion(ok, ok, 77)
    d = rt.describe("g", bf.OP_GEMM_TF32, (1, 128, 128, 64, 0), [p, p, 0, p])
    d.smem_bytes = 300 * 1024                  # over the per-CTA budget
    with pytest.raises(bf.BfuseError) as e:
        rt.register_kernel(d)
    assert e.value.code == 3


def test_release_of_kernels_fusions_groups_and_graphs(rt):
    """bfuse_unregister_* / bfuse_graph_destroy (finalize_kernel1/2 of the reference harness): out-of-order
    releases are refused and release nothing, released handles are dead and get reused, a work-queue
    fusion's counters are freed (device memory in use returns to where it was), and the caller's buffers
    and the other registrations are untouched."""
    import torch
    spec = wl.make_pair("cfg1_softmax_layernorm", seed=5, scale=0.25)
    pair = wl.DevicePair(rt, spec)
    k1, k2 = pair.kernels
    keep = rt.register_fusion(k1, k2, bf.ZIGZAG, 1, 1)
    rt.launch_fused(keep)
    want = pair.read_outputs()
    torch.cuda.synchronize()
    queue = rt.register_fusion(k1, k2, bf.WORK_QUEUE, 1, 1)
    graph = rt.graph_create([queue], bf.MODE_FUSED)
    with pytest.raises(bf.BfuseError) as e:       # captured by a live graph
        rt.unregister_fusion(queue)
    assert e.value.code == 1
    with pytest.raises(bf.BfuseError) as e:       # used by live fusions
        rt.unregister_kernel(k1)
    assert e.value.code == 1
    pair.clear_outputs()
    rt.graph_launch(graph)                        # both refusals released nothing
    got = pair.read_outputs()
    assert all(np.array_equal(got[k][0], want[k][0]) for k in range(2))
    rt.graph_destroy(graph)
    with pytest.raises(bf.BfuseError):
        rt.graph_launch(graph)
    rt.unregister_fusion(queue)
    for call in (rt.launch_fused, rt.fusion_info, rt.unregister_fusion):
        with pytest.raises(bf.BfuseError) as e:   # the handle is dead
            call(queue)
        assert e.value.code == 1
    # re-registering in a loop does not grow what the runtime holds: handles are reused
    seen = set()
    for _ in range(50):
        f = rt.register_fusion(k1, k2, bf.WORK_QUEUE, 1, 1)
        seen.add(f)
        rt.unregister_fusion(f)
    assert len(seen) == 1
    # a group pins its kernels the same way
    pa = wl.DevicePair(rt, wl.make_pair("cfg1_softmax_layernorm", seed=6, scale=0.25))
    group = rt.register_group([k1, pa.kernels[0]], bf.ZIGZAG, 1, 1)
    with pytest.raises(bf.BfuseError):
        rt.unregister_kernel(pa.kernels[0])
    rt.unregister_group(group)
    with pytest.raises(bf.BfuseError):
        rt.launch_group(group)
    rt.unregister_kernel(pa.kernels[0])
    with pytest.raises(bf.BfuseError):
        rt.launch_kernel(pa.kernels[0])
    # the fusion that was kept still runs and gives the same bits
    pair.clear_outputs()
    rt.launch_fused(keep)
    got = pair.read_outputs()
    assert rt.read_status() == 0
    assert all(np.array_equal(got[k][0], want[k][0]) for k in range(2))
    rt.unregister_fusion(keep)
    rt.unregister_kernel(k1)
    rt.unregister_kernel(k2)


def test_dependent_launch_switch_changes_no_result(rt):
    """bfuse_set_dependent_launch(0): launches without programmatic dependent launch write the same bits."""
    spec = wl.make_pair("cfg3_qkt_res_layernorm", seed=8, scale=0.25)
    pair = wl.DevicePair(rt, spec)
    f = pair.fusion(bf.ZIGZAG, 1, 1)
    rt.launch_fused(f)
    want = pair.read_outputs()
    rt.set_dependent_launch(False)
    try:
        pair.clear_outputs()
        rt.launch_fused(f)
        rt.launch_kernel(pair.kernels[0])
        got = pair.read_outputs()
    finally:
        rt.set_dependent_launch(True)
    assert rt.read_status() == 0
    assert all(np.array_equal(got[k][0].view(np.uint8), want[k][0].view(np.uint8)) for k in range(2))


def test_run_fuse_batch_matches_one_call_per_pair(rt):
    """The batched host-buffer entry point (copies in, launches and copies out of neighbouring pairs on
    three streams) returns the same bits as one synchronous run_fuse per pair; duplicates are refused."""
    specs = [wl.make_pair("cfg1_softmax_layernorm", seed=s, scale=0.25) for s in range(3)] + \
            [wl.make_pair("cfg2_q_k_proj", seed=7, scale=0.25)]
    pairs = [wl.DevicePair(rt, sp) for sp in specs]
    fus = [p.fusion(bf.ZIGZAG, 1, 1) for p in pairs]

    def host_copy(sp):
        return [[None if a is None else a.copy() for a in ks.host] for ks in (sp.a, sp.b)]

    want = []
    for p, f in zip(pairs, fus):
        h = host_copy(p.spec)
        rt.run_fuse(f, h[0], h[1])
        want.append(h)
        p.clear_outputs()
    got = [host_copy(p.spec) for p in pairs]
    rt.run_fuse_batch(fus, [h[0] for h in got], [h[1] for h in got])
    for p, w, g in zip(pairs, want, got):
        for k, ks in enumerate((p.spec.a, p.spec.b)):
            for i in ks.outputs:
                assert np.array_equal(w[k][i].view(np.uint8), g[k][i].view(np.uint8))
                assert np.any(g[k][i].view(np.uint8) != 0)
    with pytest.raises(bf.BfuseError) as e:
        rt.run_fuse_batch([fus[0], fus[0]], [got[0][0], got[0][0]], [got[0][1], got[0][1]])
    assert e.value.code == 1


def test_run_fuse_batch_over_sub_shards_that_share_their_weights(rt):
    """Sub-shards of one batch (the conv pair's images in pieces, as the end-to-end bench sends them): every piece
    names the same host and device weight buffers, which the call copies once; the pieces' outputs, written into
    slices of one host array, equal the outputs of the whole batch computed in one launch."""
    import torch
    n, sub = 6, 2
    b = wl.ConvBranchBatch(rt, torch, 0, n, seed=5)
    k3, k1 = b.shard(0, n)
    rt.launch_fused(rt.register_fusion(k3, k1, bf.RANGE_SPLIT, 0, 0))
    assert rt.read_status() == 0
    want3, want1 = b.y3.cpu().numpy(), b.y1.cpu().numpy()
    assert np.any(want3 != 0) and np.any(want1 != 0)
    b.clear_outputs()
    hx, hw3, hw1 = b.x.cpu().numpy(), b.w3.cpu().numpy(), b.w1.cpu().numpy()
    b.w3.zero_(), b.w1.zero_(), b.x.zero_()          # everything the kernels read has to come from the host buffers
    hy3, hy1 = np.zeros_like(want3), np.zeros_like(want1)
    fus, h1, h2 = [], [], []
    for o in range(0, n, sub):
        s3, s1 = b.shard(o, sub)
        fus.append(rt.register_fusion(s3, s1, bf.RANGE_SPLIT, 0, 0))
        h1.append([hx[o:o + sub], hw3, hy3[o:o + sub]])
        h2.append([hx[o:o + sub], hw1, hy1[o:o + sub]])
    rt.run_fuse_batch(fus, h1, h2)
    assert np.array_equal(hy3.view(np.uint8), want3.view(np.uint8)) and np.array_equal(hy1.view(np.uint8), want1.view(np.uint8))
