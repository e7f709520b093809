"""The runtime's own scheduler (libbfuse_b200.so, no GPU needed) against the golden data parsed
from the reference's generated kernels and against the oracle: every CTA -> (kernel, virtual
block) decision must be identical (integer work: bit-exact)."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
import oracle

MASK = (1 << 64) - 1


def digest(kern, vb):
    b = np.arange(kern.size, dtype=np.uint64)
    w = ((kern.astype(np.uint64) + np.uint64(1)) << np.uint64(40)) | vb.astype(np.uint64)
    with np.errstate(over="ignore"):
        return int(np.sum(w * (b * np.uint64(2) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15), dtype=np.uint64))


def test_zigzag_matches_every_generated_kernel(golden):
    for rec in golden["zigzag_1_1"]:
        p = bf.Plan(rec["k"], bf.ZIGZAG, 1, 1)
        assert p.fused_grid == (rec["fused_grid"], 1, 1)
        assert p.fused_block == (rec["launch_bounds"], 1, 1)
        kern, vb = p.map_all()
        assert "%016x" % digest(kern, vb) == rec["digest"], rec["name"]


def test_zigzag_m_n_matches_legacy_sweep(golden):
    for rec in golden["zigzag_m_n"]:
        g = [k[0] * k[1] * k[2] for k in rec["k"]]
        ratios = [b[7] for b in rec["br"] if b[0] == 0]
        N = ratios[int(np.argmin(g))]
        M = max(max(ratios) // N, 1)
        if max(g) // min(g) < M:
            M = max(g) // min(g) + 1
        p = bf.Plan(rec["k"], bf.ZIGZAG, M, N)
        kern, vb = p.map_all()
        assert "%016x" % digest(kern, vb) == rec["digest"], rec["name"]


def test_sm_striped_matches_legacy_kernel(golden):
    rec = golden["sm_striped_84"][0]
    p = bf.Plan(rec["k"], bf.SM_STRIPED, 84)
    kern, vb = p.map_all()
    assert "%016x" % digest(kern, vb) == rec["digest"]


def test_thread_split_matches_every_generated_kernel(golden):
    for rec in golden["thread_split"]:
        ks = [[q["gx"], q["gy"], q["gxy"] // (q["gx"] * q["gy"]), q["bx"], q["by"], q["bxy"] // (q["bx"] * q["by"])]
              for q in rec["parts"]]
        p = bf.Plan(ks, bf.THREAD_SPLIT)
        assert p.fused_block == (rec["launch_bounds"], 1, 1)
        assert p.fused_grid == (max(q["grid"] for q in rec["parts"]), 1, 1)
        for i, q in enumerate(rec["parts"]):
            assert p.map_thread(i, 0, q["t_lo"]) == (0, 0)
            assert p.map_thread(i, q["grid"] - 1, q["t_hi"] - 1) == (q["grid"] - 1, q["t_hi"] - 1 - q["t_off"])
            assert p.map_thread(i, q["grid"], q["t_lo"]) is None
            assert p.map_thread(i, 0, q["t_hi"]) is None
            assert q["t_lo"] == 0 or p.map_thread(i, 0, q["t_lo"] - 1) is None
        assert [list(p.barrier(i)) for i in range(2)] == rec["bars"]


@pytest.mark.parametrize("suite", ["tests/benchmark", "tests/inception_v3", "tests/interleave_scheduler"])
def test_fused_dims_match_yaml(golden, suite):
    y = golden["yaml"][suite]
    for a, b, bfd, hfd in y["pairs"]:
        ks = [y["kernels"][a], y["kernels"][b]]
        pz = bf.Plan(ks, bf.ZIGZAG, 1, 1)
        assert list(pz.fused_grid + pz.fused_block) == bfd
        if sum(-(-(k[3] * k[4] * k[5]) // 32) * 32 for k in ks) <= 1024:
            pt = bf.Plan(ks, bf.THREAD_SPLIT)
            assert list(pt.fused_grid + pt.fused_block) == hfd


@pytest.mark.parametrize("pattern,name,kw,args", [
    (bf.ZIGZAG, "zigzag", dict(M=1, N=1), (1, 1)), (bf.ZIGZAG, "zigzag", dict(M=3, N=2), (3, 2)),
    (bf.WORK_QUEUE, "zigzag", dict(M=2, N=4), (2, 4)),
    (bf.PROPORTIONAL, "proportional", dict(min_option=1), (1, 0)),
    (bf.PROPORTIONAL, "proportional", dict(min_option=4), (4, 0)),
    (bf.SM_STRIPED, "sm_striped", dict(total_sm=148), (148, 0)),
    (bf.SM_STRIPED, "sm_striped", dict(total_sm=7), (7, 0)),
    (bf.RANGE_SPLIT, "range_split", {}, (0, 0))])
def test_runtime_scheduler_equals_oracle_on_random_pairs(pattern, name, kw, args):
    rng = np.random.default_rng(11)
    for _ in range(80):
        ks = [[int(rng.integers(1, 60)), int(rng.integers(1, 20)), int(rng.integers(1, 4)),
               32 * int(rng.integers(1, 9)), 1, 1] for _ in range(2)]
        if rng.random() < 0.2:
            ks[1][:3] = ks[0][:3]
        o = oracle.plan(name, ks, **kw)
        p = bf.Plan(ks, pattern, *args)
        ok, ovb = oracle.block_table(o)
        pk, pvb = p.map_all()
        assert np.array_equal(ok, pk) and np.array_equal(ovb, pvb), (name, ks)
        assert p.fused_grid[0] == o.fused_grid and p.fused_block[0] == o.fused_block
        assert p.map_block(o.fused_grid) is None


@pytest.mark.parametrize("cluster", [2, 4, 6, 8])
@pytest.mark.parametrize("pattern,args", [(bf.ZIGZAG, (1, 1)), (bf.ZIGZAG, (3, 2)), (bf.PROPORTIONAL, (2, 0)),
                                          (bf.SM_STRIPED, (5, 0)), (bf.RANGE_SPLIT, (0, 0))])
def test_cluster_granular_dispatch(pattern, args, cluster):
    """With dispatch units of `cluster` CTAs the patterns schedule whole hardware clusters: all CTAs of
    a cluster run one operator on consecutive virtual blocks, every real block runs exactly once,
    and the unit-level order is exactly the oracle's order for the unit counts."""
    rng = np.random.default_rng(5)
    for _ in range(25):
        ks = [[int(rng.integers(1, 50)), int(rng.integers(1, 6)), 1, 192, 1, 1],
              [int(rng.integers(1, 90)), 1, int(rng.integers(1, 3)), 256, 1, 1]]
        p = bf.Plan(ks, pattern, *args, cluster=cluster)
        kern, vb = p.map_all()
        g = [k[0] * k[1] * k[2] for k in ks]
        units = [-(-x // cluster) for x in g]
        assert p.fused_grid[0] == sum(units) * cluster
        for i in range(2):
            assert np.array_equal(np.sort(vb[kern == i]), np.arange(g[i]))
        name = {bf.ZIGZAG: "zigzag", bf.PROPORTIONAL: "proportional", bf.SM_STRIPED: "sm_striped", bf.RANGE_SPLIT: "range_split"}[pattern]
        kw = {bf.ZIGZAG: dict(M=args[0], N=args[1]), bf.PROPORTIONAL: dict(min_option=args[0]),
              bf.SM_STRIPED: dict(total_sm=args[0]), bf.RANGE_SPLIT: {}}[pattern]
        o = oracle.plan(name, [[units[0], 1, 1, 192, 1, 1], [units[1], 1, 1, 256, 1, 1]], **kw)
        ok, ovu = oracle.block_table(o)
        for u in range(sum(units)):
            ck, cvb = kern[u * cluster:(u + 1) * cluster], vb[u * cluster:(u + 1) * cluster]
            real = ck >= 0
            assert real[0] and np.all(ck[real] == ok[u])
            assert np.array_equal(cvb[real], ovu[u] * cluster + np.arange(cluster)[real])
    with pytest.raises(bf.BfuseError):
        bf.Plan(ks, bf.THREAD_SPLIT, cluster=2)
    with pytest.raises(bf.BfuseError):
        bf.Plan(ks, bf.WORK_QUEUE, 1, 1, cluster=2)


def test_baseline_config1_dims():
    # softmax [6144, 512] (8 rows per CTA) x LayerNorm [512, 768] (4 rows per CTA)
    ks = [[768, 1, 1, 32, 8, 1], [128, 1, 1, 64, 4, 1]]
    z = bf.Plan(ks, bf.ZIGZAG, 1, 1)
    assert z.fused_grid == (896, 1, 1) and z.fused_block == (256, 1, 1)
    assert z.map_block(0) == (0, 0) and z.map_block(1) == (1, 0) and z.map_block(255) == (1, 127)
    assert z.map_block(256) == (0, 128) and z.map_block(895) == (0, 767)
    r = bf.Plan(ks, bf.RANGE_SPLIT)
    assert r.map_block(767) == (0, 767) and r.map_block(768) == (1, 0)
    t = bf.Plan(ks, bf.THREAD_SPLIT)
    assert t.fused_grid == (768, 1, 1) and t.fused_block == (512, 1, 1)


def test_bad_plans_are_rejected():
    with pytest.raises(bf.BfuseError):
        bf.Plan([[0, 1, 1, 32, 1, 1], [4, 1, 1, 32, 1, 1]], bf.ZIGZAG, 1, 1)
    with pytest.raises(bf.BfuseError):
        bf.Plan([[4, 1, 1, 32, 1, 1], [4, 1, 1, 32, 1, 1]], 99, 1, 1)
    with pytest.raises(bf.BfuseError):
        bf.Plan([[4, 1, 1, 1024, 1, 1], [4, 1, 1, 64, 1, 1]], bf.THREAD_SPLIT)
    with pytest.raises(bf.BfuseError):
        bf.Plan([[4, 1, 1, 32, 1, 1], [4, 1, 1, 32, 1, 1]], bf.SM_STRIPED, 0)
