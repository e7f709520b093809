"""Pins the dispatch oracle against known answers taken from the reference itself:
the constants its fuser printed into generated kernels, a digest of the CTA -> (kernel,
virtual block) map evaluated from those printed conditions, and the fused dims in its
YAML outputs (tests/golden/dispatch_golden.json, made by make_dispatch_golden.py)."""
import numpy as np
import pytest

import oracle

F = ("kind", "kernel", "b_lo", "b_hi", "rot", "r_lo", "r_hi", "ratio", "base", "sm", "stripe_n", "stripe_idx")


def branches_of(p):
    return [[getattr(p.br[i], f) for f in F] for i in range(p.n_branches)]


def check_record(rec, p):
    assert branches_of(p) == rec["br"], rec["name"]
    assert p.fused_grid == rec["fused_grid"]
    assert p.fused_block == rec["launch_bounds"]
    assert "%016x" % oracle.digest(p) == rec["digest"], rec["name"]


def test_zigzag_1_1_all_generated_kernels(golden):
    assert golden["zigzag_1_1_files"] == 1764
    for rec in golden["zigzag_1_1"]:
        p = oracle.plan("zigzag", rec["k"], M=1, N=1)
        check_record(rec, p)
        # guard: KernelID_ == k && threadIdx.x < B_k
        assert rec["guards"] == [k[3] * k[4] * k[5] for k in rec["k"]]


def test_unequal_grid_example(golden):
    # dense1_0 (384 CTAs) x dense2_6 (7168): interleaved below 768, tail b - 768 + 384
    rec = next(r for r in golden["zigzag_1_1"] if r["name"] == "dense1_0_dense2_6_bfuse")
    p = oracle.plan("zigzag", rec["k"])
    assert oracle.map_block(p, 0) == (0, 0)
    assert oracle.map_block(p, 1) == (1, 0)
    assert oracle.map_block(p, 767) == (1, 383)
    assert oracle.map_block(p, 768) == (1, 384)
    assert oracle.map_block(p, 7551) == (1, 7167)
    assert oracle.map_block(p, 7552) is None


def _infer_m_n(rec):
    """ratio_k = min(G_k / min G, M) * N  ->  recover (M, N) from the printed ratios."""
    g = [k[0] * k[1] * k[2] for k in rec["k"]]
    ratios = [b[7] for b in rec["br"] if b[0] == 0]
    small = int(np.argmin(g))
    n = ratios[small]  # quotient 1 -> (1 < M ? 1*N : M*N) = N either way
    m = max(ratios) // n
    return max(m, 1), n


def test_zigzag_m_n_legacy_sweep(golden):
    assert len(golden["zigzag_m_n"]) >= 30
    seen = set()
    for rec in golden["zigzag_m_n"]:
        M, N = _infer_m_n(rec)
        g = [k[0] * k[1] * k[2] for k in rec["k"]]
        if max(g) // min(g) < M:   # ratio capped by the grid quotient: M not recoverable
            M = max(g) // min(g) + 1
        p = oracle.plan("zigzag", rec["k"], M=M, N=N)
        check_record(rec, p)
        seen.add((M, N))
    assert len(seen) > 5


def test_sm_striped_84(golden):
    rec = golden["sm_striped_84"][0]
    p = oracle.plan("sm_striped", rec["k"], total_sm=84)
    check_record(rec, p)


def test_thread_split_all_generated_kernels(golden):
    assert golden["thread_split_files"] == 1764
    for rec in golden["thread_split"]:
        ks = [[q["gx"], q["gy"], q["gxy"] // (q["gx"] * q["gy"]), q["bx"], q["by"], q["bxy"] // (q["bx"] * q["by"])]
              for q in rec["parts"]]
        p = oracle.plan("thread_split", ks)
        assert p.thread_split == 1
        for i, q in enumerate(rec["parts"]):
            br = p.br[i]
            assert (br.t_lo, br.t_hi, br.b_hi) == (q["t_lo"], q["t_hi"], q["grid"])
            assert q["t_off"] == br.t_lo
        assert p.fused_block == rec["launch_bounds"]
        # bar.sync <k+1>, <round32(B_k)> for kernels that synchronise
        assert [list(oracle.named_barrier(p, i)) for i in range(len(ks))] == rec["bars"]


@pytest.mark.parametrize("suite", ["tests/benchmark", "tests/inception_v3", "tests/interleave_scheduler"])
def test_yaml_fused_dims(golden, suite):
    y = golden["yaml"][suite]
    assert len(y["pairs"]) in (1764, 900, 64)
    for a, b, bf, hf in y["pairs"]:
        ks = [y["kernels"][a], y["kernels"][b]]
        pz = oracle.plan("zigzag", ks)
        assert [pz.fused_grid, 1, 1, pz.fused_block, 1, 1] == bf
        pt = oracle.plan("thread_split", ks)
        assert [pt.fused_grid, 1, 1, pt.fused_block, 1, 1] == hf


@pytest.mark.parametrize("pattern,kw", [("zigzag", {}), ("zigzag", dict(M=4, N=2)), ("proportional", {}),
                                        ("proportional", dict(min_option=3)), ("sm_striped", dict(total_sm=148)),
                                        ("sm_striped", dict(total_sm=84)), ("range_split", {})])
def test_every_pattern_is_a_bijection(pattern, kw):
    rng = np.random.default_rng(7)
    for _ in range(60):
        ks = [[int(rng.integers(1, 40)), int(rng.integers(1, 30)), int(rng.integers(1, 4)),
               int(rng.integers(1, 9)) * 16, 1, 1] for _ in range(2)]
        p = oracle.plan(pattern, ks, **kw)
        kern, vb = oracle.block_table(p)
        for i, k in enumerate(ks):
            got = np.sort(vb[kern == i])
            assert np.array_equal(got, np.arange(k[0] * k[1] * k[2])), (pattern, ks)


def test_three_kernels_and_degenerate():
    ks = [[5, 1, 1, 64, 1, 1], [17, 1, 1, 128, 1, 1], [9, 2, 1, 32, 1, 1]]
    for pattern in ("zigzag", "proportional", "range_split", "sm_striped"):
        p = oracle.plan(pattern, ks, total_sm=4) if pattern == "sm_striped" else oracle.plan(pattern, ks)
        kern, vb = oracle.block_table(p)
        for i, k in enumerate(ks):
            assert np.array_equal(np.sort(vb[kern == i]), np.arange(k[0] * k[1] * k[2]))
    with pytest.raises(ValueError):
        oracle.plan("zigzag", [[0, 1, 1, 32, 1, 1], [1, 1, 1, 32, 1, 1]])
