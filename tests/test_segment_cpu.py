"""Host logic of the n-way groups and of the model-segment driver (no GPU)."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
import oracle
from bfuse_project_b200 import segment as sg


def _random_kernels(rng, n):
    return [[int(rng.integers(1, 40)), int(rng.integers(1, 6)), int(rng.integers(1, 4)),
             int(rng.integers(1, 257)), int(rng.integers(1, 3)), 1] for _ in range(n)]


def test_group_plans_match_the_oracle_for_two_to_four_kernels():
    """Zig-zag M:N, proportional and range split of 2, 3 and 4 kernels: fused dims and the kernel /
    virtual block of every CTA equal the oracle's if / else-if chain (Algorithms.cc:323-375, 538-587)."""
    rng = np.random.default_rng(11)
    for _ in range(400):
        ks = _random_kernels(rng, int(rng.integers(2, 5)))
        M, N, opt = int(rng.integers(1, 4)), int(rng.integers(1, 4)), int(rng.integers(1, 4))
        for pat, name, kw, pm, pn in ((bf.ZIGZAG, "zigzag", dict(M=M, N=N), M, N),
                                      (bf.PROPORTIONAL, "proportional", dict(min_option=opt), opt, 1),
                                      (bf.RANGE_SPLIT, "range_split", {}, 0, 0)):
            p = oracle.plan(name, ks, **kw)
            grid, block, kernel_of, vblock_of = bf.plan_group(ks, pat, pm, pn)
            want_k, want_vb = oracle.block_table(p)
            assert (grid, block) == (p.fused_grid, p.fused_block)
            assert np.array_equal(kernel_of, want_k) and np.array_equal(vblock_of, want_vb)


def test_group_of_two_equals_the_pair_plan():
    rng = np.random.default_rng(12)
    for _ in range(200):
        ks = _random_kernels(rng, 2)
        for pat, pm, pn in ((bf.ZIGZAG, 2, 3), (bf.PROPORTIONAL, 2, 1), (bf.RANGE_SPLIT, 0, 0)):
            grid, block, kernel_of, vblock_of = bf.plan_group(ks, pat, pm, pn)
            plan = bf.Plan(ks, pat, pm, pn)
            pk, pvb = plan.map_all()
            assert grid == plan.fused_grid[0] and block == plan.fused_block[0]
            assert np.array_equal(kernel_of, pk) and np.array_equal(vblock_of, pvb)


def test_clustered_group_keeps_clusters_whole_and_covers_every_block():
    ks = [[12, 1, 1, 192, 1, 1], [7, 1, 1, 192, 1, 1], [20, 1, 1, 192, 1, 1]]   # 7 CTAs: one padded cluster of 4
    grid, block, kernel_of, vblock_of = bf.plan_group(ks, bf.ZIGZAG, 1, 1, cluster=4)
    assert grid % 4 == 0 and grid == 4 * (3 + 2 + 5)
    for c in range(grid // 4):
        owners = {int(k) for k in kernel_of[4 * c:4 * c + 4] if k >= 0}
        assert len(owners) == 1
        vbs = [int(v) for v in vblock_of[4 * c:4 * c + 4] if v >= 0]
        assert vbs == list(range(vbs[0], vbs[0] + len(vbs))) and vbs[0] % 4 == 0
    for k, (g, *_rest) in enumerate(ks):
        assert sorted(int(v) for kk, v in zip(kernel_of, vblock_of) if kk == k) == list(range(g))
    assert int((kernel_of < 0).sum()) == 1   # the padding CTA of the 7-block kernel


def test_group_rejects_bad_input():
    ks = [[4, 1, 1, 64, 1, 1]] * 3
    for bad in (lambda: bf.plan_group(ks[:1], bf.ZIGZAG), lambda: bf.plan_group(ks * 2, bf.ZIGZAG),
                lambda: bf.plan_group(ks, bf.SM_STRIPED, 148, 0), lambda: bf.plan_group(ks, bf.THREAD_SPLIT),
                lambda: bf.plan_group(ks, bf.ZIGZAG, 0, 1)):
        with pytest.raises(bf.BfuseError):
            bad()


def _ops(spec):
    return [sg.SegmentOp(n, op, i, r, w) for i, (n, op, r, w) in enumerate(spec)]


def test_dependencies_cover_raw_war_waw():
    ops = _ops([("w1", 0, ["a"], ["b"]), ("r1", 0, ["b"], ["c"]), ("waw", 0, ["a"], ["b"]), ("war", 1, ["z"], ["a"]),
                ("free", 1, ["q"], ["r"])])
    deps = sg.dependencies(ops)
    assert deps[1] == {0} and deps[2] == {0, 1} and deps[3] == {0, 2} and deps[4] == set()


def test_schedule_respects_dependencies_and_groups_by_body():
    for name, build in sg.SEGMENTS.items():
        _, ops = build(None, None)
        deps = sg.dependencies(ops)
        steps = sg.schedule(ops)
        seen, step_of = [], {}
        for si, step in enumerate(steps):
            for kind, idx in step:
                assert 1 <= len(idx) <= 4
                assert (kind == "single") == (len(idx) == 1)
                if kind == "group":
                    assert len({ops[i].op for i in idx}) <= 2
                if kind == "pair":
                    assert len(idx) == 2 and ops[idx[0]].op != ops[idx[1]].op
                for i in idx:
                    step_of[i] = si
                seen.extend(idx)
        assert sorted(seen) == list(range(len(ops))), name
        for j, d in enumerate(deps):
            assert all(step_of[i] < step_of[j] for i in d), name


def test_bert_layer_fuses_qkv_three_ways_and_replicas_across_requests():
    _, ops = sg.bert_layer(None, None)
    steps = sg.schedule(ops)
    assert steps[0] == [("group", [0, 1, 2])] and [ops[i].name for i in (0, 1, 2)] == ["q_proj", "k_proj", "v_proj"]
    assert sum(len(s) for s in steps) == len(ops) - 2
    _, ops4 = sg.bert_layer(None, None, replicas=4)
    steps4 = sg.schedule(ops4)
    assert len(ops4) == 44 and sum(len(s) for s in steps4) == 11
    assert [len(idx) for _, idx in steps4[0]] == [4, 4, 4]


def test_rule_and_group_width_are_honoured():
    ops = _ops([("c%d" % i, bf.OP_CONV2D_F32_SIMT, ["x"], ["y%d" % i]) for i in range(3)] +
               [("s", bf.OP_SOFTMAX_F32, ["x"], ["p"]), ("l", bf.OP_LAYERNORM_F32, ["x"], ["q"])])
    steps = sg.schedule(ops)
    kinds = sorted(k for k, _ in steps[0])
    assert kinds == ["pair", "single", "single", "single"]        # CUDA-core convs stay alone; softmax pairs with LayerNorm
    five = _ops([("g%d" % i, bf.OP_GEMM_TF32, ["x"], ["y%d" % i]) for i in range(5)])
    assert [len(i) for _, i in sg.schedule(five)[0]] == [3, 2]
    assert [len(i) for _, i in sg.schedule(five, max_group=2)[0]] == [2, 2, 1]
    assert [k for k, _ in sg.schedule(five, max_group=1)[0]] == ["single"] * 5


def test_pairing_model_arithmetic():
    from bfuse_project_b200 import pairing
    assert pairing.ctas_per_sm(192, 198656) == 1 and pairing.ctas_per_sm(192, 100352) == 2
    assert pairing.ctas_per_sm(256, 256) == 8 and pairing.ctas_per_sm(1024, 0) == 2
    assert pairing.ctas_per_sm(256, 256, regs_per_thread=64) == 4
    assert pairing.fill(48, 192, 198656) == pytest.approx(48 / 148) and pairing.fill(1000, 192, 198656) == 1.0
    # two operators that each leave two thirds of the SMs idle overlap completely: the longer one plus the overhead
    a = pairing.advise(8.0, 6.0, (48, 192, 198656), (48, 192, 198656), model={})       # model = {}: the analytic core alone
    assert a["predicted_fused_us"] == pytest.approx(8.0 + pairing.OVERHEAD_US) and a["fuse"] and a["pattern"] == "zigzag"
    # two operators that fill the GPU alone gain nothing
    b = pairing.advise(50.0, 50.0, (300, 192, 198656), (300, 192, 198656), model={})
    assert b["predicted_fused_us"] == pytest.approx(101.0) and not b["fuse"]
    recs = [dict(t_a=8.0, t_b=6.0, launch_a=(48, 192, 198656), launch_b=(48, 192, 198656), fused_us=9.0, sequential_us=14.0),
            dict(t_a=50.0, t_b=50.0, launch_a=(300, 192, 198656), launch_b=(300, 192, 198656), fused_us=102.0, sequential_us=100.0),
            dict(t_a=50.0, t_b=50.0, launch_a=(300, 192, 198656), launch_b=(300, 192, 198656), fused_us=95.0, sequential_us=100.0)]
    ev = pairing.evaluate(recs, model={})
    assert (ev["pairs"], ev["advice_fuse_and_pays"], ev["advice_alone_and_slower"], ev["advice_alone_but_pays"]) == (3, 1, 1, 1)
    assert ev["median_rel_err"] == pytest.approx(1.0 / 102.0)


def test_pairing_model_fit_recovers_a_planted_rule_and_names_patterns():
    """Least-squares fit per pattern and class pair: planted linear rules come back, the advice names the pattern
    with the smaller predicted time, and the coefficients shipped with the package load and cover every pattern."""
    import random
    from bfuse_project_b200 import pairing
    rnd = random.Random(0)
    recs = []
    for i in range(200):
        ta, tb = rnd.uniform(3, 40), rnd.uniform(3, 40)
        la, lb = (rnd.choice([24, 48, 96, 300]), 192, 198656), (rnd.choice([24, 48, 96, 300]), 192, 198656)
        fa, fb = pairing.fill(*la), pairing.fill(*lb)
        core = max(max(ta, tb), fa * ta + fb * tb)
        # planted: zig-zag = core + 1; range split is better by 10 % of the shorter operator when one operator is twice the other
        zz = core + 1.0
        rg = core + 1.0 - 0.1 * min(ta, tb) + 0.02 * (ta + tb)
        recs.append(dict(pair="p%03d" % i, t_a=ta, t_b=tb, launch_a=la, launch_b=lb, op_a=6, op_b=6, fused_us=zz, sequential_us=ta + tb,
                         fused_us_by_pattern={"zigzag": zz, "range": rg}))
    w = pairing.fit(recs)
    assert set(w) == set(pairing.PATTERNS) and w["zigzag"]["gemm|gemm"][:4] == pytest.approx([1.0, 1.0, 0.0, 0.0], abs=1e-3)
    assert w["range"]["*"][:4] == pytest.approx([1.0, 1.0, -0.1, 0.02], abs=1e-3) and not w["striped"]
    ev = pairing.evaluate(recs, model=w)
    assert ev["median_rel_err"] < 1e-3 and ev["pattern_within_2_pct_of_best"] == 1.0
    shipped = pairing.load_model()
    assert shipped and set(shipped) == set(pairing.PATTERNS) and all("*" in t and len(t["*"]) == 5 for t in shipped.values())
    adv = pairing.advise(7.3, 7.3, (48, 192, 198656), (48, 192, 198656), op_a=6, op_b=6)
    assert adv["pattern"] in pairing.PATTERNS and adv["fuse"] and 7.0 < adv["predicted_fused_us"] < 10.0


def test_leftovers_of_two_bodies_share_one_group():
    """Ready operators that no same-body group took: two of different bodies are a pair, three or four drawn from
    two bodies one group; a third body waits for its own launch."""
    ops = [sg.SegmentOp("g%d" % i, bf.OP_GEMM_TF32, None, ["x"], ["y%d" % i]) for i in range(5)] + \
          [sg.SegmentOp("ln", bf.OP_LAYERNORM_F32, None, ["x"], ["z"]), sg.SegmentOp("sm", bf.OP_SOFTMAX_F32, None, ["x"], ["p"]),
           sg.SegmentOp("sm2", bf.OP_SOFTMAX_F32, None, ["x"], ["p2"]), sg.SegmentOp("sm3", bf.OP_SOFTMAX_F32, None, ["x"], ["p3"])]
    steps = sg.schedule(ops, rule=lambda group: True)
    assert len(steps) == 1
    kinds = sorted((kind, tuple(idx)) for kind, idx in steps[0])
    # 5 GEMMs -> 3 + 2; 3 softmaxes -> one group; the LayerNorm, for which no partner is left, joins the first group with room
    assert kinds == [("group", (0, 1, 2, 5)), ("group", (3, 4)), ("group", (6, 7, 8))]
    ops2 = [sg.SegmentOp("g", bf.OP_GEMM_TF32, None, ["x"], ["y"]), sg.SegmentOp("ln", bf.OP_LAYERNORM_F32, None, ["x"], ["z"]),
            sg.SegmentOp("r1", bf.OP_ROPE_BF16, None, ["x"], ["a"]), sg.SegmentOp("n1", bf.OP_RMSNORM_BF16, None, ["x"], ["b"]),
            sg.SegmentOp("cv", bf.OP_CONV2D_TF32, None, ["x"], ["c"])]
    steps = sg.schedule(ops2, rule=lambda group: True)
    assert sorted((kind, tuple(idx)) for kind, idx in steps[0]) == [("pair", (0, 1)), ("pair", (2, 3)), ("single", (4,))]
