"""Host logic of the operator cross-product sweep (no GPU): enumeration, partition, body choice, summary."""
from bfuse_project_b200 import partition, sweep


def test_sweep_enumerates_the_upper_triangle_of_42_operators():
    assert len(sweep.SWEEP_OPS) == 42
    kinds = [n.split("_")[0] for n, _ in sweep.SWEEP_OPS]
    assert (kinds.count("dense"), kinds.count("bgemm"), kinds.count("conv2d")) == (8, 12, 22)
    pairs = sweep.pair_indices()
    assert len(pairs) == 42 * 43 // 2 and pairs[0] == (0, 0) and pairs[-1] == (41, 41)
    assert all(j >= i for i, j in pairs) and len(set(pairs)) == len(pairs)


def test_sweep_pairs_are_dealt_to_every_rank_exactly_once():
    pairs = sweep.pair_indices()
    for world in (1, 2, 4, 8):
        dealt = [partition.assign_pairs(pairs, world, r) for r in range(world)]
        assert sorted(p for d in dealt for p in d) == sorted(pairs)
        assert max(len(d) for d in dealt) - min(len(d) for d in dealt) <= 1


def test_conv_body_choice_follows_the_tensor_core_body_limits():
    shapes = dict(sweep.SWEEP_OPS)
    assert not sweep.conv_on_tensor_cores(shapes["conv2d_0"])      # 7x7 window, K = 147
    assert sweep.conv_on_tensor_cores(shapes["conv2d_3"])          # the ResNet branch pair
    assert sweep.conv_on_tensor_cores(shapes["conv2d_5"])
    assert sweep.conv_on_tensor_cores(shapes["conv2d_4"])          # K = 1152: the offset table grows with K
    assert sweep.conv_on_tensor_cores(shapes["conv2d_10"])         # K = 4608, 7 x 7 = 49 output pixels
    assert sweep.conv_on_tensor_cores(shapes["conv2d_12"])         # 35 x 35 outputs: rows stored by the body itself
    assert sum(sweep.conv_on_tensor_cores(sh) for n, sh in sweep.SWEEP_OPS if n.startswith("conv2d")) == 21


def test_summary_counts_and_geomean():
    res = {"dense_0|dense_1": {"fused_us": 10.0, "sequential_us": 20.0, "speedup_vs_sequential": 2.0, "roofline_us": 1, "roofline_frac": .1},
           "dense_0|conv2d_1": {"fused_us": 10.0, "sequential_us": 5.0, "speedup_vs_sequential": 0.5, "roofline_us": 1, "roofline_frac": .1},
           "bgemm_0|bgemm_0": {"error": "x"}}
    s = sweep.summarise(res)
    assert s["pairs"] == 2 and s["errors"] == 1
    assert abs(s["geomean_speedup_vs_sequential"] - 1.0) < 1e-12
    assert s["pairs_5pct_faster"] == 1 and s["pairs_5pct_slower"] == 1
    assert set(s["geomean_speedup_by_kinds"]) == {"densexdense", "conv2dxdense"}
