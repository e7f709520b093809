"""n-way groups and the model-segment driver on the GPU: the scheduled program (groups, pairs,
singles) writes the same bits as one launch per operator, and the grouped projections agree with
the CPU oracle within the tensor-core tolerance."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
import oracle
from bfuse_project_b200 import segment as sg

pytestmark = pytest.mark.gpu


def _written(builder, ops):
    return sorted({w for o in ops for w in o.writes})


def _run_both(rt, torch, builder, ops, pattern=bf.ZIGZAG, max_group=4, rule=sg.default_rule):
    seg = sg.Segment(rt, ops, pattern=pattern, max_group=max_group, rule=rule)
    stream = torch.cuda.current_stream().cuda_stream
    names = _written(builder, ops)

    def run(program):
        for n in names:
            builder.buf[n].zero_()
        program(stream)
        torch.cuda.synchronize()
        assert rt.read_status() == 0
        return {n: builder.buf[n].clone() for n in names}

    unfused, alone, fused = run(seg.run_unfused), run(seg.run_sequential), run(seg.run_fused)
    for n in names:
        # same kernels launched one by one: the same bits
        assert torch.equal(fused[n].view(torch.uint8), unfused[n].view(torch.uint8)), n
        # every operator tiled for the whole GPU: the same sums in another order (k-slices), along a chain of operators
        a, f = alone[n].float(), fused[n].float()
        tol = 2e-2 if alone[n].dtype == torch.bfloat16 else 2e-3
        assert float((a - f).abs().max()) <= tol * (float(a.pow(2).mean().sqrt()) + float(a.abs().max())), n
    return seg


def test_qkv_three_way_group_matches_unfused_and_oracle():
    import torch
    rt = bf.Runtime(0)
    b, ops = sg.bert_layer(rt, torch, seq=256, hidden=384, heads=6, ffn=1024, seed=3)
    seg = _run_both(rt, torch, b, ops)
    assert seg.describe()[0] == [("group", ["q_proj", "k_proj", "v_proj"])]
    assert seg.launches_sequential == 11 and seg.launches_fused == 9
    x = b.buf["x"].cpu().numpy()
    for n in "qkv":
        want = oracle.gemm_nt(x[None], b.buf["w" + n].cpu().numpy()[None], b.buf["b" + n].cpu().numpy(), tf32=True)[0]
        got = b.buf[n].cpu().numpy()
        rms = np.sqrt((want.astype(np.float64) ** 2).mean())
        assert np.abs(got - want).max() <= 5e-3 * rms + 5e-3 * np.abs(want).max(), n
    # the group's record and its dispatch: every virtual block of every kernel exactly once
    kind, handle, idx = seg.steps[0][0]
    info = rt.group_info(handle)
    assert info["KernelName"] == "q_proj_k_proj_v_proj_fused_bfuse"
    grid = info["GridDim"][0]
    seen = {}
    for cta in range(grid):
        m = rt.group_map_block(handle, cta)
        if m is not None:
            seen.setdefault(m[0], []).append(m[1])
    assert sorted(seen) == [0, 1, 2] and all(sorted(v) == list(range(len(v))) for v in seen.values())
    assert rt.group_map_block(handle, grid) is None
    rt.close()


@pytest.mark.parametrize("pattern", [bf.ZIGZAG, bf.PROPORTIONAL, bf.RANGE_SPLIT])
def test_requests_grouped_four_ways_every_pattern(pattern):
    """Four independent requests of a (reduced) BERT layer: every operator runs as a 4-way group --
    tcgen05 GEMMs (clustered where the runtime split K), batch-matmuls, softmax and LayerNorm."""
    import torch
    rt = bf.Runtime(0)
    b, ops = sg.bert_layer(rt, torch, replicas=4, seq=128, hidden=256, heads=4, ffn=512, seed=4)
    seg = _run_both(rt, torch, b, ops, pattern=pattern)
    assert seg.launches_sequential == 44 and seg.launches_fused == 11
    rt.close()


def test_llama_projections_and_resnet_stages_full_size():
    import torch
    rt = bf.Runtime(0)
    b, ops = sg.llama_layer_projections(rt, torch, seed=5)
    seg = _run_both(rt, torch, b, ops)
    assert ("group", ["q_proj", "k_proj", "v_proj"]) in seg.describe()[1]
    assert ("group", ["rope_q", "rope_k"]) in seg.describe()[2]
    b2, ops2 = sg.resnet18_stages(rt, torch, batch=2, seed=6)
    seg2 = _run_both(rt, torch, b2, ops2)
    assert seg2.launches_fused == 12
    rt.close()


@pytest.mark.parametrize("pattern", [bf.ZIGZAG, bf.PROPORTIONAL, bf.RANGE_SPLIT])
def test_groups_of_two_bodies(pattern):
    """Up to four kernels of TWO operator bodies in one launch (the reference's patterns are written for n arbitrary
    kernels, horizontal-fuser/src/Algorithms.cc:538-587): three tensor-core projections beside a residual LayerNorm,
    two LayerNorms beside two softmaxes, a tcgen05 GEMM whose K is split over clusters beside row-wise operators
    (padding CTAs of partly filled clusters), a conv beside a GEMM.  The decode equals the n-kernel oracle, and the
    group writes the bits of the unfused launches."""
    import numpy as np
    import oracle
    from bfuse_project_b200 import workloads as wl
    rt = bf.Runtime(0)
    rng = np.random.default_rng(31)
    m, n = (1, 1) if pattern == bf.ZIGZAG else ((1, 0) if pattern == bf.PROPORTIONAL else (0, 0))
    q, k = wl.make_pair("cfg2_q_k_proj", seed=3, scale=0.5).a, wl.make_pair("cfg2_q_k_proj", seed=4, scale=0.5).b
    v = wl.gemm("v_proj", rng, bf.OP_GEMM_TF32, 1, 256, 768, 768, bias=True)
    ln = wl.layernorm("ln", rng, 256, 768, 1e-5, residual=True)
    ln2 = wl.layernorm("ln2", rng, 100, 768, 1e-5)
    sm1, sm2 = wl.softmax("sm1", rng, 1536, 512, 0.125), wl.softmax("sm2", rng, 333, 256, 1.0)
    gs = wl.gemm("gsplit", rng, bf.OP_GEMM_TF32, 1, 256, 256, 1024, w_std=1.0, bn=256, split=4)
    cv = wl.conv2d("conv", rng, bf.OP_CONV2D_TF32, 2, 64, 28, 28, 128, 3, 1, 1)
    for members in ([q, k, v, ln], [ln, sm1, ln2, sm2], [gs, ln2, ln], [cv, q], [sm2, q]):
        pairs = [wl.DevicePair(rt, wl.PairSpec("m", ks, wl.softmax("pad", rng, 8, 128, 1.0), "f32", "hbm")) for ks in members]
        kernels = [p.kernels[0] for p in pairs]
        for p in pairs:
            rt.launch_kernel(p.kernels[0])
        want = [p.read_outputs()[0][0].copy() for p in pairs]
        for p in pairs:
            p.clear_outputs()
        group = rt.register_group(kernels, pattern, m, n)
        info = rt.group_info(group)
        rt.launch_group(group)
        got = [p.read_outputs()[0][0] for p in pairs]
        assert rt.read_status() == 0
        for ks, w, g in zip(members, want, got):
            assert np.array_equal(w.view(np.uint8), g.view(np.uint8)) and np.any(g != 0), (ks.name, bf.PATTERN_NAMES[pattern])
        # every CTA of the fused grid maps to one virtual block of one member, each exactly once
        seen = {}
        for cta in range(info["GridDim"][0]):
            mapped = rt.group_map_block(group, cta)
            if mapped is not None:
                seen.setdefault(mapped[0], []).append(mapped[1])
        assert sorted(seen) == list(range(len(members)))
        for i, ks in enumerate(members):
            grid = ks.launch[0]
            assert sorted(seen[i]) == list(range(grid[0] * grid[1] * grid[2])), ks.name
        rt.unregister_group(group)
    rt.close()


def test_segment_scheduled_by_the_pair_selection_model():
    """rule = "model": every operator is timed alone at registration, the model decides what shares a launch and
    names the pattern of every pair; the program still writes the bits of its kernels launched one by one."""
    import torch
    rt = bf.Runtime(0)
    b, ops = sg.llama_layer_projections(rt, torch, seed=8)
    seg = _run_both(rt, torch, b, ops, rule="model")
    assert all(o.alone_us is not None and o.alone_us > 0 and o.launch is not None for o in ops)
    assert seg.launches_fused < seg.launches_sequential
    b2, ops2 = sg.bert_layer(rt, torch, replicas=2, seq=128, hidden=256, heads=4, ffn=512, seed=9)
    seg2 = _run_both(rt, torch, b2, ops2, rule="model")
    assert seg2.launches_fused < seg2.launches_sequential
    rt.close()


def test_group_registration_errors():
    import torch
    rt = bf.Runtime(0)
    b, ops = sg.bert_layer(rt, torch, seq=128, hidden=256, heads=4, ffn=512, seed=7)
    seg = sg.Segment(rt, ops)
    by_name = {o.name: k for o, k in zip(ops, seg.alone)}
    with pytest.raises(bf.BfuseError) as e:       # three bodies: a kernel exists per body and per pair of bodies
        rt.register_group([by_name["q_proj"], by_name["softmax"], by_name["ln1"]], bf.ZIGZAG, 1, 1)
    assert e.value.code == 7
    for pat in (bf.SM_STRIPED, bf.THREAD_SPLIT, bf.WORK_QUEUE):
        with pytest.raises(bf.BfuseError) as e:
            rt.register_group([by_name["q_proj"], by_name["k_proj"]], pat, 1, 1)
        assert e.value.code == 7
    with pytest.raises(bf.BfuseError) as e:
        rt.register_group([by_name["q_proj"]], bf.ZIGZAG, 1, 1)
    assert e.value.code == 1
    with pytest.raises(bf.BfuseError) as e:
        rt.register_group([by_name["q_proj"], 10 ** 6], bf.ZIGZAG, 1, 1)
    assert e.value.code == 1
    rt.close()


def test_trace_files_of_a_pair(tmp_path):
    """The five per-mode timing files of one pair, named and laid out as the reference's analysis expects."""
    import torch
    from bfuse_project_b200 import trace_csv
    rt = bf.Runtime(0)
    b, ops = sg.bert_layer(rt, torch, seq=128, hidden=256, heads=4, ffn=512, seed=9)
    seg = sg.Segment(rt, ops)
    k = {o.name: h for o, h in zip(ops, seg.alone)}
    paths = trace_csv.emit_pair(rt, torch, str(tmp_path), 2, 5, k["softmax"], k["ln1"], "softmax", "ln1", warmup=3, trials=5)
    names = sorted(p.rsplit("/", 1)[1] for p in paths)
    assert names == ["0_2_0_cuda_gpu_trace.csv", "1_0_5_cuda_gpu_trace.csv", "2_2_5_cuda_gpu_trace.csv", "3_2_5_cuda_gpu_trace.csv",
                     "4_2_5_cuda_gpu_trace.csv"]
    for p in paths:
        rows = trace_csv.read_gpu_trace(p)
        mode = int(p.rsplit("/", 1)[1][0])
        assert len(rows) == (16 if mode == 2 else 8)
        assert all(d > 0 for _, d, _ in rows) and all(rows[i][0] <= rows[i + 1][0] for i in range(len(rows) - 1))
        want = {0: {"softmax"}, 1: {"ln1"}, 2: {"softmax", "ln1"}, 3: {"softmax_ln1_fused_hfuse"}, 4: {"softmax_ln1_fused_bfuse"}}[mode]
        assert {n for _, _, n in rows} == want
    assert rt.read_status() == 0
    rt.close()


def test_group_with_clustered_members():
    """A group whose members split K over clusters of 4, beside an unsplit member that is scheduled in
    padded clusters: same bits as the unfused launches, every virtual block exactly once."""
    import torch
    rt = bf.Runtime(0)
    b = sg._Builder(rt, torch, seed=11)
    M, N, K = 256, 192, 1024
    b.tensor("x", (M, K))
    for i, (bn, split) in enumerate(((64, 4), (128, 4), (64, 1))):
        b.tensor("w%d" % i, (N, K), std=0.05)
        b.tensor("y%d" % i, (M, N), zero=True)
        b._add("g%d" % i, bf.OP_GEMM_TF32, (1, M, N, K, bn, split, 0), ["x", "w%d" % i, None, "y%d" % i], ["x", "w%d" % i], ["y%d" % i])
    ks = [o.register(rt, 3) for o in b.ops]
    stream = torch.cuda.current_stream().cuda_stream
    for k in ks:
        rt.launch_kernel(k, stream)
    torch.cuda.synchronize()
    want = [b.buf["y%d" % i].clone() for i in range(3)]
    for pattern in (bf.ZIGZAG, bf.RANGE_SPLIT):
        for i in range(3):
            b.buf["y%d" % i].zero_()
        g = rt.register_group(ks, pattern, 1 if pattern == bf.ZIGZAG else 0, 1 if pattern == bf.ZIGZAG else 0)
        rt.launch_group(g, stream)
        torch.cuda.synchronize()
        assert rt.read_status() == 0
        for i in range(3):
            assert torch.equal(b.buf["y%d" % i], want[i]) and bool(want[i].abs().sum() > 0)
        info = rt.group_info(g)
        assert info["GridDim"][0] % 4 == 0
        seen = {}
        for cta in range(info["GridDim"][0]):
            m = rt.group_map_block(g, cta)
            if m is not None:
                seen.setdefault(m[0], []).append(m[1])
        assert all(sorted(v) == list(range(len(v))) for v in seen.values()) and sorted(seen) == [0, 1, 2]
    ref = (b.buf["x"].double() @ b.buf["w0"].double().T).float()
    assert float((want[0] - ref).abs().max()) <= 5e-3 * float(ref.abs().max())
    with pytest.raises(bf.BfuseError) as e:       # clusters of 2 and of 4 cannot share a launch
        odd = sg.SegmentOp("g2", bf.OP_GEMM_TF32, None, ["x"], ["y2"], spec=((1, M, N, K, 64, 2, 0), [b.buf["x"].data_ptr(), b.buf["w2"].data_ptr(), None, b.buf["y2"].data_ptr()], {}))
        rt.register_group([ks[0], odd.register(rt, 2)], bf.ZIGZAG, 1, 1)
    assert e.value.code == 7
    rt.close()
