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


def _run_both(rt, torch, builder, ops, pattern=bf.ZIGZAG, max_group=4):
    seg = sg.Segment(rt, ops, pattern=pattern, max_group=max_group)
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


def test_group_registration_errors():
    import torch
    rt = bf.Runtime(0)
    b, ops = sg.bert_layer(rt, torch, seq=128, hidden=256, heads=4, ffn=512, seed=7)
    seg = sg.Segment(rt, ops)
    by_name = {o.name: k for o, k in zip(ops, seg.alone)}
    with pytest.raises(bf.BfuseError) as e:       # different bodies
        rt.register_group([by_name["q_proj"], by_name["softmax"]], bf.ZIGZAG, 1, 1)
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
