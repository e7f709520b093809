"""On the GPU: the fused grid decodes its dispatch table exactly as the oracle (and therefore the
reference's printed conditions) says, for every pattern, including the persistent work queue."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
import oracle
from bfuse_project_b200 import workloads as wl

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def rt():
    r = bf.Runtime(0)
    yield r
    r.close()


@pytest.fixture(scope="module")
def pair(rt):
    return wl.DevicePair(rt, wl.make_pair("cfg1_softmax_layernorm", seed=1, scale=0.5))


def dims_of(pair):
    out = []
    for ks in (pair.spec.a, pair.spec.b):
        g, b, _ = ks.launch
        out.append(list(g) + list(b))
    return out


@pytest.mark.parametrize("pattern,name,kw,m,n", [
    (bf.ZIGZAG, "zigzag", dict(M=1, N=1), 1, 1), (bf.ZIGZAG, "zigzag", dict(M=4, N=2), 4, 2),
    (bf.PROPORTIONAL, "proportional", dict(min_option=2), 2, 0), (bf.RANGE_SPLIT, "range_split", {}, 0, 0),
    (bf.SM_STRIPED, "sm_striped", dict(total_sm=148), 148, 0), (bf.SM_STRIPED, "sm_striped", dict(total_sm=84), 84, 0)])
def test_device_decode_equals_oracle(rt, pair, pattern, name, kw, m, n):
    f = pair.fusion(pattern, m, n)
    kern, vb, sm = rt.trace_fused(f)
    o = oracle.plan(name, dims_of(pair), **kw)
    ok, ovb = oracle.block_table(o)
    assert np.array_equal(kern, ok) and np.array_equal(vb, ovb)
    assert sm.min() >= 0 and sm.max() < rt.sm_count
    info = rt.fusion_info(f)
    assert info["GridDim"] == (o.fused_grid, 1, 1) and info["BlockDim"] == (o.fused_block, 1, 1)
    assert info["KernelName"] == "softmax_layernorm_fused_bfuse"
    for b in (0, 1, o.fused_grid - 1):
        assert rt.map_block(f, b) == (int(ok[b]), int(ovb[b]))
    assert rt.map_block(f, o.fused_grid) is None


def test_sm_striped_defaults_to_the_device_sm_count(rt, pair):
    f = pair.fusion(bf.SM_STRIPED, 0, 0)
    kern, vb, _ = rt.trace_fused(f)
    o = oracle.plan("sm_striped", dims_of(pair), total_sm=rt.sm_count)
    ok, ovb = oracle.block_table(o)
    assert np.array_equal(kern, ok) and np.array_equal(vb, ovb)


def test_work_queue_hands_out_every_ticket_once_and_resets(rt, pair):
    f = pair.fusion(bf.WORK_QUEUE, 1, 1)
    o = oracle.plan("zigzag", dims_of(pair))
    ok, ovb = oracle.block_table(o)
    info = rt.fusion_info(f)
    assert info["launched_ctas"] <= o.fused_grid
    for _ in range(3):  # the counters reset themselves, so repeated launches must agree
        kern, vb, sm = rt.trace_fused(f)
        assert np.array_equal(kern, ok) and np.array_equal(vb, ovb)
    assert len(np.unique(sm)) > rt.sm_count // 2
    assert rt.read_status() == 0


def test_thread_split_info(rt, pair):
    f = pair.fusion(bf.THREAD_SPLIT)
    info = rt.fusion_info(f)
    d = dims_of(pair)
    o = oracle.plan("thread_split", d)
    assert info["GridDim"] == (o.fused_grid, 1, 1) and info["BlockDim"] == (o.fused_block, 1, 1)
    assert info["KernelName"] == "softmax_layernorm_fused_hfuse"
    with pytest.raises(bf.BfuseError):
        rt.trace_fused(f)


def test_fused_timeline_marks_every_slot_in_launch_order(rt, pair):
    """The per-CTA time marks of the real fused kernel: every dispatch slot of every launch records
    entry <= body start <= body end, and a launch's CTAs end only after all of the previous launch's
    have (stream order holds under programmatic dependent launch: a body may set itself up while the
    previous kernel drains, but waits for it before touching global memory)."""
    fus = [pair.fusion(bf.ZIGZAG, 1, 1), pair.fusion(bf.RANGE_SPLIT, 0, 0), pair.fusion(bf.WORK_QUEUE, 1, 1)]
    marks = rt.fused_timeline(fus)
    assert len(marks) == 3
    for m, f in zip(marks, fus):
        assert m.shape == (rt.fusion_info(f)["GridDim"][0], 3)
        assert (m > 0).all() and (m[:, 0] <= m[:, 1]).all() and (m[:, 1] <= m[:, 2]).all()
    assert marks[1][:, 2].min() >= marks[0][:, 2].max() and marks[2][:, 2].min() >= marks[1][:, 2].max()
    assert rt.read_status() == 0


def test_which_operators_share_an_sm(rt):
    """The effect the patterns exist for is which operators end up on the same SM (the reference looks at
    it through %smid logs, tests/interleave_scheduler/test/test_scheduler.py:40-120).  The hardware deals
    consecutive CTAs to the two SMs of a TPC in turn, so under strict 1 : 1 alternation even CTAs -- one
    operator -- land on even SMs and odd CTAs on odd SMs: no SM hosts both operators, the pattern acts as
    a split of every TPC.  Runs of two (M = 1, N = 2) put both operators on at least 80 % of the SMs.
    The range split gives the whole first round of CTAs to the first operator."""
    rng = np.random.default_rng(2)
    a = wl.softmax("sm", rng, 6144, 512, 0.125)       # 768 CTAs
    b = wl.layernorm("ln", rng, 3072, 768, 1e-5)      # 768 CTAs
    pair = wl.DevicePair(rt, wl.PairSpec("mix", a, b, "f32", "hbm"))
    assert a.launch[0][0] == b.launch[0][0] == 768

    def sms_with_both(pattern, m, n):
        kern, _, sm = rt.trace_fused(pair.fusion(pattern, m, n))
        both = sum(len(set(kern[sm == s].tolist())) == 2 for s in range(rt.sm_count))
        return both / rt.sm_count, kern, sm

    runs_of_two, _, _ = sms_with_both(bf.ZIGZAG, 1, 2)
    strict, kern, sm = sms_with_both(bf.ZIGZAG, 1, 1)
    print("SMs that host both operators: zig-zag 2:2 %.2f, 1:1 %.2f" % (runs_of_two, strict))
    assert runs_of_two >= 0.8
    assert strict <= 0.2
    assert all(len(set((np.nonzero(sm == s)[0] % 2).tolist())) <= 1 for s in range(rt.sm_count))   # an SM sees CTAs of one parity
    _, kern, sm = sms_with_both(bf.RANGE_SPLIT, 0, 0)
    assert set(kern[:rt.sm_count].tolist()) == {0}
