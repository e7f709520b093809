"""The cross-product sweep on a handful of its operators: every pair fuses, times are positive, and
the fused launch of a mixed pair writes the same bits as the two unfused launches."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
from bfuse_project_b200 import sweep

pytestmark = pytest.mark.gpu


def test_sweep_subset_runs_and_fused_equals_unfused():
    import torch
    rt = bf.Runtime(0)
    ops = [o for o in sweep.SWEEP_OPS if o[0] in ("dense_0", "bgemm_10", "conv2d_5", "conv2d_13")]
    sets = sweep.build_operands(rt, torch, 0, seed=3, ops=ops)
    res = sweep.measure(rt, sets, sweep.pair_indices(len(ops)), 6545.0, 826.0, warmup=1, iters=3)
    assert len(res) == 10 and all("error" not in v and v["fused_us"] > 0 and v["sequential_us"] > 0 for v in res.values())
    summary = sweep.summarise(res)
    assert summary["pairs"] == 10 and summary["errors"] == 0
    # bit-exactness on the mixed tensor-core / CUDA-core pair
    a, b = sets[0][1], sets[1][3]
    f = rt.register_fusion(a.kernel, b.kernel, bf.ZIGZAG, 1, 1)
    stream = torch.cuda.current_stream().cuda_stream
    rt.launch_sequential(f, stream)
    torch.cuda.synchronize()
    want = [a.bufs[2].clone(), b.bufs[2].clone()]
    a.bufs[2].zero_(), b.bufs[2].zero_()
    rt.launch_fused(f, stream)
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert torch.equal(a.bufs[2], want[0]) and torch.equal(b.bufs[2], want[1])
    assert float(want[0].abs().max()) > 0 and float(want[1].abs().max()) > 0
    rt.close()
