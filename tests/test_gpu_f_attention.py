"""The attention-block chain (QK^T -> softmax -> PV per head group): the software-pipelined schedule
with horizontally fused steps writes the same bits as the plain sequence of launches, and both agree
with a float64 restatement within the tensor-core tolerance."""
import numpy as np
import pytest

import bfuse_project_b200 as bf
from bfuse_project_b200 import attention

pytestmark = pytest.mark.gpu


def reference_attention(q, k, vt):
    """float64 restatement: softmax(QK^T / sqrt(d) + causal mask) V, with V given transposed."""
    q, k, vt = (np.asarray(a, np.float64) for a in (q, k, vt))
    heads, seq, d = q.shape
    s = np.einsum("hmd,hnd->hmn", q, k) / np.sqrt(d)
    s = np.where(np.triu(np.ones((seq, seq), bool), 1)[None], -np.inf, s)
    p = np.exp(s - s.max(-1, keepdims=True))
    p /= p.sum(-1, keepdims=True)
    return np.einsum("hmn,hdn->hmd", p, vt)


@pytest.mark.parametrize("heads,seq,d,groups", [(4, 256, 64, 2), (6, 128, 32, 3), (12, 512, 64, 4)])
def test_pipelined_attention_equals_sequential_and_reference(heads, seq, d, groups):
    import torch
    rt = bf.Runtime(0)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(heads * 1000 + seq)
    q, k = (torch.randn(heads, seq, d, device="cuda", generator=gen) for _ in range(2))
    vt = torch.randn(heads, d, seq, device="cuda", generator=gen)
    blk = attention.AttentionBlock(rt, torch, q, k, vt, groups=groups)
    assert blk.launches_sequential == 3 * groups and blk.launches_pipelined == 2 * groups
    stream = torch.cuda.current_stream().cuda_stream
    blk.run_sequential(stream)
    torch.cuda.synchronize()
    seq_out, seq_probs = blk.out.clone(), blk.probs.clone()
    blk.out.zero_(), blk.probs.zero_(), blk.scores.zero_()
    blk.run_pipelined(stream)
    torch.cuda.synchronize()
    assert rt.read_status() == 0
    assert torch.equal(blk.out, seq_out) and torch.equal(blk.probs, seq_probs)
    want = reference_attention(q.cpu().numpy(), k.cpu().numpy(), vt.cpu().numpy())
    got = blk.out.cpu().numpy().astype(np.float64)
    rms = np.sqrt((want ** 2).mean())
    assert np.abs(got - want).max() <= 5e-3 * rms + 5e-3 * np.abs(want).max()   # tf32 operands, twice
    # rows of the probabilities sum to one and the mask holds
    p = blk.probs.cpu().numpy()
    assert np.allclose(p.sum(-1), 1.0, atol=1e-5) and np.all(np.triu(p[0], 1) == 0)
    rt.close()
