"""A causal self-attention block built from the runtime's registered operators, the step on either
side of the reference's attention pairs (the QK^T / softmax / PV chain of its GPT-2 and BERT dumps,
files/gpt2.txt:32-45, files/bert-base-uncased.txt:38-52; operator shapes bgemm_0 / bgemm_1 of
test-utils/examples/llm.yaml:38-49).

The heads are split into groups.  Per group g the chain is

    S_g = Q_g K_g^T with the causal mask     (tcgen05 batch-matmul, masked entries = -FLT_MAX)
    P_g = softmax(S_g / sqrt(d)) row-wise    (row-wise body)
    O_g = P_g V_g                            (tcgen05 batch-matmul; V is taken as V^T [heads, d, seq],
                                              the [N, K] weight layout of the reference's batch_matmul)

Within a group the three steps depend on each other; across groups they do not.  `sequential` runs
3 launches per group.  `pipelined` software-pipelines the groups so that the independent steps of
neighbouring groups share one horizontally fused launch -- QK^T(g+1) beside softmax(g), and the
last softmax beside the previous group's PV -- which is the reference's idea (fuse two independent
kernels) applied along a dependency chain: G >= 2 groups take 2 G launches instead of 3 G.
"""
import math

from . import FLAG_CAUSAL, OP_GEMM_TF32, OP_SOFTMAX_F32, ZIGZAG


class AttentionBlock:
    def __init__(self, rt, torch, q, k, vt, groups=2, device=0, pattern=ZIGZAG, gemm_bn=0, gemm_stages=4):
        """q, k: [heads, seq, d] fp32 CUDA tensors; vt: [heads, d, seq] (V transposed); groups divides heads.
        gemm_bn / gemm_stages: tile width and ring depth of the two batch-matmuls (gemm_bn = 0: the
        runtime's own choice, the default).  A fused launch charges every CTA the larger of the two
        operators' shared-memory windows, so narrow tiles with a shallow ring leave the softmax's small
        CTAs more room; measured, that is worth a few per cent at 4 groups and costs 8 % unsplit."""
        heads, seq, d = q.shape
        if heads % groups:
            raise ValueError("groups must divide heads")
        self.rt, self.torch, self.groups = rt, torch, groups
        self.hg = heads // groups
        dev = q.device
        self.scores = torch.empty(heads, seq, seq, device=dev, dtype=torch.float32)
        self.probs = torch.empty(heads, seq, seq, device=dev, dtype=torch.float32)
        self.out = torch.zeros(heads, seq, d, device=dev, dtype=torch.float32)
        self.keep = (q, k, vt)
        scale = 1.0 / math.sqrt(d)
        self.qk, self.sm, self.pv = [], [], []
        for g in range(groups):
            sl = slice(g * self.hg, (g + 1) * self.hg)
            def ring(kdim):  # shared-memory bytes of a ring of gemm_stages (or fewer, for short K) stages
                if not gemm_bn:
                    return None
                return 2048 + max(1, min(gemm_stages, -(-kdim // 32))) * (128 + gemm_bn) * 128
            dq = rt.describe("qk_g%d" % g, OP_GEMM_TF32, (self.hg, seq, seq, d, gemm_bn, 1),
                             [q[sl].data_ptr(), k[sl].data_ptr(), None, self.scores[sl].data_ptr()], flags=FLAG_CAUSAL,
                             smem=ring(d))
            ds = rt.describe("softmax_g%d" % g, OP_SOFTMAX_F32, (self.hg * seq, seq),
                             [self.scores[sl].data_ptr(), self.probs[sl].data_ptr()], fparam=(scale,))
            dp = rt.describe("pv_g%d" % g, OP_GEMM_TF32, (self.hg, seq, d, seq, min(gemm_bn, 64 if d <= 64 else 128) if gemm_bn else 0, 1),
                             [self.probs[sl].data_ptr(), vt[sl].data_ptr(), None, self.out[sl].data_ptr()], smem=None)
            self.qk.append(rt.register_kernel(dq))
            self.sm.append(rt.register_kernel(ds))
            self.pv.append(rt.register_kernel(dp))
        # the pipelined schedule: per step the operators whose inputs are ready, paired two at a time
        self.steps = []
        for t in range(groups + 2):
            ready = []
            if t < groups:
                ready.append(self.qk[t])
            if 0 <= t - 1 < groups:
                ready.append(self.sm[t - 1])
            if 0 <= t - 2 < groups:
                ready.append(self.pv[t - 2])
            step = []
            while len(ready) >= 2:
                a, b = ready.pop(0), ready.pop(0)
                step.append(("fused", rt.register_fusion(a, b, pattern, 1 if pattern == ZIGZAG else 0, 1 if pattern == ZIGZAG else 0)))
            if ready:
                step.append(("single", ready[0]))
            self.steps.append(step)

    @property
    def launches_pipelined(self):
        return sum(len(s) for s in self.steps)

    @property
    def launches_sequential(self):
        return 3 * self.groups

    def run_sequential(self, stream):
        for g in range(self.groups):
            self.rt.launch_kernel(self.qk[g], stream)
            self.rt.launch_kernel(self.sm[g], stream)
            self.rt.launch_kernel(self.pv[g], stream)

    def run_pipelined(self, stream):
        for step in self.steps:
            for kind, handle in step:
                if kind == "fused":
                    self.rt.launch_fused(handle, stream)
                else:
                    self.rt.launch_kernel(handle, stream)


def graph_time_us(torch, launch, replays=20, warm=3, repeat=1):
    """Microseconds per call of `launch(stream)` replayed from a CUDA graph (device time, CUDA events).
    repeat: calls captured per graph -- replays of a graph start about 2 us apart at the earliest, so a
    program of a few microseconds is captured several times over to be timed to better than that."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch(side.cuda_stream)          # first call outside capture: lazy module loading, attributes
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=side):
        for _ in range(repeat):
            launch(torch.cuda.current_stream().cuda_stream)
    for _ in range(warm):
        g.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (replays * repeat)
