"""Model-segment driver: the caller of the fused launches.

The reference extracts the operator lists of whole models (files/result.txt for ResNet-18, the
Relay dumps files/bert-base-uncased.txt / gpt2.txt, shapes in test-utils/examples/llm.yaml and
resnet-18.yaml) and then fuses hand-picked pairs of them (scripts/configure_kernels.py:157-159).
This module does the picking: it walks an operator list in program order, derives the dependencies
from the buffers each operator reads and writes, and at every step launches the operators whose
inputs are ready --

    * 2..4 ready operators of one body (the Q, K and V projections; the two branches of a
      down-sampling block; the same operator of independent requests) as one n-way group, the
      reference's n-kernel form of its patterns (horizontal-fuser/src/Algorithms.cc:538-587);
    * what that leaves over, when it is of two bodies: two operators as one fused pair, three or four
      as one group of two bodies;
    * what is left alone.

`run_sequential` is the unfused program (one launch per operator, program order, every operator
tiled for the whole GPU); `run_fused` the scheduled one, its operators tiled for their share of the
launch.  `run_unfused` launches the fused program's kernels one by one: same bodies, same tilings, so
bit-identical results (the two tilings of an operator can differ in their k-slices, i.e. in the order
of a sum).
Element-wise glue of the models (ReLU / GELU / SiLU, batch-norm, reshapes and transposes) has no
operator body here: buffers are reinterpreted in the layout the next operator wants, which keeps
every operator's shape and the dependency structure of the layer, not its numerical function.
"""
import math

from . import (FLAG_CAUSAL, MODE_KERNEL1, OP_CONV2D_F32_SIMT, OP_CONV2D_TF32, OP_GEMM_BF16, OP_GEMM_TF32, OP_LAYERNORM_F32,
               OP_RMSNORM_BF16, OP_ROPE_BF16, OP_SOFTMAX_F32, RANGE_SPLIT, SM_STRIPED, THREAD_SPLIT, ZIGZAG, BfuseError, flag_share, pairing)

# the pair-selection model's pattern names -> (pattern, M, N) of bfuse_register_fusion
MODEL_PATTERNS = {"zigzag": (ZIGZAG, 1, 1), "zigzag2": (ZIGZAG, 1, 2), "range": (RANGE_SPLIT, 0, 0), "striped": (SM_STRIPED, 0, 0),
                  "thread_split": (THREAD_SPLIT, 0, 0)}


class SegmentOp:
    """One operator of a segment: its body, the names of the buffers it reads / writes and, when it is
    bound to device buffers, what `Runtime.describe` needs to register it (`spec` = (shape, pointers,
    keyword arguments)).  `kernel` is a ready-made kernel handle for callers that registered it themselves."""

    def __init__(self, name, op, kernel, reads, writes, spec=None):
        self.name, self.op, self.kernel, self.spec = name, op, kernel, spec
        self.reads, self.writes = frozenset(reads), frozenset(writes)
        self.launch, self.alone_us = None, None      # (CTAs, threads, shared memory) alone; microseconds alone, once measured

    def register(self, rt, share):
        """Kernel handle of this operator tiled for `share` operators in one launch (1: alone)."""
        if self.spec is None:
            return self.kernel
        shape, ptrs, kw = self.spec
        kw = dict(kw)
        kw["flags"] = kw.get("flags", 0) | flag_share(share)
        desc = rt.describe(self.name, self.op, shape, ptrs, **kw)
        if share == 1:
            self.launch = (desc.GridDim.size(), desc.BlockDim.size(), desc.smem_bytes)   # what the pair-selection model reads
        return rt.register_kernel(desc)


def dependencies(ops):
    """deps[j] = indices i < j that j must wait for: i writes what j reads (RAW) or writes (WAW),
    or i reads what j writes (WAR)."""
    deps = []
    for j, b in enumerate(ops):
        d = set()
        for i in range(j):
            a = ops[i]
            if (a.writes & b.reads) or (a.writes & b.writes) or (a.reads & b.writes):
                d.add(i)
        deps.append(d)
    return deps


def default_rule(ops):
    """May these ready operators share a launch?  From the operator cross-product sweep: a fused launch
    beats back-to-back launches for every body except the CUDA-core conv, whose long CTAs the
    interleaved order delays."""
    return all(o.op != OP_CONV2D_F32_SIMT for o in ops)


def schedule(ops, max_group=4, rule=default_rule):
    """Steps of the fused program: [[("group" | "pair" | "single", [op indices])]].  Level by level:
    every operator whose dependencies completed in earlier steps is ready; ready operators of one
    body form groups of up to max_group, leftovers of different bodies pair up, the rest run alone."""
    deps = dependencies(ops)
    done, steps = set(), []
    while len(done) < len(ops):
        ready = [i for i in range(len(ops)) if i not in done and deps[i] <= done]
        if not ready:
            raise ValueError("dependency cycle")
        step, left = [], []
        by_body = {}
        for i in ready:
            by_body.setdefault(ops[i].op, []).append(i)
        for body, idx in by_body.items():
            # balanced groups: 5 ready operators -> 3 + 2, 6 -> 3 + 3, never 4 + 1
            ngroups = -(-len(idx) // max_group) if max_group >= 2 else 0
            while ngroups > 0 and len(idx) >= 2:
                take = idx[:-(-len(idx) // ngroups)]
                if len(take) < 2 or not rule([ops[i] for i in take]):
                    break
                step.append(("group", take))
                idx = idx[len(take):]
                ngroups -= 1
            left.extend(idx)
        left.sort()
        lonely = []
        while len(left) >= 2:
            a = left.pop(0)
            # what is left over joins operators of ONE other body: two of them are a fused pair (every pattern),
            # three or four a group of two bodies
            mates = {}
            for b in left:
                if ops[b].op != ops[a].op and rule([ops[a], ops[b]]):
                    mates.setdefault(ops[b].op, []).append(b)
            if not mates:
                lonely.append(a)
                continue
            other = max(mates.values(), key=len)[:max(1, max_group - 1)]
            for b in other:
                left.remove(b)
            step.append(("pair", [a, other[0]]) if len(other) == 1 else ("group", [a] + other))
        # an operator still alone joins a group of one other body that has room for it
        left = sorted(left + lonely)
        for a in list(left):
            host = next((g for kind, g in step if kind == "group" and len(g) < max_group and len({ops[i].op for i in g}) == 1
                         and ops[g[0]].op != ops[a].op and rule([ops[i] for i in g] + [ops[a]])), None)
            if host is not None:
                host.append(a)
                left.remove(a)
        step.extend(("single", [i]) for i in left)
        steps.append(step)
        done.update(ready)
    return steps


def model_rule(ops, sm_count=148, margin=1.0):
    """The pair-selection model as a scheduling rule: operators may share a launch when every pair of them is
    predicted to beat its two launches back to back (pairing.advise on the operators' times alone and launch
    records, which Segment measures at registration)."""
    for i, a in enumerate(ops):
        for b in ops[i + 1:]:
            if a.alone_us is None or b.alone_us is None:
                return default_rule([a, b])
            if not pairing.advise(a.alone_us, b.alone_us, a.launch, b.launch, sm_count, margin, a.op, b.op)["fuse"]:
                return False
    return True


class Segment:
    """A scheduled segment bound to a runtime.  Every operator is registered twice: tiled for the whole
    GPU (the program of one launch per operator, and operators the schedule leaves alone) and tiled for
    its share of the launch it was scheduled into.  With rule = "model" every operator is timed alone at
    registration and the pair-selection model decides what may share a launch, and under which pattern a pair
    runs; the default rule is the sweep's coarse finding and the given pattern."""

    def __init__(self, rt, ops, pattern=ZIGZAG, max_group=4, rule=default_rule):
        self.rt, self.ops = rt, list(ops)
        self.alone = [o.register(rt, 1) for o in self.ops]
        self.shared = list(self.alone)
        self.steps = []
        use_model = rule == "model"
        if use_model:
            for o, k in zip(self.ops, self.alone):
                probe = rt.register_fusion(k, k, RANGE_SPLIT, 0, 0)      # any fusion of the kernel: mode 0 times kernel 1 alone
                o.alone_us = rt.time(probe, MODE_KERNEL1, 3, 10)[0]
                rt.unregister_fusion(probe)
            rule = lambda group: model_rule(group, rt.sm_count)
        m = 1 if pattern == ZIGZAG else 0
        for step in schedule(self.ops, max_group, rule):
            out = []
            for kind, idx in step:
                if kind == "single":
                    out.append(("single", self.alone[idx[0]], idx))
                    continue
                ks = [self.ops[i].register(rt, len(idx)) for i in idx]
                try:
                    if kind == "group":
                        out.append(("group", rt.register_group(ks, pattern, m, m), idx))
                    elif use_model:
                        a, b = self.ops[idx[0]], self.ops[idx[1]]
                        preds = pairing.advise(a.alone_us, b.alone_us, a.launch, b.launch, rt.sm_count, 1.0, a.op, b.op)["predicted_by_pattern"]
                        handle, last = None, None
                        for name in sorted(preds, key=lambda p: preds[p]):     # the best predicted pattern that can host the pair
                            try:
                                handle = rt.register_fusion(ks[0], ks[1], *MODEL_PATTERNS[name])
                                break
                            except BfuseError as e:
                                if e.code not in (3, 7):
                                    raise
                                last = e
                        if handle is None:
                            raise last
                        out.append(("pair", handle, idx))
                    else:
                        out.append(("pair", rt.register_fusion(ks[0], ks[1], pattern, m, m), idx))
                    for i, k in zip(idx, ks):
                        self.shared[i] = k
                except BfuseError as e:
                    if e.code not in (3, 7):      # shared memory over budget / combination not supported: run them alone
                        raise
                    out.extend(("single", self.alone[i], [i]) for i in idx)
            self.steps.append(out)

    @property
    def launches_sequential(self):
        return len(self.ops)

    @property
    def launches_fused(self):
        return sum(len(s) for s in self.steps)

    def describe(self):
        """[[(kind, [operator names])]] of the fused program."""
        return [[(kind, [self.ops[i].name for i in idx]) for kind, _, idx in step] for step in self.steps]

    def run_sequential(self, stream=None):
        """One launch per operator in program order, each tiled for the whole GPU."""
        for k in self.alone:
            self.rt.launch_kernel(k, stream)

    def run_unfused(self, stream=None):
        """One launch per operator with the tilings of the fused program: its bit-exact reference."""
        for k in self.shared:
            self.rt.launch_kernel(k, stream)

    def run_fused(self, stream=None):
        for step in self.steps:
            for kind, h, _ in step:
                if kind == "group":
                    self.rt.launch_group(h, stream)
                elif kind == "pair":
                    self.rt.launch_fused(h, stream)
                else:
                    self.rt.launch_kernel(h, stream)


# ------------------------------------------------------------------------------ segments of the models

class _Shape:
    """Stand-in for a tensor when a segment is built without a device: arithmetic on it is a no-op."""

    def __init__(self, shape):
        self.shape = tuple(shape)

    def __mul__(self, other):
        return self
    __rmul__ = __add__ = __radd__ = __mul__

    def to(self, dtype):
        return self


class _Builder:
    """Named device buffers (torch tensors) and operators over them.  With rt = None nothing is
    allocated or registered: the operator list alone, for scheduling without a GPU."""

    def __init__(self, rt, torch, seed=0, device=0):
        self.rt, self.torch, self.ops, self.buf = rt, torch, [], {}
        if rt is None:
            return
        self.dev = torch.device("cuda", device)
        self.gen = torch.Generator(device=self.dev)
        self.gen.manual_seed(seed)

    def tensor(self, name, shape, dtype=None, std=1.0, zero=False):
        if self.rt is None:
            self.buf[name] = _Shape(shape)
            return self.buf[name]
        t = self.torch
        dtype = dtype or t.float32
        if zero:
            x = t.zeros(shape, device=self.dev, dtype=dtype)
        else:
            x = (t.randn(shape, device=self.dev, dtype=t.float32, generator=self.gen) * std).to(dtype)
        self.buf[name] = x
        return x

    def _add(self, name, op, shape, args, reads, writes, **kw):
        if self.rt is None:
            self.ops.append(SegmentOp(name, op, len(self.ops), reads, writes))
            return
        ptrs = [None if a is None else self.buf[a].data_ptr() for a in args]
        self.ops.append(SegmentOp(name, op, None, reads, writes, spec=(shape, ptrs, kw)))

    def dense(self, name, x, w, bias, y, M, N, K, op=OP_GEMM_TF32, batch=1, causal=False):
        self._add(name, op, (batch, M, N, K, 0, 0, 0), [x, w, bias, y], [x, w] + ([bias] if bias else []), [y],
                  flags=FLAG_CAUSAL if causal else 0)

    def softmax(self, name, x, y, rows, cols, scale):
        self._add(name, OP_SOFTMAX_F32, (rows, cols), [x, y], [x], [y], fparam=(scale,))

    def layernorm(self, name, x, res, gamma, beta, y, rows, cols, eps=1e-5):
        self._add(name, OP_LAYERNORM_F32, (rows, cols), [x, res, gamma, beta, y], [x, gamma, beta] + ([res] if res else []), [y],
                  fparam=(eps,))

    def rmsnorm(self, name, x, w, y, rows, cols, eps=1e-5):
        self._add(name, OP_RMSNORM_BF16, (rows, cols), [x, w, y], [x, w], [y], fparam=(eps,))

    def rope(self, name, q, inv_freq, y, seq, heads, dim):
        self._add(name, OP_ROPE_BF16, (seq, heads, dim), [q, inv_freq, y], [q, inv_freq], [y])

    def conv(self, name, x, w, y, n, ci, h, wd, co, k, stride, pad):
        self._add(name, OP_CONV2D_TF32, (n, ci, h, wd, co, k, k, stride, pad, 0, 0), [x, w, y], [x, w], [y])


def bert_layer(rt, torch, replicas=1, seq=512, hidden=768, heads=12, ffn=3072, seed=0):
    """One BERT-base encoder layer (files/bert-base-uncased.txt:38-75; dense_0..2, bgemm_0/1 of llm.yaml)
    for `replicas` independent requests: Q, K, V projections, QK^T, softmax, PV, output projection,
    residual + LayerNorm, the two FFN projections, residual + LayerNorm.  Returns (builder, ops)."""
    b = _Builder(rt, torch, seed)
    d = hidden // heads
    for r in range(replicas):
        s = "" if replicas == 1 else "_r%d" % r
        b.tensor("x" + s, (seq, hidden))
        for n in "qkv":
            b.tensor("w" + n + s, (hidden, hidden), std=0.03)
            b.tensor("b" + n + s, (hidden,), std=0.1)
            b.tensor(n + s, (seq, hidden), zero=True)
        for n, shape in (("scores", (heads, seq, seq)), ("probs", (heads, seq, seq)), ("ctx", (seq, hidden)), ("attn", (seq, hidden)),
                         ("h1", (seq, hidden)), ("f1", (seq, ffn)), ("f2", (seq, hidden)), ("out", (seq, hidden))):
            b.tensor(n + s, shape, zero=True)
        b.tensor("wo" + s, (hidden, hidden), std=0.03)
        b.tensor("w1" + s, (ffn, hidden), std=0.03)
        b.tensor("w2" + s, (hidden, ffn), std=0.02)
        for n in ("g1", "g2"):
            b.buf[n + s] = 1.0 + 0.1 * b.tensor(n + s, (hidden,))
        for n in ("be1", "be2"):
            b.tensor(n + s, (hidden,), std=0.1)
    for r in range(replicas):
        s = "" if replicas == 1 else "_r%d" % r
        for n in "qkv":
            b.dense(n + "_proj" + s, "x" + s, "w" + n + s, "b" + n + s, n + s, seq, hidden, hidden)
        # q, k as [heads, seq, d] and v as [heads, d, seq]: the reshapes of the dump, taken as reinterpretations
        b.dense("qk" + s, "q" + s, "k" + s, None, "scores" + s, seq, seq, d, batch=heads)
        b.softmax("softmax" + s, "scores" + s, "probs" + s, heads * seq, seq, 1.0 / math.sqrt(d))
        b.dense("pv" + s, "probs" + s, "v" + s, None, "ctx" + s, seq, d, seq, batch=heads)
        b.dense("o_proj" + s, "ctx" + s, "wo" + s, None, "attn" + s, seq, hidden, hidden)
        b.layernorm("ln1" + s, "attn" + s, "x" + s, "g1" + s, "be1" + s, "h1" + s, seq, hidden)
        b.dense("ffn1" + s, "h1" + s, "w1" + s, None, "f1" + s, seq, ffn, hidden)
        b.dense("ffn2" + s, "f1" + s, "w2" + s, None, "f2" + s, seq, hidden, ffn)
        b.layernorm("ln2" + s, "f2" + s, "h1" + s, "g2" + s, "be2" + s, "out" + s, seq, hidden)
    return b, b.ops


def llama_layer_projections(rt, torch, seq=512, hidden=4096, kv=1024, heads=32, kv_heads=8, ffn=14336, seed=0):
    """The projection half of a Llama-3-8B layer in bf16 (dense_4..7 of llm.yaml): RMSNorm, the Q / K / V
    projections, RoPE on Q and K, then RMSNorm and the gate / up / down projections."""
    t = torch
    b = _Builder(rt, torch, seed)
    bf = None if rt is None else t.bfloat16
    d = hidden // heads
    b.tensor("x", (seq, hidden), bf)
    b.buf["wn1"] = (1.0 + 0.1 * b.tensor("wn1", (hidden,))).to(bf)
    b.buf["wn2"] = (1.0 + 0.1 * b.tensor("wn2", (hidden,))).to(bf)
    b.tensor("xn", (seq, hidden), bf, zero=True)
    for n, width in (("q", hidden), ("k", kv), ("v", kv)):
        b.tensor("w" + n, (width, hidden), bf, std=0.02)
        b.tensor(n, (seq, width), bf, zero=True)
    b.tensor("q_rot", (seq, hidden), bf, zero=True)
    b.tensor("k_rot", (seq, kv), bf, zero=True)
    b.buf["inv_freq"] = _Shape((d // 2,)) if rt is None else (500000.0 ** (-t.arange(0, d, 2, device=b.dev, dtype=t.float32) / d)).contiguous()
    b.tensor("hn", (seq, hidden), bf, zero=True)
    for n in ("gate", "up"):
        b.tensor("w" + n, (ffn, hidden), bf, std=0.02)
        b.tensor(n, (seq, ffn), bf, zero=True)
    b.tensor("wdown", (hidden, ffn), bf, std=0.01)
    b.tensor("down", (seq, hidden), bf, zero=True)
    b.rmsnorm("input_norm", "x", "wn1", "xn", seq, hidden)
    b.dense("q_proj", "xn", "wq", None, "q", seq, hidden, hidden, OP_GEMM_BF16)
    b.dense("k_proj", "xn", "wk", None, "k", seq, kv, hidden, OP_GEMM_BF16)
    b.dense("v_proj", "xn", "wv", None, "v", seq, kv, hidden, OP_GEMM_BF16)
    b.rope("rope_q", "q", "inv_freq", "q_rot", seq, heads, d)
    b.rope("rope_k", "k", "inv_freq", "k_rot", seq, kv_heads, d)
    b.rmsnorm("post_norm", "q_rot", "wn2", "hn", seq, hidden)       # stands where attention + residual feed the MLP
    b.dense("gate_proj", "hn", "wgate", None, "gate", seq, ffn, hidden, OP_GEMM_BF16)
    b.dense("up_proj", "hn", "wup", None, "up", seq, ffn, hidden, OP_GEMM_BF16)
    b.dense("down_proj", "gate", "wdown", None, "down", seq, hidden, ffn, OP_GEMM_BF16)
    return b, b.ops


def resnet18_stages(rt, torch, batch=1, seed=0):
    """Stages 2-4 of ResNet-18 (files/result.txt; conv2d_3.. of resnet-18.yaml): per stage the stride-2
    3x3 conv and its 1x1 shortcut read the same input, then three 3x3 convs follow one another."""
    b = _Builder(rt, torch, seed)
    ci, hw = 64, 56
    b.tensor("s1", (batch, ci, hw, hw))
    prev = "s1"
    for stage, co in ((2, 128), (3, 256), (4, 512)):
        ho = hw // 2
        p = "s%d_" % stage
        b.tensor(p + "w_c1", (co, ci, 3, 3), std=0.05)
        b.tensor(p + "w_sc", (co, ci, 1, 1), std=0.1)
        for n in ("c1", "sc", "c2", "u2c1", "u2c2"):
            b.tensor(p + n, (batch, co, ho, ho), zero=True)
        for n in ("c2", "u2c1", "u2c2"):
            b.tensor(p + "w_" + n, (co, co, 3, 3), std=0.03)
        b.conv(p + "conv1", prev, p + "w_c1", p + "c1", batch, ci, hw, hw, co, 3, 2, 1)
        b.conv(p + "shortcut", prev, p + "w_sc", p + "sc", batch, ci, hw, hw, co, 1, 2, 0)
        b.conv(p + "conv2", p + "c1", p + "w_c2", p + "c2", batch, co, ho, ho, co, 3, 1, 1)
        b.conv(p + "unit2_conv1", p + "c2", p + "w_u2c1", p + "u2c1", batch, co, ho, ho, co, 3, 1, 1)
        b.conv(p + "unit2_conv2", p + "u2c1", p + "w_u2c2", p + "u2c2", batch, co, ho, ho, co, 3, 1, 1)
        prev, ci, hw = p + "u2c2", co, ho
    return b, b.ops


SEGMENTS = {"bert_layer": bert_layer, "bert_layer_x2": lambda rt, torch, **kw: bert_layer(rt, torch, replicas=2, **kw),
            "bert_layer_x4": lambda rt, torch, **kw: bert_layer(rt, torch, replicas=4, **kw),
            "llama_projections": llama_layer_projections, "resnet18_stages": resnet18_stages}
