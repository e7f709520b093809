"""The operator cross-product sweep: every operator of the reference's benchmark suite against
every other one (upper triangle, diagonal included), fused vs back-to-back.

The reference sweeps 42 shapes x 42 shapes at batch 1024 (test-utils/examples/benchmark.yaml:1-88:
8 dense, 12 batch-matmul, 22 conv2d; pairs (K1, K2 >= K1) as in scripts/profile_test_suite.py:37-46).
Here the same 42 operators run at the single-sequence sizes of the reference's model studies
(test-utils/examples/llm.yaml: 512 tokens, per-model head counts; test-utils/examples/resnet-18.yaml
and the Inception-v3 shapes of benchmark.yaml at one image), on tensor cores where the tcgen05
bodies cover the shape (dense / batch-matmul: fp32 in, tf32 MMA; conv: tf32 implicit GEMM) and on
the CUDA-core conv body otherwise.  Inputs are seeded synthetic tensors created on the device.

Timing follows the reference's protocol -- 3 warm-up launches, then 30 timed ones, mean
(scripts/profile_test_suite.py:10-11) -- on the same buffers every launch, i.e. operands that fit
stay in L2 as they do in the reference's own loop.
"""
import math

from . import (BfuseError, FLAG_CAUSAL, MODE_FUSED, MODE_KERNEL1, MODE_SEQUENTIAL, OP_CONV2D_F32_SIMT, OP_CONV2D_TF32, OP_GEMM_BF16,
               OP_GEMM_TF32, OP_LAYERNORM_F32, OP_RMSNORM_BF16, OP_ROPE_BF16, OP_SOFTMAX_F32, PROPORTIONAL, RANGE_SPLIT, SM_STRIPED,
               THREAD_SPLIT, ZIGZAG)

# the fused forms a pair is timed in when every pattern is asked for: (label, pattern, M, N)
ALL_PATTERNS = (("zigzag", ZIGZAG, 1, 1), ("zigzag2", ZIGZAG, 1, 2), ("range", RANGE_SPLIT, 0, 0), ("striped", SM_STRIPED, 0, 0),
                ("thread_split", THREAD_SPLIT, 0, 0))

# name -> shape.  dense: (M, K, N); bgemm: (batch, M, K, N); conv2d: (N, H, W, CO, CI, KH, KW, stride, pad)
SWEEP_OPS = (
    ("dense_0", (512, 768, 768)), ("dense_1", (512, 768, 3072)), ("dense_2", (512, 3072, 768)),
    ("dense_3", (512, 768, 2304)), ("dense_4", (512, 4096, 4096)), ("dense_5", (512, 4096, 1024)),
    ("dense_6", (512, 4096, 14336)), ("dense_7", (512, 14336, 4096)),
    ("bgemm_0", (12, 512, 64, 512)), ("bgemm_1", (12, 512, 512, 64)), ("bgemm_2", (32, 512, 128, 512)),
    ("bgemm_3", (32, 512, 512, 128)), ("bgemm_4", (16, 256, 64, 256)), ("bgemm_5", (16, 256, 256, 64)),
    ("bgemm_6", (16, 256, 80, 256)), ("bgemm_7", (16, 256, 256, 80)), ("bgemm_8", (16, 208, 64, 208)),
    ("bgemm_9", (16, 208, 208, 64)), ("bgemm_10", (16, 208, 80, 208)), ("bgemm_11", (16, 208, 208, 80)),
    ("conv2d_0", (1, 224, 224, 64, 3, 7, 7, 2, 3)), ("conv2d_1", (1, 56, 56, 64, 64, 3, 3, 1, 1)),
    ("conv2d_2", (1, 56, 56, 64, 64, 1, 1, 1, 0)), ("conv2d_3", (1, 56, 56, 128, 64, 3, 3, 2, 1)),
    ("conv2d_4", (1, 28, 28, 128, 128, 3, 3, 1, 1)), ("conv2d_5", (1, 56, 56, 128, 64, 1, 1, 2, 0)),
    ("conv2d_6", (1, 28, 28, 256, 128, 3, 3, 2, 1)), ("conv2d_7", (1, 14, 14, 256, 256, 3, 3, 1, 1)),
    ("conv2d_8", (1, 28, 28, 256, 128, 1, 1, 2, 0)), ("conv2d_9", (1, 14, 14, 512, 256, 3, 3, 2, 1)),
    ("conv2d_10", (1, 7, 7, 512, 512, 3, 3, 1, 1)), ("conv2d_11", (1, 14, 14, 512, 256, 1, 1, 2, 0)),
    ("conv2d_12", (1, 35, 35, 64, 256, 1, 1, 1, 0)), ("conv2d_13", (1, 35, 35, 48, 256, 1, 1, 1, 0)),
    ("conv2d_14", (1, 35, 35, 64, 288, 1, 1, 1, 0)), ("conv2d_15", (1, 35, 35, 48, 288, 1, 1, 1, 0)),
    ("conv2d_16", (1, 35, 35, 384, 288, 3, 3, 2, 0)), ("conv2d_17", (1, 35, 35, 96, 96, 3, 3, 2, 0)),
    ("conv2d_18", (1, 17, 17, 192, 768, 1, 1, 1, 0)), ("conv2d_19", (1, 17, 17, 128, 768, 1, 1, 1, 0)),
    ("conv2d_20", (1, 17, 17, 160, 768, 1, 1, 1, 0)), ("conv2d_21", (1, 17, 17, 320, 192, 3, 3, 2, 0)),
)


# Operators beyond the reference's suite, for the pair-selection model only: the memory-bound bodies and the bf16
# projections of the model studies, which the reference's 42 shapes (dense / batch-matmul / conv2d) do not contain.
# softmax: (rows, cols); layernorm: (rows, cols, residual); rmsnorm: (rows, cols); rope: (seq, heads, dim);
# dense16 (bf16 GEMM): (M, K, N); causal (QK^T with mask): (batch, M, K, N)
MODEL_EXTRA_OPS = (
    ("softmax_0", (6144, 512)), ("softmax_1", (16384, 512)), ("softmax_2", (1536, 1024)),
    ("layernorm_0", (512, 768, 0)), ("layernorm_1", (512, 768, 1)), ("layernorm_2", (4096, 1024, 1)),
    ("rmsnorm_0", (512, 4096)), ("rmsnorm_1", (2048, 4096)), ("rope_0", (512, 32, 128)), ("rope_1", (512, 8, 128)),
    ("dense16_0", (512, 4096, 1024)), ("dense16_1", (512, 4096, 14336)), ("dense16_2", (512, 4096, 4096)),
    ("causal_0", (12, 512, 64, 512)),
)


def pair_indices(n=len(SWEEP_OPS)):
    """(i, j) with j >= i, in the reference's enumeration order."""
    return [(i, j) for i in range(n) for j in range(i, n)]


def conv_on_tensor_cores(shape):
    """Whether the tcgen05 implicit-GEMM body takes this conv (the TMA stride rule for the weight
    rows, its offset table and its tap mask limit what it covers); otherwise the CUDA-core body
    runs it."""
    n, h, w, co, ci, kh, kw, stride, pad = shape
    k = ci * kh * kw
    return k % 4 == 0 and k <= 8192 and kh * kw <= 31


class SweepOperand:
    """One operator of the sweep resident on the device and registered with the runtime."""

    def __init__(self, rt, torch, device, name, shape, gen):
        self.name, self.shape = name, shape
        dev = torch.device("cuda", device)

        def randn(*dims, std=1.0):
            return torch.randn(*dims, device=dev, dtype=torch.float32, generator=gen) * std

        self.flops = 0.0
        kind = name.split("_")[0]
        if kind in ("softmax", "layernorm", "rmsnorm", "rope"):
            bf16 = kind in ("rmsnorm", "rope")
            dt = torch.bfloat16 if bf16 else torch.float32
            if kind == "rope":
                seq, heads, dim = shape
                inv = (500000.0 ** (-2.0 * torch.arange(dim // 2, device=dev, dtype=torch.float64) / dim)).float()
                self.bufs = [randn(seq, heads, dim).to(dt), inv, torch.zeros(seq, heads, dim, device=dev, dtype=dt)]
                self.op, args, oshape, fparam = OP_ROPE_BF16, [0, 1, 2], (seq, heads, dim), ()
            else:
                rows, cols = shape[0], shape[1]
                x, y = randn(rows, cols).to(dt), torch.zeros(rows, cols, device=dev, dtype=dt)
                if kind == "softmax":
                    self.bufs, self.op, args, fparam = [x, y], OP_SOFTMAX_F32, [0, 1], (0.125,)
                elif kind == "rmsnorm":
                    self.bufs, self.op, args, fparam = [x, (torch.rand(cols, device=dev, generator=gen) + 0.5).to(dt), y], OP_RMSNORM_BF16, [0, 1, 2], (1e-5,)
                else:
                    res = randn(rows, cols) if shape[2] else None
                    g, b = torch.rand(cols, device=dev, generator=gen) + 0.5, torch.rand(cols, device=dev, generator=gen) + 0.5
                    self.bufs, self.op, fparam = [x, g, b, y] + ([res] if res is not None else []), OP_LAYERNORM_F32, (1e-5,)
                    args = [0, 4 if res is not None else None, 1, 2, 3]
                oshape = (rows, cols)
            desc = rt.describe(name, self.op, oshape, [None if i is None else self.bufs[i].data_ptr() for i in args], fparam)
        elif kind in ("dense16", "causal"):
            if kind == "dense16":
                (m, k, nn), b, dt = shape, 1, torch.bfloat16
                self.op, flags = OP_GEMM_BF16, 0
            else:
                (b, m, k, nn), dt = shape, torch.float32
                self.op, flags = OP_GEMM_TF32, FLAG_CAUSAL
            self.bufs = [randn(b, m, k).to(dt), randn(b, nn, k, std=0.02 if b == 1 else 1.0).to(dt), torch.zeros(b, m, nn, device=dev, dtype=dt)]
            self.flops = 2.0 * b * m * nn * k
            desc = rt.describe(name, self.op, (b, m, nn, k, 0, 0), [self.bufs[0].data_ptr(), self.bufs[1].data_ptr(), None, self.bufs[2].data_ptr()],
                               flags=flags)
        elif name.startswith("conv2d"):
            n, h, w, co, ci, kh, kw, stride, pad = shape
            oh, ow = (h + 2 * pad - kh) // stride + 1, (w + 2 * pad - kw) // stride + 1
            self.bufs = [randn(n, ci, h, w), randn(co, ci, kh, kw, std=math.sqrt(2.0 / (ci * kh * kw))),
                         torch.zeros(n, co, oh, ow, device=dev)]
            self.op = OP_CONV2D_TF32 if conv_on_tensor_cores(shape) else OP_CONV2D_F32_SIMT
            self.flops = 2.0 * n * co * oh * ow * ci * kh * kw
            desc = rt.describe(name, self.op, (n, ci, h, w, co, kh, kw, stride, pad), [b.data_ptr() for b in self.bufs])
        else:
            b, (m, k, nn) = (1, shape) if name.startswith("dense") else (shape[0], shape[1:])
            self.bufs = [randn(b, m, k), randn(b, nn, k, std=0.02 if b == 1 else 1.0), torch.zeros(b, m, nn, device=dev)]
            self.op = OP_GEMM_TF32
            self.flops = 2.0 * b * m * nn * k
            desc = rt.describe(name, self.op, (b, m, nn, k, 0, 0), [self.bufs[0].data_ptr(), self.bufs[1].data_ptr(), None,
                                                                    self.bufs[2].data_ptr()])
        self.bytes = sum(t.numel() * t.element_size() for t in self.bufs)
        self.launch = (desc.GridDim.tuple(), desc.BlockDim.tuple(), desc.smem_bytes)
        self.kernel = rt.register_kernel(desc)


def build_operands(rt, torch, device=0, seed=0, ops=SWEEP_OPS):
    """Two independent sets of the sweep's operators (the reference's kernel1 / kernel2 sets)."""
    gen = torch.Generator(device=torch.device("cuda", device))
    gen.manual_seed(seed)
    return [[SweepOperand(rt, torch, device, name + suffix, shape, gen) for name, shape in ops] for suffix in ("_k1", "_k2")]


def alone_times(rt, sets, warmup=3, iters=30):
    """Microseconds of every operator of the first set launched alone (same protocol as the pairs)."""
    out = []
    for a, b in zip(sets[0], sets[1]):
        f = rt.register_fusion(a.kernel, b.kernel, RANGE_SPLIT, 0, 0)     # any fusion of the operator: mode 0 times kernel 1 alone
        out.append(rt.time(f, MODE_KERNEL1, warmup, iters)[0])
    return out


def pairing_records(sets, results, alone, sm_count):
    """The sweep's measurements in the form `pairing.evaluate` takes."""
    by_name = {a.name[:-3]: i for i, a in enumerate(sets[0])}
    recs = []
    for key, v in results.items():
        if "error" in v:
            continue
        i, j = (by_name[n] for n in key.split("|"))
        la, lb = sets[0][i].launch, sets[1][j].launch
        dims = lambda l: (l[0][0] * l[0][1] * l[0][2], l[1][0] * l[1][1] * l[1][2], l[2])
        recs.append({"pair": key, "t_a": alone[i], "t_b": alone[j], "launch_a": dims(la), "launch_b": dims(lb), "sm_count": sm_count,
                     "op_a": sets[0][i].op, "op_b": sets[1][j].op, "bytes_a": sets[0][i].bytes, "bytes_b": sets[1][j].bytes,
                     "flops_a": sets[0][i].flops, "flops_b": sets[1][j].flops,
                     "fused_us": v["fused_us"], "sequential_us": v["sequential_us"], "fused_us_by_pattern": v.get("fused_us_by_pattern")})
    return recs


def measure(rt, sets, pairs, hbm_gbs, tf32_tflops, pattern=ZIGZAG, warmup=3, iters=30):
    """{"<k1>|<k2>": {...}} for the given (i, j) pairs: fused and sequential microseconds (mean of
    `iters` launches after `warmup`), speed-up, and the pair's roofline time.  pattern = "all" times every
    form of ALL_PATTERNS (`fused_us_by_pattern`; `fused_us` is then the zig-zag figure, as in a one-pattern sweep)."""
    out = {}
    for i, j in pairs:
        a, b = sets[0][i], sets[1][j]
        key = "%s|%s" % (a.name[:-3], b.name[:-3])   # without the set suffix
        forms = ALL_PATTERNS if pattern == "all" else (("one", pattern, 1 if pattern in (ZIGZAG, PROPORTIONAL) else 0,
                                                        1 if pattern in (ZIGZAG, PROPORTIONAL) else 0),)
        by_pattern, seq, first_error = {}, None, None
        for label, pat, m, n in forms:
            try:
                f = rt.register_fusion(a.kernel, b.kernel, pat, m, n)
            except BfuseError as e:
                first_error = first_error or str(e)[:120]
                continue
            by_pattern[label] = rt.time(f, MODE_FUSED, warmup, iters)[0]
            if seq is None and not any(rt.fusion_info(f)["retiled_unsplit"]):
                seq = rt.time(f, MODE_SEQUENTIAL, warmup, iters)[0]
            rt.unregister_fusion(f)
        if not by_pattern or seq is None:
            out[key] = {"error": first_error or "no pattern could host the pair"}
            continue
        fused = by_pattern.get("zigzag", by_pattern.get("one", min(by_pattern.values())))
        roof = max((a.bytes + b.bytes) / (hbm_gbs * 1e3), (a.flops + b.flops) / (tf32_tflops * 1e6))
        out[key] = {"fused_us": fused, "sequential_us": seq, "speedup_vs_sequential": seq / fused, "roofline_us": roof,
                    "roofline_frac": roof / fused}
        if pattern == "all":
            out[key]["fused_us_by_pattern"] = by_pattern
    return out


def summarise(results):
    """Counts and geometric means over a sweep's result dict."""
    ok = [v for v in results.values() if "error" not in v]
    if not ok:
        return {"pairs": 0, "errors": len(results)}
    sp = [v["speedup_vs_sequential"] for v in ok]
    by_kind = {}
    for k, v in results.items():
        if "error" in v:
            continue
        kinds = "x".join(sorted(n.split("_")[0] for n in k.split("|")))
        by_kind.setdefault(kinds, []).append(v["speedup_vs_sequential"])
    gm = lambda xs: math.exp(sum(math.log(x) for x in xs) / len(xs))
    return {"pairs": len(ok), "errors": len(results) - len(ok), "geomean_speedup_vs_sequential": gm(sp),
            "min_speedup": min(sp), "max_speedup": max(sp), "pairs_faster_than_sequential": sum(1 for x in sp if x > 1.0),
            "pairs_5pct_faster": sum(1 for x in sp if x > 1.05), "pairs_5pct_slower": sum(1 for x in sp if x < 0.95),
            "total_fused_us": sum(v["fused_us"] for v in ok), "total_sequential_us": sum(v["sequential_us"] for v in ok),
            "geomean_speedup_by_kinds": {k: gm(v) for k, v in sorted(by_kind.items())}}
