"""The operator pairs the runtime is measured on, with seeded synthetic inputs.

Shapes come from the reference's model studies (test-utils/examples/llm.yaml:8-64,
test-utils/examples/resnet-18.yaml:37-66; Relay dumps under files/): BERT-base attention softmax
and LayerNorm, BERT Q/K projections, GPT-2 QK^T with causal mask and residual+LayerNorm, Llama-3-8B
gate/up and k/v projections, RMSNorm and RoPE, and the ResNet-18 3x3-s2 / 1x1-s2 branch pair.
No model weights or datasets are used: activations ~N(0,1), weights ~N(0,0.02), gamma/beta
~U(0.5,1.5), conv weights Kaiming-normal, all from numpy's default_rng(seed).

Device memory is held in torch tensors (plumbing only); all compute goes through the C ABI.
"""
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

from . import (FLAG_CAUSAL, OP_CONV2D_F32_SIMT, OP_CONV2D_TF32, OP_GEMM_BF16, OP_GEMM_F32_SIMT, OP_GEMM_TF32, OP_LAYERNORM_F32,
               OP_RMSNORM_BF16, OP_ROPE_BF16, OP_SOFTMAX_F32)


def f32_to_bf16_bits(x):
    """fp32 -> bf16 bit patterns (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def rope_inv_freq(dim, theta):
    i = np.arange(dim // 2, dtype=np.float64)
    return (theta ** (-2.0 * i / dim)).astype(np.float32)


@dataclass
class KernelSpec:
    name: str
    op: int
    shape: tuple
    host: List[Optional[np.ndarray]]      # one array per argument, outputs zero-filled, None = absent
    outputs: List[int]                     # indices of the output arguments
    fparam: tuple = ()
    flags: int = 0
    grid: Optional[tuple] = None
    block: Optional[tuple] = None
    smem: Optional[int] = None
    flops: float = 0.0

    @property
    def bytes(self):
        return sum(a.nbytes for a in self.host if a is not None)


@dataclass
class PairSpec:
    name: str
    a: KernelSpec
    b: KernelSpec
    dtype: str            # arithmetic type of the path: "f32", "tf32", "bf16"
    bound: str            # "hbm" or "tensor": which roofline bounds the pair
    note: str = ""

    @property
    def bytes(self):       # algorithmic bytes: every input read once, every output written once
        return self.a.bytes + self.b.bytes

    @property
    def flops(self):
        return self.a.flops + self.b.flops


# ------------------------------------------------------------------------------ kernel builders

def softmax(name, rng, rows, cols, scale):
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    return KernelSpec(name, OP_SOFTMAX_F32, (rows, cols), [x, np.zeros_like(x)], [1], fparam=(scale,))


def layernorm(name, rng, rows, cols, eps, residual=False):
    x = rng.standard_normal((rows, cols), dtype=np.float32)
    r = rng.standard_normal((rows, cols), dtype=np.float32) if residual else None
    g = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    b = rng.uniform(0.5, 1.5, cols).astype(np.float32)
    return KernelSpec(name, OP_LAYERNORM_F32, (rows, cols), [x, r, g, b, np.zeros_like(x)], [4], fparam=(eps,))


def rmsnorm(name, rng, rows, cols, eps):
    x = f32_to_bf16_bits(rng.standard_normal((rows, cols), dtype=np.float32))
    w = f32_to_bf16_bits(rng.uniform(0.5, 1.5, cols).astype(np.float32))
    return KernelSpec(name, OP_RMSNORM_BF16, (rows, cols), [x, w, np.zeros_like(x)], [2], fparam=(eps,))


def rope(name, rng, seq, heads, dim, theta):
    q = f32_to_bf16_bits(rng.standard_normal((seq, heads, dim), dtype=np.float32))
    return KernelSpec(name, OP_ROPE_BF16, (seq, heads, dim), [q, rope_inv_freq(dim, theta), np.zeros_like(q)], [2])


def gemm(name, rng, op, batch, M, N, K, bias=False, causal=False, w_std=0.02, a=None, bn=0, split=0, bm=0):
    """out[b, M, N] = A[b, M, K] . W[b, N, K]^T (+ bias).  bn / split / bm = 0: chosen by the runtime."""
    A = rng.standard_normal((batch, M, K), dtype=np.float32) if a is None else a
    W = (w_std * rng.standard_normal((batch, N, K), dtype=np.float32)).astype(np.float32)
    bvec = rng.standard_normal(N, dtype=np.float32) * 0.1 if bias else None
    if op == OP_GEMM_BF16:
        A = f32_to_bf16_bits(A) if A.dtype != np.uint16 else A
        W = f32_to_bf16_bits(W)
        out = np.zeros((batch, M, N), np.uint16)
    else:
        out = np.zeros((batch, M, N), np.float32)
    shape = (batch, M, N, K, bn, split, bm) if op in (OP_GEMM_TF32, OP_GEMM_BF16) else (batch, M, N, K)
    return KernelSpec(name, op, shape, [A, W, bvec, out], [3], flags=FLAG_CAUSAL if causal else 0,
                      flops=2.0 * batch * M * N * K)


def conv2d(name, rng, op, n, ci, h, w, co, k, stride, pad, x=None, bn=0, split=0, mode=0):
    X = rng.standard_normal((n, ci, h, w), dtype=np.float32) if x is None else x
    Wt = (np.sqrt(2.0 / (ci * k * k)) * rng.standard_normal((co, ci, k, k), dtype=np.float32)).astype(np.float32)
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    # mode: how the tensor-core body builds its im2col operand (0 the runtime's choice, 1 staged, 2 gathered)
    shape = (n, ci, h, w, co, k, k, stride, pad, bn, split, mode) if op == OP_CONV2D_TF32 else (n, ci, h, w, co, k, k, stride, pad)
    return KernelSpec(name, op, shape, [X, Wt, np.zeros((n, co, oh, ow), np.float32)],
                      [2], flops=2.0 * n * co * oh * ow * ci * k * k)


# -------------------------------------------------------------------------------- the configs

def pair_names():
    return ["cfg1_softmax_layernorm", "cfg2_q_k_proj", "cfg3_qkt_res_layernorm", "cfg4a_gate_up_proj",
            "cfg4b_k_v_proj", "cfg4c_rmsnorm_rope", "cfg5_conv_branches"]


def make_pair(name, seed=0, scale=1.0, tensor_cores=True, conv_batch=1, split=0, conv_mode=0):
    """Build one pair.  scale < 1 shrinks the row / token dimension for quick tests (512 tokens ->
    512 * scale); tensor_cores=False swaps the tcgen05 GEMM bodies for the CUDA-core fp32 bodies;
    split = 1 keeps the tcgen05 GEMMs un-split (needed under thread split and the work queue)."""
    rng = np.random.default_rng(seed)
    T = max(64, int(round(512 * scale)) // 64 * 64)  # tokens
    tf32 = OP_GEMM_TF32 if tensor_cores else OP_GEMM_F32_SIMT
    if name == "cfg1_softmax_layernorm":
        return PairSpec(name, softmax("softmax", rng, 12 * T, 512, 0.125), layernorm("layernorm", rng, T, 768, 1e-5),
                        "f32", "hbm", "BERT-base attention softmax (scale 1/8) || LayerNorm")
    if name == "cfg2_q_k_proj":
        return PairSpec(name, gemm("q_proj", rng, tf32, 1, T, 768, 768, bias=True, split=split),
                        gemm("k_proj", rng, tf32, 1, T, 768, 768, bias=True, split=split), "tf32" if tensor_cores else "f32", "hbm",
                        "BERT-base Q projection || K projection")
    if name == "cfg3_qkt_res_layernorm":
        q = gemm("qkt", rng, tf32, 12, T, T, 64, causal=True, w_std=1.0, split=split)
        return PairSpec(name, q, layernorm("res_layernorm", rng, T, 768, 1e-5, residual=True),
                        "tf32" if tensor_cores else "f32", "hbm", "GPT-2 QK^T with causal mask || residual + LayerNorm")
    if name in ("cfg4a_gate_up_proj", "cfg4b_k_v_proj"):
        if not tensor_cores:
            raise ValueError("the bf16 pairs exist on tensor cores only")
        n_out = 14336 if name == "cfg4a_gate_up_proj" else 1024
        a = f32_to_bf16_bits(rng.standard_normal((1, T, 4096), dtype=np.float32))
        na, nb = ("gate_proj", "up_proj") if n_out == 14336 else ("k_proj", "v_proj")
        return PairSpec(name, gemm(na, rng, OP_GEMM_BF16, 1, T, n_out, 4096, a=a, split=split),
                        gemm(nb, rng, OP_GEMM_BF16, 1, T, n_out, 4096, a=a, split=split), "bf16", "tensor",
                        "Llama-3-8B %s || %s (same activations)" % (na, nb))
    if name == "cfg4c_rmsnorm_rope":
        return PairSpec(name, rmsnorm("rmsnorm", rng, T, 4096, 1e-5), rope("rope_q", rng, T, 32, 128, 500000.0),
                        "bf16", "hbm", "Llama-3-8B RMSNorm || RoPE on Q")
    if name == "cfg5_conv_branches":
        x = rng.standard_normal((conv_batch, 64, 56, 56), dtype=np.float32)
        op = OP_CONV2D_TF32 if tensor_cores else OP_CONV2D_F32_SIMT
        return PairSpec(name, conv2d("conv3x3_s2", rng, op, conv_batch, 64, 56, 56, 128, 3, 2, 1, x=x, mode=conv_mode, bn=128 if conv_mode == 1 else 0),
                        conv2d("conv1x1_s2", rng, op, conv_batch, 64, 56, 56, 128, 1, 2, 0, x=x),
                        "tf32" if tensor_cores else "f32", "hbm", "ResNet-18 3x3 s2 conv || 1x1 s2 downsample (same input)")
    raise KeyError(name)


# ------------------------------------------------------------------------------ device binding

class DevicePair:
    """A PairSpec resident on one GPU: buffers uploaded, both kernels registered."""

    def __init__(self, rt, spec, device=0):
        import torch
        self.rt, self.spec, self.torch = rt, spec, torch
        self.dev = torch.device("cuda", device)
        self._shared = {}
        self.buffers = [self._upload(spec.a), self._upload(spec.b)]
        self.kernels = [self._register(spec.a, self.buffers[0]), self._register(spec.b, self.buffers[1])]
        self.fusions = {}

    def _upload(self, ks):
        t = self.torch
        out = []
        for arr in ks.host:
            if arr is None:
                out.append(None)
                continue
            key = id(arr)  # the same host array (shared activations) is uploaded once
            if key not in self._shared:
                self._shared[key] = t.from_numpy(np.ascontiguousarray(arr).view(np.uint8).reshape(-1)).to(self.dev)
            out.append(self._shared[key])
        return out

    def _register(self, ks, bufs):
        ptrs = [None if b is None else b.data_ptr() for b in bufs]
        d = self.rt.describe(ks.name, ks.op, ks.shape, ptrs, ks.fparam, ks.flags, ks.grid, ks.block, ks.smem)
        ks.launch = (d.GridDim.tuple(), d.BlockDim.tuple(), d.smem_bytes)
        return self.rt.register_kernel(d)

    def fusion(self, pattern, m=0, n=0):
        key = (pattern, m, n)
        if key not in self.fusions:
            self.fusions[key] = self.rt.register_fusion(self.kernels[0], self.kernels[1], pattern, m, n)
        return self.fusions[key]

    def clear_outputs(self):
        for ks, bufs in ((self.spec.a, self.buffers[0]), (self.spec.b, self.buffers[1])):
            for i in ks.outputs:
                bufs[i].zero_()

    def read_outputs(self):
        """[[outputs of kernel 1], [outputs of kernel 2]] as numpy arrays shaped like the host arrays."""
        self.torch.cuda.synchronize(self.dev)
        res = []
        for ks, bufs in ((self.spec.a, self.buffers[0]), (self.spec.b, self.buffers[1])):
            res.append([bufs[i].cpu().numpy().view(ks.host[i].dtype).reshape(ks.host[i].shape) for i in ks.outputs])
        return res


class ConvBranchBatch:
    """The ResNet-18 branch pair (3x3 stride-2 conv || 1x1 stride-2 downsample, 64 -> 128 channels on
    56 x 56 images) over ONE seeded batch of n images resident on a GPU, with both outputs.  A shard
    -- images [first, first + count), the partition of `partition.shard_batch` -- is a pair of kernels
    registered on the same buffers at a pointer offset: every shard reads its slice of the one batch and
    writes its slice of the one output, each with the whole (328 KB) weights, and no shard touches
    another's bytes."""

    CI, H, W, CO, OH, OW = 64, 56, 56, 128, 28, 28

    def __init__(self, rt, torch, device, n, seed=0, mode=0):
        self.rt, self.torch, self.n, self.mode = rt, torch, n, mode
        dev = torch.device("cuda", device)
        gen = torch.Generator(device=dev)
        gen.manual_seed(seed)
        self.x = torch.randn(n, self.CI, self.H, self.W, device=dev, generator=gen)
        self.w3 = torch.randn(self.CO, self.CI, 3, 3, device=dev, generator=gen) * float(np.sqrt(2.0 / (self.CI * 9)))
        self.w1 = torch.randn(self.CO, self.CI, 1, 1, device=dev, generator=gen) * float(np.sqrt(2.0 / self.CI))
        self.y3 = torch.zeros(n, self.CO, self.OH, self.OW, device=dev)
        self.y1 = torch.zeros(n, self.CO, self.OH, self.OW, device=dev)
        self._shards = {}

    def bytes(self, count=None):
        """Algorithmic bytes of the pair over `count` images: each operator's inputs read once (the shared
        input counted per operator) and its output written once."""
        c = self.n if count is None else count
        return 4 * (2 * c * self.CI * self.H * self.W + self.w3.numel() + self.w1.numel() + 2 * c * self.CO * self.OH * self.OW)

    def flops(self, count=None):
        c = self.n if count is None else count
        return 2.0 * c * self.CO * self.OH * self.OW * self.CI * (9 + 1)

    def shard(self, first, count):
        """(kernel handle 3x3, kernel handle 1x1) of the shard, registered once."""
        key = (first, count)
        if key not in self._shards:
            if first < 0 or count <= 0 or first + count > self.n:
                raise ValueError("shard outside the batch")
            xo = self.x.data_ptr() + 4 * first * self.CI * self.H * self.W
            yo = 4 * first * self.CO * self.OH * self.OW
            d3 = self.rt.describe("conv3x3_s2", OP_CONV2D_TF32, (count, self.CI, self.H, self.W, self.CO, 3, 3, 2, 1, 0, 0, self.mode),
                                  [xo, self.w3.data_ptr(), self.y3.data_ptr() + yo])
            d1 = self.rt.describe("conv1x1_s2", OP_CONV2D_TF32, (count, self.CI, self.H, self.W, self.CO, 1, 1, 2, 0, 0, 0, self.mode if self.mode != 1 else 0),
                                  [xo, self.w1.data_ptr(), self.y1.data_ptr() + yo])
            self.launch = [(d.GridDim.tuple(), d.BlockDim.tuple(), d.smem_bytes) for d in (d3, d1)]
            self._shards[key] = (self.rt.register_kernel(d3), self.rt.register_kernel(d1))
        return self._shards[key]

    def clear_outputs(self):
        self.y3.zero_()
        self.y1.zero_()
