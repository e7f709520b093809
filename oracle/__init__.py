"""ctypes binding of the CPU oracle (oracle/liboracle.so).

TEST INFRASTRUCTURE ONLY.  May be imported by tests/, by __graft_entry__.smoke()
and by the CPU-baseline / reference legs of bench.py -- never by the package.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

MAX_KERNELS, MAX_BRANCHES = 4, 16
BR_ROTATE, BR_RANGE, BR_STRIPE, BR_THREADS = 0, 1, 2, 3


class KernelDims(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("gx", "gy", "gz", "bx", "by", "bz")]


class Branch(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("kind", "kernel", "b_lo", "b_hi", "rot", "r_lo", "r_hi", "ratio",
                                       "base", "sm", "stripe_n", "stripe_idx", "t_lo", "t_hi")]


class Plan(C.Structure):
    _fields_ = [("n_kernels", C.c_int), ("k", KernelDims * MAX_KERNELS), ("n_branches", C.c_int),
                ("br", Branch * MAX_BRANCHES), ("fused_grid", C.c_int), ("fused_block", C.c_int),
                ("thread_split", C.c_int)]


def build(force=False):
    """Compile liboracle.so with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH):
        subprocess.check_call(["make", "-C", _HERE, "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        pk, pp = C.POINTER(KernelDims), C.POINTER(Plan)
        L.orc_plan_zigzag.argtypes = [pk, C.c_int, C.c_int, C.c_int, pp]
        L.orc_plan_proportional.argtypes = [pk, C.c_int, C.c_int, pp]
        L.orc_plan_sm_striped.argtypes = [pk, C.c_int, C.c_int, pp]
        L.orc_plan_thread_split.argtypes = [pk, C.c_int, pp]
        L.orc_plan_range_split.argtypes = [pk, C.c_int, pp]
        pi = C.POINTER(C.c_int)
        L.orc_map_block.argtypes = [pp, C.c_int, pi, pi]
        L.orc_map_thread.argtypes = [pp, C.c_int, C.c_int, C.c_int, pi, pi]
        L.orc_named_barrier.argtypes = [pp, C.c_int, pi, pi]
        L.orc_plan_digest.argtypes = [pp]
        L.orc_plan_digest.restype = C.c_uint64
        L.orc_decompose.argtypes = [pk, C.c_int, C.c_int, pi, pi]
        vp = C.c_void_p
        L.orc_softmax_f32.argtypes = [vp, vp, C.c_int, C.c_int, C.c_float]
        L.orc_layernorm_f32.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_float]
        L.orc_rmsnorm_bf16.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_float]
        L.orc_rope_bf16.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_int]
        L.orc_gemm_nt_f32.argtypes = [vp, vp, vp, vp] + [C.c_int] * 6
        L.orc_gemm_nt_bf16.argtypes = [vp, vp, vp] + [C.c_int] * 4
        L.orc_conv2d_nchw_f32.argtypes = [vp, vp, vp] + [C.c_int] * 10
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


# ------------------------------------------------------------------ dispatch

def _dims(kernels):
    arr = (KernelDims * len(kernels))()
    for i, k in enumerate(kernels):
        arr[i] = KernelDims(*[int(v) for v in k])
    return arr


def plan(pattern, kernels, M=1, N=1, min_option=1, total_sm=84):
    """kernels: [[gx,gy,gz,bx,by,bz], ...]; pattern: zigzag|proportional|sm_striped|thread_split|range_split."""
    p = Plan()
    d = _dims(kernels)
    L = lib()
    rc = {
        "zigzag": lambda: L.orc_plan_zigzag(d, len(kernels), M, N, p),
        "proportional": lambda: L.orc_plan_proportional(d, len(kernels), min_option, p),
        "sm_striped": lambda: L.orc_plan_sm_striped(d, len(kernels), total_sm, p),
        "thread_split": lambda: L.orc_plan_thread_split(d, len(kernels), p),
        "range_split": lambda: L.orc_plan_range_split(d, len(kernels), p),
    }[pattern]()
    if rc != 0:
        raise ValueError("oracle rejected the plan")
    return p


def map_block(p, b):
    k, vb = C.c_int(), C.c_int()
    if not lib().orc_map_block(p, b, k, vb):
        return None
    return k.value, vb.value


def block_table(p):
    """(kernel, vblock) of every fused CTA as two int arrays."""
    n = p.fused_grid
    ks, vbs = np.empty(n, np.int32), np.empty(n, np.int32)
    k, vb = C.c_int(), C.c_int()
    L = lib()
    for b in range(n):
        if not L.orc_map_block(p, b, k, vb):
            raise RuntimeError("unmapped CTA %d" % b)
        ks[b], vbs[b] = k.value, vb.value
    return ks, vbs


def digest(p):
    return lib().orc_plan_digest(p)


def named_barrier(p, kernel):
    a, b = C.c_int(), C.c_int()
    lib().orc_named_barrier(p, kernel, a, b)
    return a.value, b.value


# ----------------------------------------------------------------- operators

def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def f32_to_bf16(x):
    """fp32 ndarray -> uint16 bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_to_f32(h):
    return (np.ascontiguousarray(h, np.uint16).astype(np.uint32) << 16).view(np.float32)


def softmax(x, scale):
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_softmax_f32(_p(x), _p(y), x.shape[0], x.shape[1], scale)
    return y


def layernorm(x, gamma, beta, eps, res=None):
    x = np.ascontiguousarray(x, np.float32)
    res = None if res is None else np.ascontiguousarray(res, np.float32)
    y = np.empty_like(x)
    lib().orc_layernorm_f32(_p(x), _p(res), _p(np.ascontiguousarray(gamma, np.float32)),
                            _p(np.ascontiguousarray(beta, np.float32)), _p(y), x.shape[0], x.shape[1], eps)
    return y


def rmsnorm_bf16(x, w, eps):
    x = np.ascontiguousarray(x, np.uint16)
    y = np.empty_like(x)
    lib().orc_rmsnorm_bf16(_p(x), _p(np.ascontiguousarray(w, np.uint16)), _p(y), x.shape[0], x.shape[1], eps)
    return y


def rope_inv_freq(dim, theta):
    """inv_freq[i] = theta ** (-2i/dim), computed in double and rounded once to fp32."""
    i = np.arange(dim // 2, dtype=np.float64)
    return (theta ** (-2.0 * i / dim)).astype(np.float32)


def rope_bf16(q, inv_freq):
    q = np.ascontiguousarray(q, np.uint16)
    y = np.empty_like(q)
    s, h, d = q.shape
    lib().orc_rope_bf16(_p(q), _p(np.ascontiguousarray(inv_freq, np.float32)), _p(y), s, h, d)
    return y


def gemm_nt(A, W, bias=None, causal=False, tf32=False):
    """A[b,M,K] (or [M,K]), W[b,N,K] -> [b,M,N]."""
    A = np.ascontiguousarray(A, np.float32)
    W = np.ascontiguousarray(W, np.float32)
    squeeze = A.ndim == 2
    if squeeze:
        A, W = A[None], W[None]
    b, M, K = A.shape
    N = W.shape[1]
    out = np.empty((b, M, N), np.float32)
    bias = None if bias is None else np.ascontiguousarray(bias, np.float32)
    lib().orc_gemm_nt_f32(_p(A), _p(W), _p(bias), _p(out), b, M, N, K, int(causal), int(tf32))
    return out[0] if squeeze else out


def gemm_nt_bf16(A, W):
    A = np.ascontiguousarray(A, np.uint16)
    W = np.ascontiguousarray(W, np.uint16)
    M, K = A.shape
    N = W.shape[0]
    out = np.empty((M, N), np.uint16)
    lib().orc_gemm_nt_bf16(_p(A), _p(W), _p(out), 1, M, N, K)
    return out


def conv2d_nchw(x, w, stride, pad, tf32=False):
    x = np.ascontiguousarray(x, np.float32)
    w = np.ascontiguousarray(w, np.float32)
    n, ci, h, wd = x.shape
    co, _, kh, kw = w.shape
    oh, ow = (h + 2 * pad - kh) // stride + 1, (wd + 2 * pad - kw) // stride + 1
    y = np.empty((n, co, oh, ow), np.float32)
    lib().orc_conv2d_nchw_f32(_p(x), _p(w), _p(y), n, ci, h, wd, co, kh, kw, stride, pad, int(tf32))
    return y


def num_threads():
    return lib().orc_num_threads()


def set_num_threads(n):
    lib().orc_set_num_threads(int(n))
