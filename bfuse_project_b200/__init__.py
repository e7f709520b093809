"""bfuse_project_b200 -- host-side binding of libbfuse_b200.so (the C ABI in include/bfuse_b200.h).

The names follow the reference's surface for this path: KernelInfo / GridDim / BlockDim records
(horizontal-fuser/include/fuse/Contexts.h:13-50), fusions of two kernels with a dispatch pattern
(horizontal-fuser/src/Contexts.cc:56-92), and the harness calls run_kernel / run_parallel /
run_fuse (test-utils/test-suite-files/operation_cu.py:164-253).

There is no CPU fallback: if the shared library is missing this module raises on import of
`lib()`, and every compute call goes to a CUDA kernel.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libbfuse_b200.so")

MAX_ARGS, MAX_SHAPE = 6, 12

# operator bodies
OP_SOFTMAX_F32, OP_LAYERNORM_F32, OP_RMSNORM_BF16, OP_ROPE_BF16 = 0, 1, 2, 3
OP_GEMM_F32_SIMT, OP_CONV2D_F32_SIMT, OP_GEMM_TF32, OP_GEMM_BF16, OP_CONV2D_TF32 = 4, 5, 6, 7, 8
FLAG_CAUSAL = 1


def flag_share(n):
    """Hint for the default tiling: n operators (1..4) will share the launch; 1 = the operator runs alone."""
    return int(n) << 8
# dispatch patterns
ZIGZAG, PROPORTIONAL, SM_STRIPED, THREAD_SPLIT, RANGE_SPLIT, WORK_QUEUE = 0, 1, 2, 3, 4, 5
PATTERN_NAMES = {ZIGZAG: "zigzag", PROPORTIONAL: "proportional", SM_STRIPED: "sm_striped",
                 THREAD_SPLIT: "thread_split", RANGE_SPLIT: "range_split", WORK_QUEUE: "work_queue"}
# harness modes T (test-utils/test-suite-files/main_cc.py:22-36)
MODE_KERNEL1, MODE_KERNEL2, MODE_PARALLEL, MODE_SEQUENTIAL, MODE_FUSED = 0, 1, 2, 3, 4

ERRORS = {1: "invalid argument", 2: "shape / launch dims rejected", 3: "shared memory over budget",
          4: "CUDA error", 5: "no sm_100 device", 6: "device-side wait timed out", 7: "unsupported"}


class Dim3(C.Structure):
    _fields_ = [("X", C.c_int), ("Y", C.c_int), ("Z", C.c_int)]

    def size(self):
        return self.X * self.Y * self.Z

    def tuple(self):
        return (self.X, self.Y, self.Z)


class KernelDesc(C.Structure):
    """bfuse_kernel_desc: the reference's KernelInfo plus operator, smem, args and shape."""
    _fields_ = [("KernelName", C.c_char_p), ("HasBarriers", C.c_int), ("GridDim", Dim3), ("BlockDim", Dim3),
                ("Reg", C.c_int), ("ExecTime", C.c_float), ("op", C.c_int), ("smem_bytes", C.c_size_t),
                ("args", C.c_void_p * MAX_ARGS), ("nargs", C.c_int), ("shape", C.c_int * MAX_SHAPE),
                ("fparam", C.c_float * 4), ("flags", C.c_uint)]


class BfuseError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__("bfuse error %d (%s): %s" % (code, ERRORS.get(code, "?"), msg))
        self.code = code


_lib = None


def lib():
    """Load libbfuse_b200.so; raise if it has not been built (there is nothing to fall back to)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError("libbfuse_b200.so is not built: run `make -C bfuse_project_b200/csrc -j` "
                              "(or __graft_entry__.build()); this package has no CPU path")
        L = C.CDLL(LIB_PATH)
        vp, ip, pp = C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_void_p)
        kd = C.POINTER(KernelDesc)
        sig = {
            "bfuse_create": [C.c_int, pp], "bfuse_destroy": [vp], "bfuse_device_sm_count": [vp],
            "bfuse_default_launch": [vp, kd], "bfuse_arg_info": [vp, kd, C.c_int, C.POINTER(C.c_size_t), ip],
            "bfuse_register_kernel": [vp, kd, ip], "bfuse_set_kernel_args": [vp, C.c_int, pp, C.c_int],
            "bfuse_register_fusion": [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, ip],
            "bfuse_fusion_info": [vp, C.c_int, kd], "bfuse_fusion_map_block": [vp, C.c_int, C.c_int, ip, ip],
            "bfuse_fusion_map_thread": [vp, C.c_int, C.c_int, C.c_int, C.c_int, ip, ip, ip],
            "bfuse_launch_kernel": [vp, C.c_int, vp], "bfuse_launch_sequential": [vp, C.c_int, vp],
            "bfuse_launch_parallel": [vp, C.c_int, vp], "bfuse_launch_fused": [vp, C.c_int, vp],
            "bfuse_launch_list": [vp, ip, C.c_int, C.c_int, vp],
            "bfuse_graph_create": [vp, ip, C.c_int, C.c_int, ip], "bfuse_graph_launch": [vp, C.c_int, vp],
            "bfuse_graph_destroy": [vp, C.c_int], "bfuse_unregister_kernel": [vp, C.c_int],
            "bfuse_unregister_fusion": [vp, C.c_int], "bfuse_unregister_group": [vp, C.c_int],
            "bfuse_set_dependent_launch": [vp, C.c_int],
            "bfuse_trace_fused": [vp, C.c_int, ip, ip, ip, C.c_int], "bfuse_read_status": [vp, ip],
            "bfuse_debug_gemm_timeline": [vp, C.c_int, C.POINTER(C.c_longlong), C.c_int],
            "bfuse_debug_fused_timeline": [vp, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_longlong), C.POINTER(C.c_int)],
            "bfuse_run_kernel": [vp, C.c_int, pp], "bfuse_run_parallel": [vp, C.c_int, pp, pp],
            "bfuse_run_fuse": [vp, C.c_int, pp, pp],
            "bfuse_run_fuse_batch": [vp, ip, C.c_int, C.POINTER(pp), C.POINTER(pp)],
            "bfuse_time": [vp, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)],
            "bfuse_plan_create": [C.POINTER(Dim3), C.POINTER(Dim3), C.c_int, C.c_int, C.c_int, pp],
            "bfuse_plan_create_clustered": [C.POINTER(Dim3), C.POINTER(Dim3), C.c_int, C.c_int, C.c_int, C.c_int, pp],
            "bfuse_plan_fused_dims": [vp, C.POINTER(Dim3), C.POINTER(Dim3)],
            "bfuse_plan_map_block": [vp, C.c_int, ip, ip], "bfuse_plan_map_all": [vp, ip, ip, C.c_int],
            "bfuse_plan_map_thread": [vp, C.c_int, C.c_int, C.c_int, ip, ip, ip],
            "bfuse_plan_barrier": [vp, C.c_int, ip, ip],
            "bfuse_register_group": [vp, ip, C.c_int, C.c_int, C.c_int, C.c_int, ip],
            "bfuse_group_info": [vp, C.c_int, kd], "bfuse_group_map_block": [vp, C.c_int, C.c_int, ip, ip],
            "bfuse_launch_group": [vp, C.c_int, vp],
            "bfuse_plan_group": [C.POINTER(Dim3), C.POINTER(Dim3), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, ip, ip, ip, C.c_int],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        L.bfuse_last_error.argtypes = [vp]
        L.bfuse_last_error.restype = C.c_char_p
        L.bfuse_plan_destroy.argtypes = [vp]
        L.bfuse_plan_destroy.restype = None
        L.bfuse_check_matrix.argtypes = [vp, vp, C.c_size_t, C.c_float]
        L.bfuse_check_matrix.restype = C.c_long
        _lib = L
    return _lib


# --------------------------------------------------------------------------- scheduler only

class Plan:
    """The block-dispatch plan of one pair, computed on the CPU (no GPU needed)."""

    def __init__(self, kernels, pattern, param_m=1, param_n=1, cluster=1):
        """kernels: two [gx, gy, gz, bx, by, bz] lists; cluster: CTAs per dispatch unit."""
        g = (Dim3 * 2)(*[Dim3(*k[:3]) for k in kernels])
        b = (Dim3 * 2)(*[Dim3(*k[3:]) for k in kernels])
        self._h = C.c_void_p()
        rc = lib().bfuse_plan_create_clustered(g, b, pattern, param_m, param_n, cluster, C.byref(self._h))
        if rc:
            raise BfuseError(rc, "plan rejected")
        fg, fb = Dim3(), Dim3()
        lib().bfuse_plan_fused_dims(self._h, fg, fb)
        self.fused_grid, self.fused_block = fg.tuple(), fb.tuple()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().bfuse_plan_destroy(self._h)
            self._h = None

    def map_block(self, b):
        k, vb = C.c_int(), C.c_int()
        if lib().bfuse_plan_map_block(self._h, b, k, vb):
            return None
        return k.value, vb.value

    def map_all(self):
        import numpy as np
        n = self.fused_grid[0]
        ks, vbs = np.empty(n, np.int32), np.empty(n, np.int32)
        ip = C.POINTER(C.c_int)
        rc = lib().bfuse_plan_map_all(self._h, ks.ctypes.data_as(ip), vbs.ctypes.data_as(ip), n)
        if rc:
            raise BfuseError(rc, "unmapped CTA")
        return ks, vbs

    def map_thread(self, kernel, b, t):
        vb, vt, act = C.c_int(), C.c_int(), C.c_int()
        rc = lib().bfuse_plan_map_thread(self._h, kernel, b, t, vb, vt, act)
        if rc:
            raise BfuseError(rc, "not a thread-split plan")
        return (vb.value, vt.value) if act.value else None

    def barrier(self, kernel):
        a, b = C.c_int(), C.c_int()
        lib().bfuse_plan_barrier(self._h, kernel, a, b)
        return a.value, b.value


def plan_group(kernels, pattern, param_m=1, param_n=1, cluster=1):
    """The block-dispatch plan of 2..4 kernels in one launch, computed on the CPU.
    kernels: [gx, gy, gz, bx, by, bz] lists.  Returns (fused_grid, fused_block, kernel_of, vblock_of);
    padding CTAs of a clustered plan map to -1."""
    import numpy as np
    n = len(kernels)
    g = (Dim3 * n)(*[Dim3(*k[:3]) for k in kernels])
    b = (Dim3 * n)(*[Dim3(*k[3:]) for k in kernels])
    fb = C.c_int()
    ip = C.POINTER(C.c_int)
    grid = lib().bfuse_plan_group(g, b, n, pattern, param_m, param_n, cluster, fb, None, None, 0)
    if grid < 0:
        raise BfuseError(-grid, "group plan rejected")
    ks, vbs = np.empty(grid, np.int32), np.empty(grid, np.int32)
    lib().bfuse_plan_group(g, b, n, pattern, param_m, param_n, cluster, fb, ks.ctypes.data_as(ip), vbs.ctypes.data_as(ip), grid)
    return grid, fb.value, ks, vbs


# --------------------------------------------------------------------------------- runtime

class Runtime:
    """One context per device (bfuse_create)."""

    def __init__(self, device=0):
        self._L = lib()
        self._ctx = C.c_void_p()
        rc = self._L.bfuse_create(device, C.byref(self._ctx))
        if rc:
            raise BfuseError(rc, "bfuse_create failed (see stderr)")
        self.device = device
        self._names = []

    def close(self):
        if self._ctx:
            self._L.bfuse_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, rc):
        if rc:
            raise BfuseError(rc, self._L.bfuse_last_error(self._ctx).decode())

    @property
    def sm_count(self):
        return self._L.bfuse_device_sm_count(self._ctx)

    def describe(self, name, op, shape, args=(), fparam=(), flags=0, grid=None, block=None, smem=None):
        """Build a KernelDesc; dims default to the body's own tiling (bfuse_default_launch)."""
        d = KernelDesc()
        self._names.append(name.encode())
        d.KernelName = self._names[-1]
        d.op = op
        d.ExecTime = -1.0
        d.flags = flags
        for i, v in enumerate(shape):
            d.shape[i] = int(v)
        for i, v in enumerate(fparam):
            d.fparam[i] = float(v)
        self._ck(self._L.bfuse_default_launch(self._ctx, d))
        if grid is not None:
            d.GridDim = Dim3(*grid)
        if block is not None:
            d.BlockDim = Dim3(*block)
        if smem is not None:
            d.smem_bytes = smem
        for i, a in enumerate(args):
            d.args[i] = a
        return d

    def arg_info(self, desc):
        out = []
        for i in range(desc.nargs):
            n, o = C.c_size_t(), C.c_int()
            self._ck(self._L.bfuse_arg_info(self._ctx, desc, i, n, o))
            out.append((n.value, bool(o.value)))
        return out

    def register_kernel(self, desc):
        h = C.c_int()
        self._ck(self._L.bfuse_register_kernel(self._ctx, desc, h))
        return h.value

    def unregister_kernel(self, kernel):
        self._ck(self._L.bfuse_unregister_kernel(self._ctx, kernel))

    def unregister_fusion(self, fusion):
        self._ck(self._L.bfuse_unregister_fusion(self._ctx, fusion))

    def unregister_group(self, group):
        self._ck(self._L.bfuse_unregister_group(self._ctx, group))

    def graph_destroy(self, graph):
        self._ck(self._L.bfuse_graph_destroy(self._ctx, graph))

    def set_dependent_launch(self, enabled):
        """Diagnostic: False launches every later kernel without programmatic dependent launch."""
        self._ck(self._L.bfuse_set_dependent_launch(self._ctx, 1 if enabled else 0))

    def set_kernel_args(self, kernel, args):
        arr = (C.c_void_p * len(args))(*args)
        self._ck(self._L.bfuse_set_kernel_args(self._ctx, kernel, arr, len(args)))

    def register_fusion(self, k1, k2, pattern, param_m=0, param_n=0):
        h = C.c_int()
        self._ck(self._L.bfuse_register_fusion(self._ctx, k1, k2, pattern, param_m, param_n, h))
        return h.value

    def register_group(self, kernels, pattern, param_m=0, param_n=0):
        """2..4 registered kernels of one operator body in one fused launch."""
        arr = (C.c_int * len(kernels))(*kernels)
        h = C.c_int()
        self._ck(self._L.bfuse_register_group(self._ctx, arr, len(kernels), pattern, param_m, param_n, h))
        return h.value

    def group_info(self, group):
        d = KernelDesc()
        self._ck(self._L.bfuse_group_info(self._ctx, group, d))
        return {"KernelName": d.KernelName.decode(), "GridDim": d.GridDim.tuple(), "BlockDim": d.BlockDim.tuple(),
                "Reg": d.Reg, "smem_bytes": d.smem_bytes, "launched_ctas": d.shape[0]}

    def group_map_block(self, group, b):
        k, vb = C.c_int(), C.c_int()
        if self._L.bfuse_group_map_block(self._ctx, group, b, k, vb):
            return None
        return k.value, vb.value

    def launch_group(self, group, stream=None):
        self._ck(self._L.bfuse_launch_group(self._ctx, group, stream))

    def fusion_info(self, fusion):
        d = KernelDesc()
        self._ck(self._L.bfuse_fusion_info(self._ctx, fusion, d))
        return {"KernelName": d.KernelName.decode(), "GridDim": d.GridDim.tuple(), "BlockDim": d.BlockDim.tuple(),
                "Reg": d.Reg, "smem_bytes": d.smem_bytes, "launched_ctas": d.shape[0], "resident_ctas": d.shape[1],
                "retiled_unsplit": (bool(d.shape[2]), bool(d.shape[3]))}

    def map_block(self, fusion, b):
        k, vb = C.c_int(), C.c_int()
        if self._L.bfuse_fusion_map_block(self._ctx, fusion, b, k, vb):
            return None
        return k.value, vb.value

    def launch_kernel(self, kernel, stream=None):
        self._ck(self._L.bfuse_launch_kernel(self._ctx, kernel, stream))

    def launch_sequential(self, fusion, stream=None):
        self._ck(self._L.bfuse_launch_sequential(self._ctx, fusion, stream))

    def launch_parallel(self, fusion, stream=None):
        self._ck(self._L.bfuse_launch_parallel(self._ctx, fusion, stream))

    def launch_fused(self, fusion, stream=None):
        self._ck(self._L.bfuse_launch_fused(self._ctx, fusion, stream))

    def launch_list(self, fusions, mode, stream=None):
        arr = (C.c_int * len(fusions))(*fusions)
        self._ck(self._L.bfuse_launch_list(self._ctx, arr, len(fusions), mode, stream))

    def graph_create(self, fusions, mode):
        arr = (C.c_int * len(fusions))(*fusions)
        g = C.c_int()
        self._ck(self._L.bfuse_graph_create(self._ctx, arr, len(fusions), mode, g))
        return g.value

    def graph_launch(self, graph, stream=None):
        self._ck(self._L.bfuse_graph_launch(self._ctx, graph, stream))

    def trace_fused(self, fusion):
        import numpy as np
        n = self.fusion_info(fusion)["GridDim"][0]
        ks, vbs, sms = (np.empty(n, np.int32) for _ in range(3))
        ip = C.POINTER(C.c_int)
        self._ck(self._L.bfuse_trace_fused(self._ctx, fusion, ks.ctypes.data_as(ip), vbs.ctypes.data_as(ip),
                                           sms.ctypes.data_as(ip), n))
        return ks, vbs, sms

    def gemm_timeline(self, kernel):
        """Nanosecond offsets (from the first mark) of the first CTA's phases of a tcgen05 GEMM kernel."""
        names = ["start", "setup_done", "first_load_issued", "last_load_issued", "first_stage_full", "last_mma_issued",
                 "acc_ready", "partial_written", "cluster_sync1", "reduced", "cluster_sync2", "end"]
        buf = (C.c_longlong * len(names))()
        self._ck(self._L.bfuse_debug_gemm_timeline(self._ctx, kernel, buf, len(names)))
        t0 = buf[0]
        return {n: (buf[i] - t0 if buf[i] else None) for i, n in enumerate(names)}

    def fused_timeline(self, fusions):
        """Per launch of the list (run back to back, fused mode): int64 array [slots, 3] of nanosecond
        marks per dispatch slot -- kernel entry, body start, body end (0 where a slot recorded nothing)."""
        import numpy as np
        slots = [self.fusion_info(f)["GridDim"][0] for f in fusions]
        buf = np.zeros((sum(slots), 3), np.int64)
        self._ck(self._L.bfuse_debug_fused_timeline(self._ctx, (C.c_int * len(fusions))(*fusions), len(fusions),
                                                     buf.ctypes.data_as(C.POINTER(C.c_longlong)), (C.c_int * len(slots))(*slots)))
        out, off = [], 0
        for n in slots:
            out.append(buf[off:off + n])
            off += n
        return out

    def read_status(self):
        s = C.c_int()
        self._ck(self._L.bfuse_read_status(self._ctx, s))
        return s.value

    @staticmethod
    def _host_args(arrays):
        arr = (C.c_void_p * MAX_ARGS)()
        for i, a in enumerate(arrays):
            arr[i] = None if a is None else a.ctypes.data
        return arr

    def run_kernel(self, kernel, host_arrays):
        """run_kernel1/2: H2D inputs, launch, sync, D2H outputs (numpy arrays, None for absent)."""
        self._ck(self._L.bfuse_run_kernel(self._ctx, kernel, self._host_args(host_arrays)))

    def run_parallel(self, fusion, host1, host2):
        self._ck(self._L.bfuse_run_parallel(self._ctx, fusion, self._host_args(host1), self._host_args(host2)))

    def run_fuse(self, fusion, host1, host2):
        self._ck(self._L.bfuse_run_fuse(self._ctx, fusion, self._host_args(host1), self._host_args(host2)))

    def run_fuse_batch(self, fusions, hosts1, hosts2):
        """run_fuse over fusions with separate device buffers; transfers in both directions overlap the kernels
        (pinned host arrays needed for that).  hosts1[i] / hosts2[i]: the host arrays of fusion i's two kernels."""
        n = len(fusions)
        pp = C.POINTER(C.c_void_p)
        keep1, keep2 = [self._host_args(h) for h in hosts1], [self._host_args(h) for h in hosts2]
        a1 = (pp * n)(*[C.cast(k, pp) for k in keep1])
        a2 = (pp * n)(*[C.cast(k, pp) for k in keep2])
        self._ck(self._L.bfuse_run_fuse_batch(self._ctx, (C.c_int * n)(*fusions), n, a1, a2))

    def time(self, fusion, mode, warmup=3, iters=30):
        """(mean_us over back-to-back launches, min_us over individually bracketed launches)."""
        mean, mn = C.c_float(), C.c_float()
        self._ck(self._L.bfuse_time(self._ctx, fusion, mode, warmup, iters, mean, mn))
        return mean.value, mn.value


def check_matrix(value, answer, eps=1e-3):
    """Number of elements the reference's check_matrix would report (utils_cc.py:52-86)."""
    import numpy as np
    v = np.ascontiguousarray(value, np.float32)
    a = np.ascontiguousarray(answer, np.float32)
    return lib().bfuse_check_matrix(v.ctypes.data, a.ctypes.data, v.size, eps)
