"""Per-launch timings in the file format of the reference's analysis script.

The reference profiles every benchmark run with `nsys`, exports the `cuda_gpu_trace` report as CSV
(scripts/profile_test_suite.py:105-110) and its analysis reads those files: one row per kernel launch,
of which it uses `Start (ns)`, `Duration (ns)` and `Name`, skips the first three rows per kernel
(warm-up) and averages the rest (scripts/analyze_test_suite.py:57-122); files are named
`<mode>_<k1>_<k2>_cuda_gpu_trace.csv` with mode 0 = kernel1, 1 = kernel2, 2 = parallel, 3 = hfuse,
4 = bfuse (:164-230).  This module writes the same files from this runtime, so that script can be
pointed at its results.  There is no profiler here: a row's duration is the CUDA-event interval
around one launch on an otherwise idle stream, which includes about a microsecond of launch gap that
`nsys` would not count.
"""
import csv
import os

from . import MODE_FUSED, MODE_KERNEL1, MODE_KERNEL2, MODE_PARALLEL, THREAD_SPLIT, ZIGZAG

HEADER = ["Start (ns)", "Duration (ns)", "CorrId", "GrdX", "GrdY", "GrdZ", "BlkX", "BlkY", "BlkZ", "Reg/Trd", "StcSMem (MB)",
          "DymSMem (MB)", "Bytes (MB)", "Throughput (MB/s)", "SrcMemKd", "DstMemKd", "Device", "Ctx", "GreenCtx", "Strm", "Name"]


def write_gpu_trace(path, rows):
    """rows: dicts with Start (ns), Duration (ns), Name and optionally grid / block / regs / smem."""
    with open(path, "w", newline="") as f:
        w = csv.writer(f)
        w.writerow(HEADER)
        for i, r in enumerate(rows):
            g, b = r.get("grid", (1, 1, 1)), r.get("block", (1, 1, 1))
            w.writerow([int(r["start_ns"]), int(r["duration_ns"]), i + 1, g[0], g[1], g[2], b[0], b[1], b[2], r.get("regs", 0),
                        "0.000", "%.3f" % (r.get("smem", 0) / 1e6), "", "", "", "", r.get("device", "NVIDIA B200 (0)"), 1, "", 7, r["name"]])


def read_gpu_trace(path):
    """[(start_ms, duration_ms, name)] -- the fields the reference's parse_csv keeps, in its units."""
    out = []
    with open(path) as f:
        rows = list(csv.reader(f))
    idx = {h: i for i, h in enumerate(rows[0])}
    for r in rows[1:]:
        if r:
            out.append((float(r[idx["Start (ns)"]]) / 1e6, float(r[idx["Duration (ns)"]]) / 1e6, r[idx["Name"]]))
    return out


def time_launches(torch, launch, count):
    """[(start_ns, duration_ns)] of `count` calls of launch(stream), each bracketed by CUDA events."""
    s = torch.cuda.current_stream()
    origin = torch.cuda.Event(enable_timing=True)
    origin.record(s)
    ev = []
    for _ in range(count):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        launch(s.cuda_stream)
        e1.record(s)
        ev.append((e0, e1))
    torch.cuda.synchronize()
    return [(origin.elapsed_time(e0) * 1e6, e0.elapsed_time(e1) * 1e6) for e0, e1 in ev]


def emit_pair(rt, torch, out_dir, i1, i2, k1, k2, name1, name2, warmup=3, trials=30):
    """The five files of one pair (kernels k1, k2 with suite indices i1, i2).  Returns their paths."""
    os.makedirs(out_dir, exist_ok=True)
    paths = []

    def dump(mode, a, b, rows):
        p = os.path.join(out_dir, "%d_%d_%d_cuda_gpu_trace.csv" % (mode, a, b))
        write_gpu_trace(p, rows)
        paths.append(p)

    n = warmup + trials
    bfuse = rt.register_fusion(k1, k2, ZIGZAG, 1, 1)
    fusions = {4: bfuse}
    try:
        fusions[3] = rt.register_fusion(k1, k2, THREAD_SPLIT, 0, 0)
    except Exception:      # the pair has no thread-level form (clusters, tensor memory, block size): no mode-3 file
        pass
    for mode, a, b, names in ((MODE_KERNEL1, i1, 0, [name1]), (MODE_KERNEL2, 0, i2, [name2]), (MODE_PARALLEL, i1, i2, [name1, name2])):
        t = time_launches(torch, lambda st, mode=mode: rt.launch_list([bfuse], mode, st), n)
        dump(mode, a, b, [dict(start_ns=s, duration_ns=d, name=nm) for s, d in t for nm in names])
    for mode, f in sorted(fusions.items()):
        info = rt.fusion_info(f)
        t = time_launches(torch, lambda st, f=f: rt.launch_fused(f, st), n)
        dump(mode, i1, i2, [dict(start_ns=s, duration_ns=d, name=info["KernelName"], grid=info["GridDim"], block=info["BlockDim"],
                                 regs=info["Reg"], smem=info["smem_bytes"]) for s, d in t])
    return paths
