#!/usr/bin/env python3
"""Benchmark of the horizontal-fusion hot path: fused-pair microseconds, speed-up over back-to-back
unfused launches of the same bodies, fraction of the pair's roofline.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (config.workload): the BERT-base Q-projection || K-projection pair -- two independent
[512x768]x[768x768]+bias GEMMs, fp32 in, tf32 tensor cores, fp32 accumulate -- on seeded synthetic
inputs.  One "step" is one pass over R independent instances of the pair (distinct buffers, like
the layers of a model) replayed from a CUDA graph; R is chosen so the instances together are
larger than twice the 126 MB L2, so every launch reads its operands from HBM.  Multi-GPU: each fused
pair runs on one GPU and there is no exchange step, so the headline pair runs as replicas (every
rank the same step on its own GPU, max over ranks reported); the partitioned workloads ride along
in the same line: `pairs` (the other BASELINE pairs, pair i measured on rank i mod N) and
`conv_n256_sharded` (the ResNet branch pair at batch 256, images split evenly across the ranks, no
collective, time = max over ranks).  `reference_fuser_output` times the reference fuser's own
generated kernels (baseline/_ref/*.cubin, batch-1024 fp32 shapes) beside this runtime's pair at
the same shapes.

One JSON line on stdout (rank 0).  `value` = microseconds per fused pair, inputs resident in HBM;
`e2e` = the same metric through bfuse_run_fuse_batch with pinned HOST buffers (H2D of every input,
launch, D2H of every output inside the timed region; transfers of neighbouring pairs overlap).  `--impl reference` times the CPU
restatement of the same pair (the reference has no CPU operator code of its own) on the host cores.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "cfg2_q_k_proj"
NCU_TRAFFIC_BYTES = 7954944   # dram__bytes_read.sum + dram__bytes_write.sum of the fused kernel, one launch (profiles/)
L2_BYTES = 126 * 1024 * 1024
NAIVE_BODY_PAIRS = ("cfg2_q_k_proj", "cfg3_qkt_res_layernorm", "cfg5_conv_branches")   # fp32 pairs with a CUDA-core body


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """SM clock and throttle-reason samples taken during the timed region.  The region lasts
    milliseconds, so the samples come from NVML queries (read-only) polled by a thread every
    millisecond; `nvidia-smi -lms` would not deliver its first line in time."""

    REASONS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index, uuid=None):
        self.rows, self.index, self.uuid = [], index, uuid
        self.nvml, self.handle, self.thread, self.halt = None, None, None, threading.Event()

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + str(self.uuid)).encode()) if self.uuid else None
            except pynvml.NVMLError:
                self.handle = None
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self._sample(pynvml)          # one sample before the region starts, so a very short region still has one
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception:                 # no NVML on this machine: the record says so
            self.nvml = None

    def _sample(self, nv):
        self.rows.append((int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)),
                          int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))))

    def _poll(self):
        while not self.halt.is_set():
            try:
                self._sample(self.nvml)
            except Exception:
                break
            self.halt.wait(0.001)

    def stop(self):
        if not self.nvml:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self.halt.set()
        self.thread.join(timeout=1.0)
        rows = self.rows[1:] if len(self.rows) > 1 else self.rows
        mhz = sorted(r[0] for r in rows)
        reasons = [n for n, bit in self.REASONS if any(r[1] & bit for r in rows)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(rows)}


def cpu_pair_time(spec, budget_s=8.0):
    """Time the oracle's plain loops (OpenMP) on one instance of the pair; microseconds per pair."""
    import oracle
    oracle.set_num_threads(len(os.sched_getaffinity(0)))   # all host cores, whatever OMP_NUM_THREADS a launcher exported
    oracle_outputs = _load_pair_oracle().oracle_outputs
    oracle_outputs(spec.a), oracle_outputs(spec.b)  # warm-up
    best, n, t_end = None, 0, time.perf_counter() + budget_s
    while n < 5 or (time.perf_counter() < t_end and n < 50):
        t0 = time.perf_counter()
        oracle_outputs(spec.a)
        oracle_outputs(spec.b)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        n += 1
        if time.perf_counter() > t_end and n >= 5:
            break
    return best * 1e6, n, oracle.num_threads()


def run_reference(args):
    """CPU arm: the oracle port of the same pair on the host cores (rank 0 only)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from bfuse_project_b200 import workloads as wl
    spec = wl.make_pair(WORKLOAD, seed=0)
    us, n, cores = None, 0, 0
    samples = []
    for _ in range(args.warmup):
        cpu_pair_time(spec, 0.0)
    for _ in range(args.steps):
        u, n, cores = cpu_pair_time(spec, 2.0)
        samples.append(u)
    us = sum(samples) / len(samples)
    line = {
        "impl": "reference", "metric": "fused_pair_us", "value": us, "unit": "us", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD + ": BERT-base Q||K projection, 2x([512x768]x[768x768]+bias)",
                   "note": "the reference ships no CPU operator code; this is the plain C/OpenMP restatement "
                           "(oracle/), both GEMMs back to back, best of >=5 runs per step"},
        "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": "port",
                         "sample": "one full pair per run (1.2 GFLOP), best of %d runs per step" % n},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_sweep(args, rt, torch, rank, world, local, pk):
    """The operator cross-product sweep, its pairs dealt round-robin to the ranks; rank 0 prints one
    JSON line with the summary (and writes the per-pair table when asked to)."""
    from bfuse_project_b200 import partition, sweep
    n_ops = min(args.sweep_limit or len(sweep.SWEEP_OPS), len(sweep.SWEEP_OPS))
    sets = sweep.build_operands(rt, torch, local, seed=0, ops=sweep.SWEEP_OPS[:n_ops])
    todo = sweep.pair_indices(n_ops)
    mine = partition.assign_pairs(todo, world, rank)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    import bfuse_project_b200 as bfm
    pattern = {"zigzag": bfm.ZIGZAG, "range": bfm.RANGE_SPLIT, "striped": bfm.SM_STRIPED, "proportional": bfm.PROPORTIONAL}[args.sweep_pattern]
    res = sweep.measure(rt, sets, mine, pk["hbm_gbs"], pk["bf16_tflops"] * 0.5, pattern=pattern)
    wall = time.perf_counter() - t0
    alone = sweep.alone_times(rt, sets) if rank == 0 else None      # for the pair-selection model, outside the wall time
    assert rt.read_status() == 0, "a bounded device-side wait gave up during the sweep"
    if world > 1:
        import torch.distributed as dist
        gathered, walls = [None] * world, [None] * world
        dist.all_gather_object(gathered, res)
        dist.all_gather_object(walls, wall)
        res, wall = partition.merge_results(gathered), partition.max_over_ranks(walls)
        dist.destroy_process_group()
    if rank != 0:
        return
    line = {"metric": "sweep_wall_s", "value": wall, "unit": "s", "n_gpus": world, "higher_is_better": False, "scaling": "strong",
            "dtype": "tf32", "data": "synthetic",
            "config": {"workload": "operator cross-product sweep: %d operators, %d pairs (upper triangle), %s fusion vs "
                                   "back-to-back launches; 3 warm-ups + 30 timed launches per mode" % (n_ops, len(todo), args.sweep_pattern),
                       "partition": "pair i on rank i mod %d" % world},
            "sweep": sweep.summarise(res)}
    from bfuse_project_b200 import pairing
    line["pairing_model"] = pairing.evaluate(sweep.pairing_records(sets, res, alone, rt.sm_count))
    if args.sweep_out:
        with open(args.sweep_out, "w") as f:
            json.dump({"operators": [{"name": n, "shape": list(sh), "alone_us": alone[i], "launch": [list(x) if isinstance(x, tuple) else x for x in sets[0][i].launch]}
                                     for i, (n, sh) in enumerate(sweep.SWEEP_OPS[:n_ops])], "pairs": res}, f, indent=0)
    print(json.dumps(line), flush=True)


def replay_us(rt, torch, graph, launches, reps=5, warm=3):
    """Microseconds per launch of a CUDA-graph replay, CUDA events on torch's current stream."""
    s = torch.cuda.current_stream().cuda_stream
    for _ in range(warm):
        rt.graph_launch(graph, s)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        rt.graph_launch(graph, s)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * launches)


MODES = (("fused_zigzag", "ZIGZAG", 4), ("fused_range", "RANGE_SPLIT", 4), ("fused_striped", "SM_STRIPED", 4),
         ("fused_queue", "WORK_QUEUE", 4), ("fused_thread_split", "THREAD_SPLIT", 4), ("sequential", "ZIGZAG", 3),
         ("parallel", "ZIGZAG", 2))


def measure_pair(rt, torch, bf, wl, pk, name, device, conv_batch=1, max_reps=24):
    """Fused (every pattern that can host the pair) / sequential / two-stream microseconds of one
    BASELINE pair, replayed over enough instances to exceed twice the L2."""
    spec = wl.make_pair(name, seed=0, conv_batch=conv_batch)
    reps = max(2, min(max_reps, int(2.2 * L2_BYTES / spec.bytes) + 1))
    pairs = [wl.DevicePair(rt, spec if s == 0 else wl.make_pair(name, seed=s, conv_batch=conv_batch), device) for s in range(reps)]
    res = {"instances": reps, "alg_bytes": spec.bytes, "alg_flops": spec.flops, "dtype": spec.dtype,
           "launch": [list(spec.a.launch[0]) + list(spec.a.launch[1]), list(spec.b.launch[0]) + list(spec.b.launch[1])]}
    for label, pattern, mode in MODES:
        pat = getattr(bf, pattern)
        mn = 1 if pat in (bf.ZIGZAG, bf.WORK_QUEUE) else 0
        try:
            fus = [p.fusion(pat, mn, mn) for p in pairs]
        except bf.BfuseError as e:
            if e.code not in (3, 7):
                raise
            continue   # the pattern cannot host this pair (clustered operators; thread split: windows or TMEM over budget)
        res[label + "_us"] = replay_us(rt, torch, rt.graph_create(fus, mode), reps)
    best = min(v for k, v in res.items() if k.startswith("fused_"))
    res["best_fused_us"] = best
    res["speedup_vs_sequential"] = res["sequential_us"] / best
    res["speedup_vs_parallel_streams"] = res["parallel_us"] / best
    tensor_peak = pk["bf16_tflops"] * (1e6 if spec.dtype == "bf16" else 0.5e6)   # flop per us; tf32 = half of bf16
    res["roofline_us"] = max(spec.bytes / (pk["hbm_gbs"] * 1e3), spec.flops / tensor_peak)
    res["roofline_frac"] = res["roofline_us"] / best
    del pairs
    torch.cuda.empty_cache()
    if name in NAIVE_BODY_PAIRS and conv_batch == 1:
        # the reference's zig-zag dispatch around plain CUDA-core fp32 bodies of the same operators:
        # the stand-in for the reference fuser's output at this exact shape (which cannot be generated here)
        npairs = [wl.DevicePair(rt, wl.make_pair(name, seed=s, tensor_cores=False), device) for s in range(reps)]
        nf = [p.fusion(bf.ZIGZAG, 1, 1) for p in npairs]
        res["naive_bodies_zigzag_us"] = replay_us(rt, torch, rt.graph_create(nf, 4), reps)
        res["naive_bodies_sequential_us"] = replay_us(rt, torch, rt.graph_create(nf, 3), reps)
        res["speedup_vs_naive_bodies_zigzag"] = res["naive_bodies_zigzag_us"] / best
        del npairs
        torch.cuda.empty_cache()
    return res


def attention_block(rt, torch, bf):
    """The QK^T -> softmax -> PV chain of a BERT-base / GPT-2 attention block (12 heads, 512 tokens,
    head size 64, causal), as plain launches and software-pipelined over head groups with horizontally
    fused steps; CUDA-graph replay on the same buffers (they fit the L2)."""
    from bfuse_project_b200 import attention
    try:
        gen = torch.Generator(device="cuda")
        gen.manual_seed(0)
        q, k = (torch.randn(12, 512, 64, device="cuda", generator=gen) for _ in range(2))
        vt = torch.randn(12, 64, 512, device="cuda", generator=gen)
        out = {"shape": {"heads": 12, "seq": 512, "head_dim": 64, "causal": True}}
        one = attention.AttentionBlock(rt, torch, q, k, vt, groups=1)
        out["one_group_3_launches_us"] = attention.graph_time_us(torch, one.run_sequential, repeat=4)
        for groups in (2, 4, 6):
            blk = attention.AttentionBlock(rt, torch, q, k, vt, groups=groups)
            seq_us = attention.graph_time_us(torch, blk.run_sequential, repeat=4)
            pip_us = attention.graph_time_us(torch, blk.run_pipelined, repeat=4)
            blk.run_sequential(torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            want = blk.out.clone()
            blk.out.zero_()
            blk.run_pipelined(torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            out["groups_%d" % groups] = {"sequential_launches": blk.launches_sequential, "sequential_us": seq_us,
                                         "pipelined_launches": blk.launches_pipelined, "pipelined_fused_us": pip_us,
                                         "speedup": seq_us / pip_us, "bit_identical": bool(torch.equal(want, blk.out))}
        return out
    except Exception as e:   # reported, not hidden
        return {"error": str(e)[:300]}


def model_segments(rt, torch, bf):
    """Operator lists of model layers walked by the segment driver: ready operators of one body share an
    n-way launch (Q || K || V, the branches of a down-sampling block, the same operator of independent
    requests), against one launch per operator, each tiled for the whole GPU; CUDA-graph replay of the whole
    segment on the same buffers."""
    from bfuse_project_b200 import attention, segment
    out = {}
    for name, build in segment.SEGMENTS.items():
        try:
            b, ops = build(rt, torch)
            seg = segment.Segment(rt, ops)
            seq_us = attention.graph_time_us(torch, seg.run_sequential, repeat=4)
            fused_us = attention.graph_time_us(torch, seg.run_fused, repeat=4)
            stream = torch.cuda.current_stream().cuda_stream
            names = sorted({w for o in ops for w in o.writes})
            seg.run_unfused(stream)     # the fused program's kernels one by one
            torch.cuda.synchronize()
            want = {n: b.buf[n].clone() for n in names}
            for n in names:
                b.buf[n].zero_()
            seg.run_fused(stream)
            torch.cuda.synchronize()
            same = all(torch.equal(b.buf[n].view(torch.uint8), want[n].view(torch.uint8)) for n in names)
            kinds = [k for step in seg.describe() for k, _ in step]
            steps = []   # every shared launch alone, against its operators back to back
            for step, names in zip(seg.steps, seg.describe()):
                for (kind, h, idx), (_, nm) in zip(step, names):
                    if kind == "single":
                        continue
                    one = attention.graph_time_us(torch, lambda st, kind=kind, h=h: (rt.launch_group if kind == "group" else rt.launch_fused)(h, st), repeat=10)
                    b2b = attention.graph_time_us(torch, lambda st, idx=idx: [rt.launch_kernel(seg.alone[i], st) for i in idx], repeat=10)
                    steps.append({"kind": kind, "operators": nm, "one_launch_us": one, "back_to_back_us": b2b})
            out[name] = {"operators": seg.launches_sequential, "fused_launches": seg.launches_fused,
                         "groups": kinds.count("group"), "pairs": kinds.count("pair"),
                         "sequential_us": seq_us, "fused_us": fused_us, "speedup": seq_us / fused_us, "bit_identical": bool(same),
                         "steps": steps}
            del b, ops, seg, want
            torch.cuda.empty_cache()
        except Exception as e:   # reported, not hidden
            out[name] = {"error": str(e)[:300]}
    return out


def reference_fuser_output(rt, torch, bf, wl, pk):
    """The reference fuser's generated bfuse / hfuse kernels compiled for sm_100a, at their own
    batch-1024 fp32 shapes, beside this runtime's fused pair on the same shapes (fp32 in, tf32 MMA)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import numpy as np
    import ref_fuser
    out = {}
    stream = torch.cuda.current_stream().cuda_stream
    for name in ref_fuser.available():
        try:
            cfg = ref_fuser.PAIRS[name]
            sh1, sh2 = ref_fuser.shapes(name)
            bufs = [torch.randn(*s, device="cuda") * (0.02 if i % 3 == 1 else 1.0) for i, s in enumerate(sh1 + sh2)]
            ptrs = [b.data_ptr() for b in bufs]
            res = {"shape": {k: v for k, v in cfg.items() if k != "grids"}}
            for flavour in ("bfuse", "hfuse"):
                k = ref_fuser.RefKernel(name, flavour)
                for _ in range(2):
                    k.launch(ptrs, stream)
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                n = 5
                e0.record()
                for _ in range(n):
                    k.launch(ptrs, stream)
                e1.record()
                torch.cuda.synchronize()
                res["reference_%s_us" % flavour] = e0.elapsed_time(e1) * 1e3 / n
            ref_out = [bufs[2].clone(), bufs[5].clone()]
            # this runtime on the same buffers and shapes
            if cfg["kind"] == "conv":
                shapes = [(cfg["n"], cfg["ci"], cfg["h"], cfg["w"], cfg["co"], kk, kk, cfg["stride"], pp) for kk, pp in zip(cfg["k"], cfg["pad"])]
                descs = [rt.describe("conv%d" % i, bf.OP_CONV2D_TF32, shapes[i], [ptrs[3 * i], ptrs[3 * i + 1], ptrs[3 * i + 2]]) for i in range(2)]
            else:
                b = cfg.get("b", 1)
                descs = [rt.describe("gemm%d" % i, bf.OP_GEMM_TF32, (b, cfg["M"], cfg["N"], cfg["K"], 0, 0),
                                     [ptrs[3 * i], ptrs[3 * i + 1], None, ptrs[3 * i + 2]]) for i in range(2)]
            for i in (2, 5):
                bufs[i].zero_()
            f = rt.register_fusion(rt.register_kernel(descs[0]), rt.register_kernel(descs[1]), bf.ZIGZAG, 1, 1)
            rt.launch_fused(f, stream)
            torch.cuda.synchronize()
            # same operator, tf32 operands: agree with the reference's fp32 FMA output within 5e-3
            for got, ref in ((bufs[2], ref_out[0]), (bufs[5], ref_out[1])):
                rms = float(ref.float().pow(2).mean().sqrt())
                err = float((got - ref).abs().max())
                res.setdefault("max_abs_diff_over_rms", []).append(err / max(rms, 1e-30))
            g = rt.graph_create([f], bf.MODE_FUSED)
            res["ours_fused_us"] = replay_us(rt, torch, g, 1, reps=5, warm=2)
            res["speedup_vs_reference_bfuse"] = res["reference_bfuse_us"] / res["ours_fused_us"]
            res["speedup_vs_reference_hfuse"] = res["reference_hfuse_us"] / res["ours_fused_us"]
            out[name] = res
            del bufs, ref_out
            torch.cuda.empty_cache()
        except Exception as e:
            out[name] = {"error": str(e)[:300]}
    if not out:
        out["unavailable"] = "baseline/_ref/*.cubin not built (needs a reference checkout at build time)"
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="bfuse")
    ap.add_argument("--quick", action="store_true", help="skip the side measurements of the other pairs")
    ap.add_argument("--sweep", action="store_true", help="run the 42 x 42 operator cross-product sweep instead (pair i on rank i mod N)")
    ap.add_argument("--sweep-out", default="", help="with --sweep: also write the per-pair table to this JSON file")
    ap.add_argument("--sweep-limit", type=int, default=0, help="with --sweep: only the first N operators")
    ap.add_argument("--sweep-pattern", default="zigzag", choices=["zigzag", "range", "striped", "proportional"],
                    help="with --sweep: the block-level pattern of the fused launches")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch

    import bfuse_project_b200 as bf
    from bfuse_project_b200 import workloads as wl

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pk = peaks()

    rt = bf.Runtime(local)
    if args.sweep:
        return run_sweep(args, rt, torch, rank, world, local, pk)
    spec0 = wl.make_pair(WORKLOAD, seed=0)
    reps = int(2.2 * L2_BYTES / spec0.bytes) + 1           # instances per step, together > 2 x L2
    specs = [spec0] + [wl.make_pair(WORKLOAD, seed=s) for s in range(1, reps)]
    pairs = [wl.DevicePair(rt, s, local) for s in specs]
    stream = torch.cuda.current_stream().cuda_stream

    def graph_for(pattern, mode, m=1, n=1):
        try:
            return rt.graph_create([p.fusion(pattern, m, n) for p in pairs], mode)
        except bf.BfuseError as e:
            if e.code not in (3, 7):
                raise
            return None   # the pattern cannot host this pair (clustered operators; thread split: windows or TMEM over budget)

    graphs = {"fused_zigzag": graph_for(bf.ZIGZAG, bf.MODE_FUSED), "fused_range": graph_for(bf.RANGE_SPLIT, bf.MODE_FUSED, 0, 0),
              "fused_striped": graph_for(bf.SM_STRIPED, bf.MODE_FUSED, 0, 0),
              "fused_queue": graph_for(bf.WORK_QUEUE, bf.MODE_FUSED), "fused_thread_split": graph_for(bf.THREAD_SPLIT, bf.MODE_FUSED, 0, 0),
              "sequential": graph_for(bf.ZIGZAG, bf.MODE_SEQUENTIAL),
              "parallel": graph_for(bf.ZIGZAG, bf.MODE_PARALLEL)}
    graphs = {k: g for k, g in graphs.items() if g is not None}

    def timed(graph, steps, warmup):
        for _ in range(warmup):
            rt.graph_launch(graph, stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            rt.graph_launch(graph, stream)
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    # spin ~100 ms first so the clocks have left their idle state, pick the fused pattern on a short
    # trial, then time exactly K steps of it under the clock sampler
    t_spin = time.perf_counter()
    while time.perf_counter() - t_spin < 0.1:
        rt.graph_launch(graphs["sequential"], stream)
        torch.cuda.synchronize()
    trial = {k: timed(g, 3, 3) for k, g in graphs.items()}
    best = min((k for k in trial if k.startswith("fused_")), key=lambda k: trial[k])
    sampler = ClockSampler(local, getattr(torch.cuda.get_device_properties(local), "uuid", None))
    if rank == 0:
        sampler.start()
    ms = timed(graphs[best], args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    side = {k: timed(g, args.steps, 3) * 1e3 / (args.steps * reps) for k, g in graphs.items() if k != best}
    us_pair = ms * 1e3 / (args.steps * reps)
    side[best] = us_pair
    assert rt.read_status() == 0, "a bounded device-side wait gave up during the benchmark"

    # what was just timed must equal the unfused launches of the same bodies, bit for bit
    fused_out = pairs[0].read_outputs()
    pairs[0].clear_outputs()
    rt.launch_sequential(pairs[0].fusion(bf.ZIGZAG, 1, 1), stream)
    seq_out = pairs[0].read_outputs()
    for k in range(2):
        assert np.array_equal(fused_out[k][0].view(np.uint8), seq_out[k][0].view(np.uint8)), "fused != unfused"

    # end to end through the host-buffer entry point: pinned host inputs and outputs
    def pinned_like(arr):
        t = torch.from_numpy(arr.copy()).pin_memory() if arr.dtype != np.uint16 else \
            torch.from_numpy(arr.view(np.int16).copy()).pin_memory()
        return t

    e2e_pairs = pairs[: min(8, reps)]
    host = []
    for p in e2e_pairs:
        h = [[None if a is None else pinned_like(a) for a in ks.host] for ks in (p.spec.a, p.spec.b)]
        host.append([[None if t is None else t.numpy() for t in hk] for hk in h] + [h])
    best_pat = {"fused_zigzag": bf.ZIGZAG, "fused_range": bf.RANGE_SPLIT, "fused_queue": bf.WORK_QUEUE, "fused_striped": bf.SM_STRIPED,
                "fused_thread_split": bf.THREAD_SPLIT}[best]
    best_mn = 1 if best_pat in (bf.ZIGZAG, bf.WORK_QUEUE) else 0
    fus = [p.fusion(best_pat, best_mn, best_mn) for p in e2e_pairs]
    for i in range(min(3, len(fus))):
        rt.run_fuse(fus[i], host[i][0], host[i][1])
    rt.run_fuse_batch(fus, [h[0] for h in host], [h[1] for h in host])
    t0 = time.perf_counter()
    for i, f in enumerate(fus):    # the same pairs one synchronous call each, as the reference's run_fuse does
        rt.run_fuse(f, host[i][0], host[i][1])
    e2e_sync_us = (time.perf_counter() - t0) * 1e6 / len(fus)
    e2e_steps = max(3, min(args.steps, 10))
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):     # one call per step: the pairs' copies in, launches and copies out overlap on three streams
        rt.run_fuse_batch(fus, [h[0] for h in host], [h[1] for h in host])
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_us = e2e_s * 1e6 / (e2e_steps * len(fus))
    h2d = sum(a.nbytes for ks in (spec0.a, spec0.b) for i, a in enumerate(ks.host) if a is not None and i not in ks.outputs)
    d2h = sum(ks.host[i].nbytes for ks in (spec0.a, spec0.b) for i in ks.outputs)

    # ---- partitioned side workloads (no collective on the data path) --------------------------------
    side_pairs, conv256 = {}, None
    if not args.quick:
        from bfuse_project_b200 import partition
        names = [n for n in wl.pair_names() if n != WORKLOAD]
        for name in partition.assign_pairs(names, world, rank):   # pair sweep: pair i on rank i mod N
            if True:
                try:
                    side_pairs[name] = measure_pair(rt, torch, bf, wl, pk, name, local)
                    side_pairs[name]["rank"] = rank
                except Exception as e:                  # a pair that cannot run is reported, not hidden
                    side_pairs[name] = {"error": str(e)[:300], "rank": rank}
        # ResNet branch pair at batch 256, images split across the ranks
        per_rank = partition.shard_batch(256, world, rank)[1]
        try:
            r = measure_pair(rt, torch, bf, wl, pk, "cfg5_conv_branches", local, conv_batch=per_rank, max_reps=2)
            t = torch.tensor([r["best_fused_us"], r["sequential_us"]], device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            conv256 = {"images_total": 256, "images_per_rank": per_rank, "fused_us": float(t[0]), "sequential_us": float(t[1]),
                       "speedup_vs_sequential": float(t[1] / t[0]), "alg_bytes_total": r["alg_bytes"] * world,
                       "roofline_us": r["alg_bytes"] / (pk["hbm_gbs"] * 1e3), "images_per_s": 256 / (float(t[0]) * 1e-6)}
            conv256["roofline_frac"] = conv256["roofline_us"] / conv256["fused_us"]
        except Exception as e:
            conv256 = {"error": str(e)[:300]}
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, side_pairs)
            side_pairs = partition.merge_results(gathered)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu_us, cpu_n, cores = cpu_pair_time(spec0, 10.0)
    t_roof_us = max(spec0.bytes / (pk["hbm_gbs"] * 1e3), spec0.flops / (pk["bf16_tflops"] * 0.5e6))
    achieved = spec0.bytes / (us_pair * 1e-6) / 1e9
    info = rt.fusion_info(pairs[0].fusion(best_pat, best_mn, best_mn))   # the kernel that was timed
    line = {
        "metric": "fused_pair_us", "value": us_pair, "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
        "config": {"workload": WORKLOAD + ": BERT-base Q||K projection, 2x([512x768]x[768x768]+bias), fp32 in, tf32 MMA",
                   "pattern": best, "instances_per_step": reps, "launch": "CUDA graph replay of %d fused launches" % reps,
                   "l2": "inputs larger than L2: %d instances x %.1f MB = %.0f MB vs 126 MB L2" % (reps, spec0.bytes / 1e6, reps * spec0.bytes / 1e6),
                   "multi_gpu": "replicas only" if world > 1 else "n/a",
                   "fused_kernel": info},
        "speedup_vs_sequential": side["sequential"] / us_pair,
        "speedup_vs_parallel_streams": side["parallel"] / us_pair,
        "us": side,
        "roofline_pair_us": t_roof_us, "roofline_pair_frac": t_roof_us / us_pair,
        "pairs_per_s": world * 1e6 / us_pair,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": NCU_TRAFFIC_BYTES, "peak_source": pk["source"],
                     "traffic_note": "dram read + write of one launch from the ncu capture summarised in "
                                     "profiles/fused_gemm_tf32_pair_cfg2.md; the 3.15 MB of outputs are still in L2 at kernel end",
                     "alg_bytes_per_launch": spec0.bytes, "kernel": info["KernelName"]},
        "cpu_baseline": {"value": cpu_us, "unit": "us", "cores": cores, "kind": "port",
                         "sample": "one full pair (1.2 GFLOP) per run, best of %d runs" % cpu_n},
        "e2e": {"value": e2e_us, "unit": "us", "h2d_bytes_per_step": h2d * len(fus), "d2h_bytes_per_step": d2h * len(fus),
                "note": "bfuse_run_fuse_batch on pinned host buffers, %d pairs per call: H2D inputs, fused launch, D2H outputs of "
                        "neighbouring pairs overlap; per pair" % len(fus),
                "one_synchronous_call_per_pair_us": e2e_sync_us},
        "gpu_launches": args.steps * reps,
        "clocks": clocks,
    }
    if not args.quick:
        line["pairs"] = side_pairs
        line["conv_n256_sharded"] = conv256
        line["attention_block"] = attention_block(rt, torch, bf)
        line["model_segments"] = model_segments(rt, torch, bf)
        line["reference_fuser_output"] = reference_fuser_output(rt, torch, bf, wl, pk)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def _load_pair_oracle():
    import importlib.util
    spec = importlib.util.spec_from_file_location("tests_pair_oracle", os.path.join(ROOT, "tests", "pair_oracle.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    main()
