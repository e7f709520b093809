#!/usr/bin/env python3
"""Benchmark of the horizontal-fusion hot path: fused-pair microseconds, speed-up over back-to-back
unfused launches of the same bodies, fraction of the pair's roofline.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (config.workload): the largest single-GPU configuration -- the ResNet-18 branch pair, a 3x3
stride-2 conv || a 1x1 stride-2 downsample conv, 64 -> 128 channels, over ONE seeded batch of 256
images [64, 56, 56] (fp32 in, tf32 tensor cores, fp32 accumulate; 617 MB of algorithmic traffic).  With
--gpus N the images are split across the ranks (rank r takes the slice partition.shard_batch gives it,
no collective on the data path), so the job is the same 256 images at every N: strong scaling.  One
"step" is one fused launch over the rank's shard; consecutive steps rotate over R instances of the
shard (distinct buffers) so that the steps' inputs together exceed twice the 126 MB L2.  `value` =
microseconds per fused pair over the whole batch (the slowest rank), inputs resident in HBM; `e2e` =
the same metric through bfuse_run_fuse_batch with pinned HOST buffers (H2D of the shard, fused launches,
D2H of both outputs inside the timed region, the transfers of neighbouring sub-shards overlapping).

The other BASELINE pairs ride along as side measurements (pair i on rank i mod N); `per_config`, the
LAST key of the line, holds every configuration's best fused / sequential microseconds, roofline fraction
and pattern.  `reference_fuser_output` times the reference fuser's own generated kernels
(baseline/_ref/*.cubin, batch-1024 fp32 shapes) beside this runtime's pair at the same shapes.
`--impl reference` times the CPU restatement of the same pair (the reference has no CPU operator code of
its own) on the host cores, on a stated sample of the images.

One JSON line on stdout (rank 0).
"""
import argparse
import json
import os
import re
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "cfg5_conv_branches_n256"
WORKLOAD_DESC = (WORKLOAD + ": ResNet-18 3x3 s2 conv || 1x1 s2 downsample, 64->128 channels, one seeded batch of 256 x [64,56,56] "
                 "fp32 NCHW, tf32 MMA with fp32 accumulate; images split across the GPUs")
BATCH = 256
CONV_PROFILE = os.path.join(ROOT, "profiles", "fused_conv_tf32_pair_cfg5.md")
L2_BYTES = 126 * 1024 * 1024
NAIVE_BODY_PAIRS = ("cfg2_q_k_proj", "cfg3_qkt_res_layernorm", "cfg5_conv_branches")   # fp32 pairs with a CUDA-core body
CPU_SAMPLE_IMAGES = 32


def dram_bytes_per_image():
    """DRAM read + write bytes per image of the fused conv kernel, from the line `dram_bytes_per_image: N`
    of the committed ncu summary (the capture runs a smaller batch; traffic grows in proportion to it)."""
    try:
        m = re.search(r"dram_bytes_per_image:\s*([0-9.eE+]+)", open(CONV_PROFILE).read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


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


def cpu_conv_pair(images, seed=0, runs=1):
    """The oracle's plain loops (C + OpenMP, all host cores) over `images` images of the seeded batch, both
    convs back to back; (best seconds over `runs`, threads used).  The batch comes from numpy's default_rng --
    the CPU arm needs the values' distribution, not the device generator's bits."""
    import numpy as np
    import oracle
    oracle.set_num_threads(len(os.sched_getaffinity(0)))   # all host cores, whatever OMP_NUM_THREADS a launcher exported
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((images, 64, 56, 56), dtype=np.float32)
    w3 = (np.sqrt(2.0 / 576) * rng.standard_normal((128, 64, 3, 3), dtype=np.float32)).astype(np.float32)
    w1 = (np.sqrt(2.0 / 64) * rng.standard_normal((128, 64, 1, 1), dtype=np.float32)).astype(np.float32)
    best = None
    for _ in range(runs):
        t0 = time.perf_counter()
        oracle.conv2d_nchw(x, w3, 2, 1)
        oracle.conv2d_nchw(x, w1, 2, 0)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best, oracle.num_threads()


def cpu_pair_time(spec, budget_s=8.0):
    """Time the oracle's plain loops (OpenMP) on one instance of a pair; microseconds per pair."""
    import oracle
    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    oracle_outputs = _load_pair_oracle().oracle_outputs
    oracle_outputs(spec.a), oracle_outputs(spec.b)  # warm-up
    best, n, t_end = None, 0, time.perf_counter() + budget_s
    while n < 3 or (time.perf_counter() < t_end and n < 50):
        t0 = time.perf_counter()
        oracle_outputs(spec.a)
        oracle_outputs(spec.b)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
        n += 1
    return best * 1e6, n, oracle.num_threads()


def run_reference(args):
    """CPU arm: the oracle port of the same pair on the host cores (rank 0 only).  One step = the pair over
    CPU_SAMPLE_IMAGES images of the batch, scaled to the 256 images of the job."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = 0
    for _ in range(args.warmup):
        cpu_conv_pair(CPU_SAMPLE_IMAGES)
    samples = []
    for _ in range(args.steps):
        sec, cores = cpu_conv_pair(CPU_SAMPLE_IMAGES)
        samples.append(sec * 1e6 * BATCH / CPU_SAMPLE_IMAGES)
    us = sum(samples) / len(samples)
    line = {
        "impl": "reference", "metric": "fused_pair_us", "value": us, "unit": "us", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": us / 1e3, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD_DESC,
                   "note": "the reference ships no CPU operator code; this is the plain C/OpenMP restatement "
                           "(oracle/), both convs back to back on all host cores"},
        "cpu_baseline": {"value": us, "unit": "us", "cores": cores, "kind": "port",
                         "sample": "%d of the 256 images per step (%.2f GFLOP), time scaled by %d" % (
                             CPU_SAMPLE_IMAGES, CPU_SAMPLE_IMAGES * 0.1285, BATCH // CPU_SAMPLE_IMAGES)},
        "e2e": {"value": us, "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_sweep(args, rt, torch, rank, world, local, pk):
    """The operator cross-product sweep, its pairs dealt round-robin to the ranks; rank 0 prints one
    JSON line with the summary (and writes the per-pair table when asked to)."""
    from bfuse_project_b200 import partition, sweep
    n_ops = min(args.sweep_limit or len(sweep.SWEEP_OPS), len(sweep.SWEEP_OPS))
    op_list = list(sweep.SWEEP_OPS[:n_ops])
    todo = sweep.pair_indices(n_ops)
    if args.sweep_extra:
        # the pair-selection model's extra operators (memory-bound bodies, bf16 projections): only the pairs that have one
        op_list += list(sweep.MODEL_EXTRA_OPS)
        todo = [(i, j) for i, j in sweep.pair_indices(len(op_list)) if j >= n_ops]
    sets = sweep.build_operands(rt, torch, local, seed=0, ops=op_list)
    mine = partition.assign_pairs(todo, world, rank)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    import bfuse_project_b200 as bfm
    pattern = {"zigzag": bfm.ZIGZAG, "range": bfm.RANGE_SPLIT, "striped": bfm.SM_STRIPED, "proportional": bfm.PROPORTIONAL, "all": "all"}[args.sweep_pattern]
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
                                   "back-to-back launches; 3 warm-ups + 30 timed launches per mode" % (len(op_list), len(todo), args.sweep_pattern),
                       "partition": "pair i on rank i mod %d" % world},
            "sweep": sweep.summarise(res)}
    from bfuse_project_b200 import pairing
    records = sweep.pairing_records(sets, res, alone, rt.sm_count)
    line["pairing_model"] = pairing.evaluate(records)
    if args.sweep_out:
        with open(args.sweep_out, "w") as f:
            json.dump({"operators": [{"name": n, "shape": list(sh), "alone_us": alone[i], "launch": [list(x) if isinstance(x, tuple) else x for x in sets[0][i].launch]}
                                     for i, (n, sh) in enumerate(op_list)], "pairs": res, "records": records}, f, indent=0)
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


# (label, pattern, harness mode, M, N); zig-zag in runs of two puts both operators on every SM, strict
# alternation sends them to alternate SMs (the hardware deals consecutive CTAs to the two SMs of a TPC)
MODES = (("fused_zigzag", "ZIGZAG", 4, 1, 1), ("fused_zigzag2", "ZIGZAG", 4, 1, 2), ("fused_range", "RANGE_SPLIT", 4, 0, 0),
         ("fused_striped", "SM_STRIPED", 4, 0, 0), ("fused_queue", "WORK_QUEUE", 4, 1, 1), ("fused_thread_split", "THREAD_SPLIT", 4, 0, 0),
         ("sequential", "ZIGZAG", 3, 1, 1), ("parallel", "ZIGZAG", 2, 1, 1))


class L2Flusher:
    """Writes a buffer larger than the L2 so that the next launch starts cold."""

    def __init__(self, torch, device):
        self.buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=torch.device("cuda", device))

    def flush(self):
        self.buf.fill_(1)


def isolated_us(rt, torch, flusher, launch, n=5):
    """Microseconds of ONE launch, CUDA events around it, L2 flushed before: what a caller sees who launches
    the pair once, as opposed to the amortised figure of a graph replay over many instances."""
    stream = torch.cuda.current_stream().cuda_stream
    best = None
    for _ in range(n):
        flusher.flush()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch(stream)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3
        best = us if best is None else min(best, us)
    return best


def measure_pair(rt, torch, bf, wl, pk, name, device, conv_batch=1, max_reps=24, flusher=None):
    """Fused (every pattern that can host the pair) / sequential / two-stream microseconds of one
    BASELINE pair, replayed over enough instances to exceed twice the L2."""
    spec = wl.make_pair(name, seed=0, conv_batch=conv_batch)
    reps = max(2, min(max_reps, int(2.2 * L2_BYTES / spec.bytes) + 1))
    pairs = [wl.DevicePair(rt, spec if s == 0 else wl.make_pair(name, seed=s, conv_batch=conv_batch), device) for s in range(reps)]
    res = {"instances": reps, "alg_bytes": spec.bytes, "alg_flops": spec.flops, "dtype": spec.dtype,
           "launch": [list(spec.a.launch[0]) + list(spec.a.launch[1]), list(spec.b.launch[0]) + list(spec.b.launch[1])]}
    for label, pattern, mode, m, n in MODES:
        pat = getattr(bf, pattern)
        try:
            fus = [p.fusion(pat, m, n) for p in pairs]
        except bf.BfuseError as e:
            if e.code not in (3, 7):
                raise
            continue   # the pattern cannot host this pair (thread split: windows or tensor memory over budget)
        g = rt.graph_create(fus, mode)
        res[label + "_us"] = replay_us(rt, torch, g, reps)
        rt.graph_destroy(g)
    best_label = min((k for k in res if k.startswith("fused_")), key=lambda k: res[k])
    best = res[best_label]
    res["best_fused_us"] = best
    res["best_pattern"] = best_label[len("fused_"):-len("_us")]
    # the pair-selection model on this pair: its advice from the two operators' times alone, against what was measured
    try:
        from bfuse_project_b200 import pairing
        zz = [p.fusion(bf.ZIGZAG, 1, 1) for p in pairs]
        alone = []
        for mode in (bf.MODE_KERNEL1, bf.MODE_KERNEL2):
            g = rt.graph_create(zz, mode)
            alone.append(replay_us(rt, torch, g, reps))
            rt.graph_destroy(g)
        dims = lambda l: (l[0][0] * l[0][1] * l[0][2], l[1][0] * l[1][1] * l[1][2], l[2])
        hosted = [k[len("fused_"):-len("_us")] for k in res if k.startswith("fused_") and k.endswith("_us")]
        adv = pairing.advise(alone[0], alone[1], dims(spec.a.launch), dims(spec.b.launch), rt.sm_count, 1.0, spec.a.op, spec.b.op, allowed=hosted)
        got = res.get("fused_%s_us" % adv["pattern"])
        res["alone_us"] = alone
        res["model"] = {"pattern": adv["pattern"], "predicted_us": adv["predicted_fused_us"], "fuse": adv["fuse"], "measured_us": got,
                        "within_2_pct_of_best": None if got is None else bool(got <= 1.02 * best)}
    except Exception as e:   # reported, not hidden
        res["model"] = {"error": str(e)[:200]}
    if flusher is not None:
        lab = [x for x in MODES if "fused_" + res["best_pattern"] == x[0]][0]
        f0 = pairs[0].fusion(getattr(bf, lab[1]), lab[3], lab[4])
        res["isolated_fused_us"] = isolated_us(rt, torch, flusher, lambda st: rt.launch_fused(f0, st))
        res["isolated_sequential_us"] = isolated_us(rt, torch, flusher, lambda st: rt.launch_sequential(f0, st))
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


def bind_to_gpu_numa_node(torch, local):
    """Pin this process (and so the pinned buffers it allocates next, by first touch) to the CPUs of the NUMA
    node the GPU hangs off, read from sysfs for the GPU's PCI address; returns what was found."""
    info = {"pci": None, "numa_node": None, "cpus": None}
    try:
        bus = torch.cuda.get_device_properties(local).pci_bus_id
        dom = getattr(torch.cuda.get_device_properties(local), "pci_domain_id", 0)
        dev = getattr(torch.cuda.get_device_properties(local), "pci_device_id", 0)
        addr = "%04x:%02x:%02x.0" % (dom, bus, dev)
        info["pci"] = addr
        base = "/sys/bus/pci/devices/" + addr
        node = int(open(base + "/numa_node").read())
        info["numa_node"] = node
        cpus = set()
        for part in open(base + "/local_cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info["cpus"] = len(cpus)
    except Exception as e:   # no sysfs entry (containers): stay where the launcher put us, and say so
        info["note"] = str(e)[:80]
    return info


def copy_bandwidth(torch, host_in, dev_in, dev_outs, host_outs, reps=3):
    """Plain pinned-memory copies of the e2e step's bytes -- the input in, both outputs out -- in both directions at
    once on two streams: what the link delivers with no kernel in between (GB/s per direction, microseconds)."""
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    best = None
    for _ in range(reps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        with torch.cuda.stream(s1):
            dev_in.copy_(host_in, non_blocking=True)
        with torch.cuda.stream(s2):
            for h, d in zip(host_outs, dev_outs):
                h.copy_(d, non_blocking=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    out_bytes = sum(h.numel() * h.element_size() for h in host_outs)
    return {"h2d_gbs": host_in.numel() * host_in.element_size() / best / 1e9, "d2h_gbs": out_bytes / best / 1e9, "copies_alone_us": best * 1e6}


PATTERNS = (("zigzag", "ZIGZAG", 1, 1), ("zigzag2", "ZIGZAG", 1, 2), ("range", "RANGE_SPLIT", 0, 0), ("striped", "SM_STRIPED", 0, 0),
            ("queue", "WORK_QUEUE", 1, 1), ("thread_split", "THREAD_SPLIT", 0, 0))


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
    ap.add_argument("--sweep-extra", action="store_true", help="with --sweep: the pairs of the pair-selection model's extra operators "
                                                               "(memory-bound bodies, bf16 projections) with the suite's and with each other")
    ap.add_argument("--sweep-pattern", default="zigzag", choices=["zigzag", "range", "striped", "proportional", "all"],
                    help="with --sweep: the block-level pattern of the fused launches; all: every pattern per pair (what the pair-selection model is fitted on)")
    ap.add_argument("--batch", type=int, default=BATCH, help="images of the conv batch (256: the BASELINE configuration; smaller for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch

    import bfuse_project_b200 as bf
    from bfuse_project_b200 import partition
    from bfuse_project_b200 import workloads as wl

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    numa = bind_to_gpu_numa_node(torch, local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pk = peaks()

    rt = bf.Runtime(local)
    if args.sweep:
        return run_sweep(args, rt, torch, rank, world, local, pk)
    stream = torch.cuda.current_stream().cuda_stream
    flusher = L2Flusher(torch, local)

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor(v if isinstance(v, list) else [v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist() if isinstance(v, list) else float(t.item())

    # ---- the headline workload: this rank's shard of the one seeded batch, R instances of it ----------------
    batch = args.batch
    first, count = partition.shard_batch(batch, world, rank)
    proto = wl.ConvBranchBatch(rt, torch, local, 1, seed=0)
    shard_distinct = (proto.bytes(count) - 4 * count * proto.CI * proto.H * proto.W)      # x once + weights + both outputs
    reps = max(2, int(2.2 * L2_BYTES / shard_distinct) + 1)
    del proto
    batches = [wl.ConvBranchBatch(rt, torch, local, batch, seed=i) for i in range(reps)]   # instance 0 is THE batch; every rank holds the same one
    kernels = [b.shard(first, count) for b in batches]
    alg_bytes_total = batches[0].bytes(batch)
    alg_flops_total = batches[0].flops(batch)

    def fusions(pat, m, n):
        try:
            return [rt.register_fusion(k3, k1, getattr(bf, pat), m, n) for k3, k1 in kernels]
        except bf.BfuseError as e:
            if e.code not in (3, 7):
                raise
            return None   # the pattern cannot host this pair (thread split: the two windows do not fit one CTA)

    def graph_of(fus, mode, steps):
        return rt.graph_create([fus[i % reps] for i in range(steps)], mode)

    def timed(graph, steps, warm_graph=None, warm=0):
        """Exactly `steps` steps (one graph launch of that many kernel nodes), CUDA events on the launching
        stream, barrier + synchronize on both sides; milliseconds, the slowest rank."""
        for _ in range(warm):
            rt.graph_launch(warm_graph, stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rt.graph_launch(graph, stream)
        e1.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    fus = {name: fusions(pat, m, n) for name, pat, m, n in PATTERNS}
    fus = {k: v for k, v in fus.items() if v is not None}
    # spin ~100 ms first so the clocks have left their idle state, pick the fused pattern on a short
    # trial (best of the patterns, the same on every rank), then time exactly K steps of it
    one_step = {k: graph_of(v, bf.MODE_FUSED, 1) for k, v in fus.items()}
    t_spin = time.perf_counter()
    while time.perf_counter() - t_spin < 0.1:
        rt.graph_launch(one_step["range"], stream)
        torch.cuda.synchronize()
    trial_steps = 2 * reps
    trial = {k: timed(graph_of(v, bf.MODE_FUSED, trial_steps), trial_steps, one_step[k], 3) / trial_steps for k, v in fus.items()}
    best = min(trial, key=lambda k: trial[k])
    main_graph = graph_of(fus[best], bf.MODE_FUSED, args.steps)
    sampler = ClockSampler(local, getattr(torch.cuda.get_device_properties(local), "uuid", None))
    if rank == 0:
        sampler.start()
    ms = timed(main_graph, args.steps, one_step[best], args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    us_pair = ms * 1e3 / args.steps
    side = {"fused_" + k: v * 1e3 for k, v in trial.items()}
    side["fused_" + best] = us_pair
    for label, mode in (("sequential", bf.MODE_SEQUENTIAL), ("parallel", bf.MODE_PARALLEL)):
        side[label] = timed(graph_of(fus[best], mode, args.steps), args.steps, graph_of(fus[best], mode, 1), 3) * 1e3 / args.steps
    assert rt.read_status() == 0, "a bounded device-side wait gave up during the benchmark"
    iso_fused = max_over_ranks(isolated_us(rt, torch, flusher, lambda st: rt.launch_fused(fus[best][0], st)))
    iso_seq = max_over_ranks(isolated_us(rt, torch, flusher, lambda st: rt.launch_sequential(fus[best][0], st)))

    # what was just timed must equal the unfused launches of the same bodies, bit for bit
    b0 = batches[0]
    fused_out = (b0.y3[first:first + count].clone(), b0.y1[first:first + count].clone())
    b0.clear_outputs()
    rt.launch_sequential(fus[best][0], stream)
    torch.cuda.synchronize()
    assert torch.equal(fused_out[0], b0.y3[first:first + count]) and torch.equal(fused_out[1], b0.y1[first:first + count]), "fused != unfused"
    assert bool(fused_out[0].any()) and bool(fused_out[1].any())

    # ---- end to end through the host-buffer entry point: pinned host inputs and outputs ----------------------
    # The shard goes through bfuse_run_fuse_batch in sub-shards, so that the copy in of sub-shard i + 1, the fused
    # launch of sub-shard i and the copy out of sub-shard i - 1 overlap on three streams.
    hx = b0.x[first:first + count].cpu().pin_memory()
    hw3, hw1 = b0.w3.cpu().pin_memory(), b0.w1.cpu().pin_memory()
    hy3 = torch.zeros(count, b0.CO, b0.OH, b0.OW).pin_memory()
    hy1 = torch.zeros(count, b0.CO, b0.OH, b0.OW).pin_memory()
    pat_name = [x for x in PATTERNS if x[0] == best][0]

    def e2e_plan(sub):
        pieces = [(first + o, min(sub, count - o)) for o in range(0, count, sub)]
        fl, h1, h2 = [], [], []
        for f0, c0 in pieces:
            k3, k1 = b0.shard(f0, c0)
            fl.append(rt.register_fusion(k3, k1, getattr(bf, pat_name[1]), pat_name[2], pat_name[3]))
            o = f0 - first
            h1.append([hx[o:o + c0].numpy(), hw3.numpy(), hy3[o:o + c0].numpy()])
            h2.append([hx[o:o + c0].numpy(), hw1.numpy(), hy1[o:o + c0].numpy()])   # the same host and device input: copied once
        return pieces, fl, h1, h2

    # sub-shard size: the caller's choice; fewer pieces leave more of the first copy in and the last copy out
    # exposed, more pieces pay more per-copy overhead -- the best of three sizes on a short trial (best of 4 calls each)
    e2e_steps = max(3, min(args.steps, 10))
    plans = {}
    for sub in sorted({max(1, count // d) for d in (4, 8, 16)}):
        plan = e2e_plan(sub)
        b0.clear_outputs()
        hy3.zero_(), hy1.zero_()
        rt.run_fuse_batch(plan[1], plan[2], plan[3])
        assert torch.equal(hy3, fused_out[0].cpu()) and torch.equal(hy1, fused_out[1].cpu()), "e2e outputs differ from the device-resident run"
        best_of = float("inf")
        for _ in range(4):
            t0 = time.perf_counter()
            rt.run_fuse_batch(plan[1], plan[2], plan[3])
            best_of = min(best_of, time.perf_counter() - t0)
        plans[sub] = (max_over_ranks(best_of), plan)
    sub = min(plans, key=lambda k: plans[k][0])
    pieces, e2e_fus, h1, h2 = plans[sub][1]
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        rt.run_fuse_batch(e2e_fus, h1, h2)
    e2e_us = max_over_ranks((time.perf_counter() - t0) * 1e6 / e2e_steps)
    h2d = hx.numel() * 4 + (hw3.numel() + hw1.numel()) * 4   # the weights every sub-shard shares go in once per call
    d2h = (hy3.numel() + hy1.numel()) * 4
    link = copy_bandwidth(torch, hx, b0.x[first:first + count], (b0.y3[first:first + count], b0.y1[first:first + count]), (hy3, hy1))
    link["copies_alone_us"] = max_over_ranks(link["copies_alone_us"])
    link["e2e_h2d_gbs"] = h2d / (e2e_us * 1e-6) / 1e9
    link["e2e_d2h_gbs"] = d2h / (e2e_us * 1e-6) / 1e9
    link["e2e_over_copies_alone"] = e2e_us / link["copies_alone_us"]
    if world > 1:
        agg = torch.tensor([link["h2d_gbs"], link["d2h_gbs"]], device="cuda", dtype=torch.float64)
        dist.all_reduce(agg, op=dist.ReduceOp.SUM)
        link["all_ranks_h2d_gbs"], link["all_ranks_d2h_gbs"] = agg.tolist()
    del hx, hy3, hy1

    # ---- side measurements: the other BASELINE pairs (pair i on rank i mod N) ---------------------------------
    side_pairs = {}
    if not args.quick:
        names = wl.pair_names()
        for name in partition.assign_pairs(names, world, rank):
            try:
                side_pairs[name] = measure_pair(rt, torch, bf, wl, pk, name, local, flusher=flusher)
                side_pairs[name]["rank"] = rank
            except Exception as e:                  # a pair that cannot run is reported, not hidden
                side_pairs[name] = {"error": str(e)[:300], "rank": rank}
        if world > 1:
            gathered = [None] * world
            dist.all_gather_object(gathered, side_pairs)
            side_pairs = partition.merge_results(gathered)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    cpu_s, cores = cpu_conv_pair(CPU_SAMPLE_IMAGES, runs=3)
    cpu_us = cpu_s * 1e6 * batch / CPU_SAMPLE_IMAGES
    hbm_us = alg_bytes_total / (pk["hbm_gbs"] * 1e3)
    tensor_us = alg_flops_total / (pk["bf16_tflops"] * 0.5e6)
    # roofline of the dominant kernel (the fused conv pair of one rank): algorithmic bytes of one launch over
    # the launch's average duration inside the timed region
    launch_bytes = batches[0].bytes(count)
    achieved = launch_bytes / (us_pair * 1e-6) / 1e9
    per_image = dram_bytes_per_image()
    info = rt.fusion_info(fus[best][0])
    line = {
        "metric": "fused_pair_us", "value": us_pair, "unit": "us", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
        "config": {"workload": WORKLOAD_DESC if batch == BATCH else WORKLOAD_DESC.replace("256", str(batch)),
                   "pattern": best, "pattern_choice": "best of %d patterns on a %d-step trial, the same on every rank" % (len(trial), trial_steps),
                   "images_per_rank": count, "instances": reps,
                   "launch": "one CUDA graph of %d fused launches, rotating over %d instances of the shard" % (args.steps, reps),
                   "l2": "inputs larger than L2: %d instances x %.0f MB = %.0f MB touched per rotation vs 126 MB L2" % (reps, shard_distinct / 1e6, reps * shard_distinct / 1e6),
                   "multi_gpu": "images [r*256/N, (r+1)*256/N) of the one seeded batch on rank r, no collective on the data path",
                   "fused_kernel": info, "host": numa},
        "speedup_vs_sequential": side["sequential"] / us_pair,
        "speedup_vs_parallel_streams": side["parallel"] / us_pair,
        "us": side,
        "isolated_us": {"fused": iso_fused, "sequential": iso_seq,
                        "note": "one launch, CUDA events around it, L2 flushed before; `value` is the per-launch average of the graph"},
        "roofline_pair_us": max(hbm_us, tensor_us) / world, "roofline_pair_frac": max(hbm_us, tensor_us) / world / us_pair,
        "images_per_s": batch / (us_pair * 1e-6),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": None if per_image is None else per_image * count,
                     "peak_source": pk["source"] + " (HBM copy bandwidth; the pair's tf32 time, %.1f us at half the measured bf16 burst -- "
                                                   "no tf32 peak was measured --, is below its HBM time)" % tensor_us,
                     "traffic_note": "dram read + write of one launch: dram_bytes_per_image of profiles/fused_conv_tf32_pair_cfg5.md "
                                     "(ncu capture of a smaller batch; traffic grows in proportion to the images) x images per launch",
                     "alg_bytes_per_launch": launch_bytes, "kernel": info["KernelName"],
                     "note": "algorithmic bytes count the shared input once per operator (617 MB at batch 256; 411 MB if counted once)"},
        "cpu_baseline": {"value": cpu_us, "unit": "us", "cores": cores, "kind": "port",
                         "sample": "%d of the %d images, both convs, best of 3 runs; time scaled to the batch" % (CPU_SAMPLE_IMAGES, batch)},
        "e2e": {"value": e2e_us, "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "bfuse_run_fuse_batch on pinned host buffers, the shard in %d sub-shards of %d images: H2D of the input, fused launch, "
                        "D2H of both outputs of neighbouring sub-shards overlap; per 256-image pair, slowest rank" % (len(pieces), sub),
                "link": link},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    if not args.quick:
        line["pairs"] = side_pairs
        line["attention_block"] = attention_block(rt, torch, bf)
        line["model_segments"] = model_segments(rt, torch, bf)
        line["reference_fuser_output"] = reference_fuser_output(rt, torch, bf, wl, pk)
    # every configuration in one compact table, LAST in the line: [best fused us, sequential us, roofline fraction, pattern, isolated fused us]
    table = {"cfg5_conv_branches_n%d" % batch: [round(us_pair, 2), round(side["sequential"], 2), round(max(hbm_us, tensor_us) / world / us_pair, 3), best, round(iso_fused, 2)]}
    for name, r in side_pairs.items():
        if "error" in r:
            table[name] = r["error"][:60]
        else:
            table[name] = [round(r["best_fused_us"], 2), round(r["sequential_us"], 2), round(r["roofline_frac"], 3), r["best_pattern"],
                           round(r.get("isolated_fused_us", 0.0), 2)]
    scored = [r["model"]["within_2_pct_of_best"] for r in side_pairs.values() if isinstance(r.get("model"), dict) and r["model"].get("within_2_pct_of_best") is not None]
    if scored:
        line["pairing_model_on_baseline_pairs"] = {"pairs": len(scored), "pattern_within_2_pct_of_best": sum(scored),
                                                   "advice": {n: r["model"].get("pattern") for n, r in side_pairs.items() if isinstance(r.get("model"), dict)}}
    line["per_config"] = table
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
