"""The YAML front end against the reference's own records: kernels.yaml / fusions.yaml written in the
reference's input schema from the committed golden dims, planned on the CPU, must reproduce the fused
dims of the reference's bfuse_kernels.yaml / hfuse_kernels.yaml for all 2 728 pairs of its three suites."""
import json
import os
import subprocess
import sys

import pytest
import yaml

from bfuse_project_b200 import yaml_frontend as yf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def golden():
    with open(os.path.join(ROOT, "tests", "golden", "dispatch_golden.json")) as f:
        return json.load(f)["yaml"]


def write_inputs(tmp, suite):
    kernels = {n: {"KernelName": n, "HasBarriers": True, "GridDim": dict(zip("XYZ", d[:3])), "BlockDim": dict(zip("XYZ", d[3:])),
                   "Reg": 32, "ExecTime": -1} for n, d in suite["kernels"].items()}
    fusions = [{"File": "kernels.cu", "Kernels": [a, b]} for a, b, _, _ in suite["pairs"]]
    kp, fp = os.path.join(tmp, "kernels.yaml"), os.path.join(tmp, "fusions.yaml")
    with open(kp, "w") as f:
        yaml.safe_dump(kernels, f)
    with open(fp, "w") as f:
        yaml.safe_dump(fusions, f)
    return kp, fp


@pytest.mark.parametrize("name", ["tests/benchmark", "tests/inception_v3", "tests/interleave_scheduler"])
def test_fused_records_equal_the_reference_yaml(golden, tmp_path, name):
    suite = golden[name]
    kp, fp = write_inputs(str(tmp_path), suite)
    kernels, fusions = yf.load_kernels(kp), yf.load_fusions(fp)
    assert len(kernels) == len(suite["kernels"]) and len(fusions) == len(suite["pairs"])
    for block_level, col, suffix in ((True, 2, "_fused_bfuse"), (False, 3, "_fused_hfuse")):
        recs = yf.fuse_records(kernels, fusions, block_level=block_level)
        assert len(recs) == len({(p[0], p[1]) for p in suite["pairs"]})
        for p in suite["pairs"]:
            r = recs["%s_%s%s" % (p[0], p[1], suffix)]
            assert list(r["GridDim"]) + list(r["BlockDim"]) == p[col]
            assert r["HasBarriers"] is True and r["Reg"] == 32
        out = os.path.join(str(tmp_path), "out%s.yaml" % suffix)
        yf.dump_kernels(recs, out)
        back = yf.load_kernels(out)                      # the output parses with the input schema's reader
        assert back.keys() == recs.keys()
        k = next(iter(recs))
        assert back[k]["GridDim"] == tuple(recs[k]["GridDim"]) and back[k]["ExecTime"] == -1


def test_command_line_mirrors_the_fuser_switch(golden, tmp_path):
    suite = {"kernels": golden["tests/interleave_scheduler"]["kernels"], "pairs": golden["tests/interleave_scheduler"]["pairs"][:5]}
    kp, fp = write_inputs(str(tmp_path), suite)
    out = os.path.join(str(tmp_path), "bfuse_kernels.yaml")
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, "-m", "bfuse_project_b200.yaml_frontend", "-b", "-y", str(tmp_path), fp, kp, "unused_compile_commands"],
                       capture_output=True, text=True, env=env)
    assert r.returncode == 0, r.stderr
    doc = yaml.safe_load(open(out))
    a, b, bdims, _ = suite["pairs"][0]
    rec = doc["%s_%s_fused_bfuse" % (a, b)]
    assert [rec["GridDim"][x] for x in "XYZ"] + [rec["BlockDim"][x] for x in "XYZ"] == bdims and "ExecTime" not in rec
    # a fusion naming an unknown kernel is an error exit, not a crash
    with open(fp, "w") as f:
        yaml.safe_dump([{"File": "kernels.cu", "Kernels": ["nope", a]}], f)
    r = subprocess.run([sys.executable, "-m", "bfuse_project_b200.yaml_frontend", "-y", str(tmp_path), fp, kp], capture_output=True, text=True, env=env)
    assert r.returncode == 1 and "unknown kernel" in r.stderr


def test_gpu_trace_csv_round_trip_in_the_reference_layout(tmp_path):
    """The per-launch timing files carry the header of nsys' cuda_gpu_trace report and parse back to the
    fields the reference's analysis keeps (start / duration in ms, name); its statistic -- skip the
    first three rows of a kernel, average the rest (analyze_test_suite.py:104-122) -- comes out right."""
    from bfuse_project_b200 import trace_csv
    rows = [dict(start_ns=1000 * i, duration_ns=(50000 if i < 3 else 8000 + i), name="a_b_fused_bfuse", grid=(96, 1, 1),
                 block=(192, 1, 1), regs=114, smem=199680) for i in range(10)]
    p = tmp_path / "4_0_1_cuda_gpu_trace.csv"
    trace_csv.write_gpu_trace(str(p), rows)
    first = p.read_text().splitlines()[0]
    assert first.startswith("Start (ns),Duration (ns),CorrId,GrdX,GrdY,GrdZ,BlkX,BlkY,BlkZ,Reg/Trd") and first.endswith(",Strm,Name")
    back = trace_csv.read_gpu_trace(str(p))
    assert len(back) == 10 and back[4] == (0.004, 0.008004, "a_b_fused_bfuse")
    kept = [d for i, (_, d, n) in enumerate(back) if n == "a_b_fused_bfuse" and i >= 3]
    assert abs(sum(kept) / len(kept) - (8000 + 6.0) / 1e6) < 1e-12


def test_fused_names_come_from_the_map_keys_and_records_are_sorted(tmp_path):
    """The reference builds a fused name from the kernels.yaml map keys a fusion lists, not from the
    KernelName fields (Contexts.cc:67-84), and writes its records sorted by name (a std::map)."""
    from bfuse_project_b200 import yaml_frontend as yf
    dims = {"GridDim": {"X": 8, "Y": 1, "Z": 1}, "BlockDim": {"X": 128, "Y": 1, "Z": 1}, "Reg": 32, "HasBarriers": True}
    kernels = {"zeta": dict(dims, KernelName="real_kernel_z"), "alpha": dict(dims, KernelName="real_kernel_a"),
               "mid": dict(dims, KernelName="real_kernel_m")}
    kp, fp, out = (str(tmp_path / n) for n in ("kernels.yaml", "fusions.yaml", "bfuse_kernels.yaml"))
    with open(kp, "w") as f:
        yaml.safe_dump(kernels, f)
    with open(fp, "w") as f:
        yaml.safe_dump([{"File": "k.cu", "Kernels": ["zeta", "alpha"]}, {"File": "k.cu", "Kernels": ["alpha", "mid"]}], f)
    recs = yf.fuse_records(yf.load_kernels(kp), yf.load_fusions(fp), block_level=True)
    assert set(recs) == {"zeta_alpha_fused_bfuse", "alpha_mid_fused_bfuse"}
    yf.dump_kernels(recs, out)
    names = [ln[:-1] for ln in open(out).read().splitlines() if ln.endswith("_fused_bfuse:")]
    assert names == ["alpha_mid_fused_bfuse", "zeta_alpha_fused_bfuse"]
