#!/usr/bin/env python3
"""Build tests/golden/dispatch_golden.json from the reference checkout.

Reads, as text, the dispatch headers the reference's fuser printed into its
generated kernels and the fused dims it wrote to YAML, and stores them as
known-answer data for the dispatch oracle and for the runtime's scheduler:

  * tests/benchmark/cuda/*_bfuse.cu   -- M:N zig-zag pattern (Algorithms.cc:528-739)
  * tests/benchmark/cuda/*_hfuse.cu   -- thread-range split + bar.sync operands
  * tests/*/config/{kernels,bfuse_kernels,hfuse_kernels}.yaml -- fused grid / block
  * legacy/tests/single_bgemm_conv2d/case-0_0/M_diff/case-*/cuda/bfuse_kernels.cu -- M:N != 1:1
  * legacy/tests/block_scheduler_test/cuda/bfuse_kernels.cu -- SM-striped pattern

For every block-level kernel the C conditions are also *evaluated* here (numpy,
independently of the oracle) for every CTA, and a position-sensitive digest of
the (KernelID_, NewBlockIdx_) sequence is stored.

Usage (only where the reference checkout exists):
    python tests/golden/make_dispatch_golden.py /path/to/reference
"""
import glob
import json
import os
import re
import sys

import numpy as np
import yaml

BX = r"\(int\)blockIdx\.x"
TX = r"\(int\)threadIdx\.x"
RE_ROT = re.compile(rf"if \(\({BX} < (\d+)\) && \({BX} % (\d+) >= (\d+)\) && \({BX} % (\d+) < (\d+)\)\)")
RE_ROT_NB = re.compile(rf"NewBlockIdx_ = int\({BX} / (\d+)\) \* (\d+) \+ \({BX} % (\d+) - (\d+)\);")
RE_RANGE = re.compile(rf"if \({BX} >= (\d+) && {BX} < (\d+)\)$")
RE_RANGE_NB = re.compile(rf"NewBlockIdx_ = {BX} - (\d+) \+ (\d+);")
RE_STRIPE = re.compile(rf"if \(\({BX} >= (\d+) && {BX} < (\d+)\) && \(int\(\({BX} - (\d+)\) % (\d+) / (\d+)\) == (\d+)\)\)")
RE_STRIPE_NB = re.compile(rf"NewBlockIdx_ = (\d+) \+ \({BX} - (\d+)\) % (\d+) \+ int\(\({BX} - (\d+)\) / (\d+)\) \* (\d+);")
RE_KID = re.compile(r"KernelID_\s+= (\d+);")
RE_DIM = re.compile(r"(gridDim|blockDim)_([xyz])_ = (\d+);")
RE_GUARD = re.compile(rf"if \(\(KernelID_ == (\d+)\) && \((?:{TX} >= 0 && )?{TX} < (\d+)\)\)")
RE_HF = re.compile(rf"if \(\({TX} >= (\d+) && {TX} < (\d+)\) && \({BX} >= 0 && {BX} < (\d+)\)\)")
RE_HF_B = re.compile(rf"int blockIdx_([xyz])_ = {BX} (?:% (\d+)|/ (\d+)(?: % (\d+))?);")
RE_HF_T = re.compile(rf"int threadIdx_([xyz])_ = \({TX} - (\d+)\) (?:% (\d+)|/ (\d+)(?: % (\d+))?);")
RE_BAR = re.compile(r'bar\.sync (\d+), (\d+);')
RE_LB = re.compile(r"__launch_bounds__\((\d+)\)")

ROTATE, RANGE, STRIPE = 0, 1, 2
MASK = (1 << 64) - 1


def digest(kernel, vblock):
    """sum_b ((kernel+1) << 40 | vblock) * (2b+1) * 0x9E3779B97F4A7C15  (mod 2^64)."""
    b = np.arange(kernel.size, dtype=np.uint64)
    w = ((kernel.astype(np.uint64) + np.uint64(1)) << np.uint64(40)) | vblock.astype(np.uint64)
    with np.errstate(over="ignore"):
        return int(np.sum(w * (b * np.uint64(2) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15), dtype=np.uint64))


def evaluate(branches, grid):
    """Evaluate the parsed if / else-if chain for every CTA, first match wins."""
    b = np.arange(grid, dtype=np.int64)
    kern = np.full(grid, -1, dtype=np.int64)
    vb = np.full(grid, -1, dtype=np.int64)
    for br in branches:
        if br["kind"] == ROTATE:
            cond = (b < br["b_hi"]) & (b % br["rot"] >= br["r_lo"]) & (b % br["rot"] < br["r_hi"])
            val = b // br["rot"] * br["ratio"] + (b % br["rot"] - br["r_lo"])
        elif br["kind"] == RANGE:
            cond = (b >= br["b_lo"]) & (b < br["b_hi"])
            val = b - br["b_lo"] + br["base"]
        else:
            cond = (b >= br["b_lo"]) & (b < br["b_hi"]) & (
                (b - br["b_lo"]) % (br["sm"] * br["stripe_n"]) // br["sm"] == br["stripe_idx"])
            val = br["base"] + (b - br["b_lo"]) % br["sm"] + (b - br["b_lo"]) // (br["stripe_n"] * br["sm"]) * br["sm"]
        take = cond & (kern < 0)
        kern[take] = br["kernel"]
        vb[take] = val[take]
    assert (kern >= 0).all(), "unmapped CTA in reference kernel"
    return kern, vb


def parse_block_level(lines):
    """Parse one generated block-level fused kernel header -> (kernel dims, branches, guards)."""
    branches, dims, guards = [], {}, {}
    cur = None
    for ln in lines:
        s = ln.strip()
        if s.startswith("else "):
            s = s[5:]
        m = RE_ROT.match(s)
        if m:
            e, r1, lo, r2, hi = map(int, m.groups())
            assert r1 == r2
            cur = dict(kind=ROTATE, b_lo=0, b_hi=e, rot=r1, r_lo=lo, r_hi=hi)
            branches.append(cur)
            continue
        m = RE_STRIPE.match(s)
        if m:
            s0, e, s1, tn, t, idx = map(int, m.groups())
            assert s0 == s1 and tn % t == 0
            cur = dict(kind=STRIPE, b_lo=s0, b_hi=e, sm=t, stripe_n=tn // t, stripe_idx=idx)
            branches.append(cur)
            continue
        m = RE_RANGE.match(s)
        if m:
            cur = dict(kind=RANGE, b_lo=int(m.group(1)), b_hi=int(m.group(2)))
            branches.append(cur)
            continue
        m = RE_ROT_NB.match(s)
        if m:
            r1, ratio, r2, lo = map(int, m.groups())
            assert r1 == r2 == cur["rot"] and lo == cur["r_lo"]
            cur["ratio"] = ratio
            continue
        m = RE_STRIPE_NB.match(s)
        if m:
            base, s0, t, s1, tn, t2 = map(int, m.groups())
            assert s0 == s1 == cur["b_lo"] and t == t2 == cur["sm"] and tn == cur["sm"] * cur["stripe_n"]
            cur["base"] = base
            continue
        m = RE_RANGE_NB.match(s)
        if m:
            assert int(m.group(1)) == cur["b_lo"]
            cur["base"] = int(m.group(2))
            continue
        m = RE_KID.match(s)
        if m and cur is not None:
            cur["kernel"] = int(m.group(1))
            dims.setdefault(cur["kernel"], {})
            continue
        m = RE_DIM.match(s)
        if m and cur is not None and "kernel" in cur:
            dims[cur["kernel"]][m.group(1)[0] + m.group(2)] = int(m.group(3))
            continue
        m = RE_GUARD.search(s)
        if m:
            guards[int(m.group(1))] = int(m.group(2))
    kd = [[dims[k][f] for f in ("gx", "gy", "gz", "bx", "by", "bz")] for k in sorted(dims)]
    return kd, branches, [guards[k] for k in sorted(guards)]


BR_FIELDS = ("kind", "kernel", "b_lo", "b_hi", "rot", "r_lo", "r_hi", "ratio", "base", "sm", "stripe_n", "stripe_idx")


def block_level_record(name, text_lines, launch_bounds, body_text=None):
    kd, branches, guards = parse_block_level(text_lines)
    if body_text is not None:  # the per-kernel guards sit after the shared-memory union
        g = {int(a): int(b) for a, b in RE_GUARD.findall(body_text)}
        guards = [g[k] for k in sorted(g)]
    grid = sum(k[0] * k[1] * k[2] for k in kd)
    kern, vb = evaluate(branches, grid)
    packed = [[br.get(f, 0) for f in BR_FIELDS] for br in branches]
    return dict(name=name, k=kd, br=packed, guards=guards, launch_bounds=launch_bounds,
                fused_grid=grid, digest="%016x" % digest(kern, vb))


def read_header(path, stop="typedef struct"):
    out = []
    with open(path) as f:
        for ln in f:
            if stop in ln:
                break
            out.append(ln)
    return out


def split_kernels(path):
    """Yield (name, lines) per extern "C" __global__ kernel of a multi-kernel file."""
    name, buf = None, []
    with open(path) as f:
        for ln in f:
            if ln.startswith('extern "C" __global__'):
                if name:
                    yield name, buf
                name = re.search(r"void (\w+)\(", ln).group(1)
                buf = [ln]
            elif name:
                buf.append(ln)
    if name:
        yield name, buf


def hfuse_record(path):
    text = open(path).read()
    name = re.search(r"void (\w+)\(", text).group(1)
    parts = []
    for m in RE_HF.finditer(text):
        seg = text[m.end():m.end() + 700]
        bd = {g[0]: g for g in RE_HF_B.findall(seg)}
        td = {g[0]: g for g in RE_HF_T.findall(seg)}
        gx = int(bd["x"][1])
        gy = int(bd["y"][3]) if bd["y"][3] else 1
        bx = int(td["x"][2])
        by = int(td["y"][4]) if td["y"][4] else 1
        parts.append(dict(t_lo=int(m.group(1)), t_hi=int(m.group(2)), grid=int(m.group(3)),
                          gx=gx, gy=gy, gxy=int(bd["z"][2]), bx=bx, by=by, bxy=int(td["z"][3]),
                          t_off=int(td["x"][1])))
    bars = sorted(set((int(a), int(b)) for a, b in RE_BAR.findall(text)))
    return dict(name=name, parts=parts, bars=bars, launch_bounds=int(RE_LB.search(text).group(1)))


def yaml_dims(ref, suite):
    cfg = os.path.join(ref, suite, "config")
    kernels = yaml.safe_load(open(os.path.join(cfg, "kernels.yaml")))
    fusions = yaml.safe_load(open(os.path.join(cfg, "fusions.yaml")))
    bf = yaml.safe_load(open(os.path.join(cfg, "bfuse_kernels.yaml")))
    hf = yaml.safe_load(open(os.path.join(cfg, "hfuse_kernels.yaml")))
    kd = {n: [v["GridDim"][a] for a in "XYZ"] + [v["BlockDim"][a] for a in "XYZ"] for n, v in kernels.items()}
    pairs = []
    for fu in fusions:
        a, b = fu["Kernels"]
        nb, nh = f"{a}_{b}_fused_bfuse", f"{a}_{b}_fused_hfuse"
        if nb not in bf or nh not in hf:
            continue
        pairs.append([a, b,
                      [bf[nb]["GridDim"][x] for x in "XYZ"] + [bf[nb]["BlockDim"][x] for x in "XYZ"],
                      [hf[nh]["GridDim"][x] for x in "XYZ"] + [hf[nh]["BlockDim"][x] for x in "XYZ"]])
    return dict(kernels=kd, pairs=pairs)


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("BFUSE_REFERENCE_DIR", "")
    if not os.path.isdir(os.path.join(ref, "tests", "benchmark", "cuda")):
        sys.exit("usage: make_dispatch_golden.py <reference checkout>   (or set BFUSE_REFERENCE_DIR)")
    out = {"source": "parsed from the reference's generated kernels and YAML outputs; see this script",
           "br_fields": list(BR_FIELDS)}

    zig = []
    for p in sorted(glob.glob(os.path.join(ref, "tests/benchmark/cuda/*_bfuse.cu"))):
        hdr = read_header(p)
        lb = int(RE_LB.search(hdr[0]).group(1))
        zig.append(block_level_record(os.path.basename(p)[:-3], hdr, lb, open(p).read()))
    # many pairs share (dims, branches): keep one representative per distinct record
    seen, uniq = set(), []
    for r in zig:
        key = json.dumps([r["k"], r["br"]], sort_keys=True)
        if key not in seen:
            seen.add(key)
            uniq.append(r)
    out["zigzag_1_1"] = uniq
    out["zigzag_1_1_files"] = len(zig)

    ratio = []
    for p in sorted(glob.glob(os.path.join(ref, "legacy/tests/single_bgemm_conv2d/case-*/*_diff/case-*/cuda/bfuse_kernels.cu"))):
        rel = os.path.relpath(p, ref)
        for name, lines in split_kernels(p):
            hdr = []
            for ln in lines:
                if "typedef struct" in ln:
                    break
                hdr.append(ln)
            try:
                rec = block_level_record(rel + ":" + name, hdr, int(RE_LB.search(hdr[0]).group(1)))
            except Exception:
                continue
            ratio.append(rec)
    seen, uniq = set(), []
    for r in ratio:
        key = json.dumps([r["k"], r["br"]], sort_keys=True)
        if key not in seen:
            seen.add(key)
            uniq.append(r)
    out["zigzag_m_n"] = uniq

    striped = []
    p = os.path.join(ref, "legacy/tests/block_scheduler_test/cuda/bfuse_kernels.cu")
    for name, lines in split_kernels(p):
        hdr = []
        for ln in lines:
            if "typedef struct" in ln or "__shared__" in ln:
                break
            hdr.append(ln)
        try:
            striped.append(block_level_record(name, hdr, int(RE_LB.search(hdr[0]).group(1))))
        except Exception:
            continue
    out["sm_striped_84"] = striped

    hf = []
    for p in sorted(glob.glob(os.path.join(ref, "tests/benchmark/cuda/*_hfuse.cu"))):
        hf.append(hfuse_record(p))
    seen, uniq = set(), []
    for r in hf:
        key = json.dumps([r["parts"], r["bars"]], sort_keys=True)
        if key not in seen:
            seen.add(key)
            uniq.append(r)
    out["thread_split"] = uniq
    out["thread_split_files"] = len(hf)

    out["yaml"] = {s: yaml_dims(ref, s) for s in
                   ("tests/benchmark", "tests/inception_v3", "tests/interleave_scheduler")}

    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dispatch_golden.json")
    with open(dst, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print("wrote", dst, os.path.getsize(dst), "bytes;",
          {k: (len(v) if isinstance(v, list) else "-") for k, v in out.items()})


if __name__ == "__main__":
    main()
