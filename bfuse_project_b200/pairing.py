"""Pair-selection model: will two operators gain from sharing a launch, and under which pattern?

The reference leaves this as its open question and answers it with profiler counters: a pair is a
candidate when the time-weighted sums of the two kernels' LSU and FMA pipe utilisation stay under
thresholds, i.e. when the shared resource has head-room for both
(scripts/analyze_test_suite.py:20-25, 436-479).  On B200 the scarce resource of these short
operators is not a pipe but the SMs themselves -- most of them leave SMs idle -- so the model here
works on each operator's launch record (CTAs, threads, shared-memory window, operator body) and its
time alone.  Two parts:

  * the analytic core: fill_k = CTAs_k / (SMs * CTAs of k that fit one SM) is the share of the GPU
    operator k occupies; a fused launch takes at least the longer operator (critical path) and at
    least the SM-time both need (area):  core = max(max(t_a, t_b), fill_a * t_a + fill_b * t_b);
  * a per-pattern correction fitted by least squares on measured pairs: for pattern p and the class
    pair of the two bodies (row-wise / CUDA-core / tensor-core GEMM / tensor-core conv),
        fused_p = w0 + w1 * core + w2 * min(t_a, t_b) + w3 * (t_a + t_b) + w4 * sum_k (slow_k - 1) * t_k
    where slow_k is how many times more waves operator k needs once every CTA is charged the union of
    the two shared-memory windows (`union_slowdown`)
    (`fit`, from the per-pattern times of the operator sweep, `python bench.py --sweep
    --sweep-pattern all --sweep-out F`; `python -m bfuse_project_b200.pairing F` writes the
    coefficients to pairing_model.json beside this file and prints the held-out evaluation).

`advise` returns the pattern with the smallest predicted time and whether that beats the two
launches back to back.  Without coefficients it falls back to the analytic core plus 1 us for every
pattern (and names the zig-zag).
"""
import json
import os

SM_SMEM_BYTES = 227 * 1024
SM_THREADS = 2048
OVERHEAD_US = 1.0
PATTERNS = ("zigzag", "zigzag2", "range", "striped", "thread_split")
MODEL_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "pairing_model.json")

# operator body -> class (ids of include/bfuse_b200.h: 0..3 row-wise, 4 / 5 CUDA-core, 6 / 7 tcgen05 GEMM, 8 tcgen05 conv)
BODY_CLASS = {0: "row", 1: "row", 2: "row", 3: "row", 4: "simt", 5: "simt", 6: "gemm", 7: "gemm", 8: "conv"}


def ctas_per_sm(threads, smem_bytes, regs_per_thread=0):
    """CTAs of one operator that fit an SM: by shared memory (1 KB reserved per CTA), threads and registers."""
    by_smem = SM_SMEM_BYTES // (int(smem_bytes) + 1024)
    by_thr = SM_THREADS // max(1, int(threads))
    by_regs = 65536 // (int(regs_per_thread) * max(1, int(threads))) if regs_per_thread else 32
    return max(1, min(by_smem, by_thr, by_regs, 32))


def fill(ctas, threads, smem_bytes, sm_count=148, regs_per_thread=0):
    """Share of the GPU the operator occupies while it runs alone (1.0: every SM slot taken, or more than one wave)."""
    return min(1.0, ctas / float(sm_count * ctas_per_sm(threads, smem_bytes, regs_per_thread)))


def predict_fused_us(t_a, t_b, fill_a, fill_b, overhead_us=OVERHEAD_US):
    """The analytic core plus a constant: the model without fitted coefficients."""
    return max(max(t_a, t_b), fill_a * t_a + fill_b * t_b) + overhead_us


def class_pair(op_a, op_b):
    return "|".join(sorted((BODY_CLASS.get(op_a, "row"), BODY_CLASS.get(op_b, "row"))))


def union_slowdown(launch, other, sm_count=148):
    """How many times more waves an operator needs when every CTA of the fused grid is charged the larger of the
    two shared-memory windows and the larger block (block-level fusion keeps the union of the windows): a
    memory-bound operator of thousands of small CTAs beside a tensor-core tile with a whole-SM ring drops from
    eight CTAs per SM to one."""
    ctas, thr, smem = launch
    per_alone = sm_count * ctas_per_sm(thr, smem)
    per_union = sm_count * ctas_per_sm(max(thr, other[1]), max(smem, other[2]))
    waves = lambda per: -(-int(ctas) // per)
    return min(16.0, waves(per_union) / float(waves(per_alone)))


def features(t_a, t_b, fill_a, fill_b, slow_a=1.0, slow_b=1.0):
    core = max(max(t_a, t_b), fill_a * t_a + fill_b * t_b)
    return [1.0, core, min(t_a, t_b), t_a + t_b, (slow_a - 1.0) * t_a + (slow_b - 1.0) * t_b]


_model = None


def load_model(path=MODEL_PATH):
    """{pattern: {class pair | "*": [w0..w3]}} or None when no coefficients have been fitted."""
    global _model
    if _model is None and os.path.exists(path):
        with open(path) as f:
            _model = json.load(f)["weights"]
    return _model


def predict_by_pattern(t_a, t_b, launch_a, launch_b, op_a=None, op_b=None, sm_count=148, model=None):
    """{pattern: predicted fused microseconds}.  launch_k = (ctas, threads, smem_bytes)."""
    fa, fb = fill(*launch_a, sm_count=sm_count), fill(*launch_b, sm_count=sm_count)
    model = load_model() if model is None else model
    if not model:
        return {"zigzag": predict_fused_us(t_a, t_b, fa, fb)}
    x = features(t_a, t_b, fa, fb, union_slowdown(launch_a, launch_b, sm_count), union_slowdown(launch_b, launch_a, sm_count))
    cp = class_pair(op_a, op_b)
    out = {}
    for p, table in model.items():
        w = table.get(cp, table.get("*"))
        if w is not None:
            out[p] = max(0.5 * max(t_a, t_b), sum(wi * xi for wi, xi in zip(w, x)))
    return out


def advise(t_a, t_b, launch_a, launch_b, sm_count=148, margin=1.0, op_a=None, op_b=None, model=None, allowed=None):
    """The pattern with the smallest predicted fused time, the prediction, and whether to fuse (predicted
    speed-up over back-to-back launches above `margin`).  allowed: the patterns that can host the pair (a thread
    split needs both shared-memory windows and both tensor-memory allocations in one CTA); default all."""
    fa, fb = fill(*launch_a, sm_count=sm_count), fill(*launch_b, sm_count=sm_count)
    preds = predict_by_pattern(t_a, t_b, launch_a, launch_b, op_a, op_b, sm_count, model)
    if allowed is not None and any(p in preds for p in allowed):
        preds = {p: v for p, v in preds.items() if p in allowed}
    pattern = min(preds, key=lambda p: preds[p])
    fused = preds[pattern]
    speedup = (t_a + t_b) / fused
    return {"fill": (fa, fb), "pattern": pattern, "predicted_fused_us": fused, "predicted_by_pattern": preds,
            "predicted_speedup": speedup, "fuse": speedup > margin}


# ---------------------------------------------------------------------------------------------- fitting

def _solve(rows, ys):
    """Least squares with a small ridge term, by normal equations: no dependency beyond the standard library."""
    n = len(rows[0])
    a = [[sum(r[i] * r[j] for r in rows) + (1e-6 if i == j else 0.0) for j in range(n)] for i in range(n)]
    b = [sum(r[i] * y for r, y in zip(rows, ys)) for i in range(n)]
    for i in range(n):                      # Gauss-Jordan with partial pivoting
        piv = max(range(i, n), key=lambda r: abs(a[r][i]))
        a[i], a[piv], b[i], b[piv] = a[piv], a[i], b[piv], b[i]
        d = a[i][i]
        a[i] = [v / d for v in a[i]]
        b[i] /= d
        for r in range(n):
            if r != i and a[r][i] != 0.0:
                f = a[r][i]
                a[r] = [vr - f * vi for vr, vi in zip(a[r], a[i])]
                b[r] -= f * b[i]
    return b


def fit(records, min_bucket=12):
    """Coefficients from records that carry `fused_us_by_pattern` (see sweep.pairing_records): per pattern one
    weight vector for every class pair with at least `min_bucket` records, and one over all records ("*")."""
    weights = {}
    for p in PATTERNS:
        rows = {}
        for r in records:
            t = (r.get("fused_us_by_pattern") or {}).get(p)
            if t is None:
                continue
            fa, fb = fill(*r["launch_a"], sm_count=r.get("sm_count", 148)), fill(*r["launch_b"], sm_count=r.get("sm_count", 148))
            sm = r.get("sm_count", 148)
            x = features(r["t_a"], r["t_b"], fa, fb, union_slowdown(r["launch_a"], r["launch_b"], sm), union_slowdown(r["launch_b"], r["launch_a"], sm))
            for bucket in (class_pair(r.get("op_a"), r.get("op_b")), "*"):
                rows.setdefault(bucket, ([], []))
                # relative error is what matters: weight every record by 1 / measured time
                rows[bucket][0].append([v / t for v in x])
                rows[bucket][1].append(1.0)
        weights[p] = {bucket: _solve(xs, ys) for bucket, (xs, ys) in rows.items() if len(xs) >= min_bucket or bucket == "*"}
    return weights


def evaluate(records, margin=1.0, model=None, tolerance=0.02):
    """records: dicts with t_a, t_b, launch_a, launch_b, fused_us, sequential_us (measured; optionally op_a,
    op_b and fused_us_by_pattern).  Median / 90th-percentile relative error of the predicted time of the advised
    pattern, the confusion counts of "fusing pays" (measured speed-up of the best measured pattern > margin)
    against the advice, and how often the advised pattern is within `tolerance` of the best measured one."""
    errs, tp, fp, fn, tn, pat_ok, pat_n, zz_losers, zz_rescued = [], 0, 0, 0, 0, 0, 0, 0, 0
    for r in records:
        a = advise(r["t_a"], r["t_b"], r["launch_a"], r["launch_b"], r.get("sm_count", 148), margin, r.get("op_a"), r.get("op_b"), model)
        by = r.get("fused_us_by_pattern") or {}
        measured = by.get(a["pattern"], r["fused_us"])
        best = min(by.values()) if by else r["fused_us"]
        errs.append(abs(a["predicted_fused_us"] - measured) / measured)
        if by:
            pat_n += 1
            pat_ok += measured <= best * (1.0 + tolerance)
            if "zigzag" in by and r["sequential_us"] / by["zigzag"] <= margin:      # the reference's one pattern loses here
                zz_losers += 1
                zz_rescued += (not a["fuse"]) or r["sequential_us"] / measured > margin
        pays = r["sequential_us"] / best > margin
        if a["fuse"] and pays:
            tp += 1
        elif a["fuse"]:
            fp += 1
        elif pays:
            fn += 1
        else:
            tn += 1
    if not errs:
        return {"pairs": 0}
    errs.sort()
    out = {"pairs": len(errs), "median_rel_err": errs[len(errs) // 2], "p90_rel_err": errs[(len(errs) * 9) // 10],
           "advice_fuse_and_pays": tp, "advice_fuse_but_slower": fp, "advice_alone_but_pays": fn, "advice_alone_and_slower": tn}
    if pat_n:
        out["pattern_within_%d_pct_of_best" % round(100 * tolerance)] = pat_ok / pat_n
        # pairs that lose under strict zig-zag (the reference's pattern), and how many of them the advice turns
        # around: another pattern that beats back-to-back launches, or "alone"
        out["pairs_losing_under_zigzag"] = zz_losers
        out["of_those_won_or_left_alone_by_the_advice"] = zz_rescued
    return out


def main(argv=None):
    """python -m bfuse_project_b200.pairing SWEEP.json [--margin M]: fit on every second record (by pair name),
    report on the other half, then fit on all records and write pairing_model.json."""
    import argparse
    ap = argparse.ArgumentParser(prog="pairing")
    ap.add_argument("sweep_json", nargs="+", help="files written by `python bench.py --sweep --sweep-pattern all [--sweep-extra] --sweep-out F`")
    ap.add_argument("--margin", type=float, default=1.0)
    ap.add_argument("--out", default=MODEL_PATH)
    args = ap.parse_args(argv)
    records = []
    for path in args.sweep_json:
        with open(path) as f:
            records += [r for r in json.load(f)["records"] if r.get("fused_us_by_pattern")]
    records.sort(key=lambda r: r["pair"])
    train, held = records[0::2], records[1::2]
    report = {"records": len(records), "held_out": evaluate(held, args.margin, fit(train)),
              "analytic_only_on_the_same_half": evaluate(held, args.margin, {})}
    weights = fit(records)
    report["all_records_refit"] = evaluate(records, args.margin, weights)
    with open(args.out, "w") as f:
        json.dump({"fitted_on": [os.path.basename(p) for p in args.sweep_json], "records": len(records), "features": ["1", "core", "min(t_a,t_b)", "t_a+t_b", "sum (union_slowdown-1)*t"],
                   "weights": weights, "held_out_report": report["held_out"]}, f, indent=1)
    print(json.dumps(report, indent=1))
    return 0


if __name__ == "__main__":
    import sys
    sys.exit(main())
