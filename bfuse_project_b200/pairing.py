"""Pair-selection model: will two operators gain from sharing a launch?

The reference leaves this as its open question and answers it with profiler counters: a pair is a
candidate when the time-weighted sums of the two kernels' LSU and FMA pipe utilisation stay under
thresholds, i.e. when the shared resource has head-room for both
(scripts/analyze_test_suite.py:20-25, 436-479).  On B200 the scarce resource of these short
operators is not a pipe but the SMs themselves -- most of them leave SMs idle -- so the model here
works on each operator's launch record (CTAs, threads, shared-memory window) and its time alone:

    fill_k      = CTAs_k / (SMs * CTAs of k that fit one SM)          share of the GPU k occupies
    fused       = max( max(t_a, t_b),  fill_a * t_a + fill_b * t_b ) + overhead
    sequential  = t_a + t_b

The first term is the critical path (the longer operator), the second the area (SM-time) both need
when they do not fit side by side.  `overhead` (1 us) is what a fused CTA pays over an unfused one:
the larger shared-memory window and block, the dispatch decode.  Fitted on nothing: checked against
the 903 pairs of the operator sweep (`python bench.py --sweep` reports the error and the confusion
counts under `pairing_model`).
"""

SM_SMEM_BYTES = 227 * 1024
SM_THREADS = 2048
OVERHEAD_US = 1.0


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
    return max(max(t_a, t_b), fill_a * t_a + fill_b * t_b) + overhead_us


def advise(t_a, t_b, launch_a, launch_b, sm_count=148, margin=1.0):
    """launch_k = (ctas, threads, smem_bytes).  Returns the prediction and whether to fuse
    (predicted speed-up over back-to-back launches above `margin`)."""
    fa, fb = fill(*launch_a, sm_count=sm_count), fill(*launch_b, sm_count=sm_count)
    fused = predict_fused_us(t_a, t_b, fa, fb)
    speedup = (t_a + t_b) / fused
    return {"fill": (fa, fb), "predicted_fused_us": fused, "predicted_speedup": speedup, "fuse": speedup > margin}


def evaluate(records, margin=1.0):
    """records: iterable of dicts with t_a, t_b, launch_a, launch_b, fused_us, sequential_us (measured).
    Median / 90th-percentile relative error of the predicted fused time and the confusion counts of
    "fusing pays" (measured speed-up > margin) against the advice."""
    errs, tp, fp, fn, tn = [], 0, 0, 0, 0
    for r in records:
        a = advise(r["t_a"], r["t_b"], r["launch_a"], r["launch_b"], r.get("sm_count", 148), margin)
        errs.append(abs(a["predicted_fused_us"] - r["fused_us"]) / r["fused_us"])
        pays = r["sequential_us"] / r["fused_us"] > margin
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
    return {"pairs": len(errs), "median_rel_err": errs[len(errs) // 2], "p90_rel_err": errs[(len(errs) * 9) // 10],
            "advice_fuse_and_pays": tp, "advice_fuse_but_slower": fp, "advice_alone_but_pays": fn, "advice_alone_and_slower": tn}
