"""Checker side of the GPU parity tests: oracle outputs for a KernelSpec and the comparison rules.

What "rel 5e-3" means here.  A dot product of K terms of typical size s carries an absolute rounding error
of order s * sqrt(K) * u (u = 2^-11 for operands truncated to tf32, 2^-8 for bf16) however close to zero
the sum itself lands, so a tolerance relative to each element's own value alone cannot hold for elements
that cancel.  The tolerance is therefore relative to the element's value plus the scale of the output:

    |got - ref| <= tol * (|ref| + rms(ref))

with rms taken over the whole output tensor.  Every comparison against the oracle AND against the
reference's own kernels uses this one rule (`within`, `assert_close`); max|got - ref| / rms(ref) alone, which
ignores the |ref| term, reads up to about 6e-3 for a K = 64 tf32 product of N(0, 1) operands and is not
the rule.

Tolerances (stated once here, used by every GPU test):
  * fused vs unfused launches of the same body: bit-exact (the arithmetic order is unchanged);
  * fp32 memory-bound operators vs the oracle: |d| <= 1e-5 * (|ref| + rms(ref));
  * tf32 / bf16 tensor-core GEMMs vs the fp32 oracle: |d| <= 5e-3 * (|ref| + rms(ref)); tf32 GEMMs
    additionally vs the oracle with operands truncated to tf32: |d| <= 2e-4 * (|ref| + rms(ref));
    a bf16 output may in addition sit one bf16 ulp (2^-7 relative) from the oracle's, because the
    two fp32 sums can fall on either side of a rounding boundary;
  * bf16 outputs of memory-bound operators: equal to the oracle's bf16 except for at most 0.1 % of
    the elements, which may differ by one bf16 ulp plus 1e-5 absolute (a few-ulp fp32 difference in
    sin / cos or in the row sum before rounding, visible where two products cancel).
"""
import numpy as np

import bfuse_project_b200 as bf
import oracle

FLT_MAX = np.finfo(np.float32).max


def oracle_outputs(ks, tf32=False):
    h = ks.host
    if ks.op == bf.OP_SOFTMAX_F32:
        return [oracle.softmax(h[0], ks.fparam[0])]
    if ks.op == bf.OP_LAYERNORM_F32:
        return [oracle.layernorm(h[0], h[2], h[3], ks.fparam[0], res=h[1])]
    if ks.op == bf.OP_RMSNORM_BF16:
        return [oracle.rmsnorm_bf16(h[0], h[1], ks.fparam[0])]
    if ks.op == bf.OP_ROPE_BF16:
        return [oracle.rope_bf16(h[0], h[1])]
    if ks.op in (bf.OP_GEMM_F32_SIMT, bf.OP_GEMM_TF32):
        return [oracle.gemm_nt(h[0], h[1], bias=h[2], causal=bool(ks.flags & bf.FLAG_CAUSAL), tf32=tf32)]
    if ks.op == bf.OP_GEMM_BF16:
        return [np.stack([oracle.gemm_nt_bf16(h[0][b], h[1][b]) for b in range(h[0].shape[0])])]
    if ks.op in (bf.OP_CONV2D_F32_SIMT, bf.OP_CONV2D_TF32):
        return [oracle.conv2d_nchw(h[0], h[1], ks.shape[7], ks.shape[8], tf32=tf32)]
    raise KeyError(ks.op)


def within(got, ref, tol):
    """The rule above on torch tensors (device side, for outputs too large to bring to the host):
    (passes, worst |got - ref| / (|ref| + rms))."""
    ref64 = ref.double()
    rms = float(ref64.pow(2).mean().sqrt())
    worst = float(((got.double() - ref64).abs() / (ref64.abs() + rms)).max())
    return worst <= tol, worst


def assert_close(got, ref, tol, what, ulp_rel=0.0):
    got = got.astype(np.float64)
    ref64 = ref.astype(np.float64)
    masked = ref == -FLT_MAX
    assert np.array_equal(got[masked], ref64[masked]), what + ": causal mask entries differ"
    g, r = got[~masked], ref64[~masked]
    rms = np.sqrt(np.mean(r * r)) if r.size else 0.0
    err = np.abs(g - r)
    lim = np.maximum(tol * (np.abs(r) + rms), ulp_rel * np.abs(r))
    bad = err > lim
    assert not bad.any(), "%s: %d / %d outside %.0e (worst %.3e vs limit %.3e)" % (
        what, bad.sum(), r.size, tol, err[bad].max(), lim[bad][np.argmax(err[bad])])


def assert_bf16_close(got, ref, what, frac=1e-3):
    g = oracle.bf16_to_f32(got.reshape(-1)).astype(np.float64)
    r = oracle.bf16_to_f32(ref.reshape(-1)).astype(np.float64)
    diff = got.reshape(-1) != ref.reshape(-1)
    if diff.any():
        ulp = np.abs(r[diff]) * 2.0 ** -7 + 1e-5
        assert np.all(np.abs(g[diff] - r[diff]) <= ulp), what + ": bf16 mismatch larger than one ulp"
    assert diff.mean() <= frac, "%s: %.4f %% of bf16 outputs differ by one ulp" % (what, 100 * diff.mean())


def check_against_oracle(ks, got, what):
    """got: list of output arrays of kernel ks as produced by the CUDA path."""
    if ks.op in (bf.OP_SOFTMAX_F32, bf.OP_LAYERNORM_F32, bf.OP_GEMM_F32_SIMT, bf.OP_CONV2D_F32_SIMT):
        assert_close(got[0], oracle_outputs(ks)[0], 1e-5, what)
    elif ks.op in (bf.OP_RMSNORM_BF16, bf.OP_ROPE_BF16):
        assert_bf16_close(got[0], oracle_outputs(ks)[0], what)
    elif ks.op in (bf.OP_GEMM_TF32, bf.OP_CONV2D_TF32):
        assert_close(got[0], oracle_outputs(ks, tf32=True)[0], 2e-4, what + " (tf32-truncated oracle)")
        assert_close(got[0], oracle_outputs(ks)[0], 5e-3, what + " (fp32 oracle)")
    elif ks.op == bf.OP_GEMM_BF16:
        g = oracle.bf16_to_f32(got[0].reshape(-1)).reshape(got[0].shape)
        r = oracle.bf16_to_f32(oracle_outputs(ks)[0].reshape(-1)).reshape(got[0].shape)
        assert_close(g, r, 5e-3, what, ulp_rel=2.0 ** -7)
    else:
        raise KeyError(ks.op)
