"""The operator oracle has no reference golden outputs to pin against (the reference ships
no CPU implementation of any operator), so it is cross-checked here against float64 numpy
restatements of the same definitions, plus closed-form cases."""
import numpy as np

import oracle


def test_bf16_roundtrip_and_rounding():
    x = np.array([1.0, 1.00390625, 1.005859375, -2.5, 3.1415927, 0.0, 65504.0], np.float32)
    h = oracle.f32_to_bf16(x)
    back = oracle.bf16_to_f32(h)
    assert back[0] == 1.0 and back[3] == -2.5
    assert back[1] == 1.0          # 1 + 2^-8 is a tie -> even mantissa
    assert back[2] == 1.0078125    # above the tie -> rounds up
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)


def test_softmax():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((37, 512)).astype(np.float32)
    y = oracle.softmax(x, 0.125)
    z = np.exp((x.astype(np.float64) * 0.125) - (x.astype(np.float64) * 0.125).max(1, keepdims=True))
    z /= z.sum(1, keepdims=True)
    assert np.allclose(y, z, rtol=1e-5, atol=0)
    assert np.allclose(y.sum(1), 1.0, atol=1e-5)


def test_layernorm_with_and_without_residual():
    rng = np.random.default_rng(2)
    x = rng.standard_normal((19, 768)).astype(np.float32)
    r = rng.standard_normal((19, 768)).astype(np.float32)
    g = rng.uniform(0.5, 1.5, 768).astype(np.float32)
    b = rng.uniform(0.5, 1.5, 768).astype(np.float32)
    for res in (None, r):
        v = x.astype(np.float64) + (0 if res is None else res.astype(np.float64))
        z = (v - v.mean(1, keepdims=True)) / np.sqrt(v.var(1, keepdims=True) + 1e-5) * g + b
        y = oracle.layernorm(x, g, b, 1e-5, res)
        assert np.allclose(y, z, rtol=1e-5, atol=1e-5)


def test_rmsnorm_bf16():
    rng = np.random.default_rng(3)
    x = oracle.f32_to_bf16(rng.standard_normal((11, 4096)).astype(np.float32))
    w = oracle.f32_to_bf16(rng.uniform(0.5, 1.5, 4096).astype(np.float32))
    y = oracle.bf16_to_f32(oracle.rmsnorm_bf16(x, w, 1e-5)).astype(np.float64)
    xf, wf = oracle.bf16_to_f32(x).astype(np.float64), oracle.bf16_to_f32(w).astype(np.float64)
    z = xf / np.sqrt((xf * xf).mean(1, keepdims=True) + 1e-5) * wf
    assert np.all(np.abs(y - z) <= np.abs(z) * 2.0 ** -8 + 1e-30)


def test_rope_bf16_rotate_half():
    rng = np.random.default_rng(4)
    q = oracle.f32_to_bf16(rng.standard_normal((33, 4, 128)).astype(np.float32))
    inv = oracle.rope_inv_freq(128, 500000.0)
    assert inv[0] == 1.0 and abs(inv[-1] - 500000.0 ** (-126 / 128)) < 1e-9
    y = oracle.bf16_to_f32(oracle.rope_bf16(q, inv)).astype(np.float64)
    x = oracle.bf16_to_f32(q).astype(np.float64)
    ang = np.arange(33, dtype=np.float64)[:, None] * inv.astype(np.float64)[None, :]
    cos = np.concatenate([np.cos(ang), np.cos(ang)], -1)[:, None, :]
    sin = np.concatenate([np.sin(ang), np.sin(ang)], -1)[:, None, :]
    rot = np.concatenate([-x[..., 64:], x[..., :64]], -1)
    z = x * cos + rot * sin
    assert np.all(np.abs(y - z) <= np.abs(z) * 2.0 ** -8 + 2e-5)
    # position 0 is the identity
    assert np.array_equal(oracle.rope_bf16(q, inv)[0], q[0])


def test_gemm_nt_bias_causal_tf32():
    rng = np.random.default_rng(5)
    A = rng.standard_normal((2, 40, 64)).astype(np.float32)
    W = rng.standard_normal((2, 48, 64)).astype(np.float32)
    bias = rng.standard_normal(48).astype(np.float32)
    ref = np.einsum("bmk,bnk->bmn", A.astype(np.float64), W.astype(np.float64))
    assert np.allclose(oracle.gemm_nt(A, W), ref, rtol=1e-5, atol=1e-4)
    assert np.allclose(oracle.gemm_nt(A, W, bias=bias), ref + bias, rtol=1e-5, atol=1e-4)
    c = oracle.gemm_nt(A, W, causal=True)
    mask = np.arange(48)[None, :] > np.arange(40)[:, None]
    assert np.all(c[:, mask] == -np.finfo(np.float32).max)
    assert np.allclose(c[:, ~mask], ref[:, ~mask], rtol=1e-5, atol=1e-4)
    t = oracle.gemm_nt(A, W, tf32=True)
    At = (A.view(np.uint32) & 0xFFFFE000).view(np.float32).astype(np.float64)
    Wt = (W.view(np.uint32) & 0xFFFFE000).view(np.float32).astype(np.float64)
    assert np.allclose(t, np.einsum("bmk,bnk->bmn", At, Wt), rtol=1e-5, atol=1e-4)
    assert np.abs(t - ref).max() < 5e-3 * np.sqrt((ref ** 2).mean()) * 4


def test_gemm_bf16():
    rng = np.random.default_rng(6)
    A = oracle.f32_to_bf16(rng.standard_normal((24, 96)).astype(np.float32))
    W = oracle.f32_to_bf16((0.02 * rng.standard_normal((40, 96))).astype(np.float32))
    y = oracle.bf16_to_f32(oracle.gemm_nt_bf16(A, W)).astype(np.float64)
    z = oracle.bf16_to_f32(A).astype(np.float64) @ oracle.bf16_to_f32(W).astype(np.float64).T
    assert np.all(np.abs(y - z) <= np.abs(z) * 2.0 ** -8 + 1e-6)


def test_conv2d_nchw_both_branches():
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 8, 14, 14)).astype(np.float32)
    for (k, s, p) in ((3, 2, 1), (1, 2, 0)):
        w = rng.standard_normal((6, 8, k, k)).astype(np.float32)
        y = oracle.conv2d_nchw(x, w, s, p)
        xp = np.pad(x.astype(np.float64), ((0, 0), (0, 0), (p, p), (p, p)))
        oh = (14 + 2 * p - k) // s + 1
        z = np.zeros((2, 6, oh, oh))
        for r in range(k):
            for c in range(k):
                patch = xp[:, :, r:r + s * oh:s, c:c + s * oh:s]
                z += np.einsum("nchw,oc->nohw", patch, w[:, :, r, c].astype(np.float64))
        assert y.shape == z.shape
        assert np.allclose(y, z, rtol=1e-5, atol=1e-4)


def test_empty_inputs_are_noops():
    assert oracle.softmax(np.zeros((0, 16), np.float32), 1.0).shape == (0, 16)
    assert oracle.gemm_nt(np.zeros((0, 8), np.float32), np.zeros((4, 8), np.float32)).shape == (0, 4)
