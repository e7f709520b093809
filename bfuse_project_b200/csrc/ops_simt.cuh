// CUDA-core fp32 bodies for dense / batch_matmul / conv2d: the same operators the reference's
// generated kernels compute (tests/benchmark/cuda/*.cu: 128-thread 32x64x16 shared-memory tiles,
// fp32 FMA, NT layout).  They exist as the like-for-like baseline ("the reference's dispatch
// pattern around straightforward non-tensor-core bodies") and as the GPU-side cross-check of the
// tcgen05 bodies; the tensor-core bodies in ops_umma.cuh are the product path for these shapes.
//
// BlockDim = (16, 16, 1); a CTA computes a 64x64 output tile, 4x4 outputs per thread, K in steps
// of 16 through shared memory.  GridDim = (ceil(N/64), ceil(M/64), batch).
#pragma once

#include <float.h>

#include "tile.h"

namespace bfuse {

constexpr int kSimtTile = 64, kSimtK = 16, kSimtPad = 4;
constexpr int kSimtSmemBytes = 2 * kSimtK * (kSimtTile + kSimtPad) * 4;

// acc[i][j] += sum_k a(m0 + ty*4 + i, k) * b(n0 + tx*4 + j, k); fa / fb fetch one element (0 when
// out of range).
template <class FA, class FB>
__device__ __forceinline__ void simt_tile_mainloop(const TileCtx &c, int K, FA fa, FB fb, float (&acc)[4][4]) {
  float(*As)[kSimtTile + kSimtPad] = reinterpret_cast<float(*)[kSimtTile + kSimtPad]>(c.smem);
  float(*Bs)[kSimtTile + kSimtPad] = As + kSimtK;
  const int tx = c.tid & 15, ty = c.tid >> 4;
  const int lr = c.tid >> 2, lk = (c.tid & 3) * 4;  // loader: row lr, k lk..lk+3
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kSimtK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      As[lk + q][lr] = fa(lr, k0 + lk + q);
      Bs[lk + q][lr] = fb(lr, k0 + lk + q);
    }
    c.sync();
#pragma unroll
    for (int kk = 0; kk < kSimtK; ++kk) {
      const float4 a = *reinterpret_cast<const float4 *>(&As[kk][ty * 4]);
      const float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    c.sync();
  }
}

// out[b, m, n] = sum_k A[b, m, k] * W[b, n, k] (+ bias[n]); causal: n > m -> -FLT_MAX.
struct GemmSimtF32 {
  struct Params {
    const float *A;
    const float *W;
    const float *bias;
    float *out;
    int batch, M, N, K;
    int causal;
  };
  static constexpr int kMaxThreads = 256;
  static constexpr int kMinBlocks = 2;
  static constexpr bool kMemoryBound = false;
  static constexpr bool kUsesTmem = false;   // allocates tensor memory (see fused_block_kernel)

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    c.dependency_wait();
    const int n0 = c.block_x() * kSimtTile, m0 = c.block_y() * kSimtTile, bz = c.block_z();
    const int tx = c.tid & 15, ty = c.tid >> 4;
    float *out = p.out + (size_t)bz * p.M * p.N;
    if (p.causal && n0 > m0 + kSimtTile - 1) {  // tile entirely above the diagonal
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
          if (m < p.M && n < p.N) out[(size_t)m * p.N + n] = -FLT_MAX;
        }
      return;
    }
    const float *A = p.A + (size_t)bz * p.M * p.K, *W = p.W + (size_t)bz * p.N * p.K;
    float acc[4][4];
    simt_tile_mainloop(
        c, p.K,
        [&](int r, int k) { return (m0 + r < p.M && k < p.K) ? __ldg(A + (size_t)(m0 + r) * p.K + k) : 0.f; },
        [&](int r, int k) { return (n0 + r < p.N && k < p.K) ? __ldg(W + (size_t)(n0 + r) * p.K + k) : 0.f; }, acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
        if (m < p.M && n < p.N) {
          float v = p.bias ? acc[i][j] + __ldg(p.bias + n) : acc[i][j];
          if (p.causal && n > m) v = -FLT_MAX;
          out[(size_t)m * p.N + n] = v;
        }
      }
  }
};

// NCHW convolution as an implicit GEMM: rows = output channels (weights [co, ci*kh*kw] are
// K-contiguous), columns = output pixels (n, oh, ow) gathered from x on the fly.
struct ConvSimtF32 {
  struct Params {
    const float *x;
    const float *w;
    float *y;
    int n, ci, h, wd, co, kh, kw, stride, pad, oh, ow;
  };
  static constexpr int kMaxThreads = 256;
  static constexpr int kMinBlocks = 2;
  static constexpr bool kMemoryBound = false;
  static constexpr bool kUsesTmem = false;   // allocates tensor memory (see fused_block_kernel)

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    c.dependency_wait();
    const int px0 = c.block_x() * kSimtTile, co0 = c.block_y() * kSimtTile;
    const int tx = c.tid & 15, ty = c.tid >> 4;
    const int K = p.ci * p.kh * p.kw, ohw = p.oh * p.ow, npix = p.n * ohw, khw = p.kh * p.kw;
    float acc[4][4];
    simt_tile_mainloop(
        c, K, [&](int r, int k) { return (co0 + r < p.co && k < K) ? __ldg(p.w + (size_t)(co0 + r) * K + k) : 0.f; },
        [&](int r, int k) {
          const int px = px0 + r;
          if (px >= npix || k >= K) return 0.f;
          const int img = px / ohw, pr = px % ohw, oy = pr / p.ow, ox = pr % p.ow;
          const int ch = k / khw, kr = k % khw / p.kw, ks = k % p.kw;
          const int iy = oy * p.stride + kr - p.pad, ix = ox * p.stride + ks - p.pad;
          if (iy < 0 || iy >= p.h || ix < 0 || ix >= p.wd) return 0.f;
          return __ldg(p.x + (((size_t)img * p.ci + ch) * p.h + iy) * p.wd + ix);
        },
        acc);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int oc = co0 + ty * 4 + i, px = px0 + tx * 4 + j;
        if (oc < p.co && px < npix) {
          const int img = px / ohw, pr = px % ohw;
          p.y[((size_t)img * p.co + oc) * ohw + pr] = acc[i][j];
        }
      }
  }
};

}  // namespace bfuse
