// Memory-bound operator bodies: row softmax, LayerNorm (optionally fused with a residual add),
// RMSNorm and rotate-half RoPE.  The reference has no kernels for these (its generator only emits
// dense / batch_matmul / conv2d, scripts/configure_kernels.py:40-68); the arithmetic follows the
// operator definitions in its Relay dumps (files/bert-base-uncased.txt:34-41,61-70,
// files/gpt2.txt:9-17, files/Meta-Llama-3-8B.txt:7-28).
//
// Common shape of a body: BlockDim = (threads per row, rows per CTA, 1), GridDim.X = ceil(rows /
// rows per CTA).  Every thread keeps its slice of the row in registers as 128-bit vectors, so each
// input byte is read from HBM once and each output byte written once; reductions are warp
// shuffles plus, for rows wider than a warp, one shared-memory exchange on the operator's named
// barrier.
#pragma once

#include "tile.h"

namespace bfuse {

constexpr int kRowMaxVec = 4;  // 128-bit vectors a thread may hold per row (rows up to 4096 fp32 / 8192 bf16)

// ---------------------------------------------------------------------------------- softmax
struct SoftmaxF32 {
  struct Params {
    const float *x;
    float *y;
    int rows, cols;
    float scale;
  };
  static constexpr int kMaxThreads = 256;
  static constexpr int kMinBlocks = 6;   // 6 x 256 threads per SM: registers per thread <= 40 (32 spills badly; 5 CTAs of 48 registers lose more in waves than the spills cost)
  static constexpr bool kMemoryBound = true;
  static constexpr bool kUsesTmem = false;   // allocates tensor memory (see fused_block_kernel)

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    c.dependency_wait();
    const int tpr = c.bx, lane = c.tid % tpr, row = c.vblock * c.by + c.tid / tpr;
    const int nvec = p.cols / (4 * tpr);
    const bool live = row < p.rows;
    const float4 *xr = reinterpret_cast<const float4 *>(p.x + (size_t)row * p.cols);
    float4 v[kRowMaxVec];
    // every load of the row is issued before the first use of any of them: a use between two loads
    // would make the second one wait for the first one's trip to DRAM
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i)
      if (i < nvec && live) v[i] = ld_stream_f4(xr + i * tpr + lane);
    float m = -INFINITY;
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      if (i < nvec && live) {
        v[i].x *= p.scale, v[i].y *= p.scale, v[i].z *= p.scale, v[i].w *= p.scale;
        m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
      }
    }
    m = row_reduce<OpMax>(m, c, tpr, 0);
    constexpr float kLog2e = 1.4426950408889634f;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      if (i < nvec && live) {
        v[i].x = exp2f((v[i].x - m) * kLog2e);
        v[i].y = exp2f((v[i].y - m) * kLog2e);
        v[i].z = exp2f((v[i].z - m) * kLog2e);
        v[i].w = exp2f((v[i].w - m) * kLog2e);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    s = row_reduce<OpSum>(s, c, tpr, 1);
    const float inv = 1.f / s;
    float4 *yr = reinterpret_cast<float4 *>(p.y + (size_t)row * p.cols);
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      if (i < nvec && live) {
        v[i].x *= inv, v[i].y *= inv, v[i].z *= inv, v[i].w *= inv;
        st_stream_f4(yr + i * tpr + lane, v[i]);
      }
    }
  }
};

// -------------------------------------------------------------------- (residual +) LayerNorm
struct LayerNormF32 {
  struct Params {
    const float *x;
    const float *res;  // nullptr: plain LayerNorm
    const float *gamma;
    const float *beta;
    float *y;
    int rows, cols;
    float eps;
  };
  static constexpr int kMaxThreads = 256;
  static constexpr int kMinBlocks = 6;   // 6 x 256 threads per SM: registers per thread <= 40 (32 spills badly; 5 CTAs of 48 registers lose more in waves than the spills cost)
  static constexpr bool kMemoryBound = true;
  static constexpr bool kUsesTmem = false;   // allocates tensor memory (see fused_block_kernel)

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    c.dependency_wait();
    const int tpr = c.bx, lane = c.tid % tpr, row = c.vblock * c.by + c.tid / tpr;
    const int nvec = p.cols / (4 * tpr);
    const bool live = row < p.rows;
    const float4 *xr = reinterpret_cast<const float4 *>(p.x + (size_t)row * p.cols);
    const float4 *rr = reinterpret_cast<const float4 *>(p.res + (size_t)row * p.cols);
    const bool has_res = p.res != nullptr;
    const float4 *g4 = reinterpret_cast<const float4 *>(p.gamma);
    const float4 *b4 = reinterpret_cast<const float4 *>(p.beta);
    if (c.tid < tpr) {  // one row's worth of threads touches every line of gamma and beta
      for (int i = 0; i < nvec; ++i) {
        prefetch_l1(g4 + i * tpr + lane);
        prefetch_l1(b4 + i * tpr + lane);
      }
    }
    float4 v[kRowMaxVec];
    // every load of the row is issued before the first use of any of them (see SoftmaxF32)
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i)
      if (i < nvec && live) v[i] = ld_stream_f4(xr + i * tpr + lane);
    if (has_res) {
      float4 r[kRowMaxVec];
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i)
        if (i < nvec && live) r[i] = ld_stream_f4(rr + i * tpr + lane);
#pragma unroll
      for (int i = 0; i < kRowMaxVec; ++i)
        if (i < nvec && live) v[i].x += r[i].x, v[i].y += r[i].y, v[i].z += r[i].z, v[i].w += r[i].w;
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i)
      if (i < nvec && live) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = row_reduce<OpSum>(s, c, tpr, 0) / (float)p.cols;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      if (i < nvec && live) {
        v[i].x -= mean, v[i].y -= mean, v[i].z -= mean, v[i].w -= mean;
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
    const float rstd = 1.f / sqrtf(row_reduce<OpSum>(q, c, tpr, 1) / (float)p.cols + p.eps);
    float4 *yr = reinterpret_cast<float4 *>(p.y + (size_t)row * p.cols);
#pragma unroll
    for (int i = 0; i < kRowMaxVec; ++i) {
      if (i < nvec && live) {
        const float4 g = __ldg(g4 + i * tpr + lane), b = __ldg(b4 + i * tpr + lane);
        float4 o;
        o.x = v[i].x * rstd * g.x + b.x;
        o.y = v[i].y * rstd * g.y + b.y;
        o.z = v[i].z * rstd * g.z + b.z;
        o.w = v[i].w * rstd * g.w + b.w;
        st_stream_f4(yr + i * tpr + lane, o);
      }
    }
  }
};

// ---------------------------------------------------------------------------------- RMSNorm
__device__ __forceinline__ float2 bf16x2_to_f2(uint32_t u) {
  return make_float2(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));
}
__device__ __forceinline__ uint32_t f2_to_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t *>(&h);
}

struct RmsNormBf16 {
  struct Params {
    const uint16_t *x;
    const uint16_t *w;
    uint16_t *y;
    int rows, cols;
    float eps;
  };
  static constexpr int kMaxThreads = 256;
  static constexpr int kMinBlocks = 6;   // 6 x 256 threads per SM: registers per thread <= 40 (32 spills badly; 5 CTAs of 48 registers lose more in waves than the spills cost)
  static constexpr bool kMemoryBound = true;
  static constexpr bool kUsesTmem = false;   // allocates tensor memory (see fused_block_kernel)
  static constexpr int kMaxVec = 4;  // 8 bf16 per vector

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    c.dependency_wait();
    const int tpr = c.bx, lane = c.tid % tpr, row = c.vblock * c.by + c.tid / tpr;
    const int nvec = p.cols / (8 * tpr);
    const bool live = row < p.rows;
    const uint4 *xr = reinterpret_cast<const uint4 *>(p.x + (size_t)row * p.cols);
    const uint4 *w4 = reinterpret_cast<const uint4 *>(p.w);
    if (c.tid < tpr)  // one row's worth of threads touches every line of the weight vector
      for (int i = 0; i < nvec; ++i) prefetch_l1(w4 + i * tpr + lane);
    uint4 v[kMaxVec];
    // every load of the row is issued before the first use of any of them (see SoftmaxF32)
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i)
      if (i < nvec && live) v[i] = ld_stream_u4(xr + i * tpr + lane);
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      if (i < nvec && live) {
        const uint32_t u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = bf16x2_to_f2(u[j]);
          q += f.x * f.x + f.y * f.y;
        }
      }
    }
    const float rinv = 1.f / sqrtf(row_reduce<OpSum>(q, c, tpr, 0) / (float)p.cols + p.eps);
    uint4 *yr = reinterpret_cast<uint4 *>(p.y + (size_t)row * p.cols);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      if (i < nvec && live) {
        const uint4 wv = __ldg(w4 + i * tpr + lane);
        const uint32_t u[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
        const uint32_t g[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = bf16x2_to_f2(u[j]), wf = bf16x2_to_f2(g[j]);
          o[j] = f2_to_bf16x2(f.x * rinv * wf.x, f.y * rinv * wf.y);
        }
        st_stream_u4(yr + i * tpr + lane, make_uint4(o[0], o[1], o[2], o[3]));
      }
    }
  }
};

// ------------------------------------------------------------------------------------- RoPE
// q[seq, heads, dim] bf16.  BlockDim = (chunks * head_groups, positions per CTA, 1) where a chunk
// is 8 consecutive rotary pairs (dim / 16 chunks per head); a thread computes the 8 sin/cos of its
// (position, chunk) once and applies them to heads / head_groups heads.
struct RopeBf16 {
  struct Params {
    const uint16_t *q;
    const float *inv_freq;  // [dim / 2]
    uint16_t *y;
    int seq, heads, dim;
  };
  static constexpr int kMaxThreads = 256;
  static constexpr int kMinBlocks = 6;   // 6 x 256 threads per SM: registers per thread <= 40 (32 spills badly; 5 CTAs of 48 registers lose more in waves than the spills cost)
  static constexpr bool kMemoryBound = true;
  static constexpr bool kUsesTmem = false;   // allocates tensor memory (see fused_block_kernel)

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    c.dependency_wait();
    const int half = p.dim >> 1, chunks = half >> 3;
    const int tx = c.tid % c.bx, chunk = tx % chunks, hg = tx / chunks, ngroups = c.bx / chunks;
    const int pos = c.vblock * c.by + c.tid / c.bx;
    if (pos >= p.seq) return;
    // The frequency table first (the sin / cos arithmetic waits for it), then all of this thread's
    // rows as L1 prefetches that tie up no register; the arithmetic runs while they travel and the
    // loads in the head loop find their lines in L1.  A load first issued after the arithmetic would
    // queue behind everything the grid already has in flight and cost another trip to DRAM per head.
    const float4 f0 = __ldg(reinterpret_cast<const float4 *>(p.inv_freq) + chunk * 2);
    const float4 f1 = __ldg(reinterpret_cast<const float4 *>(p.inv_freq) + chunk * 2 + 1);
    const int hpt = p.heads / ngroups, h_begin = hg * hpt, h_end = h_begin + hpt;
    const size_t o0 = ((size_t)pos * p.heads + h_begin) * p.dim + chunk * 8;
    for (int h = 0; h < hpt; ++h) {
      prefetch_l1(p.q + o0 + (size_t)h * p.dim);
      prefetch_l1(p.q + o0 + (size_t)h * p.dim + half);
    }
    float cs[8], sn[8];
    const float fr[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) sincosf((float)pos * fr[j], &sn[j], &cs[j]);
    for (int h = h_begin; h < h_end; ++h) {
      const size_t o = ((size_t)pos * p.heads + h) * p.dim + chunk * 8;
      const uint4 a4 = ld_stream_u4(reinterpret_cast<const uint4 *>(p.q + o));
      const uint4 b4 = ld_stream_u4(reinterpret_cast<const uint4 *>(p.q + o + half));
      const uint32_t a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
      uint32_t oa[4], ob[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = bf16x2_to_f2(a[j]), fb = bf16x2_to_f2(b[j]);
        oa[j] = f2_to_bf16x2(fa.x * cs[2 * j] - fb.x * sn[2 * j], fa.y * cs[2 * j + 1] - fb.y * sn[2 * j + 1]);
        ob[j] = f2_to_bf16x2(fb.x * cs[2 * j] + fa.x * sn[2 * j], fb.y * cs[2 * j + 1] + fa.y * sn[2 * j + 1]);
      }
      st_stream_u4(reinterpret_cast<uint4 *>(p.y + o), make_uint4(oa[0], oa[1], oa[2], oa[3]));
      st_stream_u4(reinterpret_cast<uint4 *>(p.y + o + half), make_uint4(ob[0], ob[1], ob[2], ob[3]));
    }
  }
};

}  // namespace bfuse
