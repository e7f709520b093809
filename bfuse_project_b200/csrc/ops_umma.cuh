// Tensor-core bodies for dense / batch_matmul on sm_100a: TMA loads into a shared-memory ring,
// tcgen05.mma issued by one thread with the fp32 accumulator in tensor memory, tcgen05.ld back to
// registers for the epilogue (bias, causal mask, bf16 down-convert).  They compute the operators
// of the reference's dense / batch_matmul kernels (NT layout, scripts/configure_kernels.py:14-26)
// with tf32 or bf16 operands instead of CUDA-core fp32 FMAs.
//
// BlockDim = (192, 1, 1): warps 0-3 read the accumulator (one TMEM lane quadrant each), warp 4 is
// the TMA producer, warp 5 allocates tensor memory and issues the MMAs.  A CTA owns one 128 x BN
// output tile: GridDim = (ceil(N/BN), ceil(M/128), batch).  The ring depth comes from the
// shared-memory size the caller registered for the operator.
//
// Every wait on an mbarrier is bounded: when it gives up it writes a code to the status word and
// the body falls through to its normal exit (barrier, TMEM free) instead of spinning.
#pragma once

#include <cuda.h>
#include <float.h>

#include "tile.h"

namespace bfuse {

constexpr int kUmmaThreads = 192;
constexpr int kUmmaBM = 128;
constexpr int kUmmaRowBytes = 128;                      // one swizzle-128B row of K per stage
constexpr int kUmmaABytes = kUmmaBM * kUmmaRowBytes;    // 16 KB of A per stage
constexpr int kUmmaHeaderBytes = 1024;                  // barriers + tmem pointer, keeps tiles 1 KB aligned
constexpr int kUmmaMaxStages = 8;

enum UmmaStatus : int {
  UMMA_WAIT_EMPTY_TIMEOUT = 0x101,
  UMMA_WAIT_FULL_TIMEOUT = 0x102,
  UMMA_WAIT_ACC_TIMEOUT = 0x103,
};

__host__ __device__ constexpr int umma_stage_bytes(int bn) { return kUmmaABytes + bn * kUmmaRowBytes; }
__host__ __device__ constexpr int umma_smem_bytes(int bn, int stages) {
  return kUmmaHeaderBytes + stages * umma_stage_bytes(bn);
}

// ---- PTX wrappers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Wait for phase `parity` of an mbarrier, for at most ~1 s.  Returns false after reporting.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int *status, int code) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if ((it & 1023u) == 1023u) {
      const uint64_t now = global_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > 1000000000ull) {
        if (status) atomicExch(status, code);
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(cols) : "memory");
}
// Lets co-resident CTAs allocate while this one still holds its columns.  A CTA that will allocate
// again (a persistent CTA, once per tile) must NOT call this: allocating after it is illegal.
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int KIND>  // 0: tf32, 1: bf16
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  if (KIND == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 32 lanes x 16 consecutive fp32 columns of the accumulator: thread i of the warp gets lane i.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major, 128B-swizzled operand tile whose rows are 128
// bytes: 8-row groups are 1024 bytes apart (stride byte offset), version 1, layout SWIZZLE_128B.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, both operands K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t umma_idesc(int kind, int bn) {
  return (1u << 4) | ((kind == 0 ? 2u : 1u) << 7) | ((kind == 0 ? 2u : 1u) << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(kUmmaBM >> 4) << 24);
}

struct GemmUmmaParams {
  alignas(64) CUtensorMap map_a;  // {K, M, batch}, box {128 B of K, 128, 1}, 128B swizzle
  alignas(64) CUtensorMap map_b;  // {K, N, batch}, box {128 B of K, BN, 1}, 128B swizzle
  const float *bias;              // [N] or nullptr
  void *out;                      // [batch, M, N] fp32 (tf32 kind) or bf16 (bf16 kind)
  int batch, M, N, K;
  int causal;
  int stages;
  int bn;  // output-tile width: 32, 64, 128 or 256 (also the TMEM columns allocated)
};

template <int KIND>
struct GemmUmma {
  using Params = GemmUmmaParams;
  static constexpr int kMaxThreads = kUmmaThreads;
  static constexpr int kMinBlocks = 1;
  static constexpr int kElem = KIND == 0 ? 4 : 2;
  static constexpr int kBK = kUmmaRowBytes / kElem;  // K elements per stage

  // 16 consecutive outputs of one row, starting at column n0
  __device__ __forceinline__ static void store_row(const Params &p, float *dst_f32, uint16_t *dst_bf16, const uint32_t (&v)[16], int n0) {
    if (KIND == 0) {
      if (n0 + 16 <= p.N) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<uint4 *>(dst_f32 + 4 * j) = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
      } else {
        for (int j = 0; j < 16; ++j)
          if (n0 + j < p.N) dst_f32[j] = __uint_as_float(v[j]);
      }
    } else {
      if (n0 + 16 <= p.N) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint4 o;
          o.x = f2_to_bf16x2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1]));
          o.y = f2_to_bf16x2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
          o.z = f2_to_bf16x2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
          o.w = f2_to_bf16x2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
          *reinterpret_cast<uint4 *>(dst_bf16 + 8 * j) = o;
        }
      } else {
        for (int j = 0; j < 16; ++j)
          if (n0 + j < p.N) {
            const __nv_bfloat16 h = __float2bfloat16_rn(__uint_as_float(v[j]));
            dst_bf16[j] = *reinterpret_cast<const uint16_t *>(&h);
          }
      }
    }
  }

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    const int warp = c.tid >> 5, lane = c.tid & 31;
    const int BN = p.bn, kStageBytes = umma_stage_bytes(BN);
    const uint32_t idesc = umma_idesc(KIND, BN);
    const int n0 = c.block_x() * BN, m0 = c.block_y() * kUmmaBM, bz = c.block_z();
    float *out_f32 = reinterpret_cast<float *>(p.out) + (size_t)bz * p.M * p.N;
    uint16_t *out_bf16 = reinterpret_cast<uint16_t *>(p.out) + (size_t)bz * p.M * p.N;

    if (p.causal && n0 > m0 + kUmmaBM - 1) {
      // tile entirely above the diagonal: nothing to multiply, only the mask value to write
      if (warp < 4) {
        const int m = m0 + warp * 32 + lane;
        if (m < p.M) {
          uint32_t v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(-FLT_MAX);
          for (int cc = 0; cc < BN / 16; ++cc)
            if (n0 + cc * 16 < p.N)
              store_row(p, out_f32 + (size_t)m * p.N + n0 + cc * 16, out_bf16 + (size_t)m * p.N + n0 + cc * 16, v, n0 + cc * 16);
        }
      }
      return;
    }

    // operator window: [0,1024) barriers + tmem pointer, then `stages` x (A tile, B tile)
    uint64_t *bars = reinterpret_cast<uint64_t *>(c.smem);
    const int stages = p.stages;
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kUmmaMaxStages, acc_bar = empty0 + 8 * kUmmaMaxStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c.smem + 8 * (2 * kUmmaMaxStages + 1));
    const uint32_t tiles = smem_u32(c.smem) + kUmmaHeaderBytes;
    const int num_kb = (p.K + kBK - 1) / kBK;

    if (c.tid == 0) {
      for (int s = 0; s < stages; ++s) {
        mbar_init(full0 + 8 * s, 1);
        mbar_init(empty0 + 8 * s, 1);
      }
      mbar_init(acc_bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
      tmem_alloc(smem_u32(tmem_slot), BN);
      if (!c.persistent) tmem_relinquish();
    }
    tc_fence_before();
    c.sync();
    tc_fence_after();
    const uint32_t tmem_acc = *reinterpret_cast<volatile uint32_t *>(tmem_slot);

    // Producer and MMA warps run their loops with all 32 lanes (so the warp reaches the closing
    // barrier converged); lane 0 alone issues the copies / MMAs.
    if (warp == 4) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (kb / stages) & 1;
        ok = mbar_wait(empty0 + 8 * s, ph ^ 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT);
        if (ok && lane == 0) {
          mbar_expect_tx(full0 + 8 * s, kStageBytes);
          const uint32_t a_dst = tiles + s * kStageBytes;
          tma_load_3d(a_dst, &p.map_a, full0 + 8 * s, kb * kBK, m0, bz);
          tma_load_3d(a_dst + kUmmaABytes, &p.map_b, full0 + 8 * s, kb * kBK, n0, bz);
        }
        __syncwarp();
      }
    } else if (warp == 5) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (kb / stages) & 1;
        ok = mbar_wait(full0 + 8 * s, ph, c.status, UMMA_WAIT_FULL_TIMEOUT);
        tc_fence_after();
        if (ok && lane == 0) {
          const uint64_t a_desc = umma_smem_desc(tiles + s * kStageBytes);
          const uint64_t b_desc = umma_smem_desc(tiles + s * kStageBytes + kUmmaABytes);
#pragma unroll
          for (int j = 0; j < 4; ++j)  // 4 x 32 bytes of K per stage; +2 = 32 bytes in descriptor units
            umma_ss<KIND>(tmem_acc, a_desc + 2 * j, b_desc + 2 * j, idesc, (kb | j) != 0);
          umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
        }
        __syncwarp();
      }
      if (lane == 0) umma_commit(acc_bar);  // accumulator complete (also arrives if the loop bailed out)
      __syncwarp();
      // The stage-release arrivals of the last ring pass are asynchronous and nobody consumes them;
      // wait for them here so that none is still in flight when the barriers are invalidated and
      // the shared memory is handed to the next tile or the next CTA.
      for (int kb = max(0, num_kb - stages); kb < num_kb && ok; ++kb)
        ok = mbar_wait(empty0 + 8 * (kb % stages), (kb / stages) & 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT);
    } else {
      // epilogue: hardware warp w may only touch TMEM lanes [32 * (w % 4), +32)
      const int quad = (threadIdx.x >> 5) & 3;
      const bool ok = mbar_wait(acc_bar, 0, c.status, UMMA_WAIT_ACC_TIMEOUT);
      tc_fence_after();
      const int m = m0 + quad * 32 + lane;
      if (ok) {
#pragma unroll 1
        for (int cc = 0; cc < BN / 16; ++cc) {
          uint32_t r[16];
          tmem_ld_32x16(tmem_acc + ((uint32_t)(quad * 32) << 16) + cc * 16, r);
          const int nb = n0 + cc * 16;
          if (m < p.M && nb < p.N) {
            if (p.bias) {
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __ldg(p.bias + min(nb + j, p.N - 1)));
            }
            if (p.causal && nb + 15 > m) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (nb + j > m) r[j] = __float_as_uint(-FLT_MAX);
            }
            store_row(p, out_f32 + (size_t)m * p.N + nb, out_bf16 + (size_t)m * p.N + nb, r, nb);
          }
        }
      }
    }
    tc_fence_before();
    c.sync();
    if (warp == 5) tmem_dealloc(tmem_acc, BN);
    if (c.tid == 0) {
      for (int s = 0; s < stages; ++s) {
        mbar_inval(full0 + 8 * s);
        mbar_inval(empty0 + 8 * s);
      }
      mbar_inval(acc_bar);
    }
  }
};

}  // namespace bfuse
