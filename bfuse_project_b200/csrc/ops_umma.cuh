// Tensor-core bodies for dense / batch_matmul on sm_100a: TMA loads into a shared-memory ring,
// tcgen05.mma issued by one thread with the fp32 accumulator in tensor memory, tcgen05.ld back to
// registers for the epilogue (bias, causal mask, bf16 down-convert).  They compute the operators
// of the reference's dense / batch_matmul kernels (NT layout, scripts/configure_kernels.py:14-26)
// with tf32 or bf16 operands instead of CUDA-core fp32 FMAs.
//
// BlockDim = (192, 1, 1): warps 0-3 read the accumulator (one TMEM lane quadrant each), warp 4 is
// the TMA producer, warp 5 allocates tensor memory and issues the MMAs.  One 128 x BN output tile
// belongs to `split` CTAs that each multiply a slice of K: GridDim = (split * ceil(M/128),
// ceil(N/BN), batch).  A tcgen05.mma of 128 x N x 32 bytes takes about the same time for N = 32
// as for N = 256, so narrow problems are fast only with wide tiles whose K loop is spread over
// several SMs.  With split > 1 the CTAs of a tile form a thread-block cluster and every CTA owns a
// share of the tile's 128-byte column chunks: after one cluster barrier (all MMAs of the tile are
// done, so every ring is free) each CTA pushes its fp32 partial sums of a chunk straight from
// tensor memory into the owner's shared memory with st.async, the owner waits on an mbarrier that
// counts the delivered bytes, sums the k-slices in order (deterministic) and stores the chunk.
// The ring depth comes from the shared-memory size the caller registered.
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
constexpr int kUmmaHeaderBytes = 2048;                  // barriers, tmem pointer, bias slice; keeps tiles 1 KB aligned
constexpr int kUmmaMaxStages = 8;

enum UmmaStatus : int {
  UMMA_WAIT_EMPTY_TIMEOUT = 0x101,
  UMMA_WAIT_FULL_TIMEOUT = 0x102,
  UMMA_WAIT_ACC_TIMEOUT = 0x103,
  UMMA_WAIT_PEERS_TIMEOUT = 0x104,
};

// bm: rows of A (and of the output tile) per CTA, 128 or 256
__host__ __device__ constexpr int umma_stage_bytes(int bn, int bm = kUmmaBM) { return (bm + bn) * kUmmaRowBytes; }
__host__ __device__ constexpr int umma_smem_bytes(int bn, int stages, int bm = kUmmaBM) {
  return kUmmaHeaderBytes + stages * umma_stage_bytes(bn, bm);
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
      // once any wait of the launch has given up, the others follow at once: a failed launch then ends
      // after about one second in all, not one second per CTA
      if (status && *reinterpret_cast<volatile int *>(status) != 0) return false;
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
// One thread of a warp, chosen by the hardware; every lane of the (converged) warp must call it.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
// High word of the shared-memory matrix descriptor of a K-major, 128B-swizzled operand tile whose
// rows are 128 bytes: 8-row groups 1024 bytes apart (stride byte offset, bits 32-45), version 1
// (bit 46), layout SWIZZLE_128B (bits 61-63).  The low word is (address >> 4) | 1 << 16.
constexpr uint32_t kUmmaDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
template <int KIND>  // 0: tf32, 1: bf16; a_lo / b_lo: low descriptor words
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  if (KIND == 0) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(kUmmaDescHi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t}" ::"r"(d_tmem),
        "r"(a_lo), "r"(b_lo), "r"(kUmmaDescHi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// The same MMA with the A operand in tensor memory: 128 lanes (rows of A) x one 32-bit column per tf32
// value of k, 8 columns per instruction; B from shared memory as above.
__device__ __forceinline__ void umma_ts_tf32(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], db, %4, p;\n\t}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(kUmmaDescHi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Registers -> tensor memory, 32 lanes x 32 consecutive 32-bit columns: thread i of the warp writes
// lane i (a warp reaches the 32 lanes of its quadrant, warp index mod 4).  Asynchronous: complete
// after tmem_st_wait().
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// the same, 4 columns
__device__ __forceinline__ void tmem_st_32x4(uint32_t taddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// 32 lanes x 16 consecutive fp32 columns of the accumulator: thread i of the warp gets lane i.
// Asynchronous: the registers are valid after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (a shared::cta address of this CTA) in the shared memory of cluster rank `rank`
__device__ __forceinline__ uint32_t peer_smem(uint32_t local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
  return r;
}
// 16-byte store into a peer's shared memory that also credits 16 bytes to the peer's mbarrier
__device__ __forceinline__ void st_async_u4(uint32_t peer_addr, uint32_t peer_bar, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%2, %3, %4, %5}, [%1];" ::"r"(peer_addr),
               "r"(peer_bar), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_shared_u4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// Instruction descriptor: fp32 accumulate, both operands K-major, M = 128, N = bn.
__host__ __device__ constexpr uint32_t umma_idesc(int kind, int bn) {
  return (1u << 4) | ((kind == 0 ? 2u : 1u) << 7) | ((kind == 0 ? 2u : 1u) << 10) | ((uint32_t)(bn >> 3) << 17) |
         ((uint32_t)(kUmmaBM >> 4) << 24);
}

struct GemmUmmaParams {
  alignas(64) CUtensorMap map_a;    // {K, M, batch}, box {128 B of K, BM, 1}, 128B swizzle
  alignas(64) CUtensorMap map_b;    // {K, N, batch}, box {128 B of K, BN, 1}, 128B swizzle
  alignas(64) CUtensorMap map_out;  // {N, M, batch}, box {128 B of N, 32, 1}, 128B swizzle (stores)
  const float *bias;                // [N] or nullptr
  void *out;                        // [batch, M, N] fp32 (tf32 kind) or bf16 (bf16 kind)
  int batch, M, N, K;
  int causal;
  int stages;
  int bn;            // output-tile width: 32, 64, 128 or 256 (also the TMEM columns allocated)
  int split;         // CTAs (k-slices) per output tile = cluster width; 1: no split
  int kb_per_slice;  // K blocks (of 128 bytes per row) per k-slice
  int bm;            // output-tile height: 128, or 256 (two MMAs per k-step share the W tile; split == 1 only)
  long long *timeline;  // diagnostic: when non-null, CTA 0 records globaltimer marks here (see UmmaMark)
};

// marks of the diagnostic timeline (nanoseconds on the global timer), written by virtual block 0
enum UmmaMark : int {
  MARK_START = 0, MARK_SETUP_DONE, MARK_FIRST_LOAD_ISSUED, MARK_LAST_LOAD_ISSUED, MARK_FIRST_FULL, MARK_LAST_MMA_ISSUED,
  MARK_ACC_READY, MARK_PARTIAL_WRITTEN, MARK_CLUSTER_SYNC1, MARK_REDUCED, MARK_CLUSTER_SYNC2, MARK_END, MARK_COUNT
};

constexpr int kUmmaStagingBytes = 4 * 4096;  // one 32-row x 128-byte store buffer per epilogue warp
// bytes of the ring that the epilogue needs: for split GEMMs the receive area -- per owned 128-byte
// output chunk one fp32 partial (128 rows x chunk columns) from every k-slice -- plus the store buffers
__host__ __device__ constexpr int umma_recv_bytes(int bn, int split, int elem) {
  return split > 1 ? ((bn * elem / 128 + split - 1) / split) * split * (128 / elem) * kUmmaBM * 4 : 0;
}
__host__ __device__ constexpr int umma_epilogue_bytes(int bn, int split, int elem) {
  return umma_recv_bytes(bn, split, elem) + kUmmaStagingBytes;
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map), "r"(src),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(PENDING) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// The epilogue of one warp: 32 rows x 128-byte chunks go through 128B-swizzled staging buffers and
// leave with one TMA store per chunk (full lines, clipped at the tensor's edges by the hardware).
// Chunks are staged in groups: one proxy fence, one warp barrier and one bulk group per GROUP of
// chunks, because each of those costs a few hundred nanoseconds of latency that a per-chunk
// sequence would pay serially.  With a buffer for every chunk of the warp nothing is ever waited
// for before the end; otherwise the buffers form two half-groups that alternate (one being filled
// while the other's stores read it).
template <int KIND>
struct ChunkWriter {
  const CUtensorMap *map_out;
  int M, N, causal;  // output rows / columns (clipping, mask) of the tensor the map describes
  uint32_t buf0;   // staging buffers of this warp (nbuf x 4096 bytes)
  int nbuf, lane, issued;  // issued: bulk groups committed so far
  int m_base, bz;  // first output row of this warp's 32 rows, batch index
  int n_tile0;     // first output column of the tile
  int nb_step;     // columns between consecutive chunks this warp writes
  int group;       // chunks per bulk group: nbuf (single group) or nbuf / 2
  // Output rows that are not 16-byte multiples cannot be described to the TMA: the staged chunks
  // then leave with 4-byte stores, 32 lanes writing 32 consecutive elements of one row (fp32 only).
  float *direct = nullptr;  // element (0, 0) of this batch entry's output matrix, or nullptr: TMA stores
  int slot = 0, pending = 0, first_nb = 0;

  __device__ __forceinline__ uint32_t begin_chunk() {
    if (!direct && pending == 0 && issued * group >= nbuf) {
      // the half-group about to be overwritten must have been read by its stores
      if (lane == 0) {
        if (group < nbuf) tma_store_wait_read<1>();
        else tma_store_wait_read<0>();
      }
      __syncwarp();
    }
    return buf0 + (uint32_t)slot * 4096u;
  }
  // 16 finished fp32 values of this lane's row: columns [nb + sub*16, +16) of the chunk at column nb;
  // bias_tile: this tile's slice of the bias vector in shared memory (zeros without a bias)
  __device__ __forceinline__ void put16(uint32_t buf, int sub, int nb, float (&v)[16], const float *bias_tile) {
    const int col0 = nb + sub * 16, m = m_base + lane;
    if (bias_tile) {
      // all four loads first: the shared-memory stores below are ordered asm statements, and a load
      // placed between them would wait out its latency there
      const float4 *b4 = reinterpret_cast<const float4 *>(bias_tile + (col0 - n_tile0));
      const float4 ba = b4[0], bb = b4[1], bc = b4[2], bd = b4[3];
      v[0] += ba.x, v[1] += ba.y, v[2] += ba.z, v[3] += ba.w;
      v[4] += bb.x, v[5] += bb.y, v[6] += bb.z, v[7] += bb.w;
      v[8] += bc.x, v[9] += bc.y, v[10] += bc.z, v[11] += bc.w;
      v[12] += bd.x, v[13] += bd.y, v[14] += bd.z, v[15] += bd.w;
    }
    if (causal && col0 + 15 > m) {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (col0 + j > m) v[j] = -FLT_MAX;
    }
    const uint32_t row = buf + (uint32_t)lane * 128u;
    if (KIND == 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j)
        st_shared_u4(row + (uint32_t)(((sub * 4 + j) ^ (lane & 7)) * 16), __float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]),
                     __float_as_uint(v[4 * j + 2]), __float_as_uint(v[4 * j + 3]));
    } else {
#pragma unroll
      for (int j = 0; j < 2; ++j)
        st_shared_u4(row + (uint32_t)(((sub * 2 + j) ^ (lane & 7)) * 16), f2_to_bf16x2(v[8 * j], v[8 * j + 1]),
                     f2_to_bf16x2(v[8 * j + 2], v[8 * j + 3]), f2_to_bf16x2(v[8 * j + 4], v[8 * j + 5]),
                     f2_to_bf16x2(v[8 * j + 6], v[8 * j + 7]));
    }
  }
  __device__ __forceinline__ void end_chunk(uint32_t buf, int nb) {
    (void)buf;
    if (pending == 0) first_nb = nb;
    ++pending;
    if (++slot == nbuf) slot = 0;
    if (pending == group) flush();
  }
  // hands the staged chunks to the TMA: every lane fences its own writes, lane 0 issues the stores
  __device__ __forceinline__ void flush() {
    if (pending == 0) return;
    if (direct) {
      __syncwarp();
      const int first_slot = (slot == 0 ? nbuf : slot) - pending;
      for (int i = 0; i < pending; ++i) {
        const int col = first_nb + i * nb_step + lane;
        const uint32_t b = buf0 + (uint32_t)(first_slot + i) * 4096u;
        if (col < N) {
#pragma unroll 4
          for (int row = 0; row < 32; ++row) {
            float v;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(b + (uint32_t)(row * 128 + (((lane >> 2) ^ (row & 7)) << 4) + ((lane & 3) << 2))) : "memory");
            if (m_base + row < M) direct[(size_t)(m_base + row) * N + col] = v;
          }
        }
      }
      __syncwarp();  // the buffers may be overwritten
      ++issued;
      pending = 0;
      return;
    }
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      const int first_slot = (slot == 0 ? nbuf : slot) - pending;
      for (int i = 0; i < pending; ++i) {
        const int nb = first_nb + i * nb_step;
        if (nb < N && m_base < M) tma_store_3d(map_out, buf0 + (uint32_t)(first_slot + i) * 4096u, nb, m_base, bz);
      }
      tma_store_commit();
    }
    ++issued;
    pending = 0;
  }
  __device__ __forceinline__ void finish() {
    flush();
    if (!direct && lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }
};

// staging buffers (per epilogue warp) and chunks per bulk group for `total` chunks when `free_bufs`
// buffers fit: a buffer per chunk in groups of two (the stores of one pair run while the next pair
// is staged, and nothing is reused), else two alternating half-groups of up to 4, else one buffer
__device__ __forceinline__ void staging_plan(int free_bufs, int total, int &nbuf, int &group) {
  if (free_bufs >= total) nbuf = total, group = min(2, total);
  else if (free_bufs >= 2) group = min(4, free_bufs / 2), nbuf = 2 * group;
  else nbuf = 1, group = 1;
}


// The cross-CTA reduction of a tile whose K range is split over the `split` CTAs of a cluster
// (k-slice = rank in the cluster); called by every thread of the operator after the MMAs.  The
// tile's 128-byte output chunks are dealt to the k-slices round-robin; `tiles` (the ring, idle by
// now) receives, per owned chunk, one fp32 partial from every k-slice, laid out
// [16-column group][quarter][row][4 floats].  After one cluster barrier (every k-slice has finished
// its MMAs, so every ring is free) each CTA pushes its partials straight from tensor memory into
// the owners' shared memory; an owner waits on its mbarrier, which counts the delivered bytes,
// sums the k-slices in order (deterministic) and stores the chunk through `w`.
template <int KIND>
__device__ __forceinline__ void umma_split_reduce(const TileCtx &c, int BN, int split, int kslice, uint32_t tiles, uint32_t recv_bar,
                                                  uint32_t tmem_row, bool acc_ok, ChunkWriter<KIND> &w, int n0,
                                                  const float *bias_tile, long long *tl) {
  constexpr int kElem = KIND == 0 ? 4 : 2, kOutCols = 128 / kElem, kSub = kOutCols / 16;
  constexpr uint32_t kChunkPartial = (uint32_t)kOutCols * kUmmaBM * 4;
  const int warp = c.tid >> 5, lane = c.tid & 31, quad = (threadIdx.x >> 5) & 3;
  const int chunks = BN / kOutCols, max_owned = (chunks + split - 1) / split;
  auto mark = [&](int what, bool who) {
    if (tl && who) tl[what] = (long long)global_ns();
  };
  cluster_sync_all();
  mark(MARK_CLUSTER_SYNC1, c.tid == 0);
  if (warp >= 4) return;
  const int row = quad * 32 + lane;
  if (acc_ok) {
#pragma unroll 1
    for (int cc = 0; cc < BN / 16; cc += 2) {
      uint32_t r0[16], r1[16];
      tmem_ld_32x16(tmem_row + cc * 16, r0);
      tmem_ld_32x16(tmem_row + (cc + 1) * 16, r1);
      tmem_ld_wait();
      const int ch = cc / kSub, owner = ch % split;
      const uint32_t slot = tiles + (uint32_t)((ch / split) * split + kslice) * kChunkPartial;
      const uint32_t dst0 = peer_smem(slot + (uint32_t)((((cc % kSub) * 4) * kUmmaBM + row) * 16), (uint32_t)owner);
      const uint32_t dst1 = dst0 + 4u * kUmmaBM * 16u;
      const uint32_t bar = peer_smem(recv_bar, (uint32_t)owner);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        st_async_u4(dst0 + (uint32_t)(j * kUmmaBM * 16), bar, r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]);
        st_async_u4(dst1 + (uint32_t)(j * kUmmaBM * 16), bar, r1[4 * j], r1[4 * j + 1], r1[4 * j + 2], r1[4 * j + 3]);
      }
    }
  }
  mark(MARK_PARTIAL_WRITTEN, c.tid == 0);
  // all partials of the chunks this CTA owns have landed (a CTA that owns none expected no bytes)
  int owned = 0;
  for (int ch = kslice; ch < chunks; ch += split) ++owned;
  const bool got = owned == 0 || mbar_wait(recv_bar, 0, c.status, UMMA_WAIT_PEERS_TIMEOUT);
  mark(MARK_CLUSTER_SYNC2, c.tid == 0);
  if (got) {
#pragma unroll 1
    for (int li = 0; li < max_owned; ++li) {
      const int ch = li * split + kslice;
      if (ch >= chunks) break;
      const uint32_t buf = w.begin_chunk();
#pragma unroll 1
      for (int sub = 0; sub < kSub; ++sub) {
        float acc[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j] = 0.f;
#pragma unroll 1
        for (int peer = 0; peer < split; ++peer) {  // k-slice order: the sum is deterministic
          const uint32_t src = tiles + (uint32_t)(li * split + peer) * kChunkPartial + (uint32_t)(((sub * 4) * kUmmaBM + row) * 16);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 v = ld_shared_f4(src + (uint32_t)(j * kUmmaBM * 16));
            acc[4 * j] += v.x, acc[4 * j + 1] += v.y, acc[4 * j + 2] += v.z, acc[4 * j + 3] += v.w;
          }
        }
        w.put16(buf, sub, n0 + ch * kOutCols, acc, bias_tile);
      }
      w.end_chunk(buf, n0 + ch * kOutCols);
    }
    w.finish();
  }
  mark(MARK_REDUCED, c.tid == 0);
}

template <int KIND>
struct GemmUmma {
  using Params = GemmUmmaParams;
  static constexpr int kMaxThreads = kUmmaThreads;
  static constexpr int kMinBlocks = 1;
  static constexpr bool kMemoryBound = false;
  static constexpr bool kUsesTmem = true;   // allocates tensor memory (see fused_block_kernel)
  static constexpr int kElem = KIND == 0 ? 4 : 2;
  static constexpr int kBK = kUmmaRowBytes / kElem;  // K elements per stage
  static constexpr int kOutCols = 128 / kElem;       // output columns per 128-byte store chunk
  static constexpr int kSub = kOutCols / 16;         // 16-column accumulator reads per chunk

  // The MMA issue loop of one k-slice, run by a single thread.  TALL: 256-row tile -- rows 128..255
  // of A (16 KB further on in the stage) against the same W tile into a second accumulator BN
  // columns on.  A separate instantiation keeps the common loop free of the extra branch and of a
  // run-time W offset: it is a chain of dependent instructions whose length sets the MMA rate of
  // narrow tiles.  Returns false when a wait gave up.
  template <bool TALL>
  __device__ __forceinline__ static bool issue_mmas(const TileCtx &c, uint32_t tiles, int stage_bytes, int stages, int num_kb,
                                                    uint32_t full0, uint32_t empty0, uint32_t tmem_acc, uint32_t idesc, int bn,
                                                    long long *tl) {
    // low descriptor word of stage 0; a stage is stage_bytes / 16 further on
    const uint32_t lo0 = ((tiles >> 4) & 0x3fffu) | (1u << 16), stage16 = (uint32_t)stage_bytes >> 4;
    constexpr uint32_t b_off = (uint32_t)(TALL ? 2 : 1) * (kUmmaABytes >> 4);
    uint32_t s = 0, ph = 0, lo = lo0, accumulate = 0;
    for (int kb = 0; kb < num_kb; ++kb) {
      if (!mbar_wait(full0 + 8 * s, ph, c.status, UMMA_WAIT_FULL_TIMEOUT)) return false;
      tc_fence_after();
      if (kb == 0 && tl) tl[MARK_FIRST_FULL] = (long long)global_ns();
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // 4 x 32 bytes of K per stage; +2 = 32 bytes in descriptor units
        umma_ss<KIND>(tmem_acc, lo + 2 * j, lo + b_off + 2 * j, idesc, accumulate);
        if (TALL) umma_ss<KIND>(tmem_acc + (uint32_t)bn, lo + (kUmmaABytes >> 4) + 2 * j, lo + b_off + 2 * j, idesc, accumulate);
        accumulate = 1;
      }
      umma_commit(empty0 + 8 * s);  // frees the stage once these MMAs have read it
      if (++s == (uint32_t)stages) s = 0, ph ^= 1, lo = lo0;
      else lo += stage16;
    }
    return true;
  }

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    const int warp = c.tid >> 5, lane = c.tid & 31;
    const int quad = (threadIdx.x >> 5) & 3;  // hardware warp w may only touch TMEM lanes [32 * (w % 4), +32)
    const int BN = p.bn, BM = p.bm, halves = BM / kUmmaBM, kABytes = BM * kUmmaRowBytes, kStageBytes = umma_stage_bytes(BN, BM);
    const uint32_t idesc = umma_idesc(KIND, BN);
    const int split = p.split, kslice = c.block_x() % split;
    // M tiles vary fastest: the (usually few) CTAs that share a W tile are launched next to each
    // other, so the tile is fetched from HBM once and the others hit L2
    const int m0 = (c.block_x() / split) * BM, n0 = c.block_y() * BN, bz = c.block_z();
    const int stages = p.stages;
    const int chunks = BN / kOutCols;

    // operator window: [0,1024) barriers + tmem pointer, then `stages` x (A tile, B tile); once the
    // MMAs are done the ring holds the partial tile (split GEMMs) and the store buffers
    uint64_t *bars = reinterpret_cast<uint64_t *>(c.smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kUmmaMaxStages, acc_bar = empty0 + 8 * kUmmaMaxStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c.smem + 8 * (2 * kUmmaMaxStages + 2));
    // Tensor memory first: the SM starts its next CTA of this kernel only when this one has given up
    // its permit to allocate, so every instruction before that delays a co-resident CTA.  A tile
    // entirely above the diagonal of a causal product needs no accumulator.
    const bool masked_tile = p.causal && n0 > m0 + BM - 1;
    if (warp == 5) {
      if (!c.tmem_given) {   // (a persistent CTA of the work queue holds its columns already)
        if (!masked_tile) tmem_alloc(smem_u32(tmem_slot), BN * halves);
        if (!c.persistent) tmem_relinquish();
      }
    }
    const uint32_t tiles = smem_u32(c.smem) + kUmmaHeaderBytes;
    const uint32_t recv_bar = acc_bar + 8;                                  // counts partial sums delivered by peers
    float *bias_tile = reinterpret_cast<float *>(c.smem + 1024);            // BN floats
    const int max_owned = (chunks + split - 1) / split;                     // store chunks a k-slice finishes
    constexpr uint32_t kChunkPartial = (uint32_t)kOutCols * kUmmaBM * 4;    // fp32 partial of one chunk from one k-slice
    const uint32_t staging = tiles + (uint32_t)umma_recv_bytes(BN, split, kElem);
    // store buffers per epilogue warp, as many as the idle ring has room for (see staging_plan)
    const int free_bufs = (stages * kStageBytes - (int)(staging - tiles)) / kUmmaStagingBytes;
    int nbuf, group;
    staging_plan(free_bufs, max_owned, nbuf, group);
    ChunkWriter<KIND> w{&p.map_out, p.M, p.N, p.causal, staging + (uint32_t)(quad * nbuf) * 4096u, nbuf, lane, 0, m0 + quad * 32, bz, n0,
                        split * kOutCols, group};
    long long *const tl = (p.timeline && c.vblock == 0) ? p.timeline : nullptr;
    auto mark = [&](int what, bool who) {
      if (tl && who) tl[what] = (long long)global_ns();
    };
    mark(MARK_START, c.tid == 0);

    if (masked_tile) {
      c.dependency_wait();
      // tile entirely above the diagonal (for every k-slice of it): only the mask value to write;
      // k-slice 0 fills one buffer once and stores it to every chunk
      if (warp < 4 && kslice == 0) {
        const uint32_t buf = w.begin_chunk();
        const uint32_t mask = KIND == 0 ? __float_as_uint(-FLT_MAX) : f2_to_bf16x2(-FLT_MAX, -FLT_MAX);
#pragma unroll
        for (int j = 0; j < 8; ++j) st_shared_u4(buf + (uint32_t)lane * 128u + j * 16, mask, mask, mask, mask);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          for (int h = 0; h < halves; ++h) {
            const int mb = w.m_base + h * kUmmaBM;
            for (int ch = 0; ch < chunks && mb < p.M; ++ch)
              if (n0 + ch * kOutCols < p.N) tma_store_3d(&p.map_out, buf, n0 + ch * kOutCols, mb, bz);
          }
          tma_store_commit();
        }
        w.finish();
      }
      return;
    }

    const int total_kb = (p.K + kBK - 1) / kBK;
    const int kb0 = kslice * p.kb_per_slice;                 // first K block of this k-slice
    const int num_kb = min(p.kb_per_slice, total_kb - kb0);  // K blocks this CTA multiplies (>= 1)

    // The producer warp sets the barriers up itself and starts the first ring pass (every slot is
    // free, nothing to wait for) before the CTA-wide barrier, so the first operands are already on
    // their way from HBM while warp 5 allocates tensor memory.
    const int npre = min(stages, num_kb);
    if (warp == 4) {
      if (lane < stages) {
        mbar_init(full0 + 8 * lane, 1);
        mbar_init(empty0 + 8 * lane, 1);
      }
      if (lane == 0) {
        mbar_init(acc_bar, 1);
        mbar_init(recv_bar, 1);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_b) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_out) : "memory");
        if (split > 1) {
          // bytes this CTA will receive: one partial per owned chunk from every k-slice (itself included)
          int owned = 0;
          for (int ch = kslice; ch < chunks; ch += split) ++owned;
          mbar_expect_tx(recv_bar, (uint32_t)owned * (uint32_t)split * kChunkPartial);
        }
      }
      c.dependency_wait();   // all of the above ran while the previous kernel drained; the loads below read its output
      if (elect_one()) {
        for (int kb = 0; kb < npre; ++kb) {
          const uint32_t dst = tiles + kb * kStageBytes, bar = full0 + 8 * kb;
          mbar_expect_tx(bar, kStageBytes);
          tma_load_3d(dst, &p.map_a, bar, (kb0 + kb) * kBK, m0, bz);
          tma_load_3d(dst + kABytes, &p.map_b, bar, (kb0 + kb) * kBK, n0, bz);
          if (kb == 0) mark(MARK_FIRST_LOAD_ISSUED, true);
        }
      }
      __syncwarp();
    } else {
      c.dependency_wait();
    }
    tc_fence_before();
    c.sync();
    tc_fence_after();
    const uint32_t tmem_acc = c.tmem_given ? c.tmem_base : *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t tmem_row = tmem_acc + ((uint32_t)(quad * 32) << 16);
    mark(MARK_SETUP_DONE, c.tid == 0);

    // The producer and the MMA issuer are ONE elected thread each (elect.sync, so the compiler knows
    // the branch is taken by a single thread and keeps descriptors in uniform registers).  Their
    // loops carry the ring slot, its phase and the low descriptor word incrementally: the issue
    // loop is a chain of dependent instructions on one thread, and every instruction saved in it is
    // time the tensor pipe does not idle (4 MMAs of N <= 128 execute faster than a careless loop
    // iteration issues them).  The other lanes wait at the __syncwarp below.
    bool acc_ok = true;
    if (warp == 4) {
      if (elect_one()) {
        // second and later ring passes (the first was issued before the barrier): slot 0 again
        uint32_t s = 0, ph = 0, dst = tiles, bar = full0;
        int kcoord = (kb0 + npre) * kBK;
        for (int kb = npre; kb < num_kb; ++kb) {
          if (!mbar_wait(empty0 + 8 * s, ph, c.status, UMMA_WAIT_EMPTY_TIMEOUT)) break;
          mbar_expect_tx(bar, kStageBytes);
          tma_load_3d(dst, &p.map_a, bar, kcoord, m0, bz);
          tma_load_3d(dst + kABytes, &p.map_b, bar, kcoord, n0, bz);
          kcoord += kBK;
          if (++s == (uint32_t)stages) s = 0, ph ^= 1, dst = tiles, bar = full0;
          else dst += kStageBytes, bar += 8;
        }
        mark(MARK_LAST_LOAD_ISSUED, true);
      }
      __syncwarp();
    } else if (warp == 5) {
      if (elect_one()) {
        bool ok = halves == 2 ? issue_mmas<true>(c, tiles, kStageBytes, stages, num_kb, full0, empty0, tmem_acc, idesc, BN, tl)
                              : issue_mmas<false>(c, tiles, kStageBytes, stages, num_kb, full0, empty0, tmem_acc, idesc, BN, tl);
        umma_commit(acc_bar);  // accumulator complete (also arrives if the loop bailed out)
        mark(MARK_LAST_MMA_ISSUED, true);
        // The stage-release arrivals of the last ring pass are asynchronous and nobody consumes them;
        // wait for them here so that none is still in flight when the barriers are invalidated and
        // the shared memory is handed to the next tile or the next CTA.
        for (int kb = max(0, num_kb - stages); kb < num_kb && ok; ++kb)
          ok = mbar_wait(empty0 + 8 * (kb % stages), (kb / stages) & 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT);
      }
      __syncwarp();
    } else {
      // the epilogue warps are idle during the main loop: they fetch the tile's bias slice meanwhile
      // (only they read it, after their own named-barrier-free hand-off below)
      for (int i = c.tid; i < BN; i += 128) bias_tile[i] = (p.bias && n0 + i < p.N) ? __ldg(p.bias + n0 + i) : 0.f;
      asm volatile("bar.sync %0, 128;" ::"r"(c.bar_id + 8) : "memory");  // the four epilogue warps only (ids 9 / 10)
      acc_ok = mbar_wait(acc_bar, 0, c.status, UMMA_WAIT_ACC_TIMEOUT);
      tc_fence_after();
      mark(MARK_ACC_READY, c.tid == 0);
      if (acc_ok && split == 1) {
#pragma unroll 1
        for (int h = 0; h < halves; ++h) {  // accumulator h holds output rows [m0 + 128 h, +128)
          const uint32_t trow = tmem_row + (uint32_t)(h * BN);
          w.m_base = m0 + h * kUmmaBM + quad * 32;
#pragma unroll 1
          for (int ch = 0; ch < chunks; ++ch) {
            const uint32_t buf = w.begin_chunk();
#pragma unroll
            for (int sub = 0; sub < kSub; sub += 2) {  // two accumulator reads in flight per wait
              uint32_t r0[16], r1[16];
              tmem_ld_32x16(trow + (ch * kSub + sub) * 16, r0);
              tmem_ld_32x16(trow + (ch * kSub + sub + 1) * 16, r1);
              tmem_ld_wait();
              float v[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r0[j]);
              w.put16(buf, sub, n0 + ch * kOutCols, v, bias_tile);
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r1[j]);
              w.put16(buf, sub + 1, n0 + ch * kOutCols, v, bias_tile);
            }
            w.end_chunk(buf, n0 + ch * kOutCols);
          }
          w.flush();  // a group never spans two row blocks
        }
        w.finish();
        mark(MARK_PARTIAL_WRITTEN, c.tid == 0);
      }
    }
    if (split > 1) umma_split_reduce<KIND>(c, BN, split, kslice, tiles, recv_bar, tmem_row, acc_ok, w, n0, bias_tile, tl);
    tc_fence_before();
    c.sync();
    if (warp == 5 && !c.tmem_given) tmem_dealloc(tmem_acc, BN * halves);
    if (c.persistent && c.tid < stages) {  // the next tile of a persistent CTA initialises them again
      mbar_inval(full0 + 8 * c.tid);
      mbar_inval(empty0 + 8 * c.tid);
      if (c.tid == 0) {
        mbar_inval(acc_bar);
        mbar_inval(recv_bar);
      }
    }
    mark(MARK_END, c.tid == 0);
  }
};

}  // namespace bfuse
