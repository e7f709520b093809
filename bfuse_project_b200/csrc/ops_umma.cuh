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
  alignas(64) CUtensorMap map_a;    // {K, M, batch}, box {128 B of K, 128, 1}, 128B swizzle
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

// The epilogue of one warp: 32 rows x 128-byte chunks go through a 128B-swizzled staging buffer
// and leave with one TMA store per chunk (full lines, clipped at the M / N edges by the hardware).
// The epilogue of one warp: 32 rows x 128-byte chunks go through a 128B-swizzled staging buffer and
// leave with one TMA store per chunk (full lines, clipped at the tensor's edges by the hardware).
template <int KIND>
struct ChunkWriter {
  const CUtensorMap *map_out;
  int M, N, causal;  // output rows / columns (clipping, mask) of the tensor the map describes
  uint32_t buf0;   // staging buffers of this warp (nbuf x 4096 bytes)
  int nbuf, lane, issued;
  int m_base, bz;  // first output row of this warp's 32 rows, batch index
  int n_tile0;     // first output column of the tile

  // nbuf is 1, 2, or at least the number of chunks this warp will ever write (then no buffer is
  // reused and nothing has to be waited for)
  __device__ __forceinline__ uint32_t begin_chunk() {
    if (issued >= nbuf) {  // the buffer about to be overwritten must have been read by its store
      if (lane == 0) {
        if (nbuf == 2) tma_store_wait_read<1>();
        else tma_store_wait_read<0>();
      }
      __syncwarp();
    }
    return buf0 + (uint32_t)(issued % nbuf) * 4096u;
  }
  // 16 finished fp32 values of this lane's row: columns [nb + sub*16, +16) of the chunk at column nb;
  // bias_tile: this tile's slice of the bias vector in shared memory (zeros without a bias)
  __device__ __forceinline__ void put16(uint32_t buf, int sub, int nb, float (&v)[16], const float *bias_tile) {
    const int col0 = nb + sub * 16, m = m_base + lane;
    if (bias_tile) {
      const float4 *b4 = reinterpret_cast<const float4 *>(bias_tile + (col0 - n_tile0));
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float4 b = b4[j];
        v[4 * j] += b.x, v[4 * j + 1] += b.y, v[4 * j + 2] += b.z, v[4 * j + 3] += b.w;
      }
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
    fence_async_smem();
    __syncwarp();
    if (lane == 0) {
      if (nb < N && m_base < M) tma_store_3d(map_out, buf, nb, m_base, bz);
      // one group per chunk, even an empty one for a chunk that lies outside the tensor: begin_chunk
      // counts groups to know when a staging buffer may be overwritten
      tma_store_commit();
    }
    ++issued;
  }
  __device__ __forceinline__ void finish() {
    if (lane == 0) tma_store_wait_read<0>();
    __syncwarp();
  }
};


// chunks one epilogue warp writes: all of the tile's chunks, or the owned share of a split tile
__device__ __forceinline__ int max_owned_or_all(int chunks, int split) { return (chunks + split - 1) / split; }

template <int KIND>
struct GemmUmma {
  using Params = GemmUmmaParams;
  static constexpr int kMaxThreads = kUmmaThreads;
  static constexpr int kMinBlocks = 1;
  static constexpr bool kMemoryBound = false;
  static constexpr int kElem = KIND == 0 ? 4 : 2;
  static constexpr int kBK = kUmmaRowBytes / kElem;  // K elements per stage
  static constexpr int kOutCols = 128 / kElem;       // output columns per 128-byte store chunk
  static constexpr int kSub = kOutCols / 16;         // 16-column accumulator reads per chunk

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    const int warp = c.tid >> 5, lane = c.tid & 31;
    const int quad = (threadIdx.x >> 5) & 3;  // hardware warp w may only touch TMEM lanes [32 * (w % 4), +32)
    const int BN = p.bn, kStageBytes = umma_stage_bytes(BN);
    const uint32_t idesc = umma_idesc(KIND, BN);
    const int split = p.split, kslice = c.block_x() % split;
    // M tiles vary fastest: the (usually few) CTAs that share a W tile are launched next to each
    // other, so the tile is fetched from HBM once and the others hit L2
    const int m0 = (c.block_x() / split) * kUmmaBM, n0 = c.block_y() * BN, bz = c.block_z();
    const int stages = p.stages;
    const int chunks = BN / kOutCols;

    // operator window: [0,1024) barriers + tmem pointer, then `stages` x (A tile, B tile); once the
    // MMAs are done the ring holds the partial tile (split GEMMs) and the store buffers
    uint64_t *bars = reinterpret_cast<uint64_t *>(c.smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kUmmaMaxStages, acc_bar = empty0 + 8 * kUmmaMaxStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c.smem + 8 * (2 * kUmmaMaxStages + 2));
    const uint32_t tiles = smem_u32(c.smem) + kUmmaHeaderBytes;
    const uint32_t recv_bar = acc_bar + 8;                                  // counts partial sums delivered by peers
    float *bias_tile = reinterpret_cast<float *>(c.smem + 1024);            // BN floats
    const int max_owned = (chunks + split - 1) / split;                     // store chunks a k-slice finishes
    constexpr uint32_t kChunkPartial = (uint32_t)kOutCols * kUmmaBM * 4;    // fp32 partial of one chunk from one k-slice
    const uint32_t staging = tiles + (uint32_t)umma_recv_bytes(BN, split, kElem);
    // store buffers per epilogue warp: one per chunk when the idle ring has the room (no waits at
    // all), else two (double buffering), else one
    const int free_bufs = (stages * kStageBytes - (int)(staging - tiles)) / kUmmaStagingBytes;
    const int nbuf = free_bufs >= max_owned_or_all(chunks, split) ? max_owned_or_all(chunks, split) : (free_bufs >= 2 ? 2 : 1);
    ChunkWriter<KIND> w{&p.map_out, p.M, p.N, p.causal, staging + (uint32_t)(quad * nbuf) * 4096u, nbuf, lane, 0, m0 + quad * 32, bz, n0};
    long long *const tl = (p.timeline && c.vblock == 0) ? p.timeline : nullptr;
    auto mark = [&](int what, bool who) {
      if (tl && who) tl[what] = (long long)global_ns();
    };
    mark(MARK_START, c.tid == 0);

    if (p.causal && n0 > m0 + kUmmaBM - 1) {
      // tile entirely above the diagonal (for every k-slice of it): only the mask value to write;
      // k-slice 0 fills one buffer once and stores it to every chunk
      if (warp < 4 && kslice == 0) {
        const uint32_t buf = w.begin_chunk();
        const uint32_t mask = KIND == 0 ? __float_as_uint(-FLT_MAX) : f2_to_bf16x2(-FLT_MAX, -FLT_MAX);
#pragma unroll
        for (int j = 0; j < 8; ++j) st_shared_u4(buf + (uint32_t)lane * 128u + j * 16, mask, mask, mask, mask);
        fence_async_smem();
        __syncwarp();
        if (lane == 0 && w.m_base < p.M) {
          for (int ch = 0; ch < chunks; ++ch)
            if (n0 + ch * kOutCols < p.N) tma_store_3d(&p.map_out, buf, n0 + ch * kOutCols, w.m_base, bz);
          tma_store_commit();
        }
        w.finish();
      }
      return;
    }

    const int total_kb = (p.K + kBK - 1) / kBK;
    const int kb0 = kslice * p.kb_per_slice;                 // first K block of this k-slice
    const int num_kb = min(p.kb_per_slice, total_kb - kb0);  // K blocks this CTA multiplies (>= 1)

    if (c.tid == 0) {
      for (int s = 0; s < stages; ++s) {
        mbar_init(full0 + 8 * s, 1);
        mbar_init(empty0 + 8 * s, 1);
      }
      mbar_init(acc_bar, 1);
      mbar_init(recv_bar, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      if (split > 1) {
        // bytes this CTA will receive: one partial per owned chunk from every k-slice (itself included)
        int owned = 0;
        for (int ch = kslice; ch < chunks; ch += split) ++owned;
        mbar_expect_tx(recv_bar, (uint32_t)owned * (uint32_t)split * kChunkPartial);
      }
    }
    if (warp == 5) {
      tmem_alloc(smem_u32(tmem_slot), BN);
      if (!c.persistent) tmem_relinquish();
    } else if (warp == 4 && lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_b) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_out) : "memory");
    }
    tc_fence_before();
    c.sync();
    tc_fence_after();
    const uint32_t tmem_acc = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t tmem_row = tmem_acc + ((uint32_t)(quad * 32) << 16);
    mark(MARK_SETUP_DONE, c.tid == 0);

    // Producer and MMA warps run their loops with all 32 lanes (so the warp reaches the closing
    // barrier converged); lane 0 alone issues the copies / MMAs.
    bool acc_ok = true;
    if (warp == 4) {
      bool ok = true;
      for (int kb = 0; kb < num_kb && ok; ++kb) {
        const int s = kb % stages;
        const uint32_t ph = (kb / stages) & 1;
        ok = mbar_wait(empty0 + 8 * s, ph ^ 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT);
        if (ok && lane == 0) {
          mbar_expect_tx(full0 + 8 * s, kStageBytes);
          const uint32_t a_dst = tiles + s * kStageBytes;
          tma_load_3d(a_dst, &p.map_a, full0 + 8 * s, (kb0 + kb) * kBK, m0, bz);
          tma_load_3d(a_dst + kUmmaABytes, &p.map_b, full0 + 8 * s, (kb0 + kb) * kBK, n0, bz);
          if (kb == 0) mark(MARK_FIRST_LOAD_ISSUED, true);
          if (kb == num_kb - 1) mark(MARK_LAST_LOAD_ISSUED, true);
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
        if (kb == 0) mark(MARK_FIRST_FULL, lane == 0);
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
      mark(MARK_LAST_MMA_ISSUED, lane == 0);
      __syncwarp();
      // The stage-release arrivals of the last ring pass are asynchronous and nobody consumes them;
      // wait for them here so that none is still in flight when the barriers are invalidated and
      // the shared memory is handed to the next tile or the next CTA.
      for (int kb = max(0, num_kb - stages); kb < num_kb && ok; ++kb)
        ok = mbar_wait(empty0 + 8 * (kb % stages), (kb / stages) & 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT);
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
        for (int ch = 0; ch < chunks; ++ch) {
          const uint32_t buf = w.begin_chunk();
#pragma unroll
          for (int sub = 0; sub < kSub; sub += 2) {  // two accumulator reads in flight per wait
            uint32_t r0[16], r1[16];
            tmem_ld_32x16(tmem_row + (ch * kSub + sub) * 16, r0);
            tmem_ld_32x16(tmem_row + (ch * kSub + sub + 1) * 16, r1);
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
        w.finish();
        mark(MARK_PARTIAL_WRITTEN, c.tid == 0);
      }
    }
    if (split > 1) {
      // (A) every k-slice of the tile has finished its MMAs, so every ring in the cluster is free
      cluster_sync_all();
      mark(MARK_CLUSTER_SYNC1, c.tid == 0);
      if (warp < 4) {
        const int row = quad * 32 + lane;
        if (acc_ok) {
          // push: chunk ch belongs to k-slice ch % split; its receive slot for this k-slice's partial
          // is [ch / split][kslice], laid out [16-column group][quarter][row][4 floats]
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
        // (B) all partials of the chunks this CTA owns have landed
        const bool got = mbar_wait(recv_bar, 0, c.status, UMMA_WAIT_PEERS_TIMEOUT);
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
      mbar_inval(recv_bar);
    }
    mark(MARK_END, c.tid == 0);
  }
};

}  // namespace bfuse
