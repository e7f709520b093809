// NCHW convolution as an implicit GEMM on the tensor cores (tcgen05, kind::tf32), the operator of
// the reference's conv2d kernels (tests/benchmark/cuda/conv2d*.cu; files/resnet-18.txt:31,36).
//
//   y[n, co, pixel] = sum_k  w[co, k] * im2col(x)[n, pixel, k],   k = (ci, kh, kw) as in w[co][ci][kh][kw]
//
// A tile is 128 output channels x BN output pixels of one image (BN = 128, or 64 / 32 for small
// images, so that a single image still spreads over many SMs).  The weight operand is K-major in
// global memory and arrives by TMA (128B swizzle).  The im2col operand does not exist in memory:
// the four epilogue warps, idle during the main loop, gather it (128 / BN threads per output pixel,
// 32 values of k per pixel and stage) with 4-byte cp.async copies straight into the swizzled K-major layout the
// MMA expects (out-of-image taps are zero-filled by the copy itself), and each thread's
// cp.async.mbarrier.arrive makes the stage's "full" barrier fire when its copies have landed, so
// the gather runs several stages ahead of the tensor core.  Per-k input offsets and tap coordinates
// are tabulated once per CTA in shared memory, so the gather does no divisions.
//
// A long K (deep layers on small images leave few tiles) can be split over the CTAs of a cluster,
// reduced through distributed shared memory like the GEMM's k-slices.
//
// BlockDim = (192, 1, 1); GridDim = (split * ceil(oh*ow / BN), ceil(co / 128), n).
#pragma once

#include "ops_umma.cuh"

namespace bfuse {

constexpr int kConvBN = 128;                 // output pixels per tile, at most
constexpr int kConvMaxK = 8192;              // ci * kh * kw the offset table may hold (64 KB of shared memory)
// header of the operator window: barriers etc., then the offset table -- int2 {input offset, tap
// index dy*kw+dx} per k, K rounded up to whole K blocks (tap 31 = padding) and to 1 KB
__host__ __device__ constexpr int conv_header_bytes(int K) { return kUmmaHeaderBytes + ((K + 31) / 32 * 32 * 8 + 1023) / 1024 * 1024; }
__host__ __device__ constexpr int conv_stage_bytes(int bn = kConvBN) { return kUmmaABytes + bn * kUmmaRowBytes; }
__host__ __device__ constexpr int conv_umma_smem_bytes(int stages, int bn, int K) {
  return conv_header_bytes(K) + stages * conv_stage_bytes(bn);
}

struct ConvUmmaParams {
  alignas(64) CUtensorMap map_w;    // {K, co, 1}, box {32 fp32, 128, 1}, 128B swizzle
  alignas(64) CUtensorMap map_out;  // {oh*ow, co, n}, box {32 fp32, 32, 1}, 128B swizzle (stores); unused when oh*ow % 4 != 0
  float *y;                         // [n, co, oh*ow]: the output rows, for images whose rows are not 16-byte multiples
  const float *x;
  int n, ci, h, wd, co, kh, kw, stride, pad, oh, ow;
  int K;
  int stages;
  int bn;               // output pixels per tile: 32, 64 or 128
  int split;            // CTAs (k-slices) per tile = cluster width; 1: no split
  int kb_per_slice;     // K blocks per k-slice
  long long *timeline;  // diagnostic: when non-null, CTA 0 records globaltimer marks (UmmaMark indices)
};

// 4-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros instead
__device__ __forceinline__ void cp_async_4(uint32_t dst, const float *src, uint32_t src_bytes) {
  // no "memory" clobber on purpose: nothing reads the destination through C++ pointers, and the
  // clobber would serialise the table look-ups of neighbouring elements behind every copy
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes));
}
// arrive on `bar` once all cp.async copies issued so far by this thread have completed
__device__ __forceinline__ void cp_async_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

struct ConvUmmaTf32 {
  using Params = ConvUmmaParams;
  static constexpr int kMaxThreads = kUmmaThreads;
  static constexpr int kMinBlocks = 1;
  static constexpr bool kMemoryBound = false;
  static constexpr bool kUsesTmem = true;   // allocates tensor memory (see fused_block_kernel)
  static constexpr int kBK = 32;  // K elements (fp32) per stage row of 128 bytes

  // The im2col gather of one tile by the four epilogue warps (gt = 0..127): 128 / BN threads share a
  // row (one output pixel) of every stage's tile; consecutive lanes take consecutive pixels, thread
  // `sub` of a row its sub-th share of the stage's 32 values of k.  A template on BN: the loop is
  // bound by the issue rate of its copies, and run-time tile arithmetic in it costs a few percent.
  template <int BN>
  __device__ __forceinline__ static bool gather(const Params &p, const TileCtx &c, int gt, int px0, int img, int num_kb, int stages,
                                                uint32_t tiles, uint32_t full0, uint32_t empty0, const int2 *tab, long long *tl) {
    constexpr int kStageBytes = conv_stage_bytes(BN), kper = kBK * BN / 128;
    const int r = gt & (BN - 1), sub = gt / BN, pix = px0 + r, ohw = p.oh * p.ow;
    const bool live = pix < ohw;
    const int oy = pix / p.ow, ox = pix % p.ow;
    const int iy0 = oy * p.stride - p.pad, ix0 = ox * p.stride - p.pad;
    const float *xb = p.x + (size_t)img * p.ci * p.h * p.wd + (ptrdiff_t)iy0 * p.wd + ix0;
    // which taps of the window fall inside the image for this pixel (bit dy*kw+dx; none for a dead row)
    uint32_t tapmask = 0;
    if (live)
      for (int dy = 0; dy < p.kh; ++dy)
        for (int dx = 0; dx < p.kw; ++dx)
          if (iy0 + dy >= 0 && iy0 + dy < p.h && ix0 + dx >= 0 && ix0 + dx < p.wd) tapmask |= 1u << (dy * p.kw + dx);
    for (int kb = 0; kb < num_kb; ++kb) {
      const int s = kb % stages;
      if (!mbar_wait(empty0 + 8 * s, ((kb / stages) & 1) ^ 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT)) return false;
      const uint32_t brow = tiles + s * kStageBytes + kUmmaABytes + (uint32_t)r * 128u;
#pragma unroll
      for (int e0 = sub * kper; e0 < (sub + 1) * kper; e0 += 8) {
        // look the 8 taps up first (the shared-memory reads overlap), then issue the 8 copies
        const float *src[8];
        uint32_t bytes[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int2 t = tab[kb * kBK + e0 + i];
          const bool in = (tapmask >> t.y) & 1u;
          src[i] = in ? xb + t.x : p.x;
          bytes[i] = in ? 4u : 0u;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i)
          cp_async_4(brow + (uint32_t)(((((e0 + i) >> 2) ^ (r & 7)) << 4) + (((e0 + i) & 3) << 2)), src[i], bytes[i]);
      }
      cp_async_arrive(full0 + 8 * s);
      if (tl && gt == 0 && kb == 0) tl[MARK_FIRST_LOAD_ISSUED] = (long long)global_ns();
      if (tl && gt == 0 && kb == num_kb - 1) tl[MARK_LAST_LOAD_ISSUED] = (long long)global_ns();
    }
    return true;
  }

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    const int warp = c.tid >> 5, lane = c.tid & 31;
    const int quad = (threadIdx.x >> 5) & 3;
    const int BN = p.bn, kStageBytes = conv_stage_bytes(BN);
    const int split = p.split, kslice = c.block_x() % split;
    const int px0 = (c.block_x() / split) * BN, co0 = c.block_y() * kUmmaBM, img = c.block_z();
    const int stages = p.stages, ohw = p.oh * p.ow, K = p.K;
    const int total_kb = (K + kBK - 1) / kBK;
    const int kb0 = kslice * p.kb_per_slice;                  // first K block of this k-slice
    const int num_kb = min(p.kb_per_slice, total_kb - kb0);   // K blocks this CTA multiplies (>= 1)
    const uint32_t idesc = umma_idesc(0, BN);

    uint64_t *bars = reinterpret_cast<uint64_t *>(c.smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kUmmaMaxStages, acc_bar = empty0 + 8 * kUmmaMaxStages;
    const uint32_t recv_bar = acc_bar + 8;  // counts partial sums delivered by the other k-slices
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c.smem + 8 * (2 * kUmmaMaxStages + 2));
    // tensor memory first: the SM starts its next CTA of this kernel only once this one has given up
    // its permit to allocate
    if (warp == 5) {
      tmem_alloc(smem_u32(tmem_slot), BN);
      if (!c.persistent) tmem_relinquish();
    }
    int2 *tab = reinterpret_cast<int2 *>(c.smem + kUmmaHeaderBytes);
    const uint32_t tiles = smem_u32(c.smem) + conv_header_bytes(K);
    // once the MMAs are done the ring holds the k-slices' partial sums (split > 1) and the store buffers
    const int chunks = BN / 32, max_owned = (chunks + split - 1) / split;
    const uint32_t staging = tiles + (uint32_t)umma_recv_bytes(BN, split, 4);
    int nbuf, group;
    staging_plan((stages * kStageBytes - (int)(staging - tiles)) / kUmmaStagingBytes, max_owned, nbuf, group);
    ChunkWriter<0> w{&p.map_out, p.co, ohw, 0, staging + (uint32_t)(quad * nbuf) * 4096u, nbuf, lane, 0, co0 + quad * 32, img, px0, split * 32, group,
                     (ohw & 3) ? p.y + (size_t)img * p.co * ohw : nullptr};

    long long *const tl = (p.timeline && c.vblock == 0) ? p.timeline : nullptr;
    auto mark = [&](int what, bool who) {
      if (tl && who) tl[what] = (long long)global_ns();
    };
    mark(MARK_START, c.tid == 0);
    if (warp == 4) {
      if (lane < stages) {
        mbar_init(full0 + 8 * lane, 1 + 128);  // the weight copy's arrive.expect_tx + one arrive per gather thread
        mbar_init(empty0 + 8 * lane, 1);
      }
      if (lane == 0) {
        mbar_init(acc_bar, 1);
        mbar_init(recv_bar, 1);
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_w) : "memory");
        if ((ohw & 3) == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_out) : "memory");
      }
      if (lane == 0 && split > 1) {
        // bytes this CTA will receive: one partial per owned 32-pixel chunk from every k-slice (itself included)
        int owned = 0;
        for (int ch = kslice; ch < chunks; ch += split) ++owned;
        mbar_expect_tx(recv_bar, (uint32_t)owned * (uint32_t)split * (32u * kUmmaBM * 4u));
      }
    }
    if (warp < 4) {
      // k -> (input offset relative to the pixel's top-left tap, tap index dy*kw+dx).  Thread t fills
      // entries t, t + 128, ...: (channel, tap) advance by the decomposition of 128, and tap -> (dy, dx)
      // is a multiply-shift (exact for taps < 32), so the loop has no division -- four chained ones
      // per entry made this set-up take 11 us for K = 4608.
      const int khw = p.kh * p.kw, step_ch = 128 / khw, step_r = 128 % khw;
      const int inv_kw = (65536 + p.kw - 1) / p.kw;
      int ch = c.tid / khw, r = c.tid % khw;
      for (int k = c.tid; k < total_kb * kBK; k += 128) {
        const int dy = (r * inv_kw) >> 16, dx = r - dy * p.kw;
        tab[k] = k < K ? make_int2((ch * p.h + dy) * p.wd + dx, r) : make_int2(0, 31);
        ch += step_ch, r += step_r;
        if (r >= khw) r -= khw, ++ch;
      }
    }
    c.dependency_wait();   // nothing above touches global memory: barriers, tensor memory and the table overlap the previous kernel
    tc_fence_before();
    c.sync();
    tc_fence_after();
    const uint32_t tmem_acc = *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t tmem_row = tmem_acc + ((uint32_t)(quad * 32) << 16);
    mark(MARK_SETUP_DONE, c.tid == 0);

    // weight producer and MMA issuer: one elected thread each, ring slot / phase / descriptor word
    // carried incrementally (the issue loop is a dependent chain on one thread; see GemmUmma)
    bool acc_ok = true;
    if (warp == 4) {
      if (elect_one()) {
        uint32_t s = 0, ph = 1, dst = tiles, bar = full0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty0 + 8 * s, ph, c.status, UMMA_WAIT_EMPTY_TIMEOUT)) break;
          mbar_expect_tx(bar, kUmmaABytes);
          tma_load_3d(dst, &p.map_w, bar, (kb0 + kb) * kBK, co0, 0);
          if (++s == (uint32_t)stages) s = 0, ph ^= 1, dst = tiles, bar = full0;
          else dst += kStageBytes, bar += 8;
        }
      }
      __syncwarp();
    } else if (warp == 5) {
      if (elect_one()) {
        const uint32_t lo0 = ((tiles >> 4) & 0x3fffu) | (1u << 16), stage16 = (uint32_t)kStageBytes >> 4;
        uint32_t s = 0, ph = 0, lo = lo0, accumulate = 0;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          ok = mbar_wait(full0 + 8 * s, ph, c.status, UMMA_WAIT_FULL_TIMEOUT);
          if (!ok) break;
          fence_async_smem();  // the gathered operand was written through the generic proxy
          tc_fence_after();
          if (kb == 0) mark(MARK_FIRST_FULL, true);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            umma_ss<0>(tmem_acc, lo + 2 * j, lo + (kUmmaABytes >> 4) + 2 * j, idesc, accumulate);
            accumulate = 1;
          }
          umma_commit(empty0 + 8 * s);
          if (++s == (uint32_t)stages) s = 0, ph ^= 1, lo = lo0;
          else lo += stage16;
        }
        umma_commit(acc_bar);
        mark(MARK_LAST_MMA_ISSUED, true);
        for (int kb = max(0, num_kb - stages); kb < num_kb && ok; ++kb)
          ok = mbar_wait(empty0 + 8 * (kb % stages), (kb / stages) & 1, c.status, UMMA_WAIT_EMPTY_TIMEOUT);
      }
      __syncwarp();
    } else {
      bool ok;
      const int2 *tab_slice = tab + kb0 * kBK;
      if (BN == 128) ok = gather<128>(p, c, quad * 32 + lane, px0, img, num_kb, stages, tiles, full0, empty0, tab_slice, tl);
      else if (BN == 64) ok = gather<64>(p, c, quad * 32 + lane, px0, img, num_kb, stages, tiles, full0, empty0, tab_slice, tl);
      else ok = gather<32>(p, c, quad * 32 + lane, px0, img, num_kb, stages, tiles, full0, empty0, tab_slice, tl);
      (void)ok;
      // epilogue: accumulator rows are output channels, columns are this tile's pixels
      acc_ok = mbar_wait(acc_bar, 0, c.status, UMMA_WAIT_ACC_TIMEOUT);
      tc_fence_after();
      mark(MARK_ACC_READY, c.tid == 0);
      if (acc_ok && split == 1) {
#pragma unroll 1
        for (int ch = 0; ch < BN / 32; ++ch) {
          const uint32_t buf = w.begin_chunk();
          uint32_t r0[16], r1[16];
          tmem_ld_32x16(tmem_row + ch * 32, r0);
          tmem_ld_32x16(tmem_row + ch * 32 + 16, r1);
          tmem_ld_wait();
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r0[j]);
          w.put16(buf, 0, px0 + ch * 32, v, nullptr);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r1[j]);
          w.put16(buf, 1, px0 + ch * 32, v, nullptr);
          w.end_chunk(buf, px0 + ch * 32);
        }
        w.finish();
      }
    }
    if (split > 1) umma_split_reduce<0>(c, BN, split, kslice, tiles, recv_bar, tmem_row, acc_ok, w, px0, nullptr, tl);
    tc_fence_before();
    c.sync();
    if (warp == 5) tmem_dealloc(tmem_acc, BN);
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
