// NCHW convolution as an implicit GEMM on the tensor cores (tcgen05, kind::tf32), the operator of
// the reference's conv2d kernels (tests/benchmark/cuda/conv2d*.cu; files/resnet-18.txt:31,36).
//
//   y[n, co, pixel] = sum_k  w[co, k] * im2col(x)[n, pixel, k],   k = (ci, kh, kw) as in w[co][ci][kh][kw]
//
// A tile is 128 output channels x BN output pixels of one image (BN = 128, or 64 / 32 for small
// images, so that a single image still spreads over many SMs).  The weights are K-major in global
// memory and arrive by TMA (128B swizzle).  The im2col matrix does not exist in memory; the four
// epilogue warps, idle during the main loop, build it, 32 values of k per pixel and K block, in one of
// two ways:
//
//   staged (run_staged: 128-pixel tiles, K a whole number of K blocks and unsplit, image rows of
//     16-byte multiples): the input rows a tile needs -- every row its output pixels' windows touch,
//     full width, a few channels at a time -- arrive by tiled TMA loads over the NCHW tensor into a ring
//     of raw slots (padding is the TMA's out-of-bounds zero fill; a one-row window with a stride loads
//     only the rows it uses through the map's element stride).  The operands' roles are swapped: thread
//     r owns pixel r, reads its window out of the raw slots (per four values of k one 16-byte table read
//     -- their byte offsets inside a slot -- and four 4-byte reads) and writes the 32 values with one
//     tcgen05.st into TENSOR memory, where they are the MMA's A operand; the weights are the B operand;
//     the accumulator holds pixels in its lanes, so the epilogue's stores are coalesced as they are.  A
//     direct TMA load of the taps is not possible: a tap's first column is  dx - pad, and a tiled TMA copy
//     must start at a multiple of 16 bytes, nor has it a traversal stride in the innermost dimension;
//   gathered (run: everything else): 4-byte cp.async copies from global memory straight into a
//     swizzled K-major operand stage in shared memory (out-of-image taps zero-filled by the copy),
//     weights as the A operand, bound by the issue rate of those copies.  Per-k offsets are tabulated
//     once per CTA in shared memory, so the loop does not divide.  A long K (deep layers on small images
//     leave few tiles) can be split over the CTAs of a cluster, reduced through distributed shared
//     memory like the GEMM's k-slices.
//
// BlockDim = (224, 1, 1); GridDim = (split * ceil(oh*ow / BN), ceil(co / 128), n).
#pragma once

#include "ops_umma.cuh"

namespace bfuse {

constexpr int kConvThreads = 224;            // warps 0-3 build the operand and run the epilogue, 4 and 6 issue loads, 5 the MMAs
constexpr int kConvBN = 128;                 // output pixels per tile, at most
constexpr int kConvMaxK = 8192;              // ci * kh * kw the offset table may hold (64 KB of shared memory)
// header of the operator window: barriers etc., then the offset table -- int2 {input offset, tap
// index dy*kw+dx} per k, K rounded up to whole K blocks (tap 31 = padding) and to 1 KB
__host__ __device__ constexpr int conv_header_bytes(int K) { return kUmmaHeaderBytes + ((K + 31) / 32 * 32 * 8 + 1023) / 1024 * 1024; }
__host__ __device__ constexpr int conv_stage_bytes(int bn = kConvBN) { return kUmmaABytes + bn * kUmmaRowBytes; }
// operator window: header (barriers, offset table), the raw ring of a staged conv, then the operand ring
__host__ __device__ constexpr int conv_umma_smem_bytes(int stages, int bn, int K, int raw_bytes = 0) {
  return conv_header_bytes(K) + raw_bytes + stages * conv_stage_bytes(bn);
}

constexpr int kConvMaxRawSlots = 6;
constexpr int kConvRawBarOffset = 256;   // byte offset of the raw ring's barriers in the header: full[6], then empty[6]
constexpr int kConvAStages = 4;          // staged convs: K blocks of the im2col operand held in tensor memory (32 columns each);
                                         // their barriers follow the raw ring's in the header: full[4], then empty[4]
constexpr int kConvTmemCols = 256;       // staged convs: 128 accumulator columns + 4 x 32 operand columns

// Geometry of the raw-input staging of a conv (shared by the host, which sizes shared memory and
// encodes the tensor map, and the kernel).  A slot holds `cc` channels x `rows` staged rows x
// `pitch` floats; staged row j, column i of a tile is input row y0 + j * ey, column x_start + i * ex,
// where y0 = (first output row of the tile) * stride - pad.
struct ConvStaging {
  int slots;        // ring depth (0: the conv is gathered from global memory instead)
  int cc;           // channels per slot (a power of two >= 4, so a slot holds a multiple of 4 values of k)
  int rows, pitch;  // staged rows per channel, floats per staged row (a multiple of 4)
  int ex, ey;       // element strides of the load: ey > 1 for one-row windows with a stride; ex is always 1 (the TMA
                    // has no traversal stride in the innermost dimension)
  int step_x, step_y;  // staged columns / rows between neighbouring output pixels / output rows
  int x_start;      // tensor column of staged column 0 (a multiple of 4, <= -pad)
  int x_off;        // staged column of tap dx = 0 of output column 0
  int slot_bytes;   // cc * rows * pitch * 4: what one TMA load delivers
  int slot_pitch;   // slot_bytes rounded up to 128
  int tile_px;      // output pixels per tile: 128, or whole output rows (the most that fit 128) when that leaves at
                    // most a quarter of the 128 lanes idle -- tiles that start at a row need fewer staged rows
};

// Fills `st` for an image of h x wd and a kh x kw window; returns false when the conv cannot be staged
// (rows that are no 16-byte multiples cannot be described to the TMA; a box is at most 256 wide / high).
__host__ __device__ inline bool conv_staging(int ci, int h, int wd, int kh, int kw, int stride, int pad, int oh, int ow, int bn,
                                             ConvStaging *st) {
  (void)h;
  st->slots = 0;
  if (wd % 4 || (ci * kh * kw) % 32 || bn != kConvBN) return false;   // whole K blocks, whole 128-pixel tiles (the lanes of tensor memory)
  st->ey = (kh == 1 && stride <= 8) ? stride : 1;   // a traversal stride is at most 8
  st->ex = 1;
  st->tile_px = bn;
  if (ow <= bn && (bn / ow) * ow >= bn - bn / 4) st->tile_px = (bn / ow) * ow;
  // output rows that tile_px consecutive pixels can touch (tiles of whole rows: exactly their rows)
  const int out_rows = st->tile_px % ow == 0 ? min(oh, st->tile_px / ow) : min(oh, (st->tile_px - 1 + ow - 1) / ow + 1);
  st->step_y = st->ey == 1 ? stride : 1;
  st->step_x = st->ex == 1 ? stride : 1;
  st->rows = (out_rows - 1) * st->step_y + (st->ey == 1 ? kh : 1);
  st->x_start = st->ex == 1 ? -((pad + 3) / 4 * 4) : 0;
  const int cols = st->ex == 1 ? (ow - 1) * stride - pad + kw - st->x_start : ow;
  st->pitch = (cols + 3) / 4 * 4;
  st->x_off = st->ex == 1 ? -pad - st->x_start : 0;
  if (st->pitch > 256 || st->rows * st->ey > 256) return false;
  const int plane = st->rows * st->pitch * 4;
  // channels per slot: about 16 KB, and enough values of k (cc * kh * kw >= 16) that one K block touches
  // at most three slots -- the repack releases the slots it passed only at the end of a K block, so a K
  // block must not need more slots than the ring holds
  int cc = 64;
  while (cc > 4 && (cc * plane > 16 * 1024 || cc / 2 >= ci) && (cc / 2) * kh * kw >= 16) cc /= 2;
  if (cc * kh * kw < 16 || cc * plane > 24 * 1024) return false;
  st->cc = cc;
  st->slot_bytes = cc * plane;
  st->slot_pitch = (st->slot_bytes + 127) / 128 * 128;
  st->slots = 3;
  return true;
}

struct ConvUmmaParams {
  alignas(64) CUtensorMap map_w;    // {K, co, 1}, box {32 fp32, 128, 1}, 128B swizzle
  alignas(64) CUtensorMap map_out;  // {oh*ow, co, n}, box {32 fp32, 32, 1}, 128B swizzle (stores); unused when oh*ow % 4 != 0
  alignas(64) CUtensorMap map_x;    // staged convs: {wd, h, ci, n}, box {pitch, rows * ey, cc, 1}, element strides {1, ey, 1, 1}
  float *y;                         // [n, co, oh*ow]: the output rows, for images whose rows are not 16-byte multiples
  const float *x;
  int n, ci, h, wd, co, kh, kw, stride, pad, oh, ow;
  int K;
  int stages;           // ring depth: operand stages (gathered) or 16 KB weight stages (staged)
  int bn;               // output pixels per tile: 32, 64 or 128
  int split;            // CTAs (k-slices) per tile = cluster width; 1: no split
  int kb_per_slice;     // K blocks per k-slice
  int ctas;             // staged: CTAs of the grid (a CTA takes every ctas-th tile)
  ConvStaging st;       // st.slots == 0: gathered from global memory
  long long *timeline;  // diagnostic: when non-null, CTA 0 records globaltimer marks (UmmaMark indices)
};

// bytes of the raw ring, rounded so that the operand ring behind it stays 1 KB aligned (128B swizzle)
__host__ __device__ constexpr int conv_raw_bytes(int slots, int slot_pitch) { return (slots * slot_pitch + 1023) / 1024 * 1024; }

// How a staged conv divides a shared-memory window of `smem` bytes: header, raw slots, 16 KB weight stages.
// Weights come out of L2 and two stages cover that; the input comes out of DRAM, whose latency under load is
// several K blocks long, so what is left goes to raw slots first (up to 6, never more than the tile loads),
// then to more weight stages (3 x 3 stride-2 branch of ResNet-18 at batch 256 in 106 KB: 5 slots + 2 stages
// 112 us, 4 + 3 118 us, 3 + 4 127 us).  A K block touches up to three slots, so fewer than three only when the
// tile has fewer.  Returns false when the window is too small.
__host__ __device__ inline bool conv_staged_ring(int smem, int K, int kslot, int slot_pitch, int *slots, int *wstages) {
  const int num_kb = K / 32, loads = (K - 1) / kslot + 1;
  const int room = smem - conv_header_bytes(K);
  const int w_min = num_kb < 2 ? num_kb : 2, s_min = loads < 3 ? loads : 3;
  int s = (room - w_min * kUmmaABytes) / slot_pitch;
  if (s > kConvMaxRawSlots) s = kConvMaxRawSlots;
  if (s > loads) s = loads;
  if (s < s_min) s = s_min;
  int w = (room - conv_raw_bytes(s, slot_pitch)) / kUmmaABytes;
  if (w > kUmmaMaxStages) w = kUmmaMaxStages;
  if (w > num_kb) w = num_kb;
  *slots = s, *wstages = w;
  return w >= (num_kb < 2 ? num_kb : 2);
}
__host__ __device__ inline int conv_staged_smem_bytes(int K, int slots, int slot_pitch, int wstages) {
  return conv_header_bytes(K) + conv_raw_bytes(slots, slot_pitch) + wstages * kUmmaABytes;
}

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

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// has phase `parity` of the barrier completed?  Never blocks.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int4 ld_shared_i4(uint32_t addr) {
  int4 v;
  asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}

struct ConvUmmaTf32 {
  using Params = ConvUmmaParams;
  static constexpr int kMaxThreads = kConvThreads;
  static constexpr int kMinBlocks = 2;      // two CTAs per SM: one tile's epilogue runs under the other's main loop (a build for three -- 96 registers --
                                            // gained 7 % at batch 256 and lost 30 % at batch 32, where every CTA has an SM's issue slots to itself)
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
    const float *const x0 = p.x;   // read once: the loop's asm statements make the compiler re-read parameters otherwise
    const float *xb = x0 + (size_t)img * p.ci * p.h * p.wd + (ptrdiff_t)iy0 * p.wd + ix0;
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
          src[i] = in ? xb + t.x : x0;
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

  // Lane 0 of a converged warp waits for phase `parity` of an mbarrier, the other lanes wait for lane 0;
  // what the barrier's completion made visible to lane 0 is visible to the whole warp after the __syncwarp.
  // Returns the wait's outcome to every lane (false: it gave up and reported).
  __device__ __forceinline__ static bool warp_wait(bool lane0, uint32_t bar, uint32_t parity, int *status, int code) {
    int ok = 1;
    if (lane0) ok = mbar_wait(bar, parity, status, code) ? 1 : 0;
    __syncwarp();
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
  }

  // The repack of a 3 x 3 window: it walks the K range four channels at a time (a whole raw slot, or a quarter,
  // an eighth ... of one) -- 36 values of k, every one's channel, row and tap known when this is compiled -- instead of one K block
  // at a time.  A slot costs 12 row addresses and 24 reads (the taps dx = 1, 2 of a row as one 8-byte read
  // where PAIR says they start at an even float), no table and no address add per value, and it is waited
  // for and released exactly once.  The 36 values go into the ring of A stages as into 128 consecutive
  // columns (nine tcgen05.st of 4 columns, each wrapped on its own), so the MMA side keeps its K blocks
  // of 32: a stage is handed over as soon as its 32nd column is written.  `rawpix_p` points at the pixel's
  // window origin in slot 0 of the ring.
  // where the four-channel walk stands, across the tiles of a CTA
  struct SlotWalk {
    uint32_t rs = 0, rph = 0;   // raw slot of the next step, its phase
    int quad_in_slot = 0;       // a slot of more than 4 channels is walked in `quads` steps of 4
    int kdone = 0;              // values of k written so far (over all tiles: the A ring's column is kdone mod 128)
    int acquired = 0;           // A stages (counted over all tiles) whose "empty" has been seen
  };
  template <bool PAIR>
  __device__ __forceinline__ static bool repack_3x3(const TileCtx &c, int K, bool lane0, const unsigned char *rawpix_p, uint32_t slot_pitch,
                                                    int nslots, int quads, uint32_t plane4, uint32_t pitch4, uint32_t a_row, uint32_t raw_full0,
                                                    uint32_t raw_empty0, uint32_t a_full0, uint32_t a_empty0, SlotWalk &walk) {
    int *const status = c.status;
    const int steps = K / 36;
    uint32_t rs = walk.rs, rph = walk.rph;
    int quad_in_slot = walk.quad_in_slot, kdone = walk.kdone, acquired = walk.acquired;
    bool seen_raw = false, seen_empty = false;
    for (int s = 0; s < steps; ++s) {
      if (quad_in_slot == 0 && !seen_raw && !warp_wait(lane0, raw_full0 + 8 * rs, rph, status, UMMA_WAIT_FULL_TIMEOUT)) return false;
      // the stages this slot's 36 columns fall into: kdone / 32 and, mostly, the one after
      const int g_last = (kdone + 35) >> 5;
      if (seen_empty) ++acquired;
      while (acquired <= g_last) {
        if (!warp_wait(lane0, a_empty0 + 8 * (acquired & (kConvAStages - 1)), (uint32_t)((acquired / kConvAStages) & 1) ^ 1u, status,
                       UMMA_WAIT_EMPTY_TIMEOUT))
          return false;
        ++acquired;
      }
      tc_fence_after();   // the MMAs that read these stages have completed (their commit): they may be written again
      const unsigned char *base = rawpix_p + rs * slot_pitch + (uint32_t)(4 * quad_in_slot) * plane4;
      uint32_t v[36];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
#pragma unroll
        for (int dy = 0; dy < 3; ++dy) {
          const unsigned char *row = base + ch * plane4 + dy * pitch4;
          const int i = 9 * ch + 3 * dy;
          v[i] = __float_as_uint(*reinterpret_cast<const float *>(row));
          if (PAIR) {
            const float2 t = *reinterpret_cast<const float2 *>(row + 4);
            v[i + 1] = __float_as_uint(t.x), v[i + 2] = __float_as_uint(t.y);
          } else {
            v[i + 1] = __float_as_uint(*reinterpret_cast<const float *>(row + 4));
            v[i + 2] = __float_as_uint(*reinterpret_cast<const float *>(row + 8));
          }
        }
      }
      // a look at the next step's barriers while the reads are in flight: a wait costs 100-200 clocks even
      // when its barrier has completed
      const uint32_t rs_old = rs;
      const bool slot_done = ++quad_in_slot == quads;
      if (slot_done) {
        quad_in_slot = 0;
        if (++rs == (uint32_t)nslots) rs = 0, rph ^= 1;
      }
      bool e = false, f = false;
      if (s + 1 < steps) {
        f = slot_done && mbar_test(raw_full0 + 8 * rs, rph);
        if (acquired <= (kdone + 36 + 35) >> 5)
          e = mbar_test(a_empty0 + 8 * (acquired & (kConvAStages - 1)), (uint32_t)((acquired / kConvAStages) & 1) ^ 1u);
      }
      const uint32_t col = (uint32_t)kdone & 127u;
#pragma unroll
      for (int q = 0; q < 9; ++q) tmem_st_32x4(a_row + ((col + 4u * q) & 127u), v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      seen_raw = __all_sync(0xffffffffu, f);
      seen_empty = __all_sync(0xffffffffu, e);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      // one arrival per warp: the slot is free (its values were written), and so is every stage whose 32nd
      // column this step wrote
      const int done_before = kdone >> 5;
      kdone += 36;
      const int done_after = kdone >> 5;
      if (lane0) {
        if (slot_done) mbar_arrive(raw_empty0 + 8 * rs_old);
        for (int g = done_before; g < done_after; ++g) mbar_arrive(a_full0 + 8 * (g & (kConvAStages - 1)));
      }
    }
    if (quad_in_slot) {   // the tile's channels end inside a slot: it is free too, and the next tile starts in a fresh one
      if (lane0) mbar_arrive(raw_empty0 + 8 * rs);
      quad_in_slot = 0;
      if (++rs == (uint32_t)nslots) rs = 0, rph ^= 1;
    }
    walk.rs = rs, walk.rph = rph, walk.quad_in_slot = quad_in_slot, walk.kdone = kdone, walk.acquired = acquired;
    return true;
  }

  // The staged form of a tile: 128 output pixels x 128 output channels with the operands' roles swapped
  // relative to run() -- the im2col rows are the A operand and live in TENSOR memory, the weights are the
  // B operand in shared memory, and the accumulator holds pixels in its lanes and output channels in its
  // columns.  Thread r of the four repack warps owns pixel r of the tile, which is also lane r of tensor
  // memory: it reads its window's 32 values of a K block out of the raw ring (one 16-byte table read per
  // four values: their byte offsets from the window's origin inside a slot), and writes them with one
  // tcgen05.st into the K block's 32 columns of a four-deep ring of A stages.  Compared with building
  // the operand in shared memory this takes the operand's write and the MMA's read of it (2 x 16 KB per K
  // block) off the shared-memory pipe, which the raw loads, the repack's reads, the weight loads and the
  // MMA's weight reads already keep busy; it needs no proxy fence; it leaves the shared memory of the
  // operand ring to four weight stages; and the epilogue's stores are coalesced as they come out of
  // tensor memory (a warp's 32 lanes are 32 consecutive pixels of one output channel), so it needs no
  // staging buffers either.
  //
  // Warps: 0-3 repack and epilogue, 4 raw loads, 5 MMA, 6 weight loads (two issuing warps: the loads a
  // single thread issues complete one after another).  All threads walk the same k, so which ring slot
  // holds a value of k is uniform and found by comparisons: a K block of 32 touches at most three slots
  // (a slot holds at least 16 values of k); a loop or a branch per chunk costs this code -- one warp per
  // scheduler, nothing to hide a branch behind -- more than the copying.  A wait costs 100-200 clocks even
  // when its barrier has completed, so every K block looks at the next one's barriers without blocking
  // while its own reads are in flight, and the next K block waits only for what was not there yet.
  __device__ __forceinline__ static void run_staged(const Params &p, const TileCtx &c) {
    const int warp = c.tid >> 5, lane = c.tid & 31;
    const int quad = (threadIdx.x >> 5) & 3;
    const int tile_px = p.st.tile_px;
    const int ohw = p.oh * p.ow, K = p.K, num_kb = K / kBK;   // staged: K is a whole number of K blocks
    // The CTA's tiles: its block index, then every p.ctas-th one (tiles numbered pixel tile fastest, then
    // channel tile, then image; a grid of one CTA per tile makes a single pass).  The rings, their barriers'
    // phases and tensor memory live across tiles, so the loads of the next tile run under this tile's
    // epilogue, and only the first tile pays for the set-up and the first loads' latency.
    const int px_tiles = (ohw + tile_px - 1) / tile_px, co_tiles = (p.co + kUmmaBM - 1) / kUmmaBM;
    const int total_tiles = px_tiles * co_tiles * p.n, tile_step = p.ctas;
    const int wstages = p.stages;                             // 16 KB weight stages behind the raw ring
    int *const status = c.status;
    const uint32_t idesc = umma_idesc(0, kUmmaBM);            // M = 128 pixels, N = 128 output channels

    uint64_t *bars = reinterpret_cast<uint64_t *>(c.smem);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * kUmmaMaxStages, acc_bar = empty0 + 8 * kUmmaMaxStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(c.smem + 8 * (2 * kUmmaMaxStages + 2));
    const uint32_t raw_full0 = full0 + kConvRawBarOffset, raw_empty0 = raw_full0 + 8 * kConvMaxRawSlots;
    const uint32_t a_full0 = raw_empty0 + 8 * kConvMaxRawSlots, a_empty0 = a_full0 + 8 * kConvAStages;
    const uint32_t acc_empty = a_empty0 + 8 * kConvAStages;   // the epilogue has read the accumulator: the next tile's MMAs may start
    const uint32_t raw0 = smem_u32(c.smem) + conv_header_bytes(K);
    const uint32_t wring = raw0 + (uint32_t)conv_raw_bytes(p.st.slots, p.st.slot_pitch);
    if (warp == 5) {
      if (!c.tmem_given) {   // (a persistent CTA of the work queue holds its columns already)
        tmem_alloc(smem_u32(tmem_slot), kConvTmemCols);
        if (!c.persistent) tmem_relinquish();
      }
    }
    long long *const tl = (p.timeline && c.vblock == 0) ? p.timeline : nullptr;
    auto mark = [&](int what, bool who) {
      if (tl && who) tl[what] = (long long)global_ns();
    };
    mark(MARK_START, c.tid == 0);
    if (warp == 4) {
      if (lane < wstages) {
        mbar_init(full0 + 8 * lane, 1);    // the weight load's arrive.expect_tx
        mbar_init(empty0 + 8 * lane, 1);   // the MMA's commit
      }
      if (lane < kConvAStages) {
        mbar_init(a_full0 + 8 * lane, 4);  // one arrival per repack warp
        mbar_init(a_empty0 + 8 * lane, 1); // the MMA's commit
      }
      if (lane < p.st.slots) {
        mbar_init(raw_full0 + 8 * lane, 1);   // the slot's TMA load (arrive.expect_tx)
        mbar_init(raw_empty0 + 8 * lane, 4);  // every repack warp, once it has moved past the slot
      }
      if (lane == 0) {
        mbar_init(acc_bar, 1);
        mbar_init(acc_empty, 4);   // one arrival per epilogue warp
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&p.map_x) : "memory");
      }
    }
    int *tab4 = reinterpret_cast<int *>(c.smem + kUmmaHeaderBytes);
    if (warp < 4) {
      // entry k: the byte offset of (channel within its slot, dy, dx) inside a raw slot.  Thread t fills
      // entries t, t + 128, ...: (channel, tap) advance by the decomposition of 128, and tap -> (dy, dx)
      // is a multiply-shift (exact for taps < 32), so the loop has no division.
      const int khw = p.kh * p.kw, step_ch = 128 / khw, step_r = 128 % khw;
      const int inv_kw = (65536 + p.kw - 1) / p.kw;
      const int plane = p.st.rows * p.st.pitch;
      int ch = c.tid / khw, r = c.tid - ch * khw;
      for (int k = c.tid; k < K; k += 128) {
        const int dy = (r * inv_kw) >> 16, dx = r - dy * p.kw;
        tab4[k] = (((ch & (p.st.cc - 1)) * plane) + dy * p.st.pitch + dx) * 4;
        ch += step_ch, r += step_r;
        if (r >= khw) r -= khw, ++ch;
      }
    }
    c.dependency_wait();   // nothing above touches global memory: barriers, tensor memory and the table overlap the previous kernel
    tc_fence_before();
    c.sync();
    tc_fence_after();
    const uint32_t tmem_acc = c.tmem_given ? c.tmem_base : *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t tmem_row = tmem_acc + ((uint32_t)(quad * 32) << 16);   // this warp's lanes; columns 0-127: accumulator, then the A stages
    mark(MARK_SETUP_DONE, c.tid == 0);

    if (warp == 4) {
      if (elect_one()) {
        const int cc = p.st.cc, kslot = cc * p.kh * p.kw, x_start = p.st.x_start, nslots = p.st.slots;
        const uint32_t slot_bytes = (uint32_t)p.st.slot_bytes, slot_pitch = (uint32_t)p.st.slot_pitch;
        const int g_end = (K - 1) / kslot + 1;
        uint32_t rs = 0, rph = 1;
        bool ok = true;
        for (int t = c.vblock; t < total_tiles && ok; t += tile_step) {
          const int px0 = (t % px_tiles) * tile_px, img = t / (px_tiles * co_tiles);
          const int y_start = (px0 / p.ow) * p.stride - p.pad;
          for (int g = 0; g < g_end; ++g) {
            if (!(ok = mbar_wait(raw_empty0 + 8 * rs, rph, status, UMMA_WAIT_EMPTY_TIMEOUT))) break;
            mbar_expect_tx(raw_full0 + 8 * rs, slot_bytes);
            tma_load_4d(raw0 + rs * slot_pitch, &p.map_x, raw_full0 + 8 * rs, x_start, y_start, g * cc, img);
            if (++rs == (uint32_t)nslots) rs = 0, rph ^= 1;
          }
        }
      }
      __syncwarp();
    } else if (warp == 6) {
      if (elect_one()) {
        uint32_t s = 0, ph = 1, dst = wring, bar = full0;
        bool ok = true;
        for (int t = c.vblock; t < total_tiles && ok; t += tile_step) {
          const int co0 = (t / px_tiles % co_tiles) * kUmmaBM;
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!(ok = mbar_wait(empty0 + 8 * s, ph, status, UMMA_WAIT_EMPTY_TIMEOUT))) break;
            mbar_expect_tx(bar, kUmmaABytes);
            tma_load_3d(dst, &p.map_w, bar, kb * kBK, co0, 0);
            if (++s == (uint32_t)wstages) s = 0, ph ^= 1, dst = wring, bar = full0;
            else dst += kUmmaABytes, bar += 8;
          }
        }
      }
      __syncwarp();
    } else if (warp == 5) {
      if (elect_one()) {
        const uint32_t lo0 = ((wring >> 4) & 0x3fffu) | (1u << 16);
        uint32_t s = 0, ph = 0, lo = lo0, as = 0, aph = 0;
        bool ok = true;
        int done = 0;   // K blocks issued so far, over all tiles
        for (int t = c.vblock, it = 0; t < total_tiles && ok; t += tile_step, ++it) {
          // the accumulator is free again once the epilogue of the tile before has read it
          if (it > 0 && !(ok = mbar_wait(acc_empty, (uint32_t)(it - 1) & 1u, status, UMMA_WAIT_ACC_TIMEOUT))) break;
          tc_fence_after();
          uint32_t accumulate = 0;
          for (int kb = 0; kb < num_kb; ++kb) {
            ok = mbar_wait(a_full0 + 8 * as, aph, status, UMMA_WAIT_FULL_TIMEOUT) && mbar_wait(full0 + 8 * s, ph, status, UMMA_WAIT_FULL_TIMEOUT);
            if (!ok) break;
            tc_fence_after();
            if (kb == 0 && it == 0) mark(MARK_FIRST_FULL, true);
            const uint32_t a_tmem = tmem_acc + (uint32_t)(kUmmaBM + as * kBK);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              umma_ts_tf32(tmem_acc, a_tmem + 8 * j, lo + 2 * j, idesc, accumulate);
              accumulate = 1;
            }
            umma_commit(empty0 + 8 * s);
            umma_commit(a_empty0 + 8 * as);
            if (++s == (uint32_t)wstages) s = 0, ph ^= 1, lo = lo0;
            else lo += (uint32_t)kUmmaABytes >> 4;
            if (++as == (uint32_t)kConvAStages) as = 0, aph ^= 1;
            ++done;
          }
          umma_commit(acc_bar);   // this tile's accumulator is complete (also arrives if the loop bailed out)
          if (it == 0) mark(MARK_LAST_MMA_ISSUED, true);
        }
        // every commit has arrived before the barriers are invalidated and the ring is given up
        for (int j = max(0, done - wstages); j < done && ok; ++j)
          ok = mbar_wait(empty0 + 8 * (j % wstages), (uint32_t)(j / wstages) & 1u, status, UMMA_WAIT_EMPTY_TIMEOUT);
        for (int j = max(0, done - kConvAStages); j < done && ok; ++j)
          ok = mbar_wait(a_empty0 + 8 * (j % kConvAStages), (uint32_t)(j / kConvAStages) & 1u, status, UMMA_WAIT_EMPTY_TIMEOUT);
      }
      __syncwarp();
    } else {
      const int r = quad * 32 + lane;
      const bool lane0 = lane == 0;
      bool ok = true;
      // Every parameter the loops need is read into registers here: they are full of asm statements that
      // clobber memory, after each of which the compiler would otherwise read the parameter block again.
      const ConvStaging st = p.st;
      const int ow = p.ow, co_total = p.co;
      float *const y = p.y;
      const uint32_t slot_pitch = (uint32_t)st.slot_pitch;
      const int kslot = st.cc * p.kh * p.kw, nslots = st.slots;
      const uint32_t tab = smem_u32(tab4), ring_bytes = (uint32_t)nslots * slot_pitch;
      const uint32_t a_row = tmem_row + (uint32_t)kUmmaBM;
      // 3 x 3 windows go four channels at a time, without the table
      extern __shared__ __align__(16) unsigned char conv_window[];
      const bool by_slot = p.kh == 3 && p.kw == 3;   // (slots hold 4, 8, 16 ... channels; K is a multiple of 32 and of 9)
      const uint32_t plane4 = (uint32_t)(st.rows * st.pitch * 4), pitch4 = (uint32_t)(st.pitch * 4);
      // taps dx = 1, 2 of every pixel start at an even float (rows, planes and slots are 16-byte multiples)
      const bool pair = (st.step_x & 1) == 0 && (st.x_off & 1) == 1;
      SlotWalk walk;
      // The rings' positions live across tiles (every tile starts in a fresh raw slot): the slot and phase of the
      // next k, how many slots from there on have been seen full, the A stage and its phase.
      int ahead = 0;
      uint32_t rs = 0, rph = 0, as = 0, aph = 1;
      for (int t = c.vblock, it = 0; t < total_tiles && ok; t += tile_step, ++it) {
        const int px0 = (t % px_tiles) * tile_px, co0 = (t / px_tiles % co_tiles) * kUmmaBM, img = t / (px_tiles * co_tiles);
        const int pix = px0 + r;
        // a lane past the tile's pixels or past the image reads the window of pixel 0 of the tile: finite
        // values, and it is not stored
        const int oy0 = px0 / ow;
        int oy = pix / ow, ox = pix - oy * ow;
        if (r >= tile_px || pix >= ohw) oy = oy0, ox = px0 - oy0 * ow;
        const uint32_t rawpix = raw0 + (uint32_t)(((oy - oy0) * st.step_y * st.pitch + ox * st.step_x + st.x_off) * 4);
        if (by_slot) {
          const unsigned char *const rawpix_p = conv_window + (rawpix - smem_u32(conv_window));
          ok = pair ? repack_3x3<true>(c, K, lane0, rawpix_p, slot_pitch, nslots, st.cc / 4, plane4, pitch4, a_row, raw_full0, raw_empty0, a_full0, a_empty0, walk)
                    : repack_3x3<false>(c, K, lane0, rawpix_p, slot_pitch, nslots, st.cc / 4, plane4, pitch4, a_row, raw_full0, raw_empty0, a_full0, a_empty0, walk);
        }
        int kin = 0;   // where the K block starts inside slot rs
        bool seen_empty = false, seen_raw = false;
        for (int kb = 0; kb < num_kb && !by_slot; ++kb) {
          // one lane per warp polls a barrier and the warp follows it (its lanes meet again at the __syncwarp
          // before the arrival below, so the outcome of a wait has to be the same for all of them anyway)
          if (!seen_empty && !(ok = warp_wait(lane0, a_empty0 + 8 * as, aph, status, UMMA_WAIT_EMPTY_TIMEOUT))) break;
          tc_fence_after();   // the MMAs that read this A stage have completed (their commit): it may be written again
          // slots the K block reads: the first one and `last` more
          const int reach = kin + kBK - 1;
          const int last = (reach >= kslot) + (reach >= 2 * kslot);
          if (seen_raw) ++ahead;
          while (ahead <= last) {
            uint32_t w = rs + (uint32_t)ahead, wph = rph;
            if (w >= (uint32_t)nslots) w -= nslots, wph ^= 1;
            if (!(ok = warp_wait(lane0, raw_full0 + 8 * w, wph, status, UMMA_WAIT_FULL_TIMEOUT))) break;
            ++ahead;
          }
          if (!ok) break;
          // the table entries (four byte offsets per chunk of four k) and which slot each chunk reads: chunk i
          // starts kin + 4 i values of k into slot rs, so the chunks from j1 on read the next slot and those
          // from j2 on the one after (all multiples of 4: exact shifts)
          const uint32_t tabk = tab + (uint32_t)(kb * kBK) * 4u;
          uint32_t b0 = rawpix + rs * slot_pitch, b1 = b0 + slot_pitch, b2 = b1 + slot_pitch;
          if (rs + 1 >= (uint32_t)nslots) b1 -= ring_bytes;
          if (rs + 2 >= (uint32_t)nslots) b2 -= ring_bytes;
          const int j1 = (kslot - kin) >> 2, j2 = j1 + (kslot >> 2);
          int4 off[8];
          uint32_t src[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            off[i] = ld_shared_i4(tabk + 16u * i);
            src[i] = i >= j2 ? b2 : i >= j1 ? b1 : b0;
          }
          // on to the next K block's position in the ring (the slots that end inside this one are released below)
          int passed = (kin + kBK >= kslot) + (kin + kBK >= 2 * kslot);
          kin += kBK - passed * kslot;
          if (kb + 1 == num_kb && kin > 0) ++passed, kin = 0;   // the tile's K ends inside a slot: it is free too
          const uint32_t rs_old = rs, as_old = as;
          ahead -= passed, rs += passed;
          if (rs >= (uint32_t)nslots) rs -= nslots, rph ^= 1;
          if (++as == (uint32_t)kConvAStages) as = 0, aph ^= 1;
          // the look at the next K block's barriers: asked here, answered (the votes below) once this K block's
          // reads have been issued, so that the answers' round trip hides behind them
          bool e = false, f = false;
          if (kb + 1 < num_kb) {
            const int reach_n = kin + kBK - 1;
            const bool more = ahead <= (reach_n >= kslot) + (reach_n >= 2 * kslot);
            uint32_t w = rs + (uint32_t)ahead, wph = rph;
            if (w >= (uint32_t)nslots) w -= nslots, wph ^= 1;
            e = mbar_test(a_empty0 + 8 * as, aph);
            f = more && mbar_test(raw_full0 + 8 * w, wph);
          }
          // the raw values, then all 32 into this lane's columns of the A stage
          uint32_t v[32];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[4 * i] = __float_as_uint(ld_shared_f32(src[i] + (uint32_t)off[i].x));
            v[4 * i + 1] = __float_as_uint(ld_shared_f32(src[i] + (uint32_t)off[i].y));
            v[4 * i + 2] = __float_as_uint(ld_shared_f32(src[i] + (uint32_t)off[i].z));
            v[4 * i + 3] = __float_as_uint(ld_shared_f32(src[i] + (uint32_t)off[i].w));
          }
          tmem_st_32x32(a_row + as_old * (uint32_t)kBK, v);
          seen_empty = __all_sync(0xffffffffu, e);
          seen_raw = __all_sync(0xffffffffu, f);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          // One arrival per warp.  The raw reads above have completed (their values were stored), so the
          // slots that end inside this K block are free.
          if (lane0) {
            mbar_arrive(a_full0 + 8 * as_old);
            if (passed > 0) mbar_arrive(raw_empty0 + 8 * rs_old);
            if (passed > 1) mbar_arrive(raw_empty0 + 8 * (rs_old + 1 < (uint32_t)nslots ? rs_old + 1 : 0u));
            if (passed > 2) mbar_arrive(raw_empty0 + 8 * ((rs_old + 2) % (uint32_t)nslots));
          }
          if (it == 0 && kb == 0) mark(MARK_FIRST_LOAD_ISSUED, r == 0);
          if (it == 0 && kb == num_kb - 1) mark(MARK_LAST_LOAD_ISSUED, r == 0);
        }
        if (ahead < 0) ahead = 0;
        // epilogue: lane = pixel, column = output channel; a warp's store covers 32 consecutive pixels of one channel
        const bool acc_ok = ok && mbar_wait(acc_bar, (uint32_t)it & 1u, status, UMMA_WAIT_ACC_TIMEOUT);
        tc_fence_after();
        if (it == 0) mark(MARK_ACC_READY, c.tid == 0);
        if (!acc_ok) {
          ok = false;
          break;
        }
        float *const yp = y + ((size_t)img * co_total + co0) * ohw + pix;
        const bool live = r < tile_px && pix < ohw;
        const int co_left = co_total - co0;
#pragma unroll 1
        for (int cc = 0; cc < kUmmaBM; cc += 32) {
          uint32_t r0[16], r1[16];
          tmem_ld_32x16(tmem_row + cc, r0);
          tmem_ld_32x16(tmem_row + cc + 16, r1);
          tmem_ld_wait();
          if (cc + 32 == kUmmaBM && t + tile_step < total_tiles) {
            // the accumulator has been read: hand it back to the MMA thread before the last stores go out
            tc_fence_before();
            __syncwarp();
            if (lane0) mbar_arrive(acc_empty);
          }
          if (live) {
            float *q = yp + (size_t)cc * ohw;
            if (cc + 32 <= co_left) {   // a whole group of 32 channels: no test per store
#pragma unroll
              for (int j = 0; j < 16; ++j) q[(size_t)j * ohw] = __uint_as_float(r0[j]);
#pragma unroll
              for (int j = 0; j < 16; ++j) q[(size_t)(16 + j) * ohw] = __uint_as_float(r1[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (cc + j < co_left) q[(size_t)j * ohw] = __uint_as_float(r0[j]);
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (cc + 16 + j < co_left) q[(size_t)(16 + j) * ohw] = __uint_as_float(r1[j]);
            }
          }
        }
      }
    }
    tc_fence_before();
    c.sync();
    if (warp == 5 && !c.tmem_given) tmem_dealloc(tmem_acc, kConvTmemCols);
    if (c.persistent) {  // the next tile of a persistent CTA initialises them again
      if (c.tid < wstages) {
        mbar_inval(full0 + 8 * c.tid);
        mbar_inval(empty0 + 8 * c.tid);
      }
      if (c.tid < kConvAStages) {
        mbar_inval(a_full0 + 8 * c.tid);
        mbar_inval(a_empty0 + 8 * c.tid);
      }
      if (c.tid < p.st.slots) {
        mbar_inval(raw_full0 + 8 * c.tid);
        mbar_inval(raw_empty0 + 8 * c.tid);
      }
      if (c.tid == 0) {
        mbar_inval(acc_bar);
        mbar_inval(acc_empty);
      }
    }
    mark(MARK_END, c.tid == 0);
  }

  __device__ __forceinline__ static void run(const Params &p, const TileCtx &c) {
    if (p.st.slots > 0) {
      run_staged(p, c);
      return;
    }
    const int warp = c.tid >> 5, lane = c.tid & 31;
    const int quad = (threadIdx.x >> 5) & 3;
    const int BN = p.bn, kStageBytes = conv_stage_bytes(BN);
    const int split = p.split, kslice = c.block_x() % split;
    const int px0 = (c.block_x() / split) * BN, co0 = c.block_y() * kUmmaBM, img = c.block_z();
    const int stages = p.stages, ohw = p.oh * p.ow, K = p.K;
    int *const status = c.status;
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
      if (!c.tmem_given) {   // (a persistent CTA of the work queue holds its columns already)
        tmem_alloc(smem_u32(tmem_slot), BN);
        if (!c.persistent) tmem_relinquish();
      }
    }
    int2 *tab = reinterpret_cast<int2 *>(c.smem + kUmmaHeaderBytes);
    const uint32_t tiles = smem_u32(c.smem) + conv_header_bytes(K);   // the operand ring
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
    const uint32_t tmem_acc = c.tmem_given ? c.tmem_base : *reinterpret_cast<volatile uint32_t *>(tmem_slot);
    const uint32_t tmem_row = tmem_acc + ((uint32_t)(quad * 32) << 16);
    mark(MARK_SETUP_DONE, c.tid == 0);

    // weight producer and MMA issuer: one elected thread each, ring slot / phase / descriptor word
    // carried incrementally (the issue loop is a dependent chain on one thread; see GemmUmma)
    bool acc_ok = true;
    if (warp == 6) {
      // idle: the staged form's second loading warp
    } else if (warp == 4) {
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
          ok = mbar_wait(full0 + 8 * s, ph, status, UMMA_WAIT_FULL_TIMEOUT);
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
      const int gt = quad * 32 + lane;
      const int2 *tab_slice = tab + kb0 * kBK;
      // (a gather that gave up has reported to the status word; the wait below then returns at once)
      if (BN == 128) (void)gather<128>(p, c, gt, px0, img, num_kb, stages, tiles, full0, empty0, tab_slice, tl);
      else if (BN == 64) (void)gather<64>(p, c, gt, px0, img, num_kb, stages, tiles, full0, empty0, tab_slice, tl);
      else (void)gather<32>(p, c, gt, px0, img, num_kb, stages, tiles, full0, empty0, tab_slice, tl);
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
    if (warp == 5 && !c.tmem_given) tmem_dealloc(tmem_acc, BN);
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
