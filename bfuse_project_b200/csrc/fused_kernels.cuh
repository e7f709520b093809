// The fused kernels.  Where the reference's fuser rewrites two kernels' source into one
// __global__ function with the dispatch chain at the top and each body under
// `if (KernelID_ == k && threadIdx.x < B_k)` (horizontal-fuser/src/Matchers.cc:464-602 for
// block-level fusion, :604-727 for thread-level fusion), this file instantiates one kernel per
// pair of operator bodies from the registry:
//
//   fused_block_kernel<A, B>   every CTA runs one operator (zig-zag, proportional, SM-striped,
//                              range split) or, with table.queue set, loops over tickets drawn
//                              from an atomic counter (persistent work queue);
//   fused_thread_kernel<A, B>  both operators inside every CTA, split by thread range, each
//                              synchronising on its own named barrier; shared memory is the sum;
//   fused_group_kernel<A>      up to four operators of one body in one launch (the reference's
//                              n-kernel form of the block-level patterns);
//   single_kernel<A>           the unfused launch of the same body (baselines, bit-exact check);
//   trace_kernel               the dispatch decode alone, recording what each CTA would run.
//
// __launch_bounds__ come from the pair (pair_min_blocks): the larger block and a CTAs-per-SM target
// that keeps the lighter operator's occupancy without starving the heavier body of registers.
#pragma once

#include "dispatch.h"
#include "tile.h"

namespace bfuse {

__device__ __forceinline__ unsigned char *align_smem_1k(unsigned char *p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  return p + ((1024u - (a & 1023u)) & 1023u);
}

// Programmatic dependent launch: every kernel here is launched with the programmatic-stream-
// serialization attribute, so its CTAs may be scheduled while the previous kernel on the stream is
// still draining.  grid_dependency_wait() blocks until that kernel has completed and its writes
// are visible -- nothing before it may touch global memory -- and grid_launch_dependents() lets
// the next kernel's CTAs start their own prologue early.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Whole warp, converged: this CTA will not allocate tensor memory (any more).
__device__ __forceinline__ void relinquish_tmem_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

template <class Op>
__device__ __forceinline__ void run_tile(const typename Op::Params &p, const DispatchTable &t, int k, int vb, int vtid,
                                         int bar_id, unsigned char *smem, int shares_cta = 0, int tmem_given = 0, unsigned tmem_base = 0) {
  TileCtx c;
  c.vblock = vb;
  c.tid = vtid;
  c.nthreads = t.n_thr[k];
  c.bar_id = bar_id;
  c.bar_count = t.bar_count[k];
  c.gx = t.grid_x[k];
  c.gy = t.grid_y[k];
  c.bx = t.blk_x[k];
  c.by = t.blk_y[k];
  c.smem = smem;
  c.status = t.status;
  c.persistent = t.queue | shares_cta;
  c.tmem_given = tmem_given;
  c.tmem_base = tmem_base;
  Op::run(p, c);
}

constexpr int cmax(int a, int b) { return a > b ? a : b; }
constexpr int cmin(int a, int b) { return a < b ? a : b; }
// Minimum CTAs per SM the pair is compiled for.  Two memory-bound bodies: the larger of their two
// wishes (occupancy is what hides HBM latency).  A memory-bound body next to a GEMM / conv body:
// at most 4, so the heavier body is not squeezed below 64 registers per thread.
template <class A, class B>
constexpr int pair_min_blocks() {
  return (A::kMemoryBound && B::kMemoryBound) ? cmax(A::kMinBlocks, B::kMinBlocks)
                                              : cmin(4, cmax(A::kMinBlocks, B::kMinBlocks));
}

// A second, register-richer build of pairs with a memory-bound body, launched when its occupancy
// still holds the whole fused grid (so nothing is lost in waves).  Two memory-bound bodies: 4 CTAs
// per SM (64 registers) -- under the 40-register cap of the 6-CTA build the two inlined bodies spill.
// A memory-bound body beside a GEMM / conv body: 2 CTAs per SM (128 registers) -- the 64 registers
// of the default build make the tensor-core body's epilogue spill.  0: the pair has no second build.
template <class A, class B>
constexpr int pair_wide_blocks() {
  return (A::kMemoryBound && B::kMemoryBound) ? (pair_min_blocks<A, B>() > 4 ? 4 : 0)
                                              : ((A::kMemoryBound || B::kMemoryBound) && pair_min_blocks<A, B>() > 2 ? 2 : 0);
}

template <class A, class B, int MINB = pair_min_blocks<A, B>()>
__global__ void __launch_bounds__(cmax(A::kMaxThreads, B::kMaxThreads), MINB)
    fused_block_kernel(const __grid_constant__ DispatchTable t, const __grid_constant__ typename A::Params pa,
                       const __grid_constant__ typename B::Params pb) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = align_smem_1k(smem_raw);
  const int tid = threadIdx.x;
  unsigned long long t_entry = 0;
  if (t.cta_times) t_entry = global_timer_ns();
  // A kernel that contains tcgen05.alloc gets its CTAs launched one at a time per SM: the next CTA
  // starts only once the resident one has given up its permit to allocate tensor memory, and a CTA
  // that never allocates holds it until it exits.  So the CTAs of an operator without tensor memory
  // give the permit up before anything else (measured: 4 such CTAs per SM ran one after the other).
  if constexpr (A::kUsesTmem != B::kUsesTmem) {
    if (!t.queue && tid < 32) {
      int k0, vb0;
      const bool mapped = decode_cta(t, blockIdx.x, k0, vb0);
      if (!mapped || (k0 == 0 ? !A::kUsesTmem : !B::kUsesTmem)) relinquish_tmem_permit();
    }
  }
  // A persistent CTA of the work queue allocates the tensor memory its operators need ONCE, for all its
  // tickets, and gives the permit up at once: the SM starts the next CTA of a tcgen05 kernel only when the
  // resident one has given the permit up, so a persistent CTA that kept it for a later ticket held the SM's
  // second CTA off for the whole launch (batch-256 conv pair: 281 us, against 161 us for a plain launch).
  __shared__ unsigned queue_tmem_s;
  unsigned queue_tmem = 0;
  const int queue_tmem_cols = (A::kUsesTmem || B::kUsesTmem) && t.queue ? t.tmem_cols : 0;
  if (queue_tmem_cols > 0) {
    if (tid < 32) {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((unsigned)__cvta_generic_to_shared(&queue_tmem_s)),
                   "r"(queue_tmem_cols)
                   : "memory");
      relinquish_tmem_permit();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    queue_tmem = *reinterpret_cast<volatile unsigned *>(&queue_tmem_s);
  }
  if (t.queue) {   // the ticket counter is global memory; otherwise the body waits and lets the next kernel in (TileCtx::dependency_wait)
    grid_dependency_wait();
    // A queue launch with a tensor-memory operator does not let the next kernel in early: CTAs of a
    // following tensor-memory kernel, started early, allocate their columns before their own
    // griddepcontrol.wait and would hold them on this SM until this grid has finished, beside persistent
    // CTAs that are here for the whole launch.  Two memory-bound bodies keep the early trigger.
    if constexpr (!A::kUsesTmem && !B::kUsesTmem) grid_launch_dependents();
  }
  // One loop serves both launch forms, so each body is inlined once (two copies cost registers and
  // made the memory-bound pairs spill): a plain launch runs it for CTA blockIdx.x and leaves; a
  // persistent CTA of the work queue draws tickets until the queue is empty.  The last CTA to drain
  // resets the counters, so the next launch on the stream starts from zero without a memset.
  __shared__ int ticket_s;
  const bool queue = t.queue != 0;
  int ticket = blockIdx.x;
  do {
    if (queue) {
      if (tid == 0) ticket_s = (int)atomicAdd(t.queue_ctr, 1u);
      __syncthreads();
      ticket = ticket_s;
      __syncthreads();
      if (ticket >= t.total) break;
    }
    int k, vb;
    if (decode_cta(t, ticket, k, vb)) {
      unsigned long long t_body = 0;
      if (t.cta_times) t_body = global_timer_ns();
      // guard of the reference: KernelID_ == k && threadIdx.x < B_k (Algorithms.cc:699-717)
      if (k == 0) {
        if (tid < t.n_thr[0]) run_tile<A>(pa, t, 0, vb, tid, 1, smem, 0, queue_tmem_cols > 0, queue_tmem);
      } else {
        if (tid < t.n_thr[1]) run_tile<B>(pb, t, 1, vb, tid, 2, smem, 0, queue_tmem_cols > 0, queue_tmem);
      }
      if (t.cta_times && tid == 0) {  // kernel entry, body start (its set-up may overlap the previous kernel), thread 0 done
        t.cta_times[3 * (size_t)ticket] = t_entry;
        t.cta_times[3 * (size_t)ticket + 1] = t_body;
        t.cta_times[3 * (size_t)ticket + 2] = global_timer_ns();
      }
    }
  } while (queue);
  if (queue_tmem_cols > 0) {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(queue_tmem), "r"(queue_tmem_cols) : "memory");
  }
  if (queue && tid == 0) {
    __threadfence();
    if (atomicAdd(t.queue_ctr + 1, 1u) == gridDim.x - 1) {
      t.queue_ctr[0] = 0;
      t.queue_ctr[1] = 0;
      __threadfence();
    }
  }
}

template <class A, class B>
__global__ void __launch_bounds__(A::kMaxThreads + B::kMaxThreads, 1)
    fused_thread_kernel(const __grid_constant__ DispatchTable t, const __grid_constant__ typename A::Params pa,
                        const __grid_constant__ typename B::Params pb) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = align_smem_1k(smem_raw);
  const int tid = threadIdx.x, b = blockIdx.x;
  // the bodies wait for the previous kernel and let the next one in themselves (TileCtx::dependency_wait)
  // thread ranges of hfusePattern (Algorithms.cc:23-49): kernel k owns [thr_lo[k], thr_lo[k] + B_k)
  // An operator keeps its permit to allocate tensor memory only while the other one may still need it
  // (both allocate); when just one of them uses tensor memory it gives the permit up as it would alone,
  // and a CTA past that operator's grid gives it up on its behalf, so that the SM can start its next CTA.
  if (tid < t.thr_lo[1]) {
    if (tid < t.n_thr[0] && b < t.n_cta[0]) run_tile<A>(pa, t, 0, b, tid, 1, smem + t.smem_off[0], B::kUsesTmem ? 1 : 0);
    else if (A::kUsesTmem && !B::kUsesTmem && b >= t.n_cta[0] && tid < 32) relinquish_tmem_permit();
  } else {
    const int vt = tid - t.thr_lo[1];
    if (vt < t.n_thr[1] && b < t.n_cta[1]) run_tile<B>(pb, t, 1, b, vt, 2, smem + t.smem_off[1], A::kUsesTmem ? 1 : 0);
    else if (B::kUsesTmem && !A::kUsesTmem && b >= t.n_cta[1] && vt < 32) relinquish_tmem_permit();
  }
}

// Parameter blocks of a group, indexed by the operator the dispatch decode returns.
template <class A>
struct GroupParams {
  typename A::Params p[kGroupMax];
};

template <class A>
__global__ void __launch_bounds__(A::kMaxThreads, A::kMinBlocks)
    fused_group_kernel(const __grid_constant__ GroupTable t, const __grid_constant__ GroupParams<A> g) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = align_smem_1k(smem_raw);
  // the body waits for the previous kernel and lets the next one in itself (TileCtx::dependency_wait)
  int k, vb;
  if (!decode_group_cta(t, blockIdx.x, k, vb)) return;
  const int tid = threadIdx.x;
  if (tid >= t.n_thr[k]) return;   // guard of the reference: KernelID_ == k && threadIdx.x < B_k
  TileCtx c;
  c.vblock = vb;
  c.tid = tid;
  c.nthreads = t.n_thr[k];
  c.bar_id = 1;
  c.bar_count = t.bar_count[k];
  c.gx = t.grid_x[k];
  c.gy = t.grid_y[k];
  c.bx = t.blk_x[k];
  c.by = t.blk_y[k];
  c.smem = smem;
  c.status = t.status;
  c.persistent = 0;
  c.tmem_given = 0;
  c.tmem_base = 0;
  A::run(g.p[k], c);
}

// Up to four operators drawn from TWO bodies in one launch: the group's dispatch decode names the
// operator, the table says which body it runs and which of that body's parameter blocks is its own.
template <class A, class B>
__global__ void __launch_bounds__(cmax(A::kMaxThreads, B::kMaxThreads), pair_min_blocks<A, B>())
    fused_mixed_group_kernel(const __grid_constant__ GroupTable t, const __grid_constant__ GroupParams<A> ga,
                             const __grid_constant__ GroupParams<B> gb) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = align_smem_1k(smem_raw);
  const int tid = threadIdx.x;
  int k = 0, vb = 0;
  const bool mapped = decode_group_cta(t, blockIdx.x, k, vb);
  // as in fused_block_kernel: a CTA that will not allocate tensor memory gives the permit up at once
  if constexpr (A::kUsesTmem != B::kUsesTmem) {
    if (tid < 32 && (!mapped || (t.body[k] == 0 ? !A::kUsesTmem : !B::kUsesTmem))) relinquish_tmem_permit();
  }
  if (!mapped || tid >= t.n_thr[k]) return;   // guard of the reference: KernelID_ == k && threadIdx.x < B_k
  TileCtx c;
  c.vblock = vb;
  c.tid = tid;
  c.nthreads = t.n_thr[k];
  c.bar_id = 1 + t.body[k];
  c.bar_count = t.bar_count[k];
  c.gx = t.grid_x[k];
  c.gy = t.grid_y[k];
  c.bx = t.blk_x[k];
  c.by = t.blk_y[k];
  c.smem = smem;
  c.status = t.status;
  c.persistent = 0;
  c.tmem_given = 0;
  c.tmem_base = 0;
  if (t.body[k] == 0) A::run(ga.p[t.slot[k]], c);
  else B::run(gb.p[t.slot[k]], c);
}

template <class A>
__global__ void __launch_bounds__(A::kMaxThreads, A::kMinBlocks)
    single_kernel(const __grid_constant__ DispatchTable t, const __grid_constant__ typename A::Params pa) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *smem = align_smem_1k(smem_raw);
  // the body waits for the previous kernel and lets the next one in itself (TileCtx::dependency_wait)
  if ((int)threadIdx.x < t.n_thr[0]) run_tile<A>(pa, t, 0, blockIdx.x, threadIdx.x, 1, smem);
}

// ---- host-side typed launchers, stored type-erased in the pair table ---------------------------

typedef cudaError_t (*PairLaunchFn)(const DispatchTable &, const void *pa, const void *pb, unsigned grid,
                                    unsigned block, size_t smem, cudaStream_t);
typedef cudaError_t (*SingleLaunchFn)(const DispatchTable &, const void *pa, unsigned grid, unsigned block,
                                      size_t smem, cudaStream_t);
typedef cudaError_t (*GroupLaunchFn)(const GroupTable &, const void *const *params, int n, unsigned grid, unsigned block,
                                     size_t smem, cudaStream_t);
typedef cudaError_t (*MixedGroupLaunchFn)(const GroupTable &, const void *const *params_a, int na, const void *const *params_b, int nb,
                                          unsigned grid, unsigned block, size_t smem, cudaStream_t);
typedef cudaError_t (*AttrFn)(cudaFuncAttributes *);
typedef int (*ClusterCapFn)(unsigned block, size_t smem, int cluster);

template <class Kernel>
cudaError_t ensure_smem(Kernel k, size_t smem) {
  if (smem <= 48 * 1024) return cudaSuccess;
  return cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
}

// Launch with `cluster` consecutive CTAs per thread-block cluster (1 = no clusters) and with
// programmatic dependent launch allowed unless the dispatch table says otherwise (no_pdl, set from the
// context's switch bfuse_set_dependent_launch: a diagnostic to tell the overlap's effect on a timeline
// from everything else).
template <class Kernel, class... Args>
cudaError_t launch_clustered(Kernel kern, unsigned grid, unsigned block, size_t smem, cudaStream_t s, int cluster, bool pdl,
                             Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = cluster > 1 ? cluster : 1;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

// Thread-block clusters of `cluster` CTAs of this kernel that can be resident at once (a cluster must
// fit one GPC, so this is less than SMs * CTAs-per-SM / cluster); -1 when the query fails.
template <class Kernel>
int max_resident_clusters(Kernel kern, unsigned block, size_t smem, int cluster) {
  if (ensure_smem(kern, smem) != cudaSuccess) return -1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)cluster, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return -1;
  }
  return n;
}
template <class A, class B>
int clusters_block_pair(unsigned block, size_t smem, int cluster) {
  return max_resident_clusters(fused_block_kernel<A, B>, block, smem, cluster);
}
template <class A, class B>
int clusters_block_pair_wide(unsigned block, size_t smem, int cluster) {
  return max_resident_clusters(fused_block_kernel<A, B, pair_wide_blocks<A, B>()>, block, smem, cluster);
}
template <class A>
int clusters_group(unsigned block, size_t smem, int cluster) {
  return max_resident_clusters(fused_group_kernel<A>, block, smem, cluster);
}

template <class A, class B>
cudaError_t launch_block_pair(const DispatchTable &t, const void *pa, const void *pb, unsigned grid, unsigned block,
                              size_t smem, cudaStream_t s) {
  cudaError_t e = ensure_smem(fused_block_kernel<A, B>, smem);
  if (e != cudaSuccess) return e;
  return launch_clustered(fused_block_kernel<A, B>, grid, block, smem, s, t.cluster, !t.no_pdl, t,
                          *static_cast<const typename A::Params *>(pa), *static_cast<const typename B::Params *>(pb));
}
template <class A, class B>
cudaError_t launch_thread_pair(const DispatchTable &t, const void *pa, const void *pb, unsigned grid, unsigned block,
                               size_t smem, cudaStream_t s) {
  cudaError_t e = ensure_smem(fused_thread_kernel<A, B>, smem);
  if (e != cudaSuccess) return e;
  return launch_clustered(fused_thread_kernel<A, B>, grid, block, smem, s, 1, !t.no_pdl, t,
                          *static_cast<const typename A::Params *>(pa), *static_cast<const typename B::Params *>(pb));
}
template <class A>
cudaError_t launch_single(const DispatchTable &t, const void *pa, unsigned grid, unsigned block, size_t smem,
                          cudaStream_t s) {
  cudaError_t e = ensure_smem(single_kernel<A>, smem);
  if (e != cudaSuccess) return e;
  return launch_clustered(single_kernel<A>, grid, block, smem, s, t.cluster, !t.no_pdl, t,
                          *static_cast<const typename A::Params *>(pa));
}
template <class A>
cudaError_t launch_group(const GroupTable &t, const void *const *params, int n, unsigned grid, unsigned block, size_t smem,
                         cudaStream_t s) {
  cudaError_t e = ensure_smem(fused_group_kernel<A>, smem);
  if (e != cudaSuccess) return e;
  GroupParams<A> g;
  for (int i = 0; i < kGroupMax; ++i) g.p[i] = *static_cast<const typename A::Params *>(params[i < n ? i : 0]);
  return launch_clustered(fused_group_kernel<A>, grid, block, smem, s, t.cluster, !t.no_pdl, t, g);
}
template <class A>
cudaError_t attr_group(cudaFuncAttributes *a) { return cudaFuncGetAttributes(a, fused_group_kernel<A>); }
template <class A, class B>
cudaError_t launch_mixed_group(const GroupTable &t, const void *const *pa, int na, const void *const *pb, int nb, unsigned grid,
                               unsigned block, size_t smem, cudaStream_t s) {
  cudaError_t e = ensure_smem(fused_mixed_group_kernel<A, B>, smem);
  if (e != cudaSuccess) return e;
  GroupParams<A> ga;
  GroupParams<B> gb;
  for (int i = 0; i < kGroupMax; ++i) {
    ga.p[i] = *static_cast<const typename A::Params *>(pa[i < na ? i : 0]);
    gb.p[i] = *static_cast<const typename B::Params *>(pb[i < nb ? i : 0]);
  }
  return launch_clustered(fused_mixed_group_kernel<A, B>, grid, block, smem, s, t.cluster, !t.no_pdl, t, ga, gb);
}
template <class A, class B>
cudaError_t attr_mixed_group(cudaFuncAttributes *a) { return cudaFuncGetAttributes(a, fused_mixed_group_kernel<A, B>); }
template <class A, class B>
int clusters_mixed_group(unsigned block, size_t smem, int cluster) {
  return max_resident_clusters(fused_mixed_group_kernel<A, B>, block, smem, cluster);
}
template <class A, class B>
cudaError_t launch_block_pair_wide(const DispatchTable &t, const void *pa, const void *pb, unsigned grid, unsigned block,
                                   size_t smem, cudaStream_t s) {
  cudaError_t e = ensure_smem(fused_block_kernel<A, B, pair_wide_blocks<A, B>()>, smem);
  if (e != cudaSuccess) return e;
  return launch_clustered(fused_block_kernel<A, B, pair_wide_blocks<A, B>()>, grid, block, smem, s, t.cluster, !t.no_pdl, t,
                          *static_cast<const typename A::Params *>(pa), *static_cast<const typename B::Params *>(pb));
}
template <class A, class B>
cudaError_t attr_block_pair_wide(cudaFuncAttributes *a) {
  return cudaFuncGetAttributes(a, fused_block_kernel<A, B, pair_wide_blocks<A, B>()>);
}
template <class A, class B>
cudaError_t attr_block_pair(cudaFuncAttributes *a) { return cudaFuncGetAttributes(a, fused_block_kernel<A, B>); }
template <class A, class B>
cudaError_t attr_thread_pair(cudaFuncAttributes *a) { return cudaFuncGetAttributes(a, fused_thread_kernel<A, B>); }
template <class A>
cudaError_t attr_single(cudaFuncAttributes *a) { return cudaFuncGetAttributes(a, single_kernel<A>); }

}  // namespace bfuse
