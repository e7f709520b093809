// The common tile interface every operator body is written against.
//
// The reference rewrites each kernel so that blockIdx / threadIdx / blockDim / gridDim become
// locals fed by the dispatcher (horizontal-fuser/src/Matchers.cc:255-286) and, for thread-level
// fusion, __syncthreads() becomes `bar.sync <k+1>, <round32(B_k)>` (Matchers.cc:288-320).  A body
// here never touches the hardware indices: it sees a TileCtx with its virtual block, its virtual
// thread, its own named barrier and its own shared-memory window, so the same body runs unfused,
// block-fused, thread-fused or from a persistent work queue and produces identical bits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace bfuse {

struct TileCtx {
  int vblock;     // linear virtual block id in [0, G_k)
  int tid;        // linear virtual thread id in [0, B_k)
  int nthreads;   // B_k
  int bar_id;     // named barrier owned by this operator (0 when it owns the whole CTA)
  int bar_count;  // B_k rounded up to a multiple of 32
  int gx, gy;     // GridDim.X / .Y for the blockIdx decomposition
  int bx, by;     // BlockDim.X / .Y for the threadIdx decomposition
  unsigned char *smem;  // this operator's shared-memory window, 1024-byte aligned
  int *status;          // device status word (bounded waits report here)
  int persistent;       // 1: more tensor-memory allocations may follow in this CTA (work queue: the next
                        // tile; thread split: the other operator), so the allocation permit must be kept
  unsigned tmem_base;   // tmem_given: the tensor-memory columns the CTA already holds for this operator (a persistent
  int tmem_given;       // CTA of the work queue allocates once for all its tickets); the body neither allocates nor frees

  // Programmatic dependent launch: the CTA may have started while the previous kernel on the stream
  // was still running.  Every thread calls this before its first access to global memory; what comes
  // before it (tensor-memory allocation, barrier set-up, tables in shared memory) overlaps that
  // kernel's tail.  Returns at once when there is nothing to wait for.
  // Only then is the next kernel allowed to start its CTAs: were it allowed earlier, CTAs of several
  // queued launches would pile up on whatever SMs had room first, holding tensor memory and slots.
  __device__ __forceinline__ void dependency_wait() const {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }

  __device__ __forceinline__ void sync() const {
    asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(bar_count) : "memory");
  }
  // blockIdx_{x,y,z}_ / threadIdx_{x,y,z}_ exactly as Algorithms.cc:687-692 derives them
  __device__ __forceinline__ int block_x() const { return vblock % gx; }
  __device__ __forceinline__ int block_y() const { return vblock / gx % gy; }
  __device__ __forceinline__ int block_z() const { return vblock / (gx * gy); }
  __device__ __forceinline__ int thread_x() const { return tid % bx; }
  __device__ __forceinline__ int thread_y() const { return tid / bx % by; }
  __device__ __forceinline__ int thread_z() const { return tid / (bx * by); }
};

// ---- small device helpers shared by the memory-bound bodies ----------------------------------

__device__ __forceinline__ float4 ld_stream_f4(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_stream_u4(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream_f4(float4 *p, float4 v) {
  asm volatile("st.global.cs.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_stream_u4(uint4 *p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Start fetching the line at p into L1 / L2 without tying up a register: for small per-column
// tables (gamma, beta, weights) that a body needs only after its reductions.  Issued next to the
// row loads, the fetch shares their trip to DRAM; left to the point of use it would queue behind
// every load the grid has in flight and cost a second full round trip.
__device__ __forceinline__ void prefetch_l1(const void *p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }

struct OpSum {
  __device__ __forceinline__ static float apply(float a, float b) { return a + b; }
};
struct OpMax {
  __device__ __forceinline__ static float apply(float a, float b) { return fmaxf(a, b); }
};

// Reduce `v` over the `tpr` consecutive threads that share a row (tpr a power of two).  Warp
// shuffles first; rows wider than a warp exchange one partial per warp through slot `slot` of the
// operator's shared-memory window and meet on the operator's named barrier.  Successive
// reductions in one tile use different slots, which keeps the barrier count at one per reduction.
template <class Op>
__device__ __forceinline__ float row_reduce(float v, const TileCtx &c, int tpr, int slot) {
  const int width = tpr < 32 ? tpr : 32;
  for (int off = width >> 1; off > 0; off >>= 1) v = Op::apply(v, __shfl_xor_sync(0xffffffffu, v, off));
  if (tpr > 32) {
    float *s = reinterpret_cast<float *>(c.smem) + slot * 32;
    if ((c.tid & 31) == 0) s[c.tid >> 5] = v;
    c.sync();
    const int wpr = tpr >> 5, w0 = (c.tid / tpr) * wpr;
    float r = s[w0];
    for (int j = 1; j < wpr; ++j) r = Op::apply(r, s[w0 + j]);
    v = r;
  }
  return v;
}

}  // namespace bfuse
