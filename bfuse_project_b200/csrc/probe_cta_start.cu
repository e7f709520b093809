// Diagnostic: when does an SM start the 2nd, 3rd ... CTA of a kernel?  Every CTA records its entry
// time and SM and then spins for spin_ns (bounded).  Variants: plain kernels of different register
// and shared-memory footprints; kernels that allocate tensor memory and give the allocation permit
// up at once, or keep it to the end; a kernel that only contains the allocation code and never runs
// it, with and without tcgen05.relinquish_alloc_permit at entry.  The answer decides how the fused
// kernels order their first instructions (fused_kernels.cuh, ops_umma.cuh).  No wait is unbounded:
// a CTA that blocks in tcgen05.alloc is released when its neighbour's bounded spin ends.
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <algorithm>
#include <cuda_runtime.h>
__device__ __forceinline__ unsigned long long gt() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
template <int TMEM, int REGS>
__global__ void __launch_bounds__(192, 1) probe(unsigned long long *t, int *sm, int spin_ns, float *sink, int use_tmem = 1) {
  extern __shared__ unsigned char smem[];
  __shared__ uint32_t slot;
  const unsigned long long t0 = gt();
  unsigned s; asm volatile("mov.u32 %0, %%smid;" : "=r"(s));
  float acc[REGS];
  #pragma unroll
  for (int i = 0; i < REGS; ++i) acc[i] = threadIdx.x * 0.5f + i;
  if (TMEM == 4 && threadIdx.x / 32 == 5) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  if (TMEM && use_tmem && threadIdx.x / 32 == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"((uint32_t)__cvta_generic_to_shared(&slot)), "r"(32u) : "memory");
    if (TMEM == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  __syncthreads();
  const unsigned long long t1 = gt();
  int guard = 0;
  while (gt() - t0 < (unsigned long long)spin_ns && guard < 2000000) {
    ++guard;
    #pragma unroll
    for (int i = 0; i < REGS; ++i) acc[i] = acc[i] * 1.0001f + 0.5f;
  }
  __syncthreads();
  if (TMEM && use_tmem && threadIdx.x / 32 == 5) {
    if (TMEM == 2) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(slot), "r"(32u) : "memory");
  }
  float sum = 0;
  #pragma unroll
  for (int i = 0; i < REGS; ++i) sum += acc[i];
  if (sum == 12345.678f) sink[0] = sum + smem[threadIdx.x];
  if (threadIdx.x == 0) { t[3 * blockIdx.x] = t0; t[3 * blockIdx.x + 1] = t1; t[3 * blockIdx.x + 2] = gt(); sm[blockIdx.x] = (int)s; }
}
template <class K>
void run(const char *tag, K kern, int grid, size_t smem, int spin_ns, int use_tmem = 1) {
  cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  cudaFuncAttributes a; cudaFuncGetAttributes(&a, kern);
  int occ = 0; cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kern, 192, smem);
  unsigned long long *t; int *sm; float *sink;
  cudaMalloc(&t, 3 * 8 * grid); cudaMalloc(&sm, 4 * grid); cudaMalloc(&sink, 4);
  for (int rep = 0; rep < 3; ++rep) { kern<<<grid, 192, smem>>>(t, sm, spin_ns, sink, use_tmem); }
  cudaError_t e = cudaDeviceSynchronize();
  std::vector<unsigned long long> h(3 * grid); std::vector<int> hs(grid);
  cudaMemcpy(h.data(), t, 3 * 8 * grid, cudaMemcpyDeviceToHost); cudaMemcpy(hs.data(), sm, 4 * grid, cudaMemcpyDeviceToHost);
  unsigned long long t0 = h[0]; for (int i = 0; i < grid; ++i) t0 = std::min(t0, h[3 * i]);
  // per SM: sort entries
  std::vector<std::vector<long long>> per(256);
  long long last_end = 0;
  for (int i = 0; i < grid; ++i) { per[hs[i]].push_back((long long)(h[3 * i] - t0)); last_end = std::max(last_end, (long long)(h[3 * i + 2] - t0)); }
  std::vector<long long> first, second, third;
  for (auto &v : per) { std::sort(v.begin(), v.end()); if (v.size() > 0) first.push_back(v[0]); if (v.size() > 1) second.push_back(v[1]); if (v.size() > 2) third.push_back(v[2]); }
  auto med = [](std::vector<long long> &v) { if (v.empty()) return -1LL; std::sort(v.begin(), v.end()); return v[v.size() / 2]; };
  auto mx = [](std::vector<long long> &v) { return v.empty() ? -1LL : *std::max_element(v.begin(), v.end()); };
  printf("%-34s regs %3d occ/SM %d grid %d smem %6zu spin %d | 1st CTA on SM: med %5lld max %5lld | 2nd: n %3zu med %5lld max %5lld | 3rd: n %3zu med %5lld | last end %6lld  %s\n",
         tag, a.numRegs, occ, grid, smem, spin_ns, med(first), mx(first), second.size(), med(second), mx(second), third.size(), med(third), last_end, e == cudaSuccess ? "" : cudaGetErrorString(e));
  cudaFree(t); cudaFree(sm); cudaFree(sink);
}
int main() {
  for (int spin : {4000}) {
    run("plain r16 smem 0", probe<0, 16>, 296, 0, spin);
    run("plain r16 smem 45K", probe<0, 16>, 296, 45056, spin);
    run("plain r16 smem 100K", probe<0, 16>, 296, 100 * 1024, spin);
    run("plain r96 smem 45K", probe<0, 96>, 296, 45056, spin);
    run("plain r96 smem 45K grid 196", probe<0, 96>, 196, 45056, spin);
    run("tmem+relinquish r16 smem 45K", probe<1, 16>, 296, 45056, spin);
    run("tmem+relinquish r96 smem 45K", probe<1, 96>, 296, 45056, spin);
    run("tmem keep permit r16 smem 45K", probe<2, 16>, 296, 45056, spin);
    run("tmem+relinquish r16 smem 0", probe<1, 16>, 296, 0, spin);
    run("alloc code present, never run", probe<3, 16>, 592, 0, spin, 0);
    run("same + relinquish at entry", probe<4, 16>, 592, 0, spin, 0);
    run("tmem+relinquish r16 grid 592", probe<1, 16>, 592, 0, spin);
  }
  return 0;
}
