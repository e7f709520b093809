// bfuse_softmax_layernorm_queue_noalloc: the persistent work-queue launch of the softmax ||
// LayerNorm pair for callers that must not allocate.
//
// Who needs this: code that runs after a process has handed all of its device memory to a pool
// (an inference server's arena, a framework's caching allocator), or inside a latency-critical
// loop where cudaMalloc / cudaFree are unacceptable because they synchronise the whole device.
// The regular path (bfuse_register_fusion with BFUSE_PATTERN_WORK_QUEUE) cudaMallocs the two
// queue counters per fusion and keeps its registry on the host heap; this entry point does
// neither.  Its only scratch -- the ticket counter and the drained-CTA counter of the queue --
// lives in the file-scope device array below, which every GPU that loads this library carries
// (256 bytes) until the process exits.
//
// Things a caller has to know:
//   * The first call on each device looks up the array's device address (cudaGetSymbolAddress)
//     and the kernel's attributes.  Make that first call outside any stream capture.
//   * All calls on a device share the one array.  Each call zeroes the two counters on the
//     caller's stream before it launches, so a launch that was aborted earlier cannot poison the
//     next one; but two calls whose kernels overlap on the GPU (different streams, no ordering
//     between them) race on the counters and will mis-distribute work.  Serialise them.
//   * The queue holds at most BFUSE_NOALLOC_MAX_TICKETS tickets (fused CTAs of both operators).
//     Larger problems are rejected with BFUSE_ERR_SHAPE and a message on stderr.
//   * Inputs and outputs are the caller's device buffers, 16-byte aligned, exactly as for the
//     registered path; results are bit-identical to it (same operator bodies, same tilings).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/bfuse_b200.h"
#include "fused_kernels.cuh"
#include "ops_rowwise.cuh"
#include "scheduler.h"

using namespace bfuse;

namespace {

constexpr int kScratchWords = 64;  // 256 bytes; words 0 and 1 are the queue counters
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned int g_noalloc_scratch[kScratchWords];

struct DeviceSetup {
  std::once_flag once;    // the first call on a device fills the rest; concurrent first calls wait for it
  int status;             // BFUSE_OK, or why the set-up failed (kept: later calls report it again)
  const char *why;
  unsigned int *scratch;  // device address of g_noalloc_scratch on this device
  int sm_count;
  int ctas_per_sm;
};
DeviceSetup g_setup[kMaxDevices];

int reject(int code, const char *msg) {
  fprintf(stderr, "bfuse_softmax_layernorm_queue_noalloc: %s\n", msg);
  return code;
}

bool misaligned(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; }

}  // namespace

extern "C" int bfuse_softmax_layernorm_queue_noalloc(const float *sm_x, float *sm_y, int sm_rows, int sm_cols,
                                                     float sm_scale, const float *ln_x, const float *ln_res,
                                                     const float *ln_gamma, const float *ln_beta, float *ln_y,
                                                     int ln_rows, int ln_cols, float ln_eps, void *stream) {
  if (!sm_x || !sm_y || !ln_x || !ln_gamma || !ln_beta || !ln_y) return reject(BFUSE_ERR_INVALID, "null buffer");
  if (misaligned(sm_x) || misaligned(sm_y) || misaligned(ln_x) || misaligned(ln_res) || misaligned(ln_gamma) ||
      misaligned(ln_beta) || misaligned(ln_y))
    return reject(BFUSE_ERR_INVALID, "buffers must be 16-byte aligned");
  if (sm_rows <= 0 || sm_cols <= 0 || ln_rows <= 0 || ln_cols <= 0) return reject(BFUSE_ERR_SHAPE, "rows and cols must be positive");
  const int tpr_a = pick_row_threads(sm_cols, 4, kRowMaxVec), tpr_b = pick_row_threads(ln_cols, 4, kRowMaxVec);  // the registered path's rule
  if (!tpr_a || !tpr_b) return reject(BFUSE_ERR_SHAPE, "cols must be a multiple of 4 * (power-of-two threads per row), at most 4096");
  const int rpc_a = 256 / tpr_a, rpc_b = 256 / tpr_b;
  const long long ctas_a = ((long long)sm_rows + rpc_a - 1) / rpc_a, ctas_b = ((long long)ln_rows + rpc_b - 1) / rpc_b;
  if (ctas_a + ctas_b > BFUSE_NOALLOC_MAX_TICKETS)
    return reject(BFUSE_ERR_SHAPE, "more than BFUSE_NOALLOC_MAX_TICKETS (1048576) work-queue tickets; split the problem");

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) return reject(BFUSE_ERR_DEVICE, "no current CUDA device");
  DeviceSetup &su = g_setup[dev];
  auto kernel = fused_block_kernel<SoftmaxF32, LayerNormF32>;
  std::call_once(su.once, [&] {
    // once per device, with that device current: the array's name is a host-side handle, the
    // kernel needs its device address
    su.status = BFUSE_OK;
    void *ptr = nullptr;
    cudaError_t e1 = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e1 != cudaSuccess || !ptr) { su.status = BFUSE_ERR_CUDA, su.why = cudaGetErrorString(e1); return; }
    int major = 0, sms = 0;
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (major != 10 || sms <= 0) { su.status = BFUSE_ERR_DEVICE, su.why = "not an sm_100 device"; return; }
    cudaFuncAttributes attr;
    e1 = cudaFuncGetAttributes(&attr, kernel);
    if (e1 != cudaSuccess) { su.status = BFUSE_ERR_CUDA, su.why = cudaGetErrorString(e1); return; }
    const int by_regs = 65536 / (attr.numRegs * 256 > 0 ? attr.numRegs * 256 : 1);
    su.ctas_per_sm = by_regs < 1 ? 1 : (by_regs > 8 ? 8 : by_regs);
    su.sm_count = sms;
    su.scratch = static_cast<unsigned int *>(ptr);
  });
  if (su.status != BFUSE_OK) return reject(su.status, su.why);

  const KernelDims kd[2] = {{(int)ctas_a, 1, 1, tpr_a, rpc_a, 1}, {(int)ctas_b, 1, 1, tpr_b, rpc_b, 1}};
  FusedPlan plan;
  if (!plan_pair(kd, PATTERN_WORK_QUEUE, 1, 1, 0, &plan, nullptr)) return reject(BFUSE_ERR_INVALID, "scheduler rejected the pair");
  plan.table.queue_ctr = su.scratch;
  plan.table.status = nullptr;  // the row-wise bodies have no bounded waits to report
  const SoftmaxF32::Params pa{sm_x, sm_y, sm_rows, sm_cols, sm_scale};
  const LayerNormF32::Params pb{ln_x, ln_res, ln_gamma, ln_beta, ln_y, ln_rows, ln_cols, ln_eps};
  const int resident = su.ctas_per_sm * su.sm_count;
  const unsigned grid = (unsigned)(plan.table.total < resident ? plan.table.total : resident);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call left: the counters must start at zero
  e = cudaMemsetAsync(su.scratch, 0, 2 * sizeof(unsigned int), s);
  if (e != cudaSuccess) return reject(BFUSE_ERR_CUDA, cudaGetErrorString(e));
  kernel<<<grid, 256, 256 + 1024, s>>>(plan.table, pa, pb);
  e = cudaGetLastError();
  if (e != cudaSuccess) return reject(BFUSE_ERR_CUDA, cudaGetErrorString(e));
  return BFUSE_OK;
}
