/*
 * bfuse_b200 -- C ABI of the B200 horizontal-fusion runtime.
 *
 * A caller registers two independent kernels (operator body, grid / block dims, shared-memory
 * size, argument buffers) and a block-dispatch pattern; the runtime launches ONE fused sm_100a
 * kernel whose CTAs run work from both.  Plain pointers and sizes only; every call returns a
 * status code (the reference exits the process on error instead:
 * test-utils/test-suite-files/operation_cu.py:111-121, horizontal-fuser/include/fuse/Utils.h:14-21).
 *
 * Each declaration cites the reference interface it replaces (paths relative to the reference
 * repository).
 */
#ifndef BFUSE_B200_H
#define BFUSE_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BFUSE_MAX_ARGS 6
#define BFUSE_MAX_SHAPE 12

/* status codes */
enum {
  BFUSE_OK = 0,
  BFUSE_ERR_INVALID = 1,     /* bad argument / handle / unknown operator            */
  BFUSE_ERR_SHAPE = 2,       /* shape or launch dims the operator body cannot run   */
  BFUSE_ERR_SMEM = 3,        /* shared memory over the per-CTA budget               */
  BFUSE_ERR_CUDA = 4,        /* a CUDA call failed; see bfuse_last_error            */
  BFUSE_ERR_DEVICE = 5,      /* not an sm_100 device / driver entry point missing   */
  BFUSE_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up (status word set) */
  BFUSE_ERR_UNSUPPORTED = 7  /* pattern not available for this pair                 */
};

/* operator bodies in the registry (replaces the generated dense / bgemm / conv2d kernels,
 * scripts/configure_kernels.py:40-68, and adds the memory-bound operators) */
enum {
  BFUSE_OP_SOFTMAX_F32 = 0,   /* args: x, y                      shape: rows, cols            fparam: scale */
  BFUSE_OP_LAYERNORM_F32 = 1, /* args: x, res|NULL, gamma, beta, y   shape: rows, cols        fparam: eps   */
  BFUSE_OP_RMSNORM_BF16 = 2,  /* args: x, w, y                   shape: rows, cols            fparam: eps   */
  BFUSE_OP_ROPE_BF16 = 3,     /* args: q, inv_freq, y            shape: seq, heads, dim                     */
  BFUSE_OP_GEMM_F32_SIMT = 4, /* args: A, W, bias|NULL, out      shape: batch, M, N, K                      */
  BFUSE_OP_CONV2D_F32_SIMT = 5, /* args: x, w, y   shape: n, ci, h, w, co, kh, kw, stride, pad             */
  BFUSE_OP_GEMM_TF32 = 6,     /* as GEMM_F32_SIMT, tcgen05 kind::tf32; shape[4] = BN tile width (32..256),   */
                              /* shape[5] = k-slices per tile (a thread-block cluster reduces them),        */
                              /* shape[6] = BM tile height (128, or 256 with one k-slice); 0 = runtime's choice */
  BFUSE_OP_GEMM_BF16 = 7,     /* bf16 A, W, out; fp32 accumulate; tcgen05 kind::f16; shape[4..6] as above    */
  BFUSE_OP_CONV2D_TF32 = 8,   /* as CONV2D_F32_SIMT on tcgen05 kind::tf32 (implicit GEMM); shape[9] = output */
                              /* pixels per tile (32, 64, 128), shape[10] = k-slices per tile (a cluster    */
                              /* reduces them), shape[11] = how the im2col operand is built: 1 staged (input */
                              /* rows by TMA into shared memory, im2col rows written from there into tensor  */
                              /* memory; needs 128-pixel tiles, one k-slice, ci*kh*kw a multiple of 32 and   */
                              /* image rows of 16-byte multiples), 2 gathered from global memory; 0: chosen  */
                              /* by bfuse_default_launch (staged wherever it can be), which writes 1 or 2    */
                              /* back; a kernel registered with 0 is gathered                                */
  BFUSE_OP_COUNT = 9
};

/* operator flags */
#define BFUSE_FLAG_CAUSAL 1u /* GEMM: out[b,m,n] = -FLT_MAX where n > m */
/* Hint to bfuse_default_launch: n operators (1..4) will share the launch, so tile this one for 1/n of
 * the SMs; 1 = it runs alone.  Absent = 2, a pair.  Never changes results except through the k-slices. */
#define BFUSE_FLAG_SHARE(n) ((unsigned)(n) << 8)

/* block-dispatch patterns (horizontal-fuser/src/Algorithms.cc) */
enum {
  BFUSE_PATTERN_ZIGZAG = 0,       /* coarseInterleaveWithoutSMPattern2, :528-739; param_m = M, param_n = N */
  BFUSE_PATTERN_PROPORTIONAL = 1, /* coarseInterleaveWithoutSMPattern,  :319-526; param_m = MinOption       */
  BFUSE_PATTERN_SM_STRIPED = 2,   /* coarseInterleavePattern, :118-317; param_m = TotalSM (0: this device)  */
  BFUSE_PATTERN_THREAD_SPLIT = 3, /* hfusePattern, :19-116, with bar.sync <k+1>, <round32(B_k)>             */
  BFUSE_PATTERN_RANGE_SPLIT = 4,  /* contiguous ranges: the tail rule of :661-685 applied to all blocks     */
  BFUSE_PATTERN_WORK_QUEUE = 5    /* persistent CTAs drawing zig-zag tickets from an atomic counter; the    */
                                  /* dynamic form of legacy/tests/thread_pooling_test/temp.cu:576-612       */
};

/* GridDim / BlockDim (horizontal-fuser/include/fuse/Contexts.h:13-25) */
typedef struct {
  int X, Y, Z;
} bfuse_dim3;

/* KernelInfo (horizontal-fuser/include/fuse/Contexts.h:27-50; YAML keys include/fuse/Utils.h:69-80)
 * extended by what the reference takes from the kernel source instead: the operator body, its
 * dynamic shared-memory size and its argument buffers. */
typedef struct {
  const char *KernelName;
  int HasBarriers;
  bfuse_dim3 GridDim;
  bfuse_dim3 BlockDim;
  int Reg;        /* filled on output with the registers per thread of the launched kernel */
  float ExecTime; /* optional, -1 when unknown */
  int op;                    /* BFUSE_OP_*                                                      */
  size_t smem_bytes;         /* dynamic shared memory of the body at these dims                 */
  void *args[BFUSE_MAX_ARGS]; /* DEVICE pointers in the operator's argument order               */
  int nargs;
  int shape[BFUSE_MAX_SHAPE];
  float fparam[4];
  unsigned flags;
} bfuse_kernel_desc;

typedef struct bfuse_context bfuse_context;

/* One context per device; owns the registry, dispatch tables, two streams for the parallel
 * baseline (S1 / S2 of operation_cu.py:126), the work-queue counters and the status word. */
int bfuse_create(int device, bfuse_context **out);
int bfuse_destroy(bfuse_context *ctx);
const char *bfuse_last_error(const bfuse_context *ctx);
int bfuse_device_sm_count(const bfuse_context *ctx); /* replaces TotalSM = 84, src/Contexts.cc:64-65 */

/* Fill GridDim / BlockDim / smem_bytes / nargs with the body's default tiling for desc->op and
 * desc->shape (the dims the reference extracts from TVM, scripts/configure_kernels.py:73-99). */
int bfuse_default_launch(const bfuse_context *ctx, bfuse_kernel_desc *desc);
/* Size in bytes and direction of argument i of a described kernel (what run_kernel1 derives from
 * I_shape / F_shape / O_shape, operation_cu.py:164-182). */
int bfuse_arg_info(const bfuse_context *ctx, const bfuse_kernel_desc *desc, int i, size_t *bytes, int *is_output);

/* kernels.yaml entry -> handle (include/fuse/Utils.h:69-80; macro_h.py ASSIGN_KERNEL1/2). */
int bfuse_register_kernel(bfuse_context *ctx, const bfuse_kernel_desc *desc, int *kernel);
/* Rebind the device buffers of a registered kernel (same shapes). */
int bfuse_set_kernel_args(bfuse_context *ctx, int kernel, void *const *args, int nargs);
/* Release a kernel / fusion / group (finalize_kernel1/2 of the reference harness,
 * test-utils/test-suite-files/operation_cu.py:146-162): frees what the runtime holds for it (records,
 * work-queue counters) and makes the handle invalid; later registrations may reuse it.  The caller's
 * buffers are untouched.  Order: graphs that captured a fusion first (bfuse_graph_destroy), then
 * fusions and groups, then their kernels; out of order returns BFUSE_ERR_INVALID and releases nothing.
 * Releasing a work-queue fusion synchronises the device. */
int bfuse_unregister_kernel(bfuse_context *ctx, int kernel);
int bfuse_unregister_fusion(bfuse_context *ctx, int fusion);
int bfuse_unregister_group(bfuse_context *ctx, int group);

/* fusions.yaml entry {Kernels: [k1, k2]} + pattern -> fused handle: the work of fuse::bfuse /
 * fuse::hfuse (horizontal-fuser/include/fuse/Fuse.h:43-49, src/Fuse.cc:64-221,223-376). */
int bfuse_register_fusion(bfuse_context *ctx, int kernel1, int kernel2, int pattern, int param_m, int param_n,
                          int *fusion);
/* The record fuse::bfuse / hfuse write to {b,h}fuse_kernels.yaml (src/Fuse.cc:203-220,358-375):
 * name "<k1>_<k2>_fused_{bfuse,hfuse}", fused GridDim / BlockDim, plus smem and registers;
 * shape[0] = CTAs launched, shape[1] = CTAs of the kernel resident at once according to cudaOccupancyMaxActiveClusters,
 * which counts one CTA per SM for kernels that allocate tensor memory (0: not asked).
 * shape[2] / shape[3] = 1 when kernel 1 / 2 runs in this fusion with ONE k-slice although it was
 * registered with several: BFUSE_PATTERN_THREAD_SPLIT and BFUSE_PATTERN_WORK_QUEUE cannot host
 * operators launched as thread-block clusters, so such an operator is re-tiled unsplit for the fusion
 * (all launch modes of the fusion use that tiling; its sums differ in the last bits from the k-split
 * kernel launched through its own handle).
 * out->KernelName points into the context and stays valid until bfuse_destroy. */
int bfuse_fusion_info(bfuse_context *ctx, int fusion, bfuse_kernel_desc *out);
/* Which operator and virtual block CTA (or queue ticket) b runs: the if / else-if chain the
 * reference prints at the top of a fused kernel (e.g. tests/benchmark/cuda/dense1_0_dense2_6_bfuse.cu:15-63).
 * Returns BFUSE_ERR_INVALID for an unmapped b. */
int bfuse_fusion_map_block(const bfuse_context *ctx, int fusion, int b, int *kernel, int *vblock);
/* Thread-split fusions: does fused thread t of CTA b run `kernel`?  Fills its virtual ids. */
int bfuse_fusion_map_thread(const bfuse_context *ctx, int fusion, int kernel, int b, int t, int *vblock,
                            int *vthread, int *active);

/* n kernels in one fused launch -- the general form the reference's patterns are written in
 * (a `Kernels:` list of any length, horizontal-fuser/src/Algorithms.cc:323-375, 538-587, 661-685),
 * here for 2..BFUSE_GROUP_MAX registered kernels of one operator body (the Q, K and V projections
 * of a layer; the branches of a block) or of two bodies (the projections beside a normalisation; a
 * tensor-core GEMM beside CUDA-core ones).  Patterns: BFUSE_PATTERN_ZIGZAG (M:N),
 * BFUSE_PATTERN_PROPORTIONAL, BFUSE_PATTERN_RANGE_SPLIT; others return BFUSE_ERR_UNSUPPORTED, as do
 * kernels of three or more bodies or of different cluster widths. */
#define BFUSE_GROUP_MAX 4
int bfuse_register_group(bfuse_context *ctx, const int *kernels, int n, int pattern, int param_m, int param_n, int *group);
/* The fused-kernel record of a group: name "<k1>_<k2>_..._fused_bfuse", fused GridDim / BlockDim, smem, registers. */
int bfuse_group_info(bfuse_context *ctx, int group, bfuse_kernel_desc *out);
/* Which kernel (index into the group's list) and virtual block CTA b runs. */
int bfuse_group_map_block(const bfuse_context *ctx, int group, int b, int *kernel, int *vblock);
int bfuse_launch_group(bfuse_context *ctx, int group, void *stream);
/* The scheduler of a group alone (no GPU): kernel and virtual block of every CTA of the fused grid.
 * Returns the fused grid size (or a negative status); fills at most `cap` entries. */
int bfuse_plan_group(const bfuse_dim3 *grid, const bfuse_dim3 *block, int n, int pattern, int param_m, int param_n,
                     int cluster, int *fused_block, int *kernel_of, int *vblock_of, int cap);

/* Device-buffer launches on a caller stream (NULL = default stream). */
int bfuse_launch_kernel(bfuse_context *ctx, int kernel, void *stream);       /* run_kernel1/2 launch, operation_cu.py:173,191 */
int bfuse_launch_sequential(bfuse_context *ctx, int fusion, void *stream);   /* k1 then k2 on one stream                       */
int bfuse_launch_parallel(bfuse_context *ctx, int fusion, void *stream);     /* run_parallel launch, operation_cu.py:203-229   */
int bfuse_launch_fused(bfuse_context *ctx, int fusion, void *stream);        /* run_fuse launch, operation_cu.py:231-253       */
/* Launch a list of fusions back to back on one stream in mode T (0 kernel1, 1 kernel2, 2 parallel,
 * 3 sequential, 4 fused): the inner loop of the harness (main_cc.py:188-238) without returning to
 * the caller between launches. */
int bfuse_launch_list(bfuse_context *ctx, const int *fusions, int n, int mode, void *stream);
/* The same list captured once into a CUDA graph and replayed with one call; for pairs whose
 * kernels last a few microseconds the per-launch host cost otherwise dominates. */
int bfuse_graph_create(bfuse_context *ctx, const int *fusions, int n, int mode, int *graph);
int bfuse_graph_launch(bfuse_context *ctx, int graph, void *stream);
int bfuse_graph_destroy(bfuse_context *ctx, int graph);
/* Run the fused grid with a recording body: per CTA the operator, virtual block and SM id it saw
 * (the %smid printf of legacy/tests/thread_pooling_test/temp2.cu:7-9, as data).  Arrays hold
 * fused-grid entries; for WORK_QUEUE they are indexed by ticket.  Synchronises. */
int bfuse_trace_fused(bfuse_context *ctx, int fusion, int *kernel_of, int *vblock_of, int *sm_of, int n);
/* Diagnostic, no reference counterpart: run a registered tcgen05 GEMM kernel once (unfused) with its
 * first CTA recording global-timer marks in nanoseconds: start, set-up done, first / last TMA load
 * issued, first stage full, last MMA issued, accumulator ready, partial tile written, cluster
 * barrier 1, reduction done, cluster barrier 2, end (12 values; unused marks stay 0). Synchronises. */
int bfuse_debug_gemm_timeline(bfuse_context *ctx, int kernel, long long *marks, int n);
/* Diagnostic, no reference counterpart: launch the n block-level fusions back to back on the
 * context's stream (fused mode), every dispatch slot (CTA, or ticket for WORK_QUEUE) of launch i
 * recording three global-timer marks in nanoseconds: kernel entry, body start (the body sets itself
 * up and then waits for the previous launch, so this may precede that launch's end), thread 0 of
 * the body done.  times holds 3 * sum(slots) values,
 * launch i's slots[i] >= its fused grid entries first to last; unused entries stay 0.  Synchronises. */
int bfuse_debug_fused_timeline(bfuse_context *ctx, const int *fusions, int n, long long *times, const int *slots);
/* Diagnostic, no reference counterpart, no GPU needed: how the tensor-core conv body would stage the input
 * of a conv of shape {n, ci, h, w, co, kh, kw, stride, pad} with bn output pixels per tile.  out (12 ints):
 * ring slots before the window is sized (0: the conv cannot be staged and is gathered from global memory), channels per slot, staged rows,
 * floats per staged row, element strides x / y of the load, staged columns / rows between neighbouring
 * output pixels / rows, tensor column of staged column 0, staged column of tap 0 of output column 0,
 * bytes per slot, slot pitch in bytes; with n >= 13 also the output pixels per tile (bn, or whole output rows). */
int bfuse_debug_conv_staging(const int *shape, int bn, int *out, int n);
/* Read and clear the device status word (0 = no bounded wait gave up). Synchronises.  A non-zero
 * status also restarts the ticket counters of every work-queue fusion from zero. */
int bfuse_read_status(bfuse_context *ctx, int *status);
/* Diagnostic, no reference counterpart: enabled = 0 makes every later launch of this context go
 * without the programmatic-dependent-launch attribute (a kernel's CTAs then start only when the
 * previous kernel on the stream has finished), to tell that overlap's effect on a timeline from
 * everything else.  Default: enabled. */
int bfuse_set_dependent_launch(bfuse_context *ctx, int enabled);

/* Host-buffer entry points with the reference harness' semantics: H2D of every input, launch,
 * device sync, D2H of every output.  host_args follow each kernel's argument order; pointers for
 * optional arguments the kernel was registered without may be NULL.  An input that both kernels of a
 * pair take from the same host buffer into the same device buffer (shared activations) is copied once. */
int bfuse_run_kernel(bfuse_context *ctx, int kernel, void *const *host_args);                    /* run_kernel1/2 */
int bfuse_run_parallel(bfuse_context *ctx, int fusion, void *const *host_args1, void *const *host_args2); /* run_parallel */
int bfuse_run_fuse(bfuse_context *ctx, int fusion, void *const *host_args1, void *const *host_args2);     /* run_fuse     */
/* run_fuse over n fusions that own different device buffers (the harness' `-n num_iterations` loop around
 * run_fuse, tests/benchmark/main.cc:183-200, for independent pairs instead of one repeated): the copies in of fusion i + 1, the fused launch of fusion i and the copies out
 * of fusion i - 1 run on three streams, so host <-> device transfers in both directions overlap the kernels.
 * host_args1[i] / host_args2[i] are the argument lists bfuse_run_fuse takes; pinned host memory is needed for the
 * overlap.  An input that an earlier fusion of the same call already takes from the same host buffer into the same
 * device buffer (weights shared by the sub-shards of a batch) is copied once.  Returns after everything has
 * completed; a fusion listed twice is rejected (its buffers would race). */
int bfuse_run_fuse_batch(bfuse_context *ctx, const int *fusions, int n, void *const *const *host_args1,
                         void *const *const *host_args2);

/* Timing in the spirit of scripts/profile_test_suite.py:10-11 + analyze_test_suite.py:103-123
 * (warm-ups, then the mean over 30 launches): `warmup` untimed launches, then a CUDA graph of `iters`
 * launches is replayed (first until the clocks have ramped, then in 8 timed batches) under CUDA
 * events on the context's stream; host launch cost is therefore not part of the figure and the
 * buffers are L2-warm.  mode is the harness' T: 0 kernel1, 1 kernel2, 2 parallel, 3 sequential,
 * 4 fused.  Mean over all batches and the best batch, in microseconds per launch. */
int bfuse_time(bfuse_context *ctx, int fusion, int mode, int warmup, int iters, float *mean_us, float *min_us);

/* check_matrix (test-utils/test-suite-files/utils_cc.py:52-86): element i is wrong iff
 * |a-b| > eps AND (b == 0 OR |(a-b)/b| > eps).  Returns the number of wrong elements. */
long bfuse_check_matrix(const float *value, const float *answer, size_t n, float eps);

/* No counterpart in the reference.  The softmax || LayerNorm pair through the persistent work queue
 * for callers that cannot allocate device memory: processes whose memory is wholly owned by a pool
 * or caching allocator, and latency-critical loops where cudaMalloc / cudaFree (which synchronise
 * the device) are off limits.  Calls no cudaMalloc / cudaFree and keeps nothing on the heap; the
 * queue's two counters live in a 256-byte static device array inside the library.  Buffers are the
 * caller's device pointers (ln_res may be NULL).  At most BFUSE_NOALLOC_MAX_TICKETS fused CTAs;
 * more is rejected with BFUSE_ERR_SHAPE.  The first call on a device performs a one-time address
 * look-up and should happen outside stream capture; calls whose kernels overlap on one GPU race
 * on the shared counters, so order them.  Output is bit-identical to bfuse_launch_fused on a
 * BFUSE_PATTERN_WORK_QUEUE fusion of the same two kernels with default tilings. */
#define BFUSE_NOALLOC_MAX_TICKETS (1 << 20)
int bfuse_softmax_layernorm_queue_noalloc(const float *sm_x, float *sm_y, int sm_rows, int sm_cols, float sm_scale,
                                          const float *ln_x, const float *ln_res, const float *ln_gamma,
                                          const float *ln_beta, float *ln_y, int ln_rows, int ln_cols, float ln_eps,
                                          void *stream);

/* The scheduler alone, usable without a GPU: what `horizontal-fuser fusions.yaml kernels.yaml`
 * computes on the CPU (FusionContext::create, src/Contexts.cc:56-92) for one pair.  param_m /
 * param_n as for bfuse_register_fusion, except that SM_STRIPED needs an explicit SM count. */
typedef struct bfuse_plan bfuse_plan;
int bfuse_plan_create(const bfuse_dim3 grid[2], const bfuse_dim3 block[2], int pattern, int param_m, int param_n,
                      bfuse_plan **out);
/* The same with dispatch units of `cluster` consecutive CTAs: what bfuse_register_fusion uses when
 * an operator is launched as thread-block clusters (split-K GEMM).  No reference counterpart; with
 * cluster = 1 it is bfuse_plan_create.  bfuse_plan_map_all marks padding CTAs of a partly filled
 * cluster with -1. */
int bfuse_plan_create_clustered(const bfuse_dim3 grid[2], const bfuse_dim3 block[2], int pattern, int param_m,
                                int param_n, int cluster, bfuse_plan **out);
void bfuse_plan_destroy(bfuse_plan *plan);
int bfuse_plan_fused_dims(const bfuse_plan *plan, bfuse_dim3 *grid, bfuse_dim3 *block);
int bfuse_plan_map_block(const bfuse_plan *plan, int b, int *kernel, int *vblock);
int bfuse_plan_map_all(const bfuse_plan *plan, int *kernel_of, int *vblock_of, int n);
int bfuse_plan_map_thread(const bfuse_plan *plan, int kernel, int b, int t, int *vblock, int *vthread, int *active);
/* bar.sync operands of operator `kernel` (src/Matchers.cc:288-320): id = kernel + 1, count = round32(B_k). */
int bfuse_plan_barrier(const bfuse_plan *plan, int kernel, int *bar_id, int *bar_count);

#ifdef __cplusplus
}
#endif
#endif
