/*
 * CPU oracle for the horizontal-fusion hot path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped library links, loads or calls this code; it exists so
 * that the tests, the smoke check and the CPU-baseline leg of the benchmark can
 * compare the CUDA path against an independent restatement.
 *
 * Two halves:
 *   1. block-dispatch math  -- restates the reference's
 *      horizontal-fuser/src/Algorithms.cc (four patterns) as "plans": an ordered
 *      list of branches with the same constants the reference prints into the
 *      if / else-if chain of a fused kernel.  Pinned against the reference's
 *      generated kernels and YAML outputs (tests/golden).
 *   2. operator arithmetic  -- plain loops for the operator pairs.  The reference
 *      has no CPU implementation of any operator (its check is fused-vs-unfused
 *      on the GPU), so the absolute values are "parity unpinned"; the op math
 *      follows the Relay dumps under files/ in the reference.
 */
#ifndef BFUSE_ORACLE_H
#define BFUSE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ dispatch */

#define ORC_MAX_KERNELS 4
#define ORC_MAX_BRANCHES 16

/* GridDim / BlockDim of one kernel (horizontal-fuser/include/fuse/Contexts.h:13-25). */
typedef struct {
  int gx, gy, gz;
  int bx, by, bz;
} orc_kernel_dims;

enum {
  ORC_BR_ROTATE = 0, /* (b < b_hi) && (b % rot >= r_lo) && (b % rot < r_hi)                 */
  ORC_BR_RANGE = 1,  /* (b >= b_lo && b < b_hi)                                              */
  ORC_BR_STRIPE = 2, /* (b >= b_lo && b < b_hi) && ((b - b_lo) % (sm*n) / sm == stripe_idx)  */
  ORC_BR_THREADS = 3 /* (t >= t_lo && t < t_hi) && (b >= 0 && b < b_hi)   (thread split)     */
};

typedef struct {
  int kind;
  int kernel;     /* KernelID_ the branch assigns */
  int b_lo, b_hi; /* blockIdx.x window */
  int rot, r_lo, r_hi, ratio; /* ROTATE: vb = b / rot * ratio + (b % rot - r_lo) */
  int base;       /* RANGE: vb = b - b_lo + base;  STRIPE: vb = base + (b-b_lo) % sm + (b-b_lo)/(n*sm)*sm */
  int sm, stripe_n, stripe_idx;
  int t_lo, t_hi; /* THREADS: vt = t - t_lo, vb = b */
} orc_branch;

typedef struct {
  int n_kernels;
  orc_kernel_dims k[ORC_MAX_KERNELS];
  int n_branches;
  orc_branch br[ORC_MAX_BRANCHES];
  int fused_grid;  /* fused GridDim.X (Y = Z = 1) */
  int fused_block; /* fused BlockDim.X */
  int thread_split; /* 1: every branch is its own `if` and selects by thread range */
} orc_plan;

/* coarseInterleaveWithoutSMPattern2 (Algorithms.cc:528-739); M = N = 1 in the reference. */
int orc_plan_zigzag(const orc_kernel_dims *k, int n, int M, int N, orc_plan *out);
/* coarseInterleaveWithoutSMPattern (Algorithms.cc:319-526); MinOption = 1 in the reference. */
int orc_plan_proportional(const orc_kernel_dims *k, int n, int min_option, orc_plan *out);
/* coarseInterleavePattern (Algorithms.cc:118-317); TotalSM = 84 in the reference. */
int orc_plan_sm_striped(const orc_kernel_dims *k, int n, int total_sm, orc_plan *out);
/* hfusePattern (Algorithms.cc:19-116). */
int orc_plan_thread_split(const orc_kernel_dims *k, int n, orc_plan *out);
/* The contiguous-tail rule (Algorithms.cc:661-685) applied to every block. */
int orc_plan_range_split(const orc_kernel_dims *k, int n, orc_plan *out);

/* First matching branch of the if / else-if chain for CTA b.  Returns 1 and fills
 * kernel / virtual block, or 0 when no branch matches. Block-level plans only. */
int orc_map_block(const orc_plan *p, int b, int *kernel, int *vblock);
/* Thread-split plans: does (b, t) run kernel `kernel`?  Fills virtual block / thread. */
int orc_map_thread(const orc_plan *p, int kernel, int b, int t, int *vblock, int *vthread);
/* Guard of a block-level plan: KernelID_ == k && t < B_k (Algorithms.cc:699-717). */
int orc_thread_active(const orc_plan *p, int kernel, int t);
/* blockIdx_{x,y,z}_ / threadIdx_{x,y,z}_ decomposition (Algorithms.cc:687-692). */
void orc_decompose(const orc_kernel_dims *k, int vblock, int vthread, int bidx[3], int tidx[3]);
/* bar.sync operands of the thread-split rewrite (Matchers.cc:288-320): id = k + 1,
 * count = BlockDim.size() rounded up to a multiple of 32. */
void orc_named_barrier(const orc_plan *p, int kernel, int *bar_id, int *bar_count);
/* Position-weighted sum over the (kernel, vblock) sequence of all fused CTAs; 0 on an unmapped CTA. */
uint64_t orc_plan_digest(const orc_plan *p);

/* --------------------------------------------------------------- operators */

/* y[r,:] = softmax(x[r,:] * scale)   (files/bert-base-uncased.txt:34,40-41) */
void orc_softmax_f32(const float *x, float *y, int rows, int cols, float scale);
/* y = ((x [+ res]) - mean) / sqrt(var + eps) * gamma + beta
 * (files/bert-base-uncased.txt:61-70, files/gpt2.txt:9-17); res may be NULL. */
void orc_layernorm_f32(const float *x, const float *res, const float *gamma, const float *beta,
                       float *y, int rows, int cols, float eps);
/* bf16 in/out, fp32 math: y = x * (1/sqrt(mean(x^2)+eps)) * w
 * (files/Meta-Llama-3-8B.txt:7-14). */
void orc_rmsnorm_bf16(const uint16_t *x, const uint16_t *w, uint16_t *y, int rows, int cols, float eps);
/* rotate-half RoPE on q[seq, heads, dim] (bf16), angle = pos * inv_freq[i], i < dim/2
 * (files/Meta-Llama-3-8B.txt:19-28). */
void orc_rope_bf16(const uint16_t *q, const float *inv_freq, uint16_t *y, int seq, int heads, int dim);
/* out[b,m,n] = sum_k A[b,m,k] * W[b,n,k] (+ bias[n]); NT layout as in the reference's
 * dense / batch_matmul kernels (scripts/configure_kernels.py:14-26).  causal: entries with
 * n > m are set to -FLT_MAX (additive mask of files/gpt2.txt:35).  tf32: truncate the
 * operands' low 13 mantissa bits first, as the tensor core does. */
void orc_gemm_nt_f32(const float *A, const float *W, const float *bias, float *out,
                     int batch, int M, int N, int K, int causal, int tf32);
/* bf16 operands and output, fp32 accumulate. */
void orc_gemm_nt_bf16(const uint16_t *A, const uint16_t *W, uint16_t *out, int batch, int M, int N, int K);
/* NCHW direct convolution, fp32 (files/resnet-18.txt:31,36). */
void orc_conv2d_nchw_f32(const float *x, const float *w, float *y, int n, int ci, int h, int wd,
                         int co, int kh, int kw, int stride, int pad, int tf32);

/* number of OpenMP threads the loops above use */
int orc_num_threads(void);
/* override OMP_NUM_THREADS (launchers such as torchrun export OMP_NUM_THREADS=1) */
void orc_set_num_threads(int n);
uint16_t orc_f32_to_bf16(float f);
float orc_bf16_to_f32(uint16_t h);

#ifdef __cplusplus
}
#endif
#endif
