// Implementation of the C ABI in include/bfuse_b200.h: the pair registry, the launch boundary
// (replacing test-utils/test-suite-files/operation_cu.py of the reference) and the timing /
// checking helpers of its harness (main_cc.py, utils_cc.py).  No CPU fallback exists: every
// compute entry point launches a CUDA kernel or returns an error.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "../../include/bfuse_b200.h"
#include "op_list.h"
#include "scheduler.h"

using namespace bfuse;

namespace {

constexpr size_t kMaxSmemPerCta = 227 * 1024 - 256;  // opt-in dynamic limit minus the kernels' few static bytes
constexpr int kParamsBytes = 640;

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct ArgInfo {
  size_t bytes;
  int is_output;
  int optional;
};

struct KernelRec {
  alignas(64) unsigned char params[kParamsBytes];
  bfuse_kernel_desc desc;
  std::string name;
  KernelDims dims;
  size_t smem;
  int cluster;  // CTAs per thread-block cluster the body needs (split-K GEMM), else 1
  int nargs;
  ArgInfo arg[BFUSE_MAX_ARGS];
  int alias_of;  // >= 0: a hidden re-tiling (one k-slice) of that registered kernel, owned by a fusion
  int users;     // live fusions / groups that launch this kernel
};

struct FusionRec {
  int k1, k2;           // the kernels the fusion launches (hidden unsplit re-tilings when retiled[k])
  int reg1, reg2;       // the kernels it was registered with
  bool retiled[2];
  int users;            // live graphs that captured it
  FusedPlan plan;
  std::string name;
  size_t smem;
  unsigned launch_grid;
  unsigned *queue_ctr;  // device, 2 words (work queue only)
  int regs;
  int stages[2];        // thread-level fusion only: ring depths that let both windows fit (0: the kernel's own)
  bool wide;            // launch the register-richer build of the pair
};

struct GroupRec {
  int n;
  int ks[kGroupMax];
  GroupPlan plan;
  std::string name;
  size_t smem;
  int regs;
  int stages[kGroupMax];  // ring depths replaced so that two CTAs share an SM (0: the kernel's own)
  int op_lo, op_hi;       // the group's operator bodies, lower id first; equal for a group of one body
};

struct GraphRec {
  cudaGraphExec_t exec;
  int launches;
  std::vector<int> fusions;  // captured fusions: they cannot be released while the graph lives
};

}  // namespace

struct bfuse_context {
  int device;
  int sm_count;
  cudaStream_t s1, s2, own;
  cudaEvent_t ev_fork, ev_j1, ev_j2;
  int *d_status;
  int *h_status;  // pinned mirror: the host-buffer entry points read the status word with the output copies
  EncodeTiledFn encode;
  bool no_pdl;     // diagnostic switch: launch without programmatic dependent launch
  std::vector<cudaEvent_t> batch_events;  // reused by bfuse_run_fuse_batch (two per pair)
  PairEntry pairs[kNumOps][kNumOps];
  SingleEntry singles[kNumOps];
  std::vector<std::unique_ptr<KernelRec>> kernels;
  std::vector<std::unique_ptr<FusionRec>> fusions;
  std::vector<std::unique_ptr<GroupRec>> groups;
  std::vector<GraphRec> graphs;
  std::string err;
};

namespace {

int fail(bfuse_context *ctx, int code, const std::string &msg) {
  if (ctx) ctx->err = msg;
  return code;
}
int fail_cuda(bfuse_context *ctx, cudaError_t e, const char *what) {
  return fail(ctx, BFUSE_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
}
#define CK(call)                                                   \
  do {                                                             \
    cudaError_t e_ = (call);                                       \
    if (e_ != cudaSuccess) return fail_cuda(ctx, e_, #call);       \
  } while (0)

bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }
int ceil_div(int a, int b) { return (a + b - 1) / b; }
bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int conv_out(int in, int k, int stride, int pad) { return (in + 2 * pad - k) / stride + 1; }

// ---- default tilings (what the reference reads back from TVM, configure_kernels.py:73-99) --------

int umma_min_stages(int bn, int split, int elem, int bm = kUmmaBM) {
  // after the MMAs the ring doubles as the store buffers and, with split > 1, as the receive area
  return ceil_div(umma_epilogue_bytes(bn, split, elem), umma_stage_bytes(bn, bm));
}

// Tile width and k-slices of a tensor-core GEMM from a small cost model fitted to measurements on
// B200.  One CTA multiplies a k-block (128 bytes of K per row) in t_kb(BN) -- set by the MMA time for
// wide tiles and by the bytes the SM can pull from L2 for narrow ones --, pays a fixed prologue +
// epilogue that grows with BN, and a split tile pays the cross-CTA reduction on top.  The operator
// is budgeted its share of the SMs (half: its pair partner takes the other half), in whole waves.  Ties go to
// the wider tile (less L2 traffic).  With bn_fixed / split_fixed > 0 only the other one is chosen.
void pick_tile(int batch, int M, int N, int K, int elem, int sm_count, int share, int bn_fixed, int split_fixed, int *bn_out, int *split_out) {
  static const int kBn[4] = {256, 128, 64, 32};
  static const double kTkbUs[4] = {0.267, 0.213, 0.153, 0.150};
  const int num_kb = ceil_div(K * elem, kUmmaRowBytes);
  const int slots = std::max(1, sm_count / share);
  double best = 1e30;
  int best_bn = 128, best_split = 1;
  for (int i = 0; i < 4; ++i) {
    const int bn = kBn[i];
    if (bn_fixed > 0 ? bn != bn_fixed : (bn * elem < 128 || (bn > 32 && bn / 2 >= N && bn / 2 * elem >= 128))) continue;
    const long long tiles = (long long)batch * ceil_div(M, kUmmaBM) * ceil_div(N, bn);
    // own choice of k-slices: 1 or 4 and no other width, so that any two operators the runtime tiled
    // can share a launch (a fused launch has one cluster width); an operator that runs alone may also take 2
    // when K is very long (the model underrates what a split costs: at 64 K blocks two slices measured 25 us
    // against 16 us unsplit and at 128 K blocks 36 us against 34 us, at 224 K blocks 58 us against 74 us with four)
    const int cand[3] = {split_fixed > 0 ? split_fixed : 1, 4, 2};
    for (int ci = 0; ci < (split_fixed > 0 ? 1 : (share == 1 && num_kb >= 192 ? 3 : 2)); ++ci) {
      const int split = cand[ci];
      if (split > num_kb) continue;
      if (umma_smem_bytes(bn, umma_min_stages(bn, split, elem)) > ((bn == 256 || share * tiles * split <= sm_count) ? 200 : 100) * 1024) continue;
      const long long waves = (tiles * split + slots - 1) / slots;
      const double per_cta = 1.0 + 0.006 * bn + ceil_div(num_kb, split) * kTkbUs[i] + (split > 1 ? 2.5 + 0.5 * split : 0.0);
      const double t = (double)waves * per_cta;
      if (t < best * 0.999) best = t, best_bn = bn, best_split = split;
    }
  }
  *bn_out = bn_fixed > 0 ? bn_fixed : best_bn;
  *split_out = split_fixed > 0 ? split_fixed : best_split;
}

int default_launch(const bfuse_context *ctx, bfuse_kernel_desc *d, std::string *err) {
  const int *s = d->shape;
  auto set = [&](int gx, int gy, int gz, int bx, int by, size_t smem, int nargs) {
    d->GridDim = {gx, gy, gz};
    d->BlockDim = {bx, by, 1};
    d->smem_bytes = smem;
    d->nargs = nargs;
    d->HasBarriers = 1;
  };
  const int sm = ctx ? ctx->sm_count : 148;
  // operators that will share the launch (BFUSE_FLAG_SHARE): 2 unless told otherwise -- a pair
  const int share = ((d->flags >> 8) & 7u) ? (int)((d->flags >> 8) & 7u) : 2;
  switch (d->op) {
    case BFUSE_OP_SOFTMAX_F32:
    case BFUSE_OP_LAYERNORM_F32: {
      const int tpr = pick_row_threads(s[1], 4, kRowMaxVec);
      if (s[0] <= 0 || !tpr) { *err = "row operator: cols must be a multiple of 4 * (power-of-two threads per row)"; return BFUSE_ERR_SHAPE; }
      const int rpc = std::max(1, 256 / tpr);
      set(ceil_div(s[0], rpc), 1, 1, tpr, rpc, 256, d->op == BFUSE_OP_SOFTMAX_F32 ? 2 : 5);
      return BFUSE_OK;
    }
    case BFUSE_OP_RMSNORM_BF16: {
      const int tpr = pick_row_threads(s[1], 8, RmsNormBf16::kMaxVec);
      if (s[0] <= 0 || !tpr) { *err = "rmsnorm: cols must be a multiple of 8 * (power-of-two threads per row)"; return BFUSE_ERR_SHAPE; }
      const int rpc = std::max(1, 256 / tpr);
      set(ceil_div(s[0], rpc), 1, 1, tpr, rpc, 256, 3);
      return BFUSE_OK;
    }
    case BFUSE_OP_ROPE_BF16: {
      if (s[0] <= 0 || s[1] <= 0 || s[2] <= 0 || s[2] % 16) { *err = "rope: dim must be a multiple of 16"; return BFUSE_ERR_SHAPE; }
      const int chunks = s[2] / 16;
      int groups = 1;
      while (groups * 2 * chunks <= 64 && s[1] % (groups * 2) == 0) groups *= 2;
      const int bx = chunks * groups, by = std::max(1, 256 / bx);
      set(ceil_div(s[0], by), 1, 1, bx, by, 0, 3);
      d->HasBarriers = 0;
      return BFUSE_OK;
    }
    case BFUSE_OP_GEMM_F32_SIMT:
      if (s[0] <= 0 || s[1] <= 0 || s[2] <= 0 || s[3] <= 0) { *err = "gemm: batch, M, N, K must be positive"; return BFUSE_ERR_SHAPE; }
      set(ceil_div(s[2], kSimtTile), ceil_div(s[1], kSimtTile), s[0], 16, 16, kSimtSmemBytes, 4);
      return BFUSE_OK;
    case BFUSE_OP_CONV2D_F32_SIMT: {
      if (s[0] <= 0 || s[1] <= 0 || s[4] <= 0 || s[7] <= 0) { *err = "conv2d: bad shape"; return BFUSE_ERR_SHAPE; }
      const int oh = conv_out(s[2], s[5], s[7], s[8]), ow = conv_out(s[3], s[6], s[7], s[8]);
      if (oh <= 0 || ow <= 0) { *err = "conv2d: empty output"; return BFUSE_ERR_SHAPE; }
      set(ceil_div(s[0] * oh * ow, kSimtTile), ceil_div(s[4], kSimtTile), 1, 16, 16, kSimtSmemBytes, 3);
      return BFUSE_OK;
    }
    case BFUSE_OP_CONV2D_TF32: {
      if (s[0] <= 0 || s[1] <= 0 || s[4] <= 0 || s[5] <= 0 || s[6] <= 0 || s[7] <= 0) { *err = "conv2d: bad shape"; return BFUSE_ERR_SHAPE; }
      const int oh = conv_out(s[2], s[5], s[7], s[8]), ow = conv_out(s[3], s[6], s[7], s[8]);
      if (oh <= 0 || ow <= 0) { *err = "conv2d: empty output"; return BFUSE_ERR_SHAPE; }
      const int num_kb = ceil_div(s[1] * s[5] * s[6], ConvUmmaTf32::kBK);
      // pixels per tile: the widest of 128 / 64 / 32 that still gives the operator about half the
      // SMs (its pair partner takes the other half); a single small image gets 32-pixel tiles
      int bn = s[9];
      if (bn <= 0 && s[11] == 1) bn = kConvBN;   // the staged form has one tile: the 128 lanes of tensor memory
      if (bn <= 0) {
        bn = 32;
        for (int cand = kConvBN; cand > 32; cand /= 2)
          if ((long long)s[0] * ceil_div(oh * ow, cand) * ceil_div(s[4], kUmmaBM) >= sm / share) { bn = cand; break; }
      }
      if (bn != 32 && bn != 64 && bn != 128) { *err = "conv2d: pixels per tile must be 32, 64 or 128"; return BFUSE_ERR_SHAPE; }
      d->shape[9] = bn;
      const int K = s[1] * s[5] * s[6];
      const long long tiles = (long long)s[0] * ceil_div(oh * ow, bn) * ceil_div(s[4], kUmmaBM);
      // k-slices per tile (a cluster): a deep layer on a small image has few tiles and a long K.  The
      // runtime's own choice is 1 or 4 -- never another width, so that any two operators it tiled can
      // share a launch (a fused launch has one cluster width): 4 when the k-slices still fit three
      // quarters of the SMs and keep at least 4 K blocks each (8-wide clusters measured slower in pairs)
      int split = s[10];
      if (split <= 0) split = (s[11] != 1 && tiles * 4 * share <= 3 * sm / 2 && num_kb >= 16) ? 4 : 1;   // the staged form does not split K
      if (split > 8 || split > num_kb) { *err = "conv2d: k-slices must be 1..8 and at most the number of K blocks"; return BFUSE_ERR_SHAPE; }
      const int q = ceil_div(num_kb, split);
      split = ceil_div(num_kb, q);
      d->shape[10] = split;
      // ring: two CTAs per SM, or the whole SM when the operator and an equal partner leave every CTA
      // an SM of its own (a long-K conv on few CTAs is bound by the ring's round trip, not by issue
      // rate); deep enough to hold the k-slices' partial sums after the MMAs
      const long long ctas = tiles * split;
      // How the im2col operand is built, shape[11]: 1 = staged (input rows by TMA into a raw ring, the im2col rows
      // written from there into tensor memory), 2 = gathered from global memory with 4-byte copies, 0 = the
      // runtime's choice: staged wherever its one tiling (128-pixel tiles, unsplit K) is what the runtime would
      // pick anyway and the geometry allows it -- 3 x 3 stride-2 branch of ResNet-18 at batch 256: 113 us staged,
      // 193 us gathered; at batch 32: 17 us and 31 us.
      ConvStaging st;
      st.slots = 0;
      if (s[11] == 1 && (split != 1 || !conv_staging(s[1], s[2], s[3], s[5], s[6], s[7], s[8], oh, ow, bn, &st))) {
        *err = "conv2d: shape[11] = 1 (staged operand) needs 128-pixel tiles, an unsplit K of whole K blocks, image rows of 16-byte multiples and a window whose rows fit a 24 KB slot";
        return BFUSE_ERR_SHAPE;
      }
      if (s[11] == 0 && split == 1 && !conv_staging(s[1], s[2], s[3], s[5], s[6], s[7], s[8], oh, ow, bn, &st)) st.slots = 0;
      if (s[11] < 0 || s[11] > 2) { *err = "conv2d: shape[11] (operand mode) must be 0, 1 or 2"; return BFUSE_ERR_SHAPE; }
      d->shape[11] = st.slots ? 1 : 2;
      // ring budget: the whole SM when the operator and an equal partner leave every CTA an SM of its own, else
      // two CTAs per SM (staged: tensor memory holds two) or three (gathered)
      const int budget = (share * ctas <= sm ? 200 : (st.slots ? 110 : 74)) * 1024;
      if (st.slots) {
        int wst;
        if (!conv_staged_ring(budget, K, st.cc * s[5] * s[6], st.slot_pitch, &st.slots, &wst)) {
          *err = "conv2d: shape[11] = 1 (staged operand): the raw ring and two weight stages do not fit the shared-memory budget";
          return BFUSE_ERR_SHAPE;
        }
        // A CTA takes several tiles (every grid-size-th one) once there are more tiles than the two CTAs per SM
        // that fit at a time: its rings and tensor memory live across them, so only the first tile pays for the
        // set-up and the first loads' latency (a third of a tile's time), and the next tile's loads run under
        // the epilogue.  Never more CTAs than fit at once: a few left over for a second round would each still
        // walk their whole share of the tiles, alone.
        const long long staged_tiles = (long long)ceil_div(oh * ow, st.tile_px) * ceil_div(s[4], kUmmaBM) * s[0];
        if (staged_tiles > 2 * sm)
          set(2 * sm, 1, 1, kConvThreads, 1, conv_staged_smem_bytes(K, st.slots, st.slot_pitch, wst), 3);
        else
          set(ceil_div(oh * ow, st.tile_px), ceil_div(s[4], kUmmaBM), s[0], kConvThreads, 1, conv_staged_smem_bytes(K, st.slots, st.slot_pitch, wst), 3);
        return BFUSE_OK;
      }
      int stages = std::max(1, std::min({q, kUmmaMaxStages, (budget - conv_header_bytes(K)) / conv_stage_bytes(bn)}));
      stages = std::max(stages, ceil_div(umma_epilogue_bytes(bn, split, 4), conv_stage_bytes(bn)));
      set(split * ceil_div(oh * ow, bn), ceil_div(s[4], kUmmaBM), s[0], kConvThreads, 1, conv_umma_smem_bytes(stages, bn, K, 0), 3);
      return BFUSE_OK;
    }
    case BFUSE_OP_GEMM_TF32:
    case BFUSE_OP_GEMM_BF16: {
      if (s[0] <= 0 || s[1] <= 0 || s[2] <= 0 || s[3] <= 0) { *err = "gemm: batch, M, N, K must be positive"; return BFUSE_ERR_SHAPE; }
      const int eb = d->op == BFUSE_OP_GEMM_TF32 ? 4 : 2;
      int bn = s[4], split = s[5], bm = s[6], q;
      if (bn <= 0 || split <= 0) pick_tile(s[0], s[1], s[2], s[3], eb, sm, share, bn, split, &bn, &split);
      if (bn != 32 && bn != 64 && bn != 128 && bn != 256) { *err = "gemm: BN must be 32, 64, 128 or 256"; return BFUSE_ERR_SHAPE; }
      d->shape[4] = bn;
      const int num_kb = ceil_div(s[3] * eb, kUmmaRowBytes);
      if (split > 8 || split > num_kb) { *err = "gemm: split must be 1..8 and at most the number of K blocks"; return BFUSE_ERR_SHAPE; }
      q = ceil_div(num_kb, split);
      split = ceil_div(num_kb, q);
      d->shape[5] = split;
      // 256-row tiles (two MMAs per k-step share one W tile: a third less operand traffic from L2 per
      // flop) once the 128-row tiles alone would fill every SM and K is long enough for the main
      // loop to dominate: that is where L2 -> SM bandwidth, not the tensor pipe, sets the pace of
      // 128 x 256 tiles (short-K shapes are bound by their output stores and prefer two CTAs per SM)
      if (bm <= 0) {
        const long long tiles = (long long)s[0] * ceil_div(s[1], kUmmaBM) * ceil_div(s[2], bn);
        const long long slots = std::max(1, sm / share);
        // ... or, for an operator that runs alone (its waves are real ones), when halving the CTA count
        // halves the waves: with every SM busy a 256-row tile takes about 1.9x a 128-row one
        const long long waves = (tiles + slots - 1) / slots, waves_tall = ((tiles + 1) / 2 + slots - 1) / slots;
        bm = (bn == 256 && split == 1 && num_kb >= 16 && s[1] > kUmmaBM &&
              (tiles >= 2 * slots || (share == 1 && 19 * waves_tall < 10 * waves))) ? 256 : kUmmaBM;
      }
      if ((bm != kUmmaBM && bm != 256) || (bm == 256 && split != 1)) { *err = "gemm: BM must be 128, or 256 with split = 1"; return BFUSE_ERR_SHAPE; }
      d->shape[6] = bm;
      // ring depth: enough to cover the k-slice, at most 8, and large enough to hold the partial tile
      // when K is split.  Within ~200 KB when the operator and an equal partner leave every CTA an SM
      // of its own (operands arriving from HBM need ~1 us of loads in flight per SM) or for the 256-wide
      // tile, else within ~100 KB so that two CTAs share an SM.
      const long long ctas = (long long)split * s[0] * ceil_div(s[1], bm) * ceil_div(s[2], bn);
      const int budget = (bn == 256 || share * ctas <= sm) ? 200 * 1024 : 100 * 1024;
      int stages = std::min({q, kUmmaMaxStages, (budget - kUmmaHeaderBytes) / umma_stage_bytes(bn, bm)});
      stages = std::max({stages, 1, umma_min_stages(bn, split, eb, bm)});
      set(split * ceil_div(s[1], bm), ceil_div(s[2], bn), s[0], kUmmaThreads, 1, umma_smem_bytes(bn, stages, bm), 4);
      return BFUSE_OK;
    }
    default:
      *err = "operator not in the registry";
      return BFUSE_ERR_INVALID;
  }
}

// ---- argument lists ---------------------------------------------------------------------------

int describe_args(const bfuse_kernel_desc &d, ArgInfo *a, std::string *err) {
  const int *s = d.shape;
  auto n = [](long long x) { return (size_t)std::max(0LL, x); };
  switch (d.op) {
    case BFUSE_OP_SOFTMAX_F32:
      a[0] = {n(4LL * s[0] * s[1]), 0, 0};
      a[1] = {n(4LL * s[0] * s[1]), 1, 0};
      return 2;
    case BFUSE_OP_LAYERNORM_F32:
      a[0] = {n(4LL * s[0] * s[1]), 0, 0};
      a[1] = {n(4LL * s[0] * s[1]), 0, 1};
      a[2] = {n(4LL * s[1]), 0, 0};
      a[3] = {n(4LL * s[1]), 0, 0};
      a[4] = {n(4LL * s[0] * s[1]), 1, 0};
      return 5;
    case BFUSE_OP_RMSNORM_BF16:
      a[0] = {n(2LL * s[0] * s[1]), 0, 0};
      a[1] = {n(2LL * s[1]), 0, 0};
      a[2] = {n(2LL * s[0] * s[1]), 1, 0};
      return 3;
    case BFUSE_OP_ROPE_BF16:
      a[0] = {n(2LL * s[0] * s[1] * s[2]), 0, 0};
      a[1] = {n(4LL * (s[2] / 2)), 0, 0};
      a[2] = {n(2LL * s[0] * s[1] * s[2]), 1, 0};
      return 3;
    case BFUSE_OP_GEMM_F32_SIMT:
    case BFUSE_OP_GEMM_TF32:
    case BFUSE_OP_GEMM_BF16: {
      const long long e = d.op == BFUSE_OP_GEMM_BF16 ? 2 : 4;
      a[0] = {n(e * s[0] * s[1] * s[3]), 0, 0};
      a[1] = {n(e * s[0] * s[2] * s[3]), 0, 0};
      a[2] = {n(4LL * s[2]), 0, 1};
      a[3] = {n(e * s[0] * s[1] * s[2]), 1, 0};
      return 4;
    }
    case BFUSE_OP_CONV2D_F32_SIMT:
    case BFUSE_OP_CONV2D_TF32: {
      const int oh = conv_out(s[2], s[5], s[7], s[8]), ow = conv_out(s[3], s[6], s[7], s[8]);
      a[0] = {n(4LL * s[0] * s[1] * s[2] * s[3]), 0, 0};
      a[1] = {n(4LL * s[4] * s[1] * s[5] * s[6]), 0, 0};
      a[2] = {n(4LL * s[0] * s[4] * oh * ow), 1, 0};
      return 3;
    }
    default:
      *err = "operator not in the registry";
      return -1;
  }
}

// ---- typed parameter blocks ---------------------------------------------------------------------

// 3-D tensor map {k (contiguous), rows, batch} with a 128-byte x box_rows box and 128B swizzle
int encode_map(bfuse_context *ctx, CUtensorMap *map, int dtype_bytes, const void *base, int k, int rows, int batch,
               int box_rows) {
  const CUtensorMapDataType dt = dtype_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const cuuint64_t dims[3] = {(cuuint64_t)k, (cuuint64_t)rows, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)k * dtype_bytes, (cuuint64_t)k * rows * dtype_bytes};
  const cuuint32_t box[3] = {(cuuint32_t)(kUmmaRowBytes / dtype_bytes), (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = ctx->encode(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(ctx, BFUSE_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
  return BFUSE_OK;
}

int build_params(bfuse_context *ctx, KernelRec &k) {
  const bfuse_kernel_desc &d = k.desc;
  const int *s = d.shape;
  const KernelDims &kd = k.dims;
  void *const *a = d.args;
  auto shape_err = [&](const char *m) { return fail(ctx, BFUSE_ERR_SHAPE, k.name + ": " + m); };
  if (kd.block() % 32) return shape_err("BlockDim.size() must be a multiple of 32 (named-barrier arrival counts)");
  if (kd.block() > ctx->singles[d.op].max_threads) return shape_err("BlockDim exceeds the body's maximum");
  for (int i = 0; i < k.nargs; ++i) {
    if (!a[i] && !k.arg[i].optional) return fail(ctx, BFUSE_ERR_INVALID, k.name + ": missing argument buffer");
    if (a[i] && !aligned16(a[i])) return fail(ctx, BFUSE_ERR_INVALID, k.name + ": argument buffers must be 16-byte aligned");
  }
  std::memset(k.params, 0, sizeof(k.params));
  k.cluster = 1;
  switch (d.op) {
    case BFUSE_OP_SOFTMAX_F32:
    case BFUSE_OP_LAYERNORM_F32:
    case BFUSE_OP_RMSNORM_BF16: {
      const int vec = d.op == BFUSE_OP_RMSNORM_BF16 ? 8 : 4;
      const int maxv = d.op == BFUSE_OP_RMSNORM_BF16 ? RmsNormBf16::kMaxVec : kRowMaxVec;
      const int tpr = kd.bx, rpc = kd.by;
      if (s[0] <= 0 || s[1] <= 0) return shape_err("rows and cols must be positive");
      if (!is_pow2(tpr) || kd.bz != 1) return shape_err("BlockDim must be (power-of-two threads per row, rows per CTA, 1)");
      if (s[1] % (vec * tpr) || s[1] / (vec * tpr) > maxv) return shape_err("cols do not fit the per-thread vector budget");
      if (kd.gy != 1 || kd.gz != 1 || (long long)kd.gx * rpc < s[0]) return shape_err("GridDim.X * rows per CTA must cover the rows");
      if (tpr > 32 && k.smem < 256) return shape_err("rows wider than a warp need 256 bytes of shared memory");
      if (d.op == BFUSE_OP_SOFTMAX_F32) {
        SoftmaxF32::Params p{(const float *)a[0], (float *)a[1], s[0], s[1], d.fparam[0]};
        std::memcpy(k.params, &p, sizeof(p));
      } else if (d.op == BFUSE_OP_LAYERNORM_F32) {
        LayerNormF32::Params p{(const float *)a[0], (const float *)a[1], (const float *)a[2], (const float *)a[3],
                               (float *)a[4], s[0], s[1], d.fparam[0]};
        std::memcpy(k.params, &p, sizeof(p));
      } else {
        RmsNormBf16::Params p{(const uint16_t *)a[0], (const uint16_t *)a[1], (uint16_t *)a[2], s[0], s[1], d.fparam[0]};
        std::memcpy(k.params, &p, sizeof(p));
      }
      return BFUSE_OK;
    }
    case BFUSE_OP_ROPE_BF16: {
      if (s[0] <= 0 || s[1] <= 0 || s[2] <= 0 || s[2] % 16) return shape_err("dim must be a positive multiple of 16");
      const int chunks = s[2] / 16;
      if (kd.bx % chunks || s[1] % (kd.bx / chunks) || kd.bz != 1) return shape_err("BlockDim.X must be chunks * (a divisor of heads)");
      if (kd.gy != 1 || kd.gz != 1 || (long long)kd.gx * kd.by < s[0]) return shape_err("GridDim.X * positions per CTA must cover seq");
      RopeBf16::Params p{(const uint16_t *)a[0], (const float *)a[1], (uint16_t *)a[2], s[0], s[1], s[2]};
      std::memcpy(k.params, &p, sizeof(p));
      return BFUSE_OK;
    }
    case BFUSE_OP_GEMM_F32_SIMT: {
      if (s[0] <= 0 || s[1] <= 0 || s[2] <= 0 || s[3] <= 0) return shape_err("batch, M, N, K must be positive");
      if (kd.bx != 16 || kd.by != 16 || kd.bz != 1) return shape_err("BlockDim must be (16, 16, 1)");
      if (kd.gx != ceil_div(s[2], kSimtTile) || kd.gy != ceil_div(s[1], kSimtTile) || kd.gz != s[0])
        return shape_err("GridDim must be (ceil(N/64), ceil(M/64), batch)");
      if (k.smem < (size_t)kSimtSmemBytes) return shape_err("needs 8704 bytes of shared memory");
      GemmSimtF32::Params p{(const float *)a[0], (const float *)a[1], (const float *)a[2], (float *)a[3],
                            s[0], s[1], s[2], s[3], (int)(d.flags & BFUSE_FLAG_CAUSAL)};
      std::memcpy(k.params, &p, sizeof(p));
      return BFUSE_OK;
    }
    case BFUSE_OP_CONV2D_F32_SIMT: {
      if (s[0] <= 0 || s[1] <= 0 || s[4] <= 0 || s[5] <= 0 || s[6] <= 0 || s[7] <= 0 || s[8] < 0) return shape_err("bad conv shape");
      const int oh = conv_out(s[2], s[5], s[7], s[8]), ow = conv_out(s[3], s[6], s[7], s[8]);
      if (oh <= 0 || ow <= 0) return shape_err("empty output");
      if (kd.bx != 16 || kd.by != 16 || kd.bz != 1) return shape_err("BlockDim must be (16, 16, 1)");
      if (kd.gx != ceil_div(s[0] * oh * ow, kSimtTile) || kd.gy != ceil_div(s[4], kSimtTile) || kd.gz != 1)
        return shape_err("GridDim must be (ceil(n*oh*ow/64), ceil(co/64), 1)");
      if (k.smem < (size_t)kSimtSmemBytes) return shape_err("needs 8704 bytes of shared memory");
      ConvSimtF32::Params p{(const float *)a[0], (const float *)a[1], (float *)a[2], s[0], s[1], s[2], s[3],
                            s[4], s[5], s[6], s[7], s[8], oh, ow};
      std::memcpy(k.params, &p, sizeof(p));
      return BFUSE_OK;
    }
    case BFUSE_OP_CONV2D_TF32: {
      if (s[0] <= 0 || s[1] <= 0 || s[4] <= 0 || s[5] <= 0 || s[6] <= 0 || s[7] <= 0 || s[8] < 0) return shape_err("bad conv shape");
      const int oh = conv_out(s[2], s[5], s[7], s[8]), ow = conv_out(s[3], s[6], s[7], s[8]);
      if (oh <= 0 || ow <= 0) return shape_err("empty output");
      const int K = s[1] * s[5] * s[6];
      if (K > kConvMaxK || K % 4) return shape_err("ci*kh*kw must be a multiple of 4 and at most 8192 (offset table, TMA stride rule)");
      if (s[5] * s[6] > 31) return shape_err("kernel window larger than 31 taps");
      if (kd.bx != kConvThreads || kd.by != 1 || kd.bz != 1) return shape_err("BlockDim must be (224, 1, 1)");
      const int bn = s[9] > 0 ? s[9] : kConvBN;
      if (bn != 32 && bn != 64 && bn != 128) return shape_err("shape[9] (pixels per tile) must be 32, 64 or 128");
      const int split = s[10] > 0 ? s[10] : 1, num_kb = ceil_div(K, ConvUmmaTf32::kBK), q = ceil_div(num_kb, split);
      if (split > 8 || (split - 1) * q >= num_kb) return shape_err("shape[10] (k-slices) must be 1..8 with every k-slice non-empty");
      ConvStaging geometry;   // a staged conv's tiles may be whole output rows: fewer than BN pixels
      const int tile_px = s[11] == 1 && conv_staging(s[1], s[2], s[3], s[5], s[6], s[7], s[8], oh, ow, bn, &geometry) ? geometry.tile_px : bn;
      if (s[11] == 1) {
        if ((long long)kd.gx * kd.gy * kd.gz > (long long)ceil_div(oh * ow, tile_px) * ceil_div(s[4], kUmmaBM) * s[0])
          return shape_err("GridDim of a staged conv must not hold more CTAs than the conv has tiles (a CTA takes every grid-size-th tile)");
      } else if (kd.gx != split * ceil_div(oh * ow, tile_px) || kd.gy != ceil_div(s[4], kUmmaBM) || kd.gz != s[0]) {
        return shape_err("GridDim must be (k-slices * ceil(oh*ow / pixels per tile), ceil(co/128), n)");
      }
      k.cluster = split;
      ConvUmmaParams p;
      std::memset(&p, 0, sizeof(p));
      // Staged (input rows by TMA into a raw ring, repacked in shared memory) when the geometry allows
      // it and the registered window has room for the raw ring beside the smallest operand ring;
      // else gathered from global memory.  The raw ring is 3 slots deep, 4 when room is left for a
      // whole-SM operand ring as well.
      const int min_stages = ceil_div(umma_epilogue_bytes(bn, split, 4), conv_stage_bytes(bn));
      if (s[11] < 0 || s[11] > 2) return shape_err("shape[11] (operand mode) must be 0 (the runtime's choice), 1 (staged) or 2 (gathered)");
      if (s[11] == 1 && (split != 1 || !conv_staging(s[1], s[2], s[3], s[5], s[6], s[7], s[8], oh, ow, bn, &p.st)))
        return shape_err("shape[11] = 1 (staged operand) needs 128-pixel tiles, an unsplit K of whole K blocks, image rows of 16-byte multiples and a window whose rows fit a 24 KB slot");
      int wstages = 0;
      if (s[11] == 1) {
        if (!conv_staged_ring((int)std::min<size_t>(k.smem, kMaxSmemPerCta), K, p.st.cc * s[5] * s[6], p.st.slot_pitch, &p.st.slots, &wstages))
          return shape_err("shape[11] = 1 (staged operand): shared memory below the raw ring plus two weight stages");
      } else if (k.smem < (size_t)conv_umma_smem_bytes(min_stages, bn, K, 0)) {
        return shape_err("shared memory below the store buffers (and, for a split conv, the receive area of the k-slices)");
      }
      int rc = encode_map(ctx, &p.map_w, 4, a[1], K, s[4], 1, kUmmaBM);
      if (rc) return rc;
      if (p.st.slots) {
        // the NCHW input as {w, h, ci, n}; a box is one slot: pitch x rows x cc elements, rows taken with element stride ey
        const cuuint64_t dims[4] = {(cuuint64_t)s[3], (cuuint64_t)s[2], (cuuint64_t)s[1], (cuuint64_t)s[0]};
        const cuuint64_t strides[3] = {(cuuint64_t)s[3] * 4, (cuuint64_t)s[3] * s[2] * 4, (cuuint64_t)s[3] * s[2] * s[1] * 4};
        const cuuint32_t box[4] = {(cuuint32_t)p.st.pitch, (cuuint32_t)(p.st.rows * p.st.ey), (cuuint32_t)p.st.cc, 1};
        const cuuint32_t estr[4] = {1, (cuuint32_t)p.st.ey, 1, 1};
        const CUresult r = ctx->encode(&p.map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, a[0], dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                       CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(ctx, BFUSE_ERR_CUDA, "cuTensorMapEncodeTiled (conv input) failed (" + std::to_string((int)r) + ")");
      }
      if ((oh * ow) % 4 == 0) {  // else the rows are no 16-byte multiples and the body stores them itself
        rc = encode_map(ctx, &p.map_out, 4, a[2], oh * ow, s[4], s[0], 32);
        if (rc) return rc;
      }
      p.y = (float *)a[2];
      p.x = (const float *)a[0];
      p.n = s[0], p.ci = s[1], p.h = s[2], p.wd = s[3], p.co = s[4], p.kh = s[5], p.kw = s[6], p.stride = s[7], p.pad = s[8];
      p.oh = oh, p.ow = ow, p.K = K;
      p.stages = wstages ? wstages : std::min<int>(kUmmaMaxStages, (int)((k.smem - conv_header_bytes(K)) / conv_stage_bytes(bn)));
      p.bn = bn;
      p.split = split;
      p.kb_per_slice = q;
      p.ctas = kd.gx * kd.gy * kd.gz;
      static_assert(sizeof(p) <= kParamsBytes, "parameter block too small");
      std::memcpy(k.params, &p, sizeof(p));
      return BFUSE_OK;
    }
    case BFUSE_OP_GEMM_TF32:
    case BFUSE_OP_GEMM_BF16: {
      const int eb = d.op == BFUSE_OP_GEMM_TF32 ? 4 : 2;
      const int bn = s[4], split = s[5] > 0 ? s[5] : 1, bm = s[6] > 0 ? s[6] : kUmmaBM;
      if (s[0] <= 0 || s[1] <= 0 || s[2] <= 0 || s[3] <= 0) return shape_err("batch, M, N, K must be positive");
      if (bn != 32 && bn != 64 && bn != 128 && bn != 256) return shape_err("shape[4] (BN) must be 32, 64, 128 or 256");
      if (bn * eb < 128) return shape_err("shape[4] (BN) must span at least 128 bytes of output (64 for bf16): stores leave in 128-byte chunks");
      if ((s[3] * eb) % 16) return shape_err("K rows must be a multiple of 16 bytes (TMA stride rule)");
      if ((s[2] * eb) % 16) return shape_err("N must make output rows a multiple of 16 bytes");
      const int num_kb = ceil_div(s[3] * eb, kUmmaRowBytes), q = ceil_div(num_kb, split);
      if (split > 8 || (split - 1) * q >= num_kb) return shape_err("shape[5] (split) must be 1..8 with every k-slice non-empty");
      if (kd.bx != kUmmaThreads || kd.by != 1 || kd.bz != 1) return shape_err("BlockDim must be (192, 1, 1)");
      if ((bm != kUmmaBM && bm != 256) || (bm == 256 && split != 1) || bn * (bm / kUmmaBM) > 512)
        return shape_err("shape[6] (BM) must be 128, or 256 with split = 1");
      if (kd.gx != split * ceil_div(s[1], bm) || kd.gy != ceil_div(s[2], bn) || kd.gz != s[0])
        return shape_err("GridDim must be (split * ceil(M/BM), ceil(N/BN), batch)");
      if (k.smem < (size_t)umma_smem_bytes(bn, umma_min_stages(bn, split, eb, bm), bm))
        return shape_err("shared memory below the store buffers (and, for a split GEMM, the receive area of the k-slices)");
      k.cluster = split;
      GemmUmmaParams p;
      std::memset(&p, 0, sizeof(p));
      int rc = encode_map(ctx, &p.map_a, eb, a[0], s[3], s[1], s[0], bm);
      if (rc) return rc;
      rc = encode_map(ctx, &p.map_b, eb, a[1], s[3], s[2], s[0], bn);
      if (rc) return rc;
      rc = encode_map(ctx, &p.map_out, eb, a[3], s[2], s[1], s[0], 32);
      if (rc) return rc;
      p.bias = (const float *)a[2];
      p.out = a[3];
      p.batch = s[0], p.M = s[1], p.N = s[2], p.K = s[3];
      p.causal = (int)(d.flags & BFUSE_FLAG_CAUSAL);
      p.stages = std::min<int>(kUmmaMaxStages, (int)((k.smem - kUmmaHeaderBytes) / umma_stage_bytes(bn, bm)));
      p.bm = bm;
      p.bn = bn;
      p.split = split;
      p.kb_per_slice = q;
      static_assert(sizeof(p) <= kParamsBytes, "parameter block too small");
      std::memcpy(k.params, &p, sizeof(p));
      return BFUSE_OK;
    }
    default:
      return fail(ctx, BFUSE_ERR_INVALID, "operator not in the registry");
  }
}

__global__ void trace_kernel(const __grid_constant__ DispatchTable t, int *kernel_of, int *vblock_of, int *sm_of) {
  unsigned smid;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  if (!t.queue) {
    int k = -1, vb = -1;
    decode_cta(t, blockIdx.x, k, vb);
    if (threadIdx.x == 0) {
      kernel_of[blockIdx.x] = k;
      vblock_of[blockIdx.x] = vb;
      sm_of[blockIdx.x] = (int)smid;
    }
    return;
  }
  __shared__ int ticket_s;
  for (;;) {
    if (threadIdx.x == 0) ticket_s = (int)atomicAdd(t.queue_ctr, 1u);
    __syncthreads();
    const int ticket = ticket_s;
    __syncthreads();
    if (ticket >= t.total) break;
    int k = -1, vb = -1;
    decode_cta(t, ticket, k, vb);
    if (threadIdx.x == 0) {
      kernel_of[ticket] = k;
      vblock_of[ticket] = vb;
      sm_of[ticket] = (int)smid;
    }
  }
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(t.queue_ctr + 1, 1u) == gridDim.x - 1) {
      t.queue_ctr[0] = 0;
      t.queue_ctr[1] = 0;
    }
  }
}

template <int I>
void fill_rows(bfuse_context *ctx) {
  fill_pair_row<I>(ctx->pairs[I], &ctx->singles[I]);
  if constexpr (I + 1 < kNumOps) fill_rows<I + 1>(ctx);
}

KernelRec *get_kernel(bfuse_context *ctx, int h) {   // nullptr for a bad or released handle
  return (ctx && h >= 0 && h < (int)ctx->kernels.size()) ? ctx->kernels[h].get() : nullptr;
}
GroupRec *get_group(const bfuse_context *ctx, int h) {
  return (ctx && h >= 0 && h < (int)ctx->groups.size()) ? ctx->groups[h].get() : nullptr;
}
// first released slot of a handle table, else a new one at the end
template <class T>
int free_slot(std::vector<std::unique_ptr<T>> &v) {
  for (size_t i = 0; i < v.size(); ++i)
    if (!v[i]) return (int)i;
  v.emplace_back();
  return (int)v.size() - 1;
}
FusionRec *get_fusion(const bfuse_context *ctx, int h) {
  return (ctx && h >= 0 && h < (int)ctx->fusions.size()) ? ctx->fusions[h].get() : nullptr;
}

DispatchTable single_table(const bfuse_context *ctx, const KernelRec &k) {
  DispatchTable t;
  std::memset(&t, 0, sizeof(t));
  t.n_cta[0] = k.dims.grid();
  t.n_thr[0] = k.dims.block();
  t.grid_x[0] = k.dims.gx, t.grid_y[0] = k.dims.gy;
  t.blk_x[0] = k.dims.bx, t.blk_y[0] = k.dims.by;
  t.bar_count[0] = round_up32(k.dims.block());
  t.total = t.n_cta[0];
  t.cluster = k.cluster;
  t.status = ctx->d_status;
  t.no_pdl = ctx->no_pdl;
  return t;
}

int launch_one(bfuse_context *ctx, KernelRec &k, cudaStream_t s) {
  const DispatchTable t = single_table(ctx, k);
  const size_t smem = k.smem + 1024;
  cudaError_t e = ctx->singles[k.desc.op].launch(t, k.params, (unsigned)k.dims.grid(), (unsigned)k.dims.block(), smem, s);
  if (e != cudaSuccess) return fail_cuda(ctx, e, ("launch " + k.name).c_str());
  return BFUSE_OK;
}

// Shared-memory ring of a tensor-core operator: header bytes, bytes per stage, fewest stages its
// epilogue can live with, stages it has now.  False for operators without a ring.
bool ring_info(const KernelRec &k, int *header, int *stage_bytes, int *min_stages, int *stages) {
  const int *s = k.desc.shape;
  if (k.desc.op == BFUSE_OP_GEMM_TF32 || k.desc.op == BFUSE_OP_GEMM_BF16) {
    const int eb = k.desc.op == BFUSE_OP_GEMM_TF32 ? 4 : 2;
    const int bm = s[6] > 0 ? s[6] : kUmmaBM;
    *header = kUmmaHeaderBytes, *stage_bytes = umma_stage_bytes(s[4], bm);
    *min_stages = umma_min_stages(s[4], std::max(1, s[5]), eb, bm);
    *stages = reinterpret_cast<const GemmUmmaParams *>(k.params)->stages;
    return true;
  }
  if (k.desc.op == BFUSE_OP_CONV2D_TF32) {
    const int bn = s[9] > 0 ? s[9] : kConvBN;
    const ConvUmmaParams *cp = reinterpret_cast<const ConvUmmaParams *>(k.params);
    const int K = s[1] * s[5] * s[6];
    if (cp->st.slots) {   // staged: the raw ring stays as registered, the 16 KB weight stages are what can be given up
      *header = conv_header_bytes(K) + conv_raw_bytes(cp->st.slots, cp->st.slot_pitch), *stage_bytes = kUmmaABytes;
      *min_stages = std::min(2, K / ConvUmmaTf32::kBK);
    } else {
      *header = conv_header_bytes(K), *stage_bytes = conv_stage_bytes(bn);
      *min_stages = std::max(1, ceil_div(umma_epilogue_bytes(bn, std::max(1, s[10]), 4), conv_stage_bytes(bn)));
    }
    *stages = cp->stages;
    return true;
  }
  return false;
}

// parameter block of `k` with the ring depth replaced (stages > 0), else k's own
const void *params_with_stages(const KernelRec &k, int stages, unsigned char *scratch) {
  if (stages <= 0) return k.params;
  std::memcpy(scratch, k.params, kParamsBytes);
  if (k.desc.op == BFUSE_OP_CONV2D_TF32) reinterpret_cast<ConvUmmaParams *>(scratch)->stages = stages;
  else reinterpret_cast<GemmUmmaParams *>(scratch)->stages = stages;
  return scratch;
}

int launch_fused_rec(bfuse_context *ctx, FusionRec &f, cudaStream_t s, const DispatchTable *table = nullptr) {
  KernelRec &a = *ctx->kernels[f.k1], &b = *ctx->kernels[f.k2];
  const PairEntry &pe = ctx->pairs[a.desc.op][b.desc.op];
  PairLaunchFn fn = f.plan.table.kind == DISPATCH_THREADS ? pe.thread : (f.wide ? pe.block_wide : pe.block);
  alignas(64) unsigned char pa[kParamsBytes], pb[kParamsBytes];
  DispatchTable with_switch;
  if (ctx->no_pdl) {
    with_switch = table ? *table : f.plan.table;
    with_switch.no_pdl = 1;
    table = &with_switch;
  }
  cudaError_t e = fn(table ? *table : f.plan.table, params_with_stages(a, f.stages[0], pa), params_with_stages(b, f.stages[1], pb), f.launch_grid,
                     (unsigned)f.plan.fused_block, f.smem, s);
  if (e != cudaSuccess) return fail_cuda(ctx, e, ("launch " + f.name).c_str());
  return BFUSE_OK;
}

int launch_parallel_rec(bfuse_context *ctx, FusionRec &f, cudaStream_t s) {
  // fork the caller's stream into S1 / S2 and join back (run_parallel, operation_cu.py:203-229)
  CK(cudaEventRecord(ctx->ev_fork, s));
  CK(cudaStreamWaitEvent(ctx->s1, ctx->ev_fork, 0));
  CK(cudaStreamWaitEvent(ctx->s2, ctx->ev_fork, 0));
  int rc = launch_one(ctx, *ctx->kernels[f.k1], ctx->s1);
  if (rc) return rc;
  rc = launch_one(ctx, *ctx->kernels[f.k2], ctx->s2);
  if (rc) return rc;
  CK(cudaEventRecord(ctx->ev_j1, ctx->s1));
  CK(cudaEventRecord(ctx->ev_j2, ctx->s2));
  CK(cudaStreamWaitEvent(s, ctx->ev_j1, 0));
  CK(cudaStreamWaitEvent(s, ctx->ev_j2, 0));
  return BFUSE_OK;
}

int launch_mode(bfuse_context *ctx, FusionRec &f, int mode, cudaStream_t s) {
  switch (mode) {
    case 0: return launch_one(ctx, *ctx->kernels[f.k1], s);
    case 1: return launch_one(ctx, *ctx->kernels[f.k2], s);
    case 2: return launch_parallel_rec(ctx, f, s);
    case 3: {
      int rc = launch_one(ctx, *ctx->kernels[f.k1], s);
      return rc ? rc : launch_one(ctx, *ctx->kernels[f.k2], s);
    }
    case 4: return launch_fused_rec(ctx, f, s);
    default: return fail(ctx, BFUSE_ERR_INVALID, "mode must be 0..4");
  }
}

}  // namespace

// ================================================================================ C ABI

extern "C" {

int bfuse_create(int device, bfuse_context **out) {
  if (!out) return BFUSE_ERR_INVALID;
  *out = nullptr;
  std::unique_ptr<bfuse_context> c(new bfuse_context());
  bfuse_context *ctx = c.get();
  static std::string create_err;
  auto bail = [&](int code) {
    create_err = ctx->err;
    fprintf(stderr, "bfuse_create: %s\n", create_err.c_str());
    return code;
  };
  ctx->device = device;
  ctx->no_pdl = false;
  cudaDeviceProp prop;
  if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    ctx->err = "no usable CUDA device " + std::to_string(device);
    return bail(BFUSE_ERR_DEVICE);
  }
  if (prop.major != 10) {
    ctx->err = std::string("device is sm_") + std::to_string(prop.major * 10 + prop.minor) + ", this library is built for sm_100a only";
    return bail(BFUSE_ERR_DEVICE);
  }
  ctx->sm_count = prop.multiProcessorCount;
  void *fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
    ctx->err = "driver entry point cuTensorMapEncodeTiled not found";
    return bail(BFUSE_ERR_DEVICE);
  }
  ctx->encode = reinterpret_cast<EncodeTiledFn>(fn);
  fill_rows<0>(ctx);
  if (cudaStreamCreateWithFlags(&ctx->s1, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ctx->s2, cudaStreamNonBlocking) != cudaSuccess ||
      cudaStreamCreateWithFlags(&ctx->own, cudaStreamNonBlocking) != cudaSuccess ||
      cudaEventCreateWithFlags(&ctx->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ctx->ev_j1, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&ctx->ev_j2, cudaEventDisableTiming) != cudaSuccess ||
      cudaMalloc(&ctx->d_status, sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_status, 0, sizeof(int)) != cudaSuccess ||
      cudaHostAlloc(&ctx->h_status, sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
    ctx->err = std::string("context set-up failed: ") + cudaGetErrorString(cudaGetLastError());
    return bail(BFUSE_ERR_CUDA);
  }
  *out = c.release();
  return BFUSE_OK;
}

int bfuse_destroy(bfuse_context *ctx) {
  if (!ctx) return BFUSE_ERR_INVALID;
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  for (auto &g : ctx->graphs)
    if (g.exec) cudaGraphExecDestroy(g.exec);
  for (auto &f : ctx->fusions)
    if (f && f->queue_ctr) cudaFree(f->queue_ctr);
  for (cudaEvent_t e : ctx->batch_events) cudaEventDestroy(e);
  cudaFree(ctx->d_status);
  cudaFreeHost(ctx->h_status);
  cudaEventDestroy(ctx->ev_fork);
  cudaEventDestroy(ctx->ev_j1);
  cudaEventDestroy(ctx->ev_j2);
  cudaStreamDestroy(ctx->s1);
  cudaStreamDestroy(ctx->s2);
  cudaStreamDestroy(ctx->own);
  delete ctx;
  return BFUSE_OK;
}

const char *bfuse_last_error(const bfuse_context *ctx) { return ctx ? ctx->err.c_str() : "null context"; }
int bfuse_device_sm_count(const bfuse_context *ctx) { return ctx ? ctx->sm_count : -1; }

int bfuse_default_launch(const bfuse_context *ctx, bfuse_kernel_desc *desc) {
  if (!desc) return BFUSE_ERR_INVALID;
  std::string err;
  const int rc = default_launch(ctx, desc, &err);
  if (rc && ctx) const_cast<bfuse_context *>(ctx)->err = err;
  return rc;
}

int bfuse_arg_info(const bfuse_context *ctx, const bfuse_kernel_desc *desc, int i, size_t *bytes, int *is_output) {
  if (!desc) return BFUSE_ERR_INVALID;
  ArgInfo a[BFUSE_MAX_ARGS];
  std::string err;
  const int n = describe_args(*desc, a, &err);
  if (n < 0 || i < 0 || i >= n) {
    if (ctx) const_cast<bfuse_context *>(ctx)->err = n < 0 ? err : "argument index out of range";
    return BFUSE_ERR_INVALID;
  }
  if (bytes) *bytes = a[i].bytes;
  if (is_output) *is_output = a[i].is_output;
  return BFUSE_OK;
}

int bfuse_register_kernel(bfuse_context *ctx, const bfuse_kernel_desc *desc, int *kernel) {
  if (!ctx || !desc || !kernel) return BFUSE_ERR_INVALID;
  if (desc->op < 0 || desc->op >= kNumOps) return fail(ctx, BFUSE_ERR_INVALID, "operator not in the registry");
  std::unique_ptr<KernelRec> k(new KernelRec());
  k->desc = *desc;
  k->name = desc->KernelName ? desc->KernelName : ("kernel" + std::to_string(ctx->kernels.size()));
  k->desc.KernelName = nullptr;
  k->dims = {desc->GridDim.X, desc->GridDim.Y, desc->GridDim.Z, desc->BlockDim.X, desc->BlockDim.Y, desc->BlockDim.Z};
  if (k->dims.gx <= 0 || k->dims.gy <= 0 || k->dims.gz <= 0 || k->dims.bx <= 0 || k->dims.by <= 0 || k->dims.bz <= 0)
    return fail(ctx, BFUSE_ERR_SHAPE, k->name + ": GridDim and BlockDim must be positive");
  k->smem = desc->smem_bytes;
  if (k->smem + 1024 > kMaxSmemPerCta) return fail(ctx, BFUSE_ERR_SMEM, k->name + ": shared memory over the 227 KB per-CTA budget");
  std::string err;
  k->nargs = describe_args(k->desc, k->arg, &err);
  if (k->nargs < 0) return fail(ctx, BFUSE_ERR_INVALID, err);
  if (desc->nargs != k->nargs) return fail(ctx, BFUSE_ERR_INVALID, k->name + ": wrong number of arguments for this operator");
  k->alias_of = -1;
  k->users = 0;
  cudaSetDevice(ctx->device);
  const int rc = build_params(ctx, *k);
  if (rc) return rc;
  *kernel = free_slot(ctx->kernels);
  ctx->kernels[*kernel] = std::move(k);
  return BFUSE_OK;
}

int bfuse_set_kernel_args(bfuse_context *ctx, int kernel, void *const *args, int nargs) {
  KernelRec *k = get_kernel(ctx, kernel);
  if (!k || !args || nargs != k->nargs) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle or argument count");
  void *saved[BFUSE_MAX_ARGS];
  std::memcpy(saved, k->desc.args, sizeof(saved));
  for (int i = 0; i < nargs; ++i) k->desc.args[i] = args[i];
  cudaSetDevice(ctx->device);
  const int rc = build_params(ctx, *k);
  if (rc) {
    std::memcpy(k->desc.args, saved, sizeof(saved));
    build_params(ctx, *k);
    return rc;
  }
  // hidden unsplit re-tilings of this kernel (thread-split / work-queue fusions) follow it
  for (auto &other : ctx->kernels)
    if (other && other->alias_of == kernel) {
      std::memcpy(other->desc.args, k->desc.args, sizeof(saved));
      const int rc2 = build_params(ctx, *other);
      if (rc2) return rc2;
    }
  return BFUSE_OK;
}

int bfuse_register_fusion(bfuse_context *ctx, int kernel1, int kernel2, int pattern, int param_m, int param_n, int *fusion) {
  KernelRec *a = get_kernel(ctx, kernel1), *b = get_kernel(ctx, kernel2);
  if (!a || !b || !fusion) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle");
  if (a->alias_of >= 0 || b->alias_of >= 0) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle");
  std::unique_ptr<FusionRec> f(new FusionRec());
  f->k1 = f->reg1 = kernel1, f->k2 = f->reg2 = kernel2;
  f->retiled[0] = f->retiled[1] = false;
  f->users = 0;
  // Thread split and the work queue cannot host operators launched as clusters (a cluster's CTAs must
  // start together; a persistent CTA or a thread range is no cluster).  An operator whose tiling splits
  // K over a cluster is therefore re-tiled with one k-slice for such a fusion -- a hidden kernel record
  // owned by the fusion, same buffers and tile width -- and the fusion's record says so.  Every launch
  // mode of this fusion (fused, sequential, parallel) then uses the unsplit tiling, so fused == unfused
  // still holds bit for bit within the fusion; the k-split kernel launched by its own handle sums in a
  // different order.
  struct Undo {   // hidden records are dropped again if the registration fails further down
    bfuse_context *c;
    int h[2] = {-1, -1};
    bool keep = false;
    ~Undo() {
      for (int x : h)
        if (x >= 0 && !keep) c->kernels[x].reset();
    }
  } undo{ctx};
  if (pattern == PATTERN_THREAD_SPLIT || pattern == PATTERN_WORK_QUEUE) {
    KernelRec **side[2] = {&a, &b};
    int *handle[2] = {&f->k1, &f->k2};
    for (int i = 0; i < 2; ++i) {
      KernelRec *orig = *side[i];
      if (orig->cluster <= 1) continue;
      std::unique_ptr<KernelRec> alt(new KernelRec(*orig));
      const bool conv = orig->desc.op == BFUSE_OP_CONV2D_TF32;
      alt->desc.shape[conv ? 10 : 5] = 1;
      if (!conv) alt->desc.shape[6] = 0;   // tile height: the runtime's choice for the unsplit form
      alt->desc.KernelName = nullptr;
      std::string err;
      int rc = default_launch(ctx, &alt->desc, &err);
      if (rc) return fail(ctx, rc, orig->name + " (re-tiled with one k-slice): " + err);
      alt->dims = {alt->desc.GridDim.X, alt->desc.GridDim.Y, alt->desc.GridDim.Z, alt->desc.BlockDim.X, alt->desc.BlockDim.Y, alt->desc.BlockDim.Z};
      alt->smem = alt->desc.smem_bytes;
      alt->alias_of = *handle[i];
      alt->users = 0;
      rc = build_params(ctx, *alt);
      if (rc) return rc;
      const int slot = free_slot(ctx->kernels);
      ctx->kernels[slot] = std::move(alt);
      undo.h[i] = slot;
      *handle[i] = slot;
      *side[i] = ctx->kernels[slot].get();
      f->retiled[i] = true;
    }
    // free_slot may have grown the table: the unique_ptrs moved, the records they own did not
    a = ctx->kernels[f->k1].get(), b = ctx->kernels[f->k2].get();
  }
  const KernelDims kd[2] = {a->dims, b->dims};
  if (pattern == PATTERN_SM_STRIPED && param_m == 0) param_m = ctx->sm_count;
  if (pattern != PATTERN_SM_STRIPED && pattern != PATTERN_THREAD_SPLIT && pattern != PATTERN_RANGE_SPLIT) {
    if (param_m == 0) param_m = 1;
    if (param_n == 0) param_n = 1;
  }
  // operators launched as clusters (split-K GEMMs) make the patterns schedule whole clusters
  const int cluster = std::max(a->cluster, b->cluster);
  if ((a->cluster != 1 && a->cluster != cluster) || (b->cluster != 1 && b->cluster != cluster))
    return fail(ctx, BFUSE_ERR_UNSUPPORTED, "the two operators need different cluster widths; register them with equal splits");
  std::string err;
  if (!plan_pair(kd, pattern, param_m, param_n, param_m, &f->plan, &err, cluster)) return fail(ctx, BFUSE_ERR_INVALID, err);
  DispatchTable &t = f->plan.table;
  t.status = ctx->d_status;
  const bool thread_split = t.kind == DISPATCH_THREADS;
  // fused kernel name as FusionContext::create builds it (src/Contexts.cc:67-84)
  f->name = a->name + "_" + b->name + (thread_split ? "_fused_hfuse" : "_fused_bfuse");
  // shared memory: union for block-level fusion, sum for thread-level fusion (Matchers.cc:512-519)
  f->stages[0] = f->stages[1] = 0;
  // tensor-memory columns an operator's CTA allocates
  auto tmem_cols = [](const KernelRec &k) {
    if (k.desc.op == BFUSE_OP_GEMM_TF32 || k.desc.op == BFUSE_OP_GEMM_BF16) return k.desc.shape[4] * std::max(1, k.desc.shape[6] / kUmmaBM);
    if (k.desc.op == BFUSE_OP_CONV2D_TF32 && k.desc.shape[11] == 1) return kConvTmemCols;   // staged: accumulator and operand stages
    return k.desc.op == BFUSE_OP_CONV2D_TF32 ? (k.desc.shape[9] > 0 ? k.desc.shape[9] : kConvBN) : 0;
  };
  // a persistent CTA of the work queue allocates once what either operator's tile may need (a power of two >= 32)
  t.tmem_cols = 0;
  if (t.queue) {
    const int need = std::max(tmem_cols(*a), tmem_cols(*b));
    for (int c = 32; need > 0 && t.tmem_cols == 0; c *= 2)
      if (c >= need) t.tmem_cols = c;
  }
  if (thread_split) {
    // both operators allocate tensor memory in the same CTA; an allocation that cannot be granted
    // would block for ever, so the sum has to fit the SM's 512 columns
    if (tmem_cols(*a) + tmem_cols(*b) > 512)
      return fail(ctx, BFUSE_ERR_UNSUPPORTED, "thread split: the two operators need more than 512 tensor-memory columns together");
    // both windows live side by side; rings registered for a whole SM each are made shallower until
    // the sum fits (the deeper one first), never below what the operator's epilogue needs
    size_t win[2] = {a->smem, b->smem};
    int hdr[2], stg[2], mn[2], st[2];
    const bool ring[2] = {ring_info(*a, &hdr[0], &stg[0], &mn[0], &st[0]), ring_info(*b, &hdr[1], &stg[1], &mn[1], &st[1])};
    auto total = [&] { return (win[0] + 1023) / 1024 * 1024 + win[1] + 1024; };
    while (total() > kMaxSmemPerCta) {
      int pick = -1;
      for (int i = 0; i < 2; ++i)
        if (ring[i] && st[i] > mn[i] && (pick < 0 || win[i] > win[pick])) pick = i;
      if (pick < 0) break;
      --st[pick];
      win[pick] = (size_t)hdr[pick] + (size_t)st[pick] * stg[pick];
      f->stages[pick] = st[pick];
    }
    t.smem_off[0] = 0;
    t.smem_off[1] = (int)((win[0] + 1023) / 1024 * 1024);
    f->smem = t.smem_off[1] + win[1] + 1024;
  } else {
    // The union is the larger window, and every CTA of the fused grid is charged for it.  A ring that
    // was sized for a CTA with an SM to itself would then keep the partner's CTAs from sharing SMs:
    // when the fused grid needs more than one CTA per SM, such rings are made shallower (never below
    // what the operator's epilogue needs, and only if at least three stages remain) until two CTAs fit.
    size_t win[2] = {a->smem, b->smem};
    constexpr size_t kHalfSm = 111 * 1024;
    // clusters have to fit a GPC each, so fewer CTAs than SMs can be resident at one CTA per SM: ask
    bool second_wave = f->plan.fused_grid > ctx->sm_count;
    if (!second_wave && cluster > 1 && std::max(win[0], win[1]) > kHalfSm) {
      cudaSetDevice(ctx->device);
      const int cap = ctx->pairs[a->desc.op][b->desc.op].block_clusters((unsigned)f->plan.fused_block, std::max(win[0], win[1]) + 1024, cluster);
      second_wave = cap > 0 && f->plan.fused_grid / cluster > cap;
    }
    if (second_wave && !t.queue) {
      KernelRec *ks[2] = {a, b};
      for (int i = 0; i < 2; ++i) {
        int hdr, stg, mn, st;
        if (win[i] <= kHalfSm || !ring_info(*ks[i], &hdr, &stg, &mn, &st)) continue;
        const int fit = (int)((kHalfSm - hdr) / stg);
        if (fit < st && fit >= std::max(mn, 3)) {  // a ring of fewer than 3 stages is no pipeline: such tiles keep their SM
          f->stages[i] = fit;
          win[i] = (size_t)hdr + (size_t)fit * stg;
        }
      }
    }
    f->smem = std::max(win[0], win[1]) + 1024;
  }
  if (f->smem > kMaxSmemPerCta) return fail(ctx, BFUSE_ERR_SMEM, f->name + ": fused shared memory over the 227 KB per-CTA budget");
  f->launch_grid = (unsigned)f->plan.fused_grid;
  cudaSetDevice(ctx->device);
  const PairEntry &pe = ctx->pairs[a->desc.op][b->desc.op];
  // the register-richer build of the pair when its occupancy still holds the whole grid in one wave
  // (or, for two memory-bound bodies, when the grid is many waves long and waves stop mattering)
  f->wide = !thread_split && pe.block_wide && !t.queue &&
            (f->launch_grid <= (unsigned)(pe.wide_min_blocks * ctx->sm_count) ||
             (pe.wide_min_blocks == 4 && f->launch_grid >= (unsigned)(12 * ctx->sm_count)));
  cudaFuncAttributes attr;
  cudaError_t e = (thread_split ? pe.thread_attr : (f->wide ? pe.block_wide_attr : pe.block_attr))(&attr);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "cudaFuncGetAttributes");
  f->regs = attr.numRegs;
  if (t.queue) {
    // persistent grid: as many CTAs as can be resident at once, never more than there are tickets
    const int threads = f->plan.fused_block;
    const int by_regs = std::max(1, 65536 / std::max(1, attr.numRegs * threads));
    const int by_thr = std::max(1, 2048 / threads);
    const int by_smem = std::max<int>(1, (int)((228 * 1024) / (f->smem + 1024)));
    const int per_sm = std::min({by_regs, by_thr, by_smem, 32});
    f->launch_grid = (unsigned)std::min(t.total, per_sm * ctx->sm_count);
    CK(cudaMalloc(&f->queue_ctr, 2 * sizeof(unsigned)));
    CK(cudaMemset(f->queue_ctr, 0, 2 * sizeof(unsigned)));
    t.queue_ctr = f->queue_ctr;
  }
  undo.keep = true;
  ++ctx->kernels[f->reg1]->users, ++ctx->kernels[f->reg2]->users;
  *fusion = free_slot(ctx->fusions);
  ctx->fusions[*fusion] = std::move(f);
  return BFUSE_OK;
}

int bfuse_register_group(bfuse_context *ctx, const int *kernels, int n, int pattern, int param_m, int param_n, int *group) {
  if (!ctx || !kernels || !group) return fail(ctx, BFUSE_ERR_INVALID, "null argument");
  if (n < 2 || n > kGroupMax) return fail(ctx, BFUSE_ERR_INVALID, "a group holds 2 to 4 kernels");
  std::unique_ptr<GroupRec> g(new GroupRec());
  g->n = n;
  KernelRec *ks[kGroupMax];
  KernelDims kd[kGroupMax];
  int cluster = 1;
  for (int i = 0; i < n; ++i) {
    ks[i] = get_kernel(ctx, kernels[i]);
    if (!ks[i] || ks[i]->alias_of >= 0) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle");
    g->ks[i] = kernels[i];
    kd[i] = ks[i]->dims;
    cluster = std::max(cluster, ks[i]->cluster);
    g->name += (i ? "_" : "") + ks[i]->name;
  }
  g->name += "_fused_bfuse";
  // one body, or two: a kernel exists per body and per unordered pair of bodies
  g->op_lo = g->op_hi = ks[0]->desc.op;
  for (int i = 1; i < n; ++i) {
    const int op = ks[i]->desc.op;
    if (op == g->op_lo || op == g->op_hi) continue;
    if (g->op_lo != g->op_hi) return fail(ctx, BFUSE_ERR_UNSUPPORTED, "the kernels of a group may use at most two operator bodies");
    if (op < g->op_lo) g->op_lo = op;
    else g->op_hi = op;
  }
  const bool mixed = g->op_lo != g->op_hi;
  for (int i = 0; i < n; ++i)
    if (ks[i]->cluster != 1 && ks[i]->cluster != cluster)
      return fail(ctx, BFUSE_ERR_UNSUPPORTED, "the operators need different cluster widths; register them with equal splits");
  if (pattern != PATTERN_ZIGZAG && pattern != PATTERN_PROPORTIONAL && pattern != PATTERN_RANGE_SPLIT)
    return fail(ctx, BFUSE_ERR_UNSUPPORTED, "a group takes the zig-zag, proportional and range-split patterns");
  if (pattern != PATTERN_RANGE_SPLIT) {
    if (param_m == 0) param_m = 1;
    if (param_n == 0) param_n = 1;
  }
  std::string err;
  if (!plan_group(kd, n, pattern, param_m, param_n, &g->plan, &err, cluster)) return fail(ctx, BFUSE_ERR_INVALID, err);
  g->plan.table.status = ctx->d_status;
  for (int i = 0, na = 0, nb = 0; i < n; ++i) {
    const bool second = mixed && ks[i]->desc.op == g->op_hi;
    g->plan.table.body[i] = second ? 1 : 0;
    g->plan.table.slot[i] = second ? nb++ : na++;
  }
  const PairEntry &mixed_entry = ctx->pairs[g->op_lo][g->op_hi];
  // shared memory: the union of the windows; rings sized for a whole SM are made shallower when the
  // fused grid needs two CTAs per SM (same rule as for a pair)
  constexpr size_t kHalfSm = 111 * 1024;
  size_t win = 0, widest = 0;
  for (int i = 0; i < n; ++i) widest = std::max(widest, ks[i]->smem);
  bool second_wave = g->plan.fused_grid > ctx->sm_count;
  if (!second_wave && cluster > 1 && widest > kHalfSm) {   // clusters fit a GPC each: fewer resident CTAs than SMs
    cudaSetDevice(ctx->device);
    const int cap = mixed ? mixed_entry.mixed_clusters((unsigned)g->plan.fused_block, widest + 1024, cluster)
                          : ctx->singles[ks[0]->desc.op].group_clusters((unsigned)g->plan.fused_block, widest + 1024, cluster);
    second_wave = cap > 0 && g->plan.fused_grid / cluster > cap;
  }
  for (int i = 0; i < n; ++i) {
    size_t w = ks[i]->smem;
    int hdr, stg, mn, st;
    g->stages[i] = 0;
    if (second_wave && w > kHalfSm && ring_info(*ks[i], &hdr, &stg, &mn, &st)) {
      const int fit = (int)((kHalfSm - hdr) / stg);
      if (fit < st && fit >= std::max(mn, 3)) {
        g->stages[i] = fit;
        w = (size_t)hdr + (size_t)fit * stg;
      }
    }
    win = std::max(win, w);
  }
  g->smem = win + 1024;
  if (g->smem > kMaxSmemPerCta) return fail(ctx, BFUSE_ERR_SMEM, g->name + ": fused shared memory over the 227 KB per-CTA budget");
  cudaSetDevice(ctx->device);
  cudaFuncAttributes attr;
  cudaError_t e = mixed ? mixed_entry.mixed_attr(&attr) : ctx->singles[ks[0]->desc.op].group_attr(&attr);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "cudaFuncGetAttributes");
  g->regs = attr.numRegs;
  for (int i = 0; i < n; ++i) ++ks[i]->users;
  *group = free_slot(ctx->groups);
  ctx->groups[*group] = std::move(g);
  return BFUSE_OK;
}

int bfuse_group_info(bfuse_context *ctx, int group, bfuse_kernel_desc *out) {
  if (!get_group(ctx, group) || !out) return fail(ctx, BFUSE_ERR_INVALID, "bad group handle");
  const GroupRec &g = *ctx->groups[group];
  std::memset(out, 0, sizeof(*out));
  out->KernelName = g.name.c_str();
  out->HasBarriers = 1;
  out->GridDim = {g.plan.fused_grid, 1, 1};
  out->BlockDim = {g.plan.fused_block, 1, 1};
  out->Reg = g.regs;
  out->ExecTime = -1.f;
  out->op = -1;
  out->smem_bytes = g.smem;
  out->shape[0] = g.plan.fused_grid;
  return BFUSE_OK;
}

int bfuse_group_map_block(const bfuse_context *ctx, int group, int b, int *kernel, int *vblock) {
  if (!get_group(ctx, group) || !kernel || !vblock || b < 0) return BFUSE_ERR_INVALID;
  const GroupRec &g = *ctx->groups[group];
  int k, vb;
  if (b >= g.plan.fused_grid || !decode_group_cta(g.plan.table, b, k, vb)) return BFUSE_ERR_INVALID;
  *kernel = k, *vblock = vb;
  return BFUSE_OK;
}

int bfuse_launch_group(bfuse_context *ctx, int group, void *stream) {
  if (!get_group(ctx, group)) return fail(ctx, BFUSE_ERR_INVALID, "bad group handle");
  GroupRec &g = *ctx->groups[group];
  alignas(64) unsigned char scratch[kGroupMax][kParamsBytes];
  const void *params[2][kGroupMax];
  int count[2] = {0, 0};
  for (int i = 0; i < g.n; ++i) {
    const int b = g.plan.table.body[i];
    params[b][count[b]++] = params_with_stages(*ctx->kernels[g.ks[i]], g.stages[i], scratch[i]);
  }
  g.plan.table.no_pdl = ctx->no_pdl;
  cudaError_t e;
  if (g.op_lo != g.op_hi)
    e = ctx->pairs[g.op_lo][g.op_hi].mixed(g.plan.table, params[0], count[0], params[1], count[1], (unsigned)g.plan.fused_grid,
                                           (unsigned)g.plan.fused_block, g.smem, (cudaStream_t)stream);
  else
    e = ctx->singles[g.op_lo].group(g.plan.table, params[0], g.n, (unsigned)g.plan.fused_grid, (unsigned)g.plan.fused_block, g.smem,
                                    (cudaStream_t)stream);
  if (e != cudaSuccess) return fail_cuda(ctx, e, ("launch " + g.name).c_str());
  return BFUSE_OK;
}

int bfuse_plan_group(const bfuse_dim3 *grid, const bfuse_dim3 *block, int n, int pattern, int param_m, int param_n,
                     int cluster, int *fused_block, int *kernel_of, int *vblock_of, int cap) {
  if (!grid || !block || n < 2 || n > kGroupMax) return -BFUSE_ERR_INVALID;
  KernelDims kd[kGroupMax];
  for (int i = 0; i < n; ++i) kd[i] = KernelDims{grid[i].X, grid[i].Y, grid[i].Z, block[i].X, block[i].Y, block[i].Z};
  GroupPlan p;
  std::string err;
  if (pattern != PATTERN_ZIGZAG && pattern != PATTERN_PROPORTIONAL && pattern != PATTERN_RANGE_SPLIT) return -BFUSE_ERR_UNSUPPORTED;
  if (!plan_group(kd, n, pattern, param_m, param_n, &p, &err, cluster < 1 ? 1 : cluster)) return -BFUSE_ERR_INVALID;
  if (fused_block) *fused_block = p.fused_block;
  for (int b = 0; b < p.fused_grid && b < cap && kernel_of && vblock_of; ++b) {
    int k, vb;
    if (decode_group_cta(p.table, b, k, vb)) kernel_of[b] = k, vblock_of[b] = vb;
    else kernel_of[b] = -1, vblock_of[b] = -1;
  }
  return p.fused_grid;
}

int bfuse_fusion_info(bfuse_context *ctx, int fusion, bfuse_kernel_desc *out) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f || !out) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  std::memset(out, 0, sizeof(*out));
  out->KernelName = f->name.c_str();
  out->HasBarriers = 1;
  out->GridDim = {f->plan.fused_grid, 1, 1};
  out->BlockDim = {f->plan.fused_block, 1, 1};
  out->Reg = f->regs;
  out->ExecTime = -1.f;
  out->op = -1;
  out->smem_bytes = f->smem;
  out->shape[0] = (int)f->launch_grid;  // CTAs actually launched (differs from GridDim for the work queue)
  // CTAs of this kernel resident at once according to the occupancy calculator (whole clusters; one CTA per SM
  // for kernels that allocate tensor memory), 0 when not asked
  out->shape[1] = 0;
  // operator 1 / 2 runs here in a one-k-slice re-tiling of the registered kernel (thread split, work queue)
  out->shape[2] = f->retiled[0] ? 1 : 0;
  out->shape[3] = f->retiled[1] ? 1 : 0;
  if (f->plan.table.kind != DISPATCH_THREADS && !f->wide) {
    const int cl = std::max(1, f->plan.table.cluster);
    cudaSetDevice(ctx->device);
    const int cap = ctx->pairs[ctx->kernels[f->k1]->desc.op][ctx->kernels[f->k2]->desc.op].block_clusters((unsigned)f->plan.fused_block, f->smem, cl);
    if (cap > 0) out->shape[1] = cap * cl;
  }
  return BFUSE_OK;
}

int bfuse_fusion_map_block(const bfuse_context *ctx, int fusion, int b, int *kernel, int *vblock) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f || !kernel || !vblock || b < 0) return BFUSE_ERR_INVALID;
  int k, vb;
  const int limit = f->plan.table.queue ? f->plan.table.total : f->plan.fused_grid;
  if (b >= limit || !decode_cta(f->plan.table, b, k, vb)) return BFUSE_ERR_INVALID;
  *kernel = k, *vblock = vb;
  return BFUSE_OK;
}

int bfuse_fusion_map_thread(const bfuse_context *ctx, int fusion, int kernel, int b, int t, int *vblock, int *vthread, int *active) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f || kernel < 0 || kernel > 1 || !active) return BFUSE_ERR_INVALID;
  const DispatchTable &tb = f->plan.table;
  if (tb.kind != DISPATCH_THREADS) return BFUSE_ERR_UNSUPPORTED;
  const int vt = t - tb.thr_lo[kernel];
  *active = vt >= 0 && vt < tb.n_thr[kernel] && b >= 0 && b < tb.n_cta[kernel];
  if (vblock) *vblock = b;
  if (vthread) *vthread = vt;
  return BFUSE_OK;
}

int bfuse_launch_kernel(bfuse_context *ctx, int kernel, void *stream) {
  KernelRec *k = get_kernel(ctx, kernel);
  if (!k) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle");
  return launch_one(ctx, *k, (cudaStream_t)stream);
}
int bfuse_launch_sequential(bfuse_context *ctx, int fusion, void *stream) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  return launch_mode(ctx, *f, 3, (cudaStream_t)stream);
}
int bfuse_launch_parallel(bfuse_context *ctx, int fusion, void *stream) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  return launch_mode(ctx, *f, 2, (cudaStream_t)stream);
}
int bfuse_launch_fused(bfuse_context *ctx, int fusion, void *stream) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  return launch_fused_rec(ctx, *f, (cudaStream_t)stream);
}

int bfuse_launch_list(bfuse_context *ctx, const int *fusions, int n, int mode, void *stream) {
  if (!ctx || !fusions || n < 0) return BFUSE_ERR_INVALID;
  for (int i = 0; i < n; ++i) {
    FusionRec *f = get_fusion(ctx, fusions[i]);
    if (!f) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle in list");
    const int rc = launch_mode(ctx, *f, mode, (cudaStream_t)stream);
    if (rc) return rc;
  }
  return BFUSE_OK;
}

int bfuse_graph_create(bfuse_context *ctx, const int *fusions, int n, int mode, int *graph) {
  if (!ctx || !fusions || n <= 0 || !graph) return BFUSE_ERR_INVALID;
  cudaSetDevice(ctx->device);
  // one plain pass first: it sets every kernel's shared-memory attribute outside the capture
  int rc0 = bfuse_launch_list(ctx, fusions, n, mode, ctx->own);
  if (rc0) return rc0;
  CK(cudaStreamSynchronize(ctx->own));
  cudaGraph_t g = nullptr;
  CK(cudaStreamBeginCapture(ctx->own, cudaStreamCaptureModeThreadLocal));
  int rc = bfuse_launch_list(ctx, fusions, n, mode, ctx->own);
  cudaError_t e = cudaStreamEndCapture(ctx->own, &g);
  if (rc) {
    if (g) cudaGraphDestroy(g);
    return rc;
  }
  if (e != cudaSuccess) return fail_cuda(ctx, e, "cudaStreamEndCapture");
  GraphRec gr{nullptr, n * (mode == 2 || mode == 3 ? 2 : 1), std::vector<int>(fusions, fusions + n)};
  e = cudaGraphInstantiate(&gr.exec, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "cudaGraphInstantiate");
  for (int h : gr.fusions) ++ctx->fusions[h]->users;
  int slot = -1;
  for (size_t i = 0; i < ctx->graphs.size() && slot < 0; ++i)
    if (!ctx->graphs[i].exec) slot = (int)i;
  if (slot < 0) {
    ctx->graphs.emplace_back();
    slot = (int)ctx->graphs.size() - 1;
  }
  ctx->graphs[slot] = std::move(gr);
  *graph = slot;
  return BFUSE_OK;
}

int bfuse_graph_destroy(bfuse_context *ctx, int graph) {
  if (!ctx || graph < 0 || graph >= (int)ctx->graphs.size() || !ctx->graphs[graph].exec) return fail(ctx, BFUSE_ERR_INVALID, "bad graph handle");
  cudaSetDevice(ctx->device);
  GraphRec &g = ctx->graphs[graph];
  CK(cudaGraphExecDestroy(g.exec));
  g.exec = nullptr;
  for (int h : g.fusions)
    if (FusionRec *f = get_fusion(ctx, h)) --f->users;
  g.fusions.clear();
  return BFUSE_OK;
}

// ---- release (finalize_kernel1/2 of the reference harness, operation_cu.py:146-162) ------------------

int bfuse_unregister_fusion(bfuse_context *ctx, int fusion) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  if (f->users > 0) return fail(ctx, BFUSE_ERR_INVALID, f->name + ": still captured by a graph; destroy the graph first");
  cudaSetDevice(ctx->device);
  if (f->queue_ctr) {
    // the counters may still be in use by a launch in flight
    CK(cudaDeviceSynchronize());
    CK(cudaFree(f->queue_ctr));
  }
  if (f->retiled[0]) ctx->kernels[f->k1].reset();
  if (f->retiled[1]) ctx->kernels[f->k2].reset();
  --ctx->kernels[f->reg1]->users, --ctx->kernels[f->reg2]->users;
  ctx->fusions[fusion].reset();
  return BFUSE_OK;
}

int bfuse_unregister_group(bfuse_context *ctx, int group) {
  GroupRec *g = get_group(ctx, group);
  if (!g) return fail(ctx, BFUSE_ERR_INVALID, "bad group handle");
  for (int i = 0; i < g->n; ++i) --ctx->kernels[g->ks[i]]->users;
  ctx->groups[group].reset();
  return BFUSE_OK;
}

int bfuse_unregister_kernel(bfuse_context *ctx, int kernel) {
  KernelRec *k = get_kernel(ctx, kernel);
  if (!k || k->alias_of >= 0) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle");
  if (k->users > 0) return fail(ctx, BFUSE_ERR_INVALID, k->name + ": still used by a fusion or group; release those first");
  ctx->kernels[kernel].reset();
  return BFUSE_OK;
}

int bfuse_graph_launch(bfuse_context *ctx, int graph, void *stream) {
  if (!ctx || graph < 0 || graph >= (int)ctx->graphs.size() || !ctx->graphs[graph].exec) return BFUSE_ERR_INVALID;
  CK(cudaGraphLaunch(ctx->graphs[graph].exec, (cudaStream_t)stream));
  return BFUSE_OK;
}

int bfuse_trace_fused(bfuse_context *ctx, int fusion, int *kernel_of, int *vblock_of, int *sm_of, int n) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f || !kernel_of || !vblock_of || !sm_of) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  const DispatchTable &t = f->plan.table;
  if (t.kind == DISPATCH_THREADS) return fail(ctx, BFUSE_ERR_UNSUPPORTED, "thread-split fusions host both operators in every CTA");
  const int cnt = t.queue ? t.total : f->plan.fused_grid;
  if (n < cnt) return fail(ctx, BFUSE_ERR_INVALID, "trace arrays shorter than the fused grid");
  cudaSetDevice(ctx->device);
  int *d = nullptr;
  CK(cudaMalloc(&d, 3 * sizeof(int) * cnt));
  cudaError_t e = cudaMemset(d, 0xff, 3 * sizeof(int) * cnt);
  if (e == cudaSuccess) {
    trace_kernel<<<f->launch_grid, 32, 0, ctx->own>>>(t, d, d + cnt, d + 2 * cnt);
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->own);
  if (e == cudaSuccess) e = cudaMemcpy(kernel_of, d, sizeof(int) * cnt, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(vblock_of, d + cnt, sizeof(int) * cnt, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(sm_of, d + 2 * cnt, sizeof(int) * cnt, cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "trace");
  return BFUSE_OK;
}

int bfuse_debug_fused_timeline(bfuse_context *ctx, const int *fusions, int n, long long *times, const int *slots) {
  if (!ctx || !fusions || !times || !slots || n <= 0) return BFUSE_ERR_INVALID;
  size_t total = 0;
  for (int i = 0; i < n; ++i) {
    FusionRec *f = get_fusion(ctx, fusions[i]);
    if (!f) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle in list");
    if (f->plan.table.kind == DISPATCH_THREADS) return fail(ctx, BFUSE_ERR_UNSUPPORTED, "thread-level fusions record no per-CTA times");
    const int cnt = f->plan.table.queue ? f->plan.table.total * f->plan.table.cluster : (int)f->launch_grid;
    if (slots[i] < cnt) return fail(ctx, BFUSE_ERR_INVALID, "times array shorter than the fused grid");
    total += (size_t)slots[i];
  }
  cudaSetDevice(ctx->device);
  unsigned long long *d = nullptr;
  CK(cudaMalloc(&d, total * 3 * sizeof(unsigned long long)));
  cudaError_t e = cudaMemsetAsync(d, 0, total * 3 * sizeof(unsigned long long), ctx->own);
  int rc = BFUSE_OK;
  size_t off = 0;
  for (int i = 0; i < n && e == cudaSuccess && !rc; ++i) {
    FusionRec *f = get_fusion(ctx, fusions[i]);
    DispatchTable t = f->plan.table;
    t.cta_times = d + off * 3;
    rc = launch_fused_rec(ctx, *f, ctx->own, &t);
    off += (size_t)slots[i];
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->own);
  if (e == cudaSuccess) e = cudaMemcpy(times, d, total * 3 * sizeof(unsigned long long), cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (rc) return rc;
  if (e != cudaSuccess) return fail_cuda(ctx, e, "fused timeline");
  return BFUSE_OK;
}

int bfuse_debug_gemm_timeline(bfuse_context *ctx, int kernel, long long *marks, int n) {
  KernelRec *k = get_kernel(ctx, kernel);
  if (!k || !marks || n < MARK_COUNT) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle or buffer shorter than 12 marks");
  const bool is_conv = k->desc.op == BFUSE_OP_CONV2D_TF32;
  if (k->desc.op != BFUSE_OP_GEMM_TF32 && k->desc.op != BFUSE_OP_GEMM_BF16 && !is_conv)
    return fail(ctx, BFUSE_ERR_UNSUPPORTED, "only the tcgen05 GEMM / conv bodies record a timeline");
  cudaSetDevice(ctx->device);
  long long *d = nullptr;
  const int held = std::max(n, (int)MARK_COUNT);
  CK(cudaMalloc(&d, sizeof(long long) * held));
  cudaMemset(d, 0, sizeof(long long) * held);
  long long **slot = is_conv ? &reinterpret_cast<ConvUmmaParams *>(k->params)->timeline
                             : &reinterpret_cast<GemmUmmaParams *>(k->params)->timeline;
  int rc = launch_one(ctx, *k, ctx->own);  // warm run
  *slot = d;
  if (!rc) rc = launch_one(ctx, *k, ctx->own);
  *slot = nullptr;
  cudaError_t e = cudaStreamSynchronize(ctx->own);
  if (!rc && e == cudaSuccess) e = cudaMemcpy(marks, d, sizeof(long long) * held, cudaMemcpyDeviceToHost);
  cudaFree(d);
  if (rc) return rc;
  if (e != cudaSuccess) return fail_cuda(ctx, e, "timeline");
  return BFUSE_OK;
}

// After a bounded wait gave up, a persistent launch may have left its ticket counters non-zero (the
// last CTA to drain resets them, and a CTA that bailed out may have skipped tickets): every later
// launch of that fusion would then find the queue "empty" and do nothing.  Start them from zero again.
static void reset_queue_counters(bfuse_context *ctx) {
  for (auto &f : ctx->fusions)
    if (f && f->queue_ctr) cudaMemset(f->queue_ctr, 0, 2 * sizeof(unsigned));
}

int bfuse_debug_conv_staging(const int *shape, int bn, int *out, int n) {
  if (!shape || !out || n < 12) return BFUSE_ERR_INVALID;
  const int *s = shape;
  const int oh = conv_out(s[2], s[5], s[7], s[8]), ow = conv_out(s[3], s[6], s[7], s[8]);
  ConvStaging st;
  std::memset(&st, 0, sizeof(st));
  const bool ok = oh > 0 && ow > 0 && conv_staging(s[1], s[2], s[3], s[5], s[6], s[7], s[8], oh, ow, bn, &st);
  const int v[13] = {ok ? st.slots : 0, st.cc, st.rows, st.pitch, st.ex, st.ey, st.step_x, st.step_y, st.x_start, st.x_off, st.slot_bytes, st.slot_pitch,
                     st.tile_px};
  std::memcpy(out, v, sizeof(int) * (n >= 13 ? 13 : 12));
  return BFUSE_OK;
}

int bfuse_read_status(bfuse_context *ctx, int *status) {
  if (!ctx || !status) return BFUSE_ERR_INVALID;
  cudaSetDevice(ctx->device);
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (*status) {
    CK(cudaMemset(ctx->d_status, 0, sizeof(int)));
    reset_queue_counters(ctx);
  }
  return BFUSE_OK;
}

int bfuse_set_dependent_launch(bfuse_context *ctx, int enabled) {
  if (!ctx) return BFUSE_ERR_INVALID;
  ctx->no_pdl = !enabled;
  return BFUSE_OK;
}

// ---- host-buffer entry points (H2D, launch, sync, D2H) --------------------------------------------

// `other` / `other_host`: the pair's first kernel, already copied in by this call -- an input of this kernel that
// is the same device buffer fed from the same host buffer (two operators sharing their activations) is not
// copied a second time.
// One host -> device copy already issued in the current call: same destination, source and size
struct CopyDone {
  const void *dev, *host;
  size_t bytes;
};
static int copy_in(bfuse_context *ctx, KernelRec &k, void *const *host, cudaStream_t s, const KernelRec *other = nullptr,
                   void *const *other_host = nullptr, std::vector<CopyDone> *seen = nullptr) {
  // small buffers (bias, per-column tables) first: each copy pays a fixed few microseconds, which
  // then overlap the previous pair's large transfer instead of trailing this pair's
  for (int pass = 0; pass < 2; ++pass)
    for (int i = 0; i < k.nargs; ++i)
      if (!k.arg[i].is_output && k.desc.args[i] && (k.arg[i].bytes <= 65536) == (pass == 0)) {
        if (!host[i]) return fail(ctx, BFUSE_ERR_INVALID, k.name + ": missing host input buffer");
        bool done = false;
        for (int j = 0; other && j < other->nargs && !done; ++j)
          done = !other->arg[j].is_output && other->desc.args[j] == k.desc.args[i] && other_host[j] == host[i] &&
                 other->arg[j].bytes == k.arg[i].bytes;
        // (a batch call: the weights that every sub-shard's pair shares go in once, not once per pair -- each
        // copy costs the copy engine a fixed ten-odd microseconds that nothing overlaps)
        for (size_t j = 0; seen && j < seen->size() && !done; ++j)
          done = (*seen)[j].dev == k.desc.args[i] && (*seen)[j].host == host[i] && (*seen)[j].bytes == k.arg[i].bytes;
        if (done) continue;
        if (seen) seen->push_back({k.desc.args[i], host[i], k.arg[i].bytes});
        CK(cudaMemcpyAsync(k.desc.args[i], host[i], k.arg[i].bytes, cudaMemcpyHostToDevice, s));
      }
  return BFUSE_OK;
}
static int copy_out(bfuse_context *ctx, KernelRec &k, void *const *host, cudaStream_t s) {
  for (int i = 0; i < k.nargs; ++i)
    if (k.arg[i].is_output) {
      if (!host[i]) return fail(ctx, BFUSE_ERR_INVALID, k.name + ": missing host output buffer");
      CK(cudaMemcpyAsync(host[i], k.desc.args[i], k.arg[i].bytes, cudaMemcpyDeviceToHost, s));
    }
  return BFUSE_OK;
}
static int finish(bfuse_context *ctx, cudaStream_t s) {
  // the status word rides behind the output copies on the same stream: one synchronisation in all
  CK(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  CK(cudaStreamSynchronize(s));
  const int st = *ctx->h_status;
  if (st) {
    cudaMemset(ctx->d_status, 0, sizeof(int));
    reset_queue_counters(ctx);
    char buf[64];
    snprintf(buf, sizeof(buf), "device status 0x%x: a bounded wait gave up", st);
    return fail(ctx, BFUSE_ERR_TIMEOUT, buf);
  }
  return BFUSE_OK;
}

int bfuse_run_kernel(bfuse_context *ctx, int kernel, void *const *host_args) {
  KernelRec *k = get_kernel(ctx, kernel);
  if (!k || !host_args) return fail(ctx, BFUSE_ERR_INVALID, "bad kernel handle");
  cudaSetDevice(ctx->device);
  int rc = copy_in(ctx, *k, host_args, ctx->own);
  if (!rc) rc = launch_one(ctx, *k, ctx->own);
  if (!rc) rc = copy_out(ctx, *k, host_args, ctx->own);
  return rc ? rc : finish(ctx, ctx->own);
}

static int run_pair(bfuse_context *ctx, int fusion, void *const *h1, void *const *h2, int mode) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f || !h1 || !h2) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle");
  cudaSetDevice(ctx->device);
  KernelRec &a = *ctx->kernels[f->k1], &b = *ctx->kernels[f->k2];
  int rc = copy_in(ctx, a, h1, ctx->own);
  if (!rc) rc = copy_in(ctx, b, h2, ctx->own, &a, h1);
  if (!rc) rc = launch_mode(ctx, *f, mode, ctx->own);
  if (!rc) rc = copy_out(ctx, a, h1, ctx->own);
  if (!rc) rc = copy_out(ctx, b, h2, ctx->own);
  return rc ? rc : finish(ctx, ctx->own);
}
int bfuse_run_fuse_batch(bfuse_context *ctx, const int *fusions, int n, void *const *const *h1, void *const *const *h2) {
  if (!ctx || !fusions || !h1 || !h2 || n <= 0) return fail(ctx, BFUSE_ERR_INVALID, "null argument");
  for (int i = 0; i < n; ++i) {
    if (!get_fusion(ctx, fusions[i]) || !h1[i] || !h2[i]) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle in batch");
    for (int j = 0; j < i; ++j)
      if (fusions[j] == fusions[i]) return fail(ctx, BFUSE_ERR_INVALID, "a fusion may appear once per batch: its device buffers would race");
  }
  cudaSetDevice(ctx->device);
  // s1 carries the copies in, the context's own stream the launches, s2 the copies out
  // (two events per pair, kept in the context and reused by later calls)
  std::vector<cudaEvent_t> &ev = ctx->batch_events;
  int rc = BFUSE_OK;
  while (ev.size() < 2 * (size_t)n && !rc) {
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) rc = fail(ctx, BFUSE_ERR_CUDA, "cudaEventCreate");
    else ev.push_back(e);
  }
  std::vector<CopyDone> seen;   // inputs already on their way in this call
  for (int i = 0; i < n && !rc; ++i) {
    FusionRec &f = *get_fusion(ctx, fusions[i]);
    KernelRec &a = *ctx->kernels[f.k1], &b = *ctx->kernels[f.k2];
    rc = copy_in(ctx, a, h1[i], ctx->s1, nullptr, nullptr, &seen);
    if (!rc) rc = copy_in(ctx, b, h2[i], ctx->s1, &a, h1[i], &seen);
    if (rc) break;
    cudaEventRecord(ev[2 * i], ctx->s1);
    cudaStreamWaitEvent(ctx->own, ev[2 * i], 0);
    rc = launch_fused_rec(ctx, f, ctx->own);
    if (rc) break;
    cudaEventRecord(ev[2 * i + 1], ctx->own);
    cudaStreamWaitEvent(ctx->s2, ev[2 * i + 1], 0);
    rc = copy_out(ctx, a, h1[i], ctx->s2);
    if (!rc) rc = copy_out(ctx, b, h2[i], ctx->s2);
  }
  cudaStreamSynchronize(ctx->s1);
  cudaStreamSynchronize(ctx->own);
  const int rc2 = finish(ctx, ctx->s2);   // status word behind the last copies out, then one synchronisation
  return rc ? rc : rc2;
}
int bfuse_run_parallel(bfuse_context *ctx, int fusion, void *const *h1, void *const *h2) { return run_pair(ctx, fusion, h1, h2, 2); }
int bfuse_run_fuse(bfuse_context *ctx, int fusion, void *const *h1, void *const *h2) { return run_pair(ctx, fusion, h1, h2, 4); }

int bfuse_time(bfuse_context *ctx, int fusion, int mode, int warmup, int iters, float *mean_us, float *min_us) {
  FusionRec *f = get_fusion(ctx, fusion);
  if (!f || iters <= 0 || warmup < 0) return fail(ctx, BFUSE_ERR_INVALID, "bad fusion handle or iteration count");
  cudaSetDevice(ctx->device);
  cudaStream_t s = ctx->own;
  // The launches are captured into a graph of `iters` nodes so that host launch cost (a few
  // microseconds per call, more than many of these kernels take) stays out of the measurement.
  for (int i = 0; i < std::max(warmup, 1); ++i) {
    const int rc = launch_mode(ctx, *f, mode, s);
    if (rc) return rc;
  }
  CK(cudaStreamSynchronize(s));
  cudaGraph_t g = nullptr;
  CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
  int rc = BFUSE_OK;
  for (int i = 0; i < iters && !rc; ++i) rc = launch_mode(ctx, *f, mode, s);
  cudaError_t e = cudaStreamEndCapture(s, &g);
  if (rc || e != cudaSuccess) {
    if (g) cudaGraphDestroy(g);
    return rc ? rc : fail_cuda(ctx, e, "cudaStreamEndCapture");
  }
  cudaGraphExec_t ex = nullptr;
  e = cudaGraphInstantiate(&ex, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "cudaGraphInstantiate");
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0);
  cudaEventCreate(&e1);
  // replay until ~30 ms have passed so that the clocks have left their idle state, then time
  // batches of replays; mean = overall, min = best batch
  float ms = 0.f, spent = 0.f;
  int per_batch = 1;
  while (spent < 30.f && e == cudaSuccess) {
    cudaEventRecord(e0, s);
    for (int i = 0; i < per_batch; ++i) cudaGraphLaunch(ex, s);
    cudaEventRecord(e1, s);
    e = cudaStreamSynchronize(s);
    cudaEventElapsedTime(&ms, e0, e1);
    spent += ms;
    if (ms < 2.f) per_batch *= 2;
  }
  float total = 0.f, best = 1e30f;
  const int batches = 8;
  for (int b = 0; b < batches && e == cudaSuccess; ++b) {
    cudaEventRecord(e0, s);
    for (int i = 0; i < per_batch; ++i) cudaGraphLaunch(ex, s);
    cudaEventRecord(e1, s);
    e = cudaStreamSynchronize(s);
    cudaEventElapsedTime(&ms, e0, e1);
    total += ms;
    best = std::min(best, ms);
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaGraphExecDestroy(ex);
  if (e != cudaSuccess) return fail_cuda(ctx, e, "timing loop");
  if (mean_us) *mean_us = total * 1000.f / ((float)batches * per_batch * iters);
  if (min_us) *min_us = best * 1000.f / ((float)per_batch * iters);
  return BFUSE_OK;
}

long bfuse_check_matrix(const float *value, const float *answer, size_t n, float eps) {
  long wrong = 0;
  for (size_t i = 0; i < n; ++i) {
    const float o = value[i], ans = answer[i];
    if (!(std::fabs(o - ans) <= eps) && (ans == 0.f || !(std::fabs((o - ans) / ans) <= eps))) ++wrong;
  }
  return wrong;
}

// ---- scheduler without a device (the fuser itself runs on the CPU) ---------------------------------

struct bfuse_plan {
  FusedPlan plan;
};

int bfuse_plan_create_clustered(const bfuse_dim3 grid[2], const bfuse_dim3 block[2], int pattern, int param_m,
                                int param_n, int cluster, bfuse_plan **out);

int bfuse_plan_create(const bfuse_dim3 grid[2], const bfuse_dim3 block[2], int pattern, int param_m, int param_n,
                      bfuse_plan **out) {
  return bfuse_plan_create_clustered(grid, block, pattern, param_m, param_n, 1, out);
}

int bfuse_plan_create_clustered(const bfuse_dim3 grid[2], const bfuse_dim3 block[2], int pattern, int param_m,
                                int param_n, int cluster, bfuse_plan **out) {
  if (!grid || !block || !out) return BFUSE_ERR_INVALID;
  const KernelDims kd[2] = {{grid[0].X, grid[0].Y, grid[0].Z, block[0].X, block[0].Y, block[0].Z},
                            {grid[1].X, grid[1].Y, grid[1].Z, block[1].X, block[1].Y, block[1].Z}};
  std::unique_ptr<bfuse_plan> p(new bfuse_plan());
  std::string err;
  if (!plan_pair(kd, pattern, param_m, param_n, param_m, &p->plan, &err, cluster)) return BFUSE_ERR_INVALID;
  *out = p.release();
  return BFUSE_OK;
}
void bfuse_plan_destroy(bfuse_plan *p) { delete p; }
int bfuse_plan_fused_dims(const bfuse_plan *p, bfuse_dim3 *grid, bfuse_dim3 *block) {
  if (!p || !grid || !block) return BFUSE_ERR_INVALID;
  *grid = {p->plan.fused_grid, 1, 1};
  *block = {p->plan.fused_block, 1, 1};
  return BFUSE_OK;
}
int bfuse_plan_map_block(const bfuse_plan *p, int b, int *kernel, int *vblock) {
  if (!p || !kernel || !vblock || b < 0 || b >= p->plan.fused_grid) return BFUSE_ERR_INVALID;
  int k, vb;
  if (!decode_cta(p->plan.table, b, k, vb)) return BFUSE_ERR_INVALID;
  *kernel = k, *vblock = vb;
  return BFUSE_OK;
}
int bfuse_plan_map_all(const bfuse_plan *p, int *kernel_of, int *vblock_of, int n) {
  if (!p || !kernel_of || !vblock_of || n < p->plan.fused_grid) return BFUSE_ERR_INVALID;
  if (p->plan.table.kind == DISPATCH_THREADS) return BFUSE_ERR_UNSUPPORTED;
  for (int b = 0; b < p->plan.fused_grid; ++b)
    if (!decode_cta(p->plan.table, b, kernel_of[b], vblock_of[b])) {
      if (p->plan.table.cluster <= 1) return BFUSE_ERR_INVALID;
      kernel_of[b] = vblock_of[b] = -1;  // padding CTA of a partly filled cluster
    }
  return BFUSE_OK;
}
int bfuse_plan_map_thread(const bfuse_plan *p, int kernel, int b, int t, int *vblock, int *vthread, int *active) {
  if (!p || kernel < 0 || kernel > 1 || !active) return BFUSE_ERR_INVALID;
  const DispatchTable &tb = p->plan.table;
  if (tb.kind != DISPATCH_THREADS) return BFUSE_ERR_UNSUPPORTED;
  const int vt = t - tb.thr_lo[kernel];
  *active = vt >= 0 && vt < tb.n_thr[kernel] && b >= 0 && b < tb.n_cta[kernel];
  if (vblock) *vblock = b;
  if (vthread) *vthread = vt;
  return BFUSE_OK;
}
int bfuse_plan_barrier(const bfuse_plan *p, int kernel, int *bar_id, int *bar_count) {
  if (!p || kernel < 0 || kernel > 1 || !bar_id || !bar_count) return BFUSE_ERR_INVALID;
  *bar_id = kernel + 1;  // bar.sync <k+1>, <round32(B_k)> (Matchers.cc:301-311)
  *bar_count = p->plan.table.bar_count[kernel];
  return BFUSE_OK;
}

}  // extern "C"
