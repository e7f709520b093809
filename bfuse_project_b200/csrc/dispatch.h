// Block-dispatch table of a fused pair and its decode, shared by host and device.
//
// The reference prints its schedule as an if / else-if chain into every fused
// kernel (horizontal-fuser/src/Algorithms.cc).  Here the schedule is data: the host
// scheduler (scheduler.cc) reduces a pattern to the closed-form constants below, the
// table travels to the kernel as a __grid_constant__ parameter, and decode_cta() maps
// a CTA index (or a work-queue ticket) to (operator, virtual block).  The host calls
// the same decode_cta() to answer "which operator runs CTA b", so host and device
// cannot disagree.
#pragma once

#if defined(__CUDACC__)
#define BFUSE_HD __host__ __device__ __forceinline__
#else
#define BFUSE_HD inline
#endif

namespace bfuse {

enum DispatchKind : int {
  DISPATCH_ROTATE = 0,   // rotating region + one contiguous tail per operator
  DISPATCH_STRIPE = 1,   // stripes of `sm` consecutive CTAs per operator
  DISPATCH_THREADS = 2,  // both operators inside every CTA, split by thread range
};

struct DispatchTable {
  int kind;
  int queue;          // 1: persistent CTAs draw tickets from queue_ctr instead of using blockIdx.x
  int total;          // dispatch units (block-level kinds) or tickets (queue); units = CTAs when cluster == 1
  int cluster;        // CTAs per dispatch unit = hardware cluster width (1: the reference's CTA-level dispatch)
  int n_cta[2];       // G_k = GridDim.size() of operator k
  int n_thr[2];       // B_k = BlockDim.size() of operator k
  int grid_x[2], grid_y[2];
  int blk_x[2], blk_y[2];
  // DISPATCH_ROTATE: CTAs [0, rot_end) rotate with period `rot`; residues [0, ratio[0]) belong to
  // operator 0, the rest to operator 1.  Then operator k owns [tail_lo[k], tail_hi[k]).
  int rot_end, rot, ratio[2];
  int tail_lo[2], tail_hi[2], tail_base[2];
  // DISPATCH_STRIPE: phase 0 alternates stripes (smaller grid first) below ph0_end; phase 1 is the
  // larger operator alone up to ph1_end; leftovers reuse tail_lo / tail_hi / tail_base.
  int sm, small, ph0_end, ph1_end, ph1_base;
  // DISPATCH_THREADS: operator k owns fused threads [thr_lo[k], thr_lo[k] + B_k).
  int thr_lo[2];
  // all kinds
  int bar_count[2];        // B_k rounded up to a multiple of 32 (named-barrier arrival count)
  int smem_off[2];         // byte offset of operator k's shared-memory window
  unsigned int *queue_ctr; // [0] next ticket, [1] CTAs that have drained (persistent queue only)
  int *status;             // device status word; non-zero = a bounded wait gave up
  unsigned long long *cta_times;  // diagnostic: when non-null, every block-level dispatch slot records 3 globaltimer marks
  int no_pdl;              // host side only: launch without the programmatic-dependent-launch attribute
  int tmem_cols;           // queue launches: tensor-memory columns a persistent CTA allocates ONCE for all its tickets
                           // (the larger need of the two operators, a power of two; 0: neither uses tensor memory)
};

// Dispatch unit (or ticket) b -> operator k and its virtual unit.  Returns false if b is unmapped.
// With cluster == 1 a unit is a CTA and this is the reference's if / else-if chain.
BFUSE_HD bool decode_unit(const DispatchTable &t, int b, int &k, int &vb) {
  if (t.kind == DISPATCH_ROTATE) {
    if (b < t.rot_end) {
      const int r = b % t.rot, q = b / t.rot;
      if (r < t.ratio[0]) {
        k = 0;
        vb = q * t.ratio[0] + r;
      } else {
        k = 1;
        vb = q * t.ratio[1] + (r - t.ratio[0]);
      }
      return true;
    }
  } else if (t.kind == DISPATCH_STRIPE) {
    if (b < t.ph0_end) {
      const int idx = b % (2 * t.sm) / t.sm;
      k = idx == 0 ? t.small : 1 - t.small;
      vb = b % t.sm + b / (2 * t.sm) * t.sm;
      return true;
    }
    if (b < t.ph1_end) {
      k = 1 - t.small;
      vb = t.ph1_base + (b - t.ph0_end);
      return true;
    }
  } else {
    return false;
  }
  if (b >= t.tail_lo[0] && b < t.tail_hi[0]) {
    k = 0;
    vb = b - t.tail_lo[0] + t.tail_base[0];
    return true;
  }
  if (b >= t.tail_lo[1] && b < t.tail_hi[1]) {
    k = 1;
    vb = b - t.tail_lo[1] + t.tail_base[1];
    return true;
  }
  return false;
}

// Hardware CTA b -> operator k and its virtual block.  When operators are launched as thread-block
// clusters (split-K GEMM tiles reduce over distributed shared memory) the patterns above schedule
// whole clusters: unit u = b / cluster goes through decode_unit, and the CTA's virtual block is
// vu * cluster + b % cluster, so the CTAs of one hardware cluster always belong to one operator
// and to consecutive virtual blocks.  Returns false for an unmapped or padding CTA.
BFUSE_HD bool decode_cta(const DispatchTable &t, int b, int &k, int &vb) {
  if (t.cluster <= 1) return decode_unit(t, b, k, vb);
  int vu;
  if (!decode_unit(t, b / t.cluster, k, vu)) return false;
  vb = vu * t.cluster + b % t.cluster;
  return vb < t.n_cta[k];
}

// ---- n operators of one body in one launch ------------------------------------------------------
// The reference writes its patterns for n kernels (Algorithms.cc:323-375, 538-587) although its
// test suite only ever fuses two.  A group is that general form for up to kGroupMax operators that
// share a body (the Q, K and V projections of one layer, the branches of one block): a rotating
// region of sum(ratio) units in which residues [ratio_lo[k], ratio_lo[k + 1]) belong to operator
// k, then what is left of each operator as one contiguous tail, in registration order.
constexpr int kGroupMax = 4;

struct GroupTable {
  int n;              // operators in the group (2..kGroupMax)
  int total;          // dispatch units
  int cluster;        // CTAs per dispatch unit (see DispatchTable::cluster)
  int n_cta[kGroupMax], n_thr[kGroupMax];
  int grid_x[kGroupMax], grid_y[kGroupMax];
  int blk_x[kGroupMax], blk_y[kGroupMax];
  int bar_count[kGroupMax];
  int rot_end, rot, ratio_lo[kGroupMax + 1];
  int tail_lo[kGroupMax], tail_hi[kGroupMax], tail_base[kGroupMax];
  // groups of two operator bodies: which of the two bodies operator i runs (0 / 1) and its index among
  // that body's parameter blocks; all zero / i for a group of one body
  int body[kGroupMax], slot[kGroupMax];
  int *status;
  int no_pdl;         // host side only: launch without the programmatic-dependent-launch attribute
};

BFUSE_HD bool decode_group_unit(const GroupTable &t, int b, int &k, int &vb) {
  if (b < t.rot_end) {
    const int r = b % t.rot, q = b / t.rot;
    for (int i = 0; i < t.n; ++i)
      if (r < t.ratio_lo[i + 1]) {
        k = i;
        vb = q * (t.ratio_lo[i + 1] - t.ratio_lo[i]) + (r - t.ratio_lo[i]);
        return true;
      }
    return false;
  }
  for (int i = 0; i < t.n; ++i)
    if (b >= t.tail_lo[i] && b < t.tail_hi[i]) {
      k = i;
      vb = b - t.tail_lo[i] + t.tail_base[i];
      return true;
    }
  return false;
}

BFUSE_HD bool decode_group_cta(const GroupTable &t, int b, int &k, int &vb) {
  if (t.cluster <= 1) return decode_group_unit(t, b, k, vb);
  int vu;
  if (!decode_group_unit(t, b / t.cluster, k, vu)) return false;
  vb = vu * t.cluster + b % t.cluster;
  return vb < t.n_cta[k];
}

}  // namespace bfuse
