// Host scheduler: turns (two kernels' dims, a pattern, its parameters) into the DispatchTable the
// fused kernel decodes.  Pure integer host code, usable without a GPU.
#pragma once

#include <string>

#include "dispatch.h"

namespace bfuse {

struct KernelDims {
  int gx, gy, gz;
  int bx, by, bz;
  int grid() const { return gx * gy * gz; }
  int block() const { return bx * by * bz; }
};

enum Pattern : int {
  PATTERN_ZIGZAG = 0,
  PATTERN_PROPORTIONAL = 1,
  PATTERN_SM_STRIPED = 2,
  PATTERN_THREAD_SPLIT = 3,
  PATTERN_RANGE_SPLIT = 4,
  PATTERN_WORK_QUEUE = 5,
};

struct FusedPlan {
  DispatchTable table;
  int fused_grid;   // GridDim.X of the fused launch (Y = Z = 1), a multiple of table.cluster
  int fused_block;  // BlockDim.X of the fused launch
  int pattern;
};

inline int round_up32(int x) { return (x + 31) / 32 * 32; }

// Threads per row of the row-wise bodies' default tiling: the smallest power of two (>= 32) that
// keeps at most 4 vectors of `vec_elems` elements per thread, else the largest one within the
// body's per-thread budget of `max_vec` vectors; 0 when cols cannot be tiled.  One definition for the
// registered path and the allocation-free entry point, whose outputs must stay bit-identical.
inline int pick_row_threads(int cols, int vec_elems, int max_vec) {
  for (int tpr = 32; tpr <= 256; tpr *= 2)
    if (cols % (vec_elems * tpr) == 0 && cols / (vec_elems * tpr) <= (max_vec < 4 ? max_vec : 4)) return tpr;
  for (int tpr = 256; tpr >= 1; tpr /= 2)
    if (cols % (vec_elems * tpr) == 0 && cols / (vec_elems * tpr) <= max_vec) return tpr;
  return 0;
}

// Returns false and sets err on invalid input.  For PATTERN_WORK_QUEUE the table describes the
// ticket order (zig-zag param_m : param_n); the caller sizes the persistent grid.
// cluster > 1 schedules units of `cluster` consecutive CTAs (see decode_cta in dispatch.h).
bool plan_pair(const KernelDims k[2], int pattern, int param_m, int param_n, int total_sm, FusedPlan *out,
               std::string *err, int cluster = 1);

struct GroupPlan {
  GroupTable table;
  int fused_grid;   // GridDim.X of the fused launch, a multiple of table.cluster
  int fused_block;  // BlockDim.X of the fused launch
  int pattern;
};

// n operators (2..kGroupMax) in one block-level launch: zig-zag M:N, proportional zig-zag and
// range split in the reference's n-kernel form (Algorithms.cc:323-375, 538-587, 661-685).
bool plan_group(const KernelDims *k, int n, int pattern, int param_m, int param_n, GroupPlan *out, std::string *err,
                int cluster = 1);

}  // namespace bfuse
