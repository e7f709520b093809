// Host scheduler.  Each pattern of the reference's horizontal-fuser/src/Algorithms.cc is reduced,
// for a pair of kernels, to closed-form constants (see dispatch.h) rather than to generated C text.
#include "scheduler.h"

#include <algorithm>
#include <cstring>

namespace bfuse {

namespace {

// Rotating region of `ratio[0] + ratio[1]` CTAs repeated `rounds` times, then what is left of
// each operator as one contiguous tail (Algorithms.cc:570-587 and :661-685).
void fill_rotate(DispatchTable &t, const int units[2], const int ratio[2], int rounds) {
  t.kind = DISPATCH_ROTATE;
  t.rot = ratio[0] + ratio[1];
  t.ratio[0] = ratio[0];
  t.ratio[1] = ratio[1];
  t.rot_end = t.rot * rounds;
  int at = t.rot_end;
  for (int k = 0; k < 2; ++k) {
    const int done = ratio[k] * rounds;
    t.tail_lo[k] = at;
    t.tail_hi[k] = at + (units[k] - done);
    t.tail_base[k] = done;
    at = t.tail_hi[k];
  }
}

}  // namespace

bool plan_pair(const KernelDims k[2], int pattern, int param_m, int param_n, int total_sm, FusedPlan *out,
               std::string *err, int cluster) {
  auto fail = [&](const char *m) {
    if (err) *err = m;
    return false;
  };
  std::memset(out, 0, sizeof(*out));
  DispatchTable &t = out->table;
  for (int i = 0; i < 2; ++i) {
    if (k[i].gx <= 0 || k[i].gy <= 0 || k[i].gz <= 0 || k[i].bx <= 0 || k[i].by <= 0 || k[i].bz <= 0)
      return fail("grid and block dims must be positive");
    if ((long long)k[i].gx * k[i].gy * k[i].gz > 0x3fffffffLL) return fail("grid too large");
    if (k[i].block() > 1024) return fail("block larger than 1024 threads");
    t.n_cta[i] = k[i].grid();
    t.n_thr[i] = k[i].block();
    t.grid_x[i] = k[i].gx;
    t.grid_y[i] = k[i].gy;
    t.blk_x[i] = k[i].bx;
    t.blk_y[i] = k[i].by;
    t.bar_count[i] = round_up32(k[i].block());
  }
  out->pattern = pattern;
  if (cluster < 1 || cluster > 8) return fail("cluster width must be 1..8");
  t.cluster = cluster;
  // the patterns schedule units of `cluster` CTAs; with cluster == 1 a unit is a CTA
  const int units[2] = {(t.n_cta[0] + cluster - 1) / cluster, (t.n_cta[1] + cluster - 1) / cluster};
  const int g0 = units[0], g1 = units[1], gmin = std::min(g0, g1);
  // block-level fusion: grid = sum, block = max (Algorithms.cc:719-736)
  out->fused_grid = (g0 + g1) * cluster;
  out->fused_block = std::max(t.n_thr[0], t.n_thr[1]);
  t.total = g0 + g1;

  switch (pattern) {
    case PATTERN_WORK_QUEUE:
      if (cluster != 1) return fail("the work queue cannot host operators launched as clusters");
      t.queue = 1;
      // fallthrough: tickets follow the zig-zag order
    case PATTERN_ZIGZAG: {
      // ratio_k = min(G_k / min G, M) * N; rounds = min_k G_k / ratio_k (Algorithms.cc:553-566)
      if (param_m < 1 || param_n < 1) return fail("zig-zag needs M >= 1 and N >= 1");
      int ratio[2], rounds = -1;
      for (int i = 0; i < 2; ++i) {
        const int q = units[i] / gmin;
        ratio[i] = q < param_m ? q * param_n : param_m * param_n;
        const int r = units[i] / ratio[i];
        rounds = rounds < 0 ? r : std::min(rounds, r);
      }
      fill_rotate(t, units, ratio, rounds);
      break;
    }
    case PATTERN_PROPORTIONAL: {
      // ratio_k = G_k / max(min G / MinOption, 1) (Algorithms.cc:323-355)
      if (param_m < 1) return fail("proportional zig-zag needs MinOption >= 1");
      const int unit = std::max(gmin / param_m, 1);
      int ratio[2], rounds = -1;
      for (int i = 0; i < 2; ++i) {
        ratio[i] = units[i] / unit;
        const int r = units[i] / ratio[i];
        rounds = rounds < 0 ? r : std::min(rounds, r);
      }
      fill_rotate(t, units, ratio, rounds);
      break;
    }
    case PATTERN_RANGE_SPLIT: {
      const int ratio[2] = {1, 1};
      fill_rotate(t, units, ratio, 0);  // no rotating region: operator 0 then operator 1
      break;
    }
    case PATTERN_SM_STRIPED: {
      // stripes of total_sm CTAs, smaller grid first; then the larger alone; then the leftovers
      // of each operator in registration order (Algorithms.cc:122-163)
      if (total_sm < 1) return fail("SM-striped needs a positive SM count");
      t.kind = DISPATCH_STRIPE;
      t.sm = total_sm;
      t.small = g1 < g0 ? 1 : 0;  // stable: equal grids keep registration order
      const int fs = units[t.small] / total_sm * total_sm;
      const int fl = units[1 - t.small] / total_sm * total_sm;
      t.ph0_end = 2 * fs;
      t.ph1_end = fs + fl;
      t.ph1_base = fs;
      int at = t.ph1_end;
      for (int i = 0; i < 2; ++i) {
        const int rem = units[i] % total_sm;
        t.tail_lo[i] = at;
        t.tail_hi[i] = at + rem;
        t.tail_base[i] = units[i] - rem;
        at = t.tail_hi[i];
      }
      break;
    }
    case PATTERN_THREAD_SPLIT: {
      // kernel k owns threads [acc_k, acc_k + B_k), acc advancing by round32(B_k); every CTA below
      // G_k hosts kernel k; grid = max G, block = sum of rounded blocks (Algorithms.cc:23-49,98-113)
      t.kind = DISPATCH_THREADS;
      t.thr_lo[0] = 0;
      t.thr_lo[1] = round_up32(t.n_thr[0]);
      if (cluster != 1) return fail("thread split cannot host operators launched as clusters");
      out->fused_grid = std::max(g0, g1);
      out->fused_block = round_up32(t.n_thr[0]) + round_up32(t.n_thr[1]);
      if (out->fused_block > 1024) return fail("thread split: the two blocks do not fit one CTA");
      t.total = out->fused_grid;
      break;
    }
    default:
      return fail("unknown pattern");
  }
  return true;
}

bool plan_group(const KernelDims *k, int n, int pattern, int param_m, int param_n, GroupPlan *out, std::string *err,
                int cluster) {
  auto fail = [&](const char *m) {
    if (err) *err = m;
    return false;
  };
  std::memset(out, 0, sizeof(*out));
  GroupTable &t = out->table;
  if (n < 2 || n > kGroupMax) return fail("a group holds 2 to 4 operators");
  if (cluster < 1 || cluster > 8) return fail("cluster width must be 1..8");
  t.n = n;
  t.cluster = cluster;
  out->pattern = pattern;
  int units[kGroupMax], umin = 0;
  long long sum = 0;
  for (int i = 0; i < n; ++i) {
    if (k[i].gx <= 0 || k[i].gy <= 0 || k[i].gz <= 0 || k[i].bx <= 0 || k[i].by <= 0 || k[i].bz <= 0)
      return fail("grid and block dims must be positive");
    if ((long long)k[i].gx * k[i].gy * k[i].gz > 0x0fffffffLL) return fail("grid too large");
    if (k[i].block() > 1024) return fail("block larger than 1024 threads");
    t.n_cta[i] = k[i].grid();
    t.n_thr[i] = k[i].block();
    t.grid_x[i] = k[i].gx, t.grid_y[i] = k[i].gy;
    t.blk_x[i] = k[i].bx, t.blk_y[i] = k[i].by;
    t.bar_count[i] = round_up32(k[i].block());
    units[i] = (t.n_cta[i] + cluster - 1) / cluster;
    umin = i == 0 ? units[i] : std::min(umin, units[i]);
    sum += units[i];
    out->fused_block = std::max(out->fused_block, t.n_thr[i]);
  }
  t.total = (int)sum;
  out->fused_grid = (int)sum * cluster;
  int ratio[kGroupMax], rounds = -1;
  switch (pattern) {
    case PATTERN_ZIGZAG:
      if (param_m < 1 || param_n < 1) return fail("zig-zag needs M >= 1 and N >= 1");
      for (int i = 0; i < n; ++i) {
        const int q = units[i] / umin;
        ratio[i] = q < param_m ? q * param_n : param_m * param_n;
      }
      break;
    case PATTERN_PROPORTIONAL: {
      if (param_m < 1) return fail("proportional zig-zag needs MinOption >= 1");
      const int unit = std::max(umin / param_m, 1);
      for (int i = 0; i < n; ++i) ratio[i] = units[i] / unit;
      break;
    }
    case PATTERN_RANGE_SPLIT:
      for (int i = 0; i < n; ++i) ratio[i] = 1;
      rounds = 0;
      break;
    default:
      return fail("a group takes the zig-zag, proportional and range-split patterns");
  }
  if (rounds < 0)
    for (int i = 0; i < n; ++i) rounds = rounds < 0 ? units[i] / ratio[i] : std::min(rounds, units[i] / ratio[i]);
  t.ratio_lo[0] = 0;
  for (int i = 0; i < n; ++i) t.ratio_lo[i + 1] = t.ratio_lo[i] + ratio[i];
  t.rot = t.ratio_lo[n];
  t.rot_end = t.rot * rounds;
  int at = t.rot_end;
  for (int i = 0; i < n; ++i) {
    const int done = ratio[i] * rounds;
    t.tail_lo[i] = at;
    t.tail_hi[i] = at + (units[i] - done);
    t.tail_base[i] = done;
    at = t.tail_hi[i];
  }
  return true;
}

}  // namespace bfuse
