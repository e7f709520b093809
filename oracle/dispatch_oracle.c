/*
 * CPU oracle, half 1: the block-dispatch math of the reference's fuser.
 * TEST INFRASTRUCTURE ONLY -- never linked into the shipped library.
 *
 * Each orc_plan_* function follows one pattern function of
 * horizontal-fuser/src/Algorithms.cc and records, instead of C text, the
 * constants that function prints into the fused kernel's if / else-if chain.
 * Parity is pinned: tests/golden holds those constants as parsed from the
 * reference's own generated kernels, and the fused dims from its YAML outputs.
 */
#include "bfuse_oracle.h"

#include <string.h>

static int grid_size(const orc_kernel_dims *k) { return k->gx * k->gy * k->gz; }
static int block_size(const orc_kernel_dims *k) { return k->bx * k->by * k->bz; }
static int round32(int x) { return x % 32 == 0 ? x : (x / 32 + 1) * 32; }

static int plan_begin(const orc_kernel_dims *k, int n, orc_plan *out) {
  if (n < 1 || n > ORC_MAX_KERNELS) return -1;
  memset(out, 0, sizeof(*out));
  out->n_kernels = n;
  for (int i = 0; i < n; ++i) {
    if (grid_size(&k[i]) <= 0 || block_size(&k[i]) <= 0) return -1;
    out->k[i] = k[i];
  }
  return 0;
}

/* Fused dims of every block-level pattern: grid = sum of grids, block = max of blocks
 * (Algorithms.cc:297-314, :506-523, :719-736). */
static void block_level_dims(orc_plan *p) {
  int acc = 0, mx = 0;
  for (int i = 0; i < p->n_kernels; ++i) {
    acc += grid_size(&p->k[i]);
    if (block_size(&p->k[i]) > mx) mx = block_size(&p->k[i]);
  }
  p->fused_grid = acc;
  p->fused_block = mx;
}

/* Shared tail of the two "WithoutSM" patterns once the per-kernel ratios are known:
 * rotate region (Algorithms.cc:570-587,628-651) then per-kernel remainders (:661-685). */
static int rotate_then_remainders(orc_plan *p, const int *ratio, int min_quot) {
  int n = p->n_kernels;
  int end_bound = 0, rotate = 0;
  int remain[ORC_MAX_KERNELS], lo[ORC_MAX_KERNELS];
  for (int i = 0; i < n; ++i) {
    remain[i] = grid_size(&p->k[i]) - ratio[i] * min_quot;
    end_bound += ratio[i] * min_quot;
    lo[i] = rotate;
    rotate += ratio[i];
  }
  for (int i = 0; i < n; ++i) {
    orc_branch *b = &p->br[p->n_branches++];
    b->kind = ORC_BR_ROTATE;
    b->kernel = i;
    b->b_lo = 0;
    b->b_hi = end_bound;
    b->rot = rotate;
    b->r_lo = lo[i];
    b->r_hi = lo[i] + ratio[i];
    b->ratio = ratio[i];
  }
  for (int i = 0; i < n; ++i) {
    orc_branch *b = &p->br[p->n_branches++];
    b->kind = ORC_BR_RANGE;
    b->kernel = i;
    b->b_lo = end_bound;
    b->b_hi = end_bound + remain[i];
    b->base = ratio[i] * min_quot;
    end_bound += remain[i];
  }
  block_level_dims(p);
  return 0;
}

int orc_plan_zigzag(const orc_kernel_dims *k, int n, int M, int N, orc_plan *out) {
  if (plan_begin(k, n, out) || M < 1 || N < 1) return -1;
  int min_g = -1;
  for (int i = 0; i < n; ++i) { /* Algorithms.cc:541-551 */
    int g = grid_size(&k[i]);
    min_g = (min_g == -1 || g < min_g) ? g : min_g;
  }
  int ratio[ORC_MAX_KERNELS], min_quot = -1;
  for (int i = 0; i < n; ++i) { /* Algorithms.cc:553-566 */
    int r = grid_size(&k[i]) / min_g;
    r = r < M ? r * N : M * N;
    int quot = grid_size(&k[i]) / r;
    ratio[i] = r;
    min_quot = (min_quot == -1 || quot < min_quot) ? quot : min_quot;
  }
  return rotate_then_remainders(out, ratio, min_quot);
}

int orc_plan_proportional(const orc_kernel_dims *k, int n, int min_option, orc_plan *out) {
  if (plan_begin(k, n, out) || min_option < 1) return -1;
  int min_ratio = -1;
  for (int i = 0; i < n; ++i) { /* Algorithms.cc:326-338 */
    int g = grid_size(&k[i]);
    min_ratio = (min_ratio == -1 || g < min_ratio) ? g : min_ratio;
  }
  min_ratio = min_ratio / min_option; /* :340-341 */
  if (min_ratio <= 0) min_ratio = 1;
  int ratio[ORC_MAX_KERNELS], min_quot = -1;
  for (int i = 0; i < n; ++i) { /* :343-355 */
    int r = grid_size(&k[i]) / min_ratio;
    int quot = grid_size(&k[i]) / r;
    ratio[i] = r;
    min_quot = (min_quot == -1 || quot < min_quot) ? quot : min_quot;
  }
  return rotate_then_remainders(out, ratio, min_quot);
}

int orc_plan_sm_striped(const orc_kernel_dims *k, int n, int total_sm, orc_plan *out) {
  if (plan_begin(k, n, out) || total_sm < 1) return -1;
  /* kernels sorted by grid size, ascending, stable (Algorithms.cc:122-131) */
  int order[ORC_MAX_KERNELS];
  for (int i = 0; i < n; ++i) order[i] = i;
  for (int i = 1; i < n; ++i) {
    int v = order[i], j = i - 1;
    while (j >= 0 && grid_size(&k[order[j]]) > grid_size(&k[v])) {
      order[j + 1] = order[j];
      --j;
    }
    order[j + 1] = v;
  }
  int b_first[ORC_MAX_KERNELS], b_second[ORC_MAX_KERNELS], my_blocks[ORC_MAX_KERNELS];
  int remains[ORC_MAX_KERNELS];
  int end_bounds = 0, my_bounds = 0, acc_bounds = 0;
  for (int i = 0; i < n; ++i) { /* :140-154 */
    const orc_kernel_dims *ki = &k[order[i]];
    int cur_total = n - i;
    int full = grid_size(ki) / total_sm * total_sm;
    b_first[i] = end_bounds;
    b_second[i] = acc_bounds + full * cur_total;
    my_blocks[i] = my_bounds;
    remains[order[i]] = grid_size(ki) % total_sm;
    end_bounds = b_second[i];
    my_bounds = full;
    acc_bounds += full;
  }
  for (int i = 0; i < n; ++i) {   /* :203-232: phase i, kernels order[i..] take turns */
    for (int j = i; j < n; ++j) {
      orc_branch *b = &out->br[out->n_branches++];
      b->kind = ORC_BR_STRIPE;
      b->kernel = order[j];
      b->b_lo = b_first[i];
      b->b_hi = b_second[i];
      b->sm = total_sm;
      b->stripe_n = n - i;
      b->stripe_idx = j - i;
      b->base = my_blocks[i];
    }
  }
  for (int i = 0; i < n; ++i) { /* :156-163, :242-263: leftovers in registration order */
    orc_branch *b = &out->br[out->n_branches++];
    b->kind = ORC_BR_RANGE;
    b->kernel = i;
    b->b_lo = end_bounds;
    b->b_hi = end_bounds + remains[i];
    b->base = grid_size(&k[i]) - grid_size(&k[i]) % total_sm;
    end_bounds = b->b_hi;
  }
  block_level_dims(out);
  return 0;
}

int orc_plan_thread_split(const orc_kernel_dims *k, int n, orc_plan *out) {
  if (plan_begin(k, n, out)) return -1;
  out->thread_split = 1;
  int acc = 0, max_blocks = 0;
  for (int i = 0; i < n; ++i) { /* Algorithms.cc:23-35, :60-74 */
    orc_branch *b = &out->br[out->n_branches++];
    b->kind = ORC_BR_THREADS;
    b->kernel = i;
    b->t_lo = acc;
    b->t_hi = acc + block_size(&k[i]);
    b->b_lo = 0;
    b->b_hi = grid_size(&k[i]);
    acc += round32(block_size(&k[i]));
    if (grid_size(&k[i]) > max_blocks) max_blocks = grid_size(&k[i]);
  }
  out->fused_grid = max_blocks; /* :98-113 */
  out->fused_block = acc;
  return 0;
}

int orc_plan_range_split(const orc_kernel_dims *k, int n, orc_plan *out) {
  if (plan_begin(k, n, out)) return -1;
  int start = 0;
  for (int i = 0; i < n; ++i) {
    orc_branch *b = &out->br[out->n_branches++];
    b->kind = ORC_BR_RANGE;
    b->kernel = i;
    b->b_lo = start;
    b->b_hi = start + grid_size(&k[i]);
    b->base = 0;
    start = b->b_hi;
  }
  block_level_dims(out);
  return 0;
}

int orc_map_block(const orc_plan *p, int b, int *kernel, int *vblock) {
  if (p->thread_split) return 0;
  for (int i = 0; i < p->n_branches; ++i) {
    const orc_branch *br = &p->br[i];
    switch (br->kind) {
      case ORC_BR_ROTATE: /* Algorithms.cc:590-602, :641-642 */
        if (b < br->b_hi && b % br->rot >= br->r_lo && b % br->rot < br->r_hi) {
          *kernel = br->kernel;
          *vblock = b / br->rot * br->ratio + (b % br->rot - br->r_lo);
          return 1;
        }
        break;
      case ORC_BR_RANGE: /* :653-659, :674 */
        if (b >= br->b_lo && b < br->b_hi) {
          *kernel = br->kernel;
          *vblock = b - br->b_lo + br->base;
          return 1;
        }
        break;
      case ORC_BR_STRIPE: /* :166-177, :220-222 */
        if (b >= br->b_lo && b < br->b_hi &&
            (b - br->b_lo) % (br->sm * br->stripe_n) / br->sm == br->stripe_idx) {
          *kernel = br->kernel;
          *vblock = br->base + (b - br->b_lo) % br->sm +
                    (b - br->b_lo) / (br->stripe_n * br->sm) * br->sm;
          return 1;
        }
        break;
      default:
        break;
    }
  }
  return 0;
}

int orc_map_thread(const orc_plan *p, int kernel, int b, int t, int *vblock, int *vthread) {
  if (!p->thread_split || kernel < 0 || kernel >= p->n_kernels) return 0;
  const orc_branch *br = &p->br[kernel];
  if (t >= br->t_lo && t < br->t_hi && b >= 0 && b < br->b_hi) { /* Algorithms.cc:38-49 */
    *vblock = b;
    *vthread = t - br->t_lo; /* :86 */
    return 1;
  }
  return 0;
}

int orc_thread_active(const orc_plan *p, int kernel, int t) {
  return t < block_size(&p->k[kernel]);
}

void orc_decompose(const orc_kernel_dims *k, int vblock, int vthread, int bidx[3], int tidx[3]) {
  bidx[0] = vblock % k->gx;
  bidx[1] = vblock / k->gx % k->gy;
  bidx[2] = vblock / (k->gx * k->gy);
  tidx[0] = vthread % k->bx;
  tidx[1] = vthread / k->bx % k->by;
  tidx[2] = vthread / (k->bx * k->by);
}

void orc_named_barrier(const orc_plan *p, int kernel, int *bar_id, int *bar_count) {
  *bar_id = kernel + 1;
  *bar_count = round32(block_size(&p->k[kernel]));
}

uint64_t orc_plan_digest(const orc_plan *p) {
  /* sum over CTAs b of ((kernel+1) << 40 | vblock) * (2b+1) * 0x9E3779B97F4A7C15 (mod 2^64):
   * the same formula the golden generator applies to the reference's printed conditions. */
  uint64_t h = 0;
  for (int b = 0; b < p->fused_grid; ++b) {
    int k = -1, vb = -1;
    if (p->thread_split) {
      k = 0; /* thread split: digest the set of kernels a CTA hosts */
      for (int i = 0; i < p->n_kernels; ++i)
        if (b < p->br[i].b_hi) k |= 1 << i;
      vb = b;
    } else if (!orc_map_block(p, b, &k, &vb)) {
      return 0;
    }
    uint64_t w = ((uint64_t)(k + 1) << 40) | (uint64_t)(uint32_t)vb;
    h += w * (2ull * (uint64_t)b + 1ull) * 0x9E3779B97F4A7C15ull;
  }
  return h;
}
