// The fused-kernel registry: the list of operator bodies and the table of fused kernels
// instantiated for every ordered pair of them.  This is the compile-time counterpart of the
// reference's generated switch tables (test-utils/test-suite-files/macro_h.py:202-324): a pair
// of operator ids selects a pre-built fused kernel instead of a function pointer into generated
// source.  Row I of the table is compiled in its own translation unit (pairs_row.cu with
// -DBFUSE_ROW=I) so the rows build in parallel.
#pragma once

#include "fused_kernels.cuh"
#include "ops_rowwise.cuh"
#include "ops_simt.cuh"
#include "ops_conv_umma.cuh"
#include "ops_umma.cuh"

namespace bfuse {

constexpr int kNumOps = 9;

template <int I> struct OpAt;
template <> struct OpAt<0> { using type = SoftmaxF32; };
template <> struct OpAt<1> { using type = LayerNormF32; };
template <> struct OpAt<2> { using type = RmsNormBf16; };
template <> struct OpAt<3> { using type = RopeBf16; };
template <> struct OpAt<4> { using type = GemmSimtF32; };
template <> struct OpAt<5> { using type = ConvSimtF32; };
template <> struct OpAt<6> { using type = GemmUmma<0>; };
template <> struct OpAt<7> { using type = GemmUmma<1>; };
template <> struct OpAt<8> { using type = ConvUmmaTf32; };

struct PairEntry {
  PairLaunchFn block, thread;
  AttrFn block_attr, thread_attr;
  PairLaunchFn block_wide;   // the register-richer build of the pair (see pair_wide_blocks), else nullptr
  AttrFn block_wide_attr;
  int wide_min_blocks;       // CTAs per SM the wide build is compiled for
  ClusterCapFn block_clusters;  // clusters of the block-level kernel that can be resident at once
  // groups of these two bodies (built once per unordered pair: for row < column only, else nullptr)
  MixedGroupLaunchFn mixed;
  AttrFn mixed_attr;
  ClusterCapFn mixed_clusters;
};
struct SingleEntry {
  SingleLaunchFn launch;
  AttrFn attr;
  GroupLaunchFn group;       // up to kGroupMax operators of this body in one launch
  AttrFn group_attr;
  ClusterCapFn group_clusters;
  int max_threads;
  size_t params_size;
};

// defined once per row by pairs_row.cu
template <int I> void fill_pair_row(PairEntry *row, SingleEntry *single);

}  // namespace bfuse
