// One row of the fused-kernel registry: operator BFUSE_ROW fused with every operator.
#include "op_list.h"

#ifndef BFUSE_ROW
#error "compile with -DBFUSE_ROW=<operator id>"
#endif

namespace bfuse {

template <class A, class B, bool HAS>
struct WideFiller {
  static void fill(PairEntry &e) {
    e.block_wide = nullptr;
    e.block_wide_attr = nullptr;
    e.wide_min_blocks = 0;
  }
};
template <class A, class B>
struct WideFiller<A, B, true> {
  static void fill(PairEntry &e) {
    e.block_wide = &launch_block_pair_wide<A, B>;
    e.block_wide_attr = &attr_block_pair_wide<A, B>;
    e.wide_min_blocks = pair_wide_blocks<A, B>();
  }
};

template <class A, class B, bool HAS>
struct MixedFiller {
  static void fill(PairEntry &e) {
    e.mixed = nullptr;
    e.mixed_attr = nullptr;
    e.mixed_clusters = nullptr;
  }
};
template <class A, class B>
struct MixedFiller<A, B, true> {
  static void fill(PairEntry &e) {
    e.mixed = &launch_mixed_group<A, B>;
    e.mixed_attr = &attr_mixed_group<A, B>;
    e.mixed_clusters = &clusters_mixed_group<A, B>;
  }
};

template <int I, int J>
struct RowFiller {
  static void fill(PairEntry *row) {
    using A = typename OpAt<I>::type;
    using B = typename OpAt<J>::type;
    row[J].block = &launch_block_pair<A, B>;
    row[J].thread = &launch_thread_pair<A, B>;
    row[J].block_attr = &attr_block_pair<A, B>;
    row[J].thread_attr = &attr_thread_pair<A, B>;
    row[J].block_clusters = &clusters_block_pair<A, B>;
    WideFiller<A, B, (pair_wide_blocks<A, B>() > 0)>::fill(row[J]);
    MixedFiller<A, B, (I < J)>::fill(row[J]);
    RowFiller<I, J + 1>::fill(row);
  }
};
template <int I>
struct RowFiller<I, kNumOps> {
  static void fill(PairEntry *) {}
};

template <>
void fill_pair_row<BFUSE_ROW>(PairEntry *row, SingleEntry *single) {
  using A = typename OpAt<BFUSE_ROW>::type;
  RowFiller<BFUSE_ROW, 0>::fill(row);
  single->launch = &launch_single<A>;
  single->attr = &attr_single<A>;
  single->group = &launch_group<A>;
  single->group_attr = &attr_group<A>;
  single->group_clusters = &clusters_group<A>;
  single->max_threads = A::kMaxThreads;
  single->params_size = sizeof(typename A::Params);
}

}  // namespace bfuse
