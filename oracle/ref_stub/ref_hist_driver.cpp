// Calls the reference's own CPU histogram step (TreeBuilder::ComputeHistogram in
// src/models/tree/build_tree.cc:258-289, which ends with its prefix scan, :291-341) on caller
// data.  The reference keeps that class in an unnamed namespace, so its unmodified source file is
// included into this translation unit instead of being linked.  TEST INFRASTRUCTURE: used to
// check the oracle's histogram and as the timed reference CPU arm of the benchmark.
#include <legate.h>

#include <chrono>
#include <cstdint>
#include <cstdio>
#include <limits>

#include "models/tree/build_tree.cc"

namespace legateboost {
auto Registry::get_registrar() -> legate::TaskRegistrar&
{
  static legate::TaskRegistrar r;
  return r;
}
}  // namespace legateboost

extern "C" {

// bins: [n_rows, F] feature-relative bin ids, every feature has `bins_per_feature` bins.  The
// reference bins a float matrix itself, so X is set to the bin id and the proposals of every
// feature to 0,1,...,bins-2,+inf: its lower_bound then returns the same id.
// out: [node_end-node_begin, K, F*bins_per_feature, 2] float64, prefix-scanned inside each feature
// as the reference leaves it.  Returns the seconds spent inside ComputeHistogram.
double ref_compute_histogram(const uint8_t* bins,
                             int64_t n_rows,
                             int F,
                             int bins_per_feature,
                             const double* g,
                             const double* h,
                             int K,
                             const int32_t* node_of_row,
                             int node_begin,
                             int node_end,
                             double* out)
{
  using namespace legateboost;
  double seconds = -1.0;
  try {
    const int B = F * bins_per_feature;
    auto props  = legate::create_buffer<float, 1>(B);
    auto rowp   = legate::create_buffer<int32_t, 1>(F + 1);
    for (int f = 0; f <= F; ++f) rowp[f] = f * bins_per_feature;
    for (int f = 0; f < F; ++f)
      for (int b = 0; b < bins_per_feature; ++b)
        props[f * bins_per_feature + b] =
          b == bins_per_feature - 1 ? std::numeric_limits<float>::infinity() : static_cast<float>(b);
    SparseSplitProposals<float> split_proposals({props.ptr(0), static_cast<std::size_t>(B)},
                                                {rowp.ptr(0), static_cast<std::size_t>(F + 1)});
    auto Xf = legate::create_buffer<float, 1>(n_rows * F);
    for (int64_t i = 0; i < n_rows * F; ++i) Xf[i] = static_cast<float>(bins[i]);

    legate::PhysicalStore xs, gs, hs;
    auto fill = [&](legate::PhysicalStore& s, const void* p, legate::Type::Code c, long long s0, long long s1, long long s2) {
      s.ptr   = const_cast<void*>(p);
      s.tcode = c;
      s.ndim  = 3;
      s.lo    = {0, 0, 0, 0};
      s.hi    = {n_rows - 1, F - 1, K - 1, 0};
      s.stride = {s0, s1, s2, 0};
    };
    fill(xs, Xf.ptr(0), legate::Type::Code::FLOAT32, F, 1, 0);
    fill(gs, g, legate::Type::Code::FLOAT64, K, 0, 1);
    fill(hs, h, legate::Type::Code::FLOAT64, K, 0, 1);
    auto X_shape = xs.shape<3>();
    auto X_acc   = xs.read_accessor<float, 3, true>();
    auto g_acc   = gs.read_accessor<double, 3, true>();
    auto h_acc   = hs.read_accessor<double, 3, true>();

    const BinnedX binned(X_acc, X_shape, split_proposals);
    const int max_nodes = node_end;
    Tree tree(max_nodes, K);
    TreeBuilder<float> builder(static_cast<int32_t>(n_rows), F, K, max_nodes, 0, split_proposals);
    builder.histogram = Histogram<GPair>(node_begin, node_end, K, B);
    for (int64_t i = 0; i < n_rows; ++i) builder.sorted_positions[i] = {node_of_row[i], static_cast<int32_t>(i)};
    NodeBatch batch{node_begin, node_end, {builder.sorted_positions.ptr(0), static_cast<std::size_t>(n_rows)}};
    legate::TaskContext context;
    auto t0 = std::chrono::steady_clock::now();
    builder.ComputeHistogram(builder.histogram, context, tree, binned, g_acc, h_acc, batch);
    seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (out) {
      const GPair* src = builder.histogram.Ptr(node_begin);
      const std::size_t n = static_cast<std::size_t>(node_end - node_begin) * K * B;
      for (std::size_t i = 0; i < n; ++i) {
        out[2 * i]     = src[i].grad;
        out[2 * i + 1] = src[i].hess;
      }
    }
  } catch (const std::exception& e) {
    std::fprintf(stderr, "reference ComputeHistogram raised: %s\n", e.what());
  }
  legate::detail::release_task_buffers();
  return seconds;
}
}
