// Driver that calls the reference's unmodified CPU task bodies (BuildTreeTask::cpu_variant,
// PredictTask::cpu_variant) through the host-only stand-in of the runtime headers.
// TEST INFRASTRUCTURE: used to check the oracle's restatement and as the timed reference CPU
// arm of the benchmark; never part of the product library.
#include <legate.h>
#include <cstdint>
#include <cstdio>
#include <exception>

#include "models/tree/build_tree.h"
#include "models/tree/predict.h"

namespace {
using legate::PhysicalArray;
using legate::Type;

PhysicalArray make_array(const void* p, Type::Code code, int ndim, const long long* extent, const long long* stride)
{
  PhysicalArray a;
  a.store.ptr   = const_cast<void*>(p);
  a.store.tcode = code;
  a.store.ndim  = ndim;
  for (int i = 0; i < ndim; ++i) {
    a.store.lo[i]     = 0;
    a.store.hi[i]     = extent[i] - 1;
    a.store.stride[i] = stride[i];
  }
  return a;
}
}  // namespace

// legate_library.cc is not compiled; the registrar is never used by the task bodies.
namespace legateboost {
auto Registry::get_registrar() -> legate::TaskRegistrar&
{
  static legate::TaskRegistrar r;
  return r;
}
}  // namespace legateboost

extern "C" {

// Argument order of the BUILD_TREE task as the reference's Python launcher sets it up
// (legateboost/models/tree.py:117-178): X promoted to (N,F,K) with stride 0 in dim 2, g and h
// promoted to (N,F,K) with stride 0 in dim 1, optional bool feature set, eight scalars, five
// outputs.
int ref_build_tree_cpu(int x_is_f64,
                       const void* X,
                       const double* g,
                       const double* h,
                       const uint8_t* feature_set,
                       int64_t N,
                       int F,
                       int K,
                       int max_depth,
                       int split_samples,
                       int seed,
                       double l1,
                       double l2,
                       double min_split_gain,
                       double* leaf_value,
                       int32_t* feature,
                       double* split_value,
                       double* gain,
                       double* hessian)
{
  try {
    legate::TaskContext ctx;
    const long long e3[3]  = {N, F, K};
    const long long sx[3]  = {F, 1, 0};
    const long long sg[3]  = {K, 0, 1};
    ctx.st->inputs.push_back(make_array(X, x_is_f64 ? Type::Code::FLOAT64 : Type::Code::FLOAT32, 3, e3, sx));
    ctx.st->inputs.push_back(make_array(g, Type::Code::FLOAT64, 3, e3, sg));
    ctx.st->inputs.push_back(make_array(h, Type::Code::FLOAT64, 3, e3, sg));
    if (feature_set) {
      const long long e1[1] = {F};
      const long long s1[1] = {1};
      ctx.st->inputs.push_back(make_array(feature_set, Type::Code::BOOL, 1, e1, s1));
    }
    const int max_nodes = (1 << (max_depth + 1)) - 1;
    ctx.st->scalars.push_back(legate::Scalar::make<int>(max_depth));
    ctx.st->scalars.push_back(legate::Scalar::make<int>(max_nodes));
    ctx.st->scalars.push_back(legate::Scalar::make<int>(split_samples));
    ctx.st->scalars.push_back(legate::Scalar::make<int>(seed));
    ctx.st->scalars.push_back(legate::Scalar::make<int64_t>(N));
    ctx.st->scalars.push_back(legate::Scalar::make<double>(l1));
    ctx.st->scalars.push_back(legate::Scalar::make<double>(l2));
    ctx.st->scalars.push_back(legate::Scalar::make<double>(min_split_gain));
    const long long e2[2] = {max_nodes, K};
    const long long s2[2] = {K, 1};
    const long long e1[1] = {max_nodes};
    const long long s1[1] = {1};
    ctx.st->outputs.push_back(make_array(leaf_value, Type::Code::FLOAT64, 2, e2, s2));
    ctx.st->outputs.push_back(make_array(feature, Type::Code::INT32, 1, e1, s1));
    ctx.st->outputs.push_back(make_array(split_value, Type::Code::FLOAT64, 1, e1, s1));
    ctx.st->outputs.push_back(make_array(gain, Type::Code::FLOAT64, 1, e1, s1));
    ctx.st->outputs.push_back(make_array(hessian, Type::Code::FLOAT64, 2, e2, s2));
    legateboost::BuildTreeTask::cpu_variant(ctx);
    legate::detail::release_task_buffers();
    return 0;
  } catch (const std::exception& e) {
    legate::detail::release_task_buffers();
    std::fprintf(stderr, "reference build_tree raised: %s\n", e.what());
    return 1;
  }
}

// PREDICT task (legateboost/models/tree.py:252-277): X (N,F,K) stride 0 in dim 2, then
// (leaf_value, feature, split_value) per tree, output pred (N,F,K) stride 0 in dim 1.
int ref_predict_cpu(int x_is_f64,
                    const void* X,
                    int64_t N,
                    int F,
                    int K,
                    int n_trees,
                    const int32_t* max_nodes,
                    const double* const* leaf,
                    const int32_t* const* feat,
                    const double* const* split,
                    double* pred)
{
  try {
    legate::TaskContext ctx;
    const long long e3[3] = {N, F, K};
    const long long sx[3] = {F, 1, 0};
    const long long sp[3] = {K, 0, 1};
    ctx.st->inputs.push_back(make_array(X, x_is_f64 ? Type::Code::FLOAT64 : Type::Code::FLOAT32, 3, e3, sx));
    for (int t = 0; t < n_trees; ++t) {
      const long long e2[2] = {max_nodes[t], K};
      const long long s2[2] = {K, 1};
      const long long e1[1] = {max_nodes[t]};
      const long long s1[1] = {1};
      ctx.st->inputs.push_back(make_array(leaf[t], Type::Code::FLOAT64, 2, e2, s2));
      ctx.st->inputs.push_back(make_array(feat[t], Type::Code::INT32, 1, e1, s1));
      ctx.st->inputs.push_back(make_array(split[t], Type::Code::FLOAT64, 1, e1, s1));
    }
    ctx.st->outputs.push_back(make_array(pred, Type::Code::FLOAT64, 3, e3, sp));
    legateboost::PredictTask::cpu_variant(ctx);
    legate::detail::release_task_buffers();
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "reference predict raised: %s\n", e.what());
    return 1;
  }
}
}
