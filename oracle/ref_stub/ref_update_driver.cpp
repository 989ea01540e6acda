// Calls the reference's own UPDATE_TREE task body (UpdateTreeTask::cpu_variant,
// src/models/tree/update_tree.cc:36-134) on caller data.  The task class lives in that source file
// only, so the unmodified file is included into this translation unit instead of being linked.
// TEST INFRASTRUCTURE: used to check the oracle's restatement; never part of the product library.
#include <legate.h>

#include <cstdint>
#include <cstdio>
#include <exception>

#include "models/tree/update_tree.cc"

namespace legateboost {
auto Registry::get_registrar() -> legate::TaskRegistrar&
{
  static legate::TaskRegistrar r;
  return r;
}
}  // namespace legateboost

namespace {
legate::PhysicalArray make_array(const void* p, legate::Type::Code code, int ndim, const long long* extent,
                                 const long long* stride)
{
  legate::PhysicalArray a;
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

extern "C" {

// Argument order of the UPDATE_TREE task as the reference's Python launcher sets it up
// (legateboost/models/tree.py:197-240): scalars l1, l2; X promoted to (N,F,K) with stride 0 in dim
// 2; g and h promoted to (N,F,K) with stride 0 in dim 1; feature, split_value; outputs leaf_value
// and hessian [max_nodes, K].
int ref_update_tree_cpu(int x_is_f64, const void* X, const double* g, const double* h, int64_t N, int F, int K,
                        int max_nodes, const int32_t* feature, const double* split_value, double l1, double l2,
                        double* leaf_value, double* hessian)
{
  using legate::Type;
  try {
    legate::TaskContext ctx;
    const long long e3[3] = {N, F, K};
    const long long sx[3] = {F, 1, 0};
    const long long sg[3] = {K, 0, 1};
    const long long e2[2] = {max_nodes, K};
    const long long s2[2] = {K, 1};
    const long long e1[1] = {max_nodes};
    const long long s1[1] = {1};
    ctx.st->scalars.push_back(legate::Scalar::make<double>(l1));
    ctx.st->scalars.push_back(legate::Scalar::make<double>(l2));
    ctx.st->inputs.push_back(make_array(X, x_is_f64 ? Type::Code::FLOAT64 : Type::Code::FLOAT32, 3, e3, sx));
    ctx.st->inputs.push_back(make_array(g, Type::Code::FLOAT64, 3, e3, sg));
    ctx.st->inputs.push_back(make_array(h, Type::Code::FLOAT64, 3, e3, sg));
    ctx.st->inputs.push_back(make_array(feature, Type::Code::INT32, 1, e1, s1));
    ctx.st->inputs.push_back(make_array(split_value, Type::Code::FLOAT64, 1, e1, s1));
    ctx.st->outputs.push_back(make_array(leaf_value, Type::Code::FLOAT64, 2, e2, s2));
    ctx.st->outputs.push_back(make_array(hessian, Type::Code::FLOAT64, 2, e2, s2));
    legateboost::UpdateTreeTask::cpu_variant(ctx);
    legate::detail::release_task_buffers();
    return 0;
  } catch (const std::exception& e) {
    legate::detail::release_task_buffers();
    std::fprintf(stderr, "reference update_tree raised: %s\n", e.what());
    return 1;
  }
}
}
