// Driver that runs the reference's unmodified GPU task bodies (BuildTreeTask::gpu_variant from
// src/models/tree/build_tree.cu, PredictTask::gpu_variant from predict.cu) on one device through
// the stand-in of the runtime headers, on host arrays that it copies to the device and back.
// TEST INFRASTRUCTURE: it produces the golden vectors that pin the quantised ("GPU variant")
// mode of the oracle and of the CUDA library; never part of the product library.
//
// build_tree.cu keeps TreeBuilder and its helpers in the translation unit, so the file is
// included here rather than linked: ref_gpu_build_tree calls the task body as it stands, and
// ref_gpu_build_tree_trace walks the same steps as the task body (build_tree.cu:1274-1359) in
// order to copy out each batch's histogram after ComputeHistogram and the quantised node sums.
#include <legate.h>

#include <cstdint>
#include <cstdio>
#include <exception>
#include <vector>

#include "models/tree/build_tree.cu"
#include "models/tree/predict.h"

namespace legateboost {
auto Registry::get_registrar() -> legate::TaskRegistrar&
{
  static legate::TaskRegistrar r;
  return r;
}
}  // namespace legateboost

// One rank never reaches NCCL (cpp_utils.cuh:107 returns before the call), but the symbols are
// referenced; define them here so that the object needs no NCCL library.
extern "C" const char* ncclGetErrorString(ncclResult_t) { return "NCCL is not part of the stand-in"; }
extern "C" ncclResult_t ncclAllReduce(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t)
{
  return ncclInternalError;
}

namespace {
using legate::PhysicalArray;
using legate::Type;

#define DRV_CUDA(call)                                                                          \
  do {                                                                                          \
    cudaError_t e_ = (call);                                                                    \
    if (e_ != cudaSuccess) throw std::runtime_error(std::string(#call ": ") + cudaGetErrorString(e_)); \
  } while (0)

// device copies of the caller's host arrays, released with the object
struct DeviceArrays {
  std::vector<void*> ptrs;
  ~DeviceArrays()
  {
    for (void* p : ptrs) cudaFree(p);
  }
  void* upload(const void* host, size_t bytes)
  {
    void* d = nullptr;
    DRV_CUDA(cudaMalloc(&d, bytes > 0 ? bytes : 1));
    ptrs.push_back(d);
    if (host && bytes) DRV_CUDA(cudaMemcpy(d, host, bytes, cudaMemcpyHostToDevice));
    return d;
  }
  void* zeros(size_t bytes)
  {
    void* d = upload(nullptr, bytes);
    DRV_CUDA(cudaMemset(d, 0, bytes > 0 ? bytes : 1));
    return d;
  }
};

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

struct TreeCall {
  DeviceArrays dev;
  legate::TaskContext ctx;
  int max_nodes = 0;
  double *d_leaf = nullptr, *d_split = nullptr, *d_gain = nullptr, *d_hess = nullptr;
  int32_t* d_feat = nullptr;
  cudaStream_t stream = nullptr;
  ~TreeCall()
  {
    if (stream) cudaStreamDestroy(stream);
  }
};

// Argument order of the BUILD_TREE task as the reference's Python launcher sets it up
// (legateboost/models/tree.py:117-178).
void setup_tree_call(TreeCall& c, int x_is_f64, const void* X, const double* g, const double* h,
                     const uint8_t* feature_set, int64_t N, int F, int K, int max_depth, int split_samples, int seed,
                     double l1, double l2, double min_split_gain)
{
  DRV_CUDA(cudaStreamCreate(&c.stream));
  c.ctx.st->stream       = c.stream;
  const size_t xsz       = x_is_f64 ? 8 : 4;
  const void* dX         = c.dev.upload(X, xsz * N * F);
  const void* dg         = c.dev.upload(g, sizeof(double) * N * K);
  const void* dh         = c.dev.upload(h, sizeof(double) * N * K);
  const long long e3[3]  = {N, F, K};
  const long long sx[3]  = {F, 1, 0};
  const long long sg[3]  = {K, 0, 1};
  c.ctx.st->inputs.push_back(make_array(dX, x_is_f64 ? Type::Code::FLOAT64 : Type::Code::FLOAT32, 3, e3, sx));
  c.ctx.st->inputs.push_back(make_array(dg, Type::Code::FLOAT64, 3, e3, sg));
  c.ctx.st->inputs.push_back(make_array(dh, Type::Code::FLOAT64, 3, e3, sg));
  if (feature_set) {
    const void* dfs       = c.dev.upload(feature_set, F);
    const long long e1[1] = {F};
    const long long s1[1] = {1};
    c.ctx.st->inputs.push_back(make_array(dfs, Type::Code::BOOL, 1, e1, s1));
  }
  c.max_nodes = (1 << (max_depth + 1)) - 1;
  c.ctx.st->scalars.push_back(legate::Scalar::make<int>(max_depth));
  c.ctx.st->scalars.push_back(legate::Scalar::make<int>(c.max_nodes));
  c.ctx.st->scalars.push_back(legate::Scalar::make<int>(split_samples));
  c.ctx.st->scalars.push_back(legate::Scalar::make<int>(seed));
  c.ctx.st->scalars.push_back(legate::Scalar::make<int64_t>(N));
  c.ctx.st->scalars.push_back(legate::Scalar::make<double>(l1));
  c.ctx.st->scalars.push_back(legate::Scalar::make<double>(l2));
  c.ctx.st->scalars.push_back(legate::Scalar::make<double>(min_split_gain));
  const int M           = c.max_nodes;
  c.d_leaf              = static_cast<double*>(c.dev.zeros(sizeof(double) * M * K));
  c.d_feat              = static_cast<int32_t*>(c.dev.zeros(sizeof(int32_t) * M));
  c.d_split             = static_cast<double*>(c.dev.zeros(sizeof(double) * M));
  c.d_gain              = static_cast<double*>(c.dev.zeros(sizeof(double) * M));
  c.d_hess              = static_cast<double*>(c.dev.zeros(sizeof(double) * M * K));
  const long long e2[2] = {M, K};
  const long long s2[2] = {K, 1};
  const long long e1[1] = {M};
  const long long s1[1] = {1};
  c.ctx.st->outputs.push_back(make_array(c.d_leaf, Type::Code::FLOAT64, 2, e2, s2));
  c.ctx.st->outputs.push_back(make_array(c.d_feat, Type::Code::INT32, 1, e1, s1));
  c.ctx.st->outputs.push_back(make_array(c.d_split, Type::Code::FLOAT64, 1, e1, s1));
  c.ctx.st->outputs.push_back(make_array(c.d_gain, Type::Code::FLOAT64, 1, e1, s1));
  c.ctx.st->outputs.push_back(make_array(c.d_hess, Type::Code::FLOAT64, 2, e2, s2));
}

void fetch_tree(const TreeCall& c, int K, double* leaf_value, int32_t* feature, double* split_value, double* gain,
                double* hessian)
{
  const int M = c.max_nodes;
  DRV_CUDA(cudaDeviceSynchronize());
  DRV_CUDA(cudaMemcpy(leaf_value, c.d_leaf, sizeof(double) * M * K, cudaMemcpyDeviceToHost));
  DRV_CUDA(cudaMemcpy(feature, c.d_feat, sizeof(int32_t) * M, cudaMemcpyDeviceToHost));
  DRV_CUDA(cudaMemcpy(split_value, c.d_split, sizeof(double) * M, cudaMemcpyDeviceToHost));
  DRV_CUDA(cudaMemcpy(gain, c.d_gain, sizeof(double) * M, cudaMemcpyDeviceToHost));
  DRV_CUDA(cudaMemcpy(hessian, c.d_hess, sizeof(double) * M * K, cudaMemcpyDeviceToHost));
}

// The steps of build_tree_fn::operator() (build_tree.cu:1276-1358) with two copies added: every
// batch's histogram after ComputeHistogram (all-reduced and scanned: what the split search reads)
// and the quantised node sums at the end.
template <typename T>
void traced_build(legate::TaskContext context, int64_t* trace_hist, int trace_nodes, int64_t* trace_node_sums,
                  int32_t* total_bins)
{
  using namespace legateboost;
  auto [X, X_shape, X_accessor] = GetInputStore<T, 3>(context.input(0).data());
  auto [g, g_shape, g_accessor] = GetInputStore<double, 3>(context.input(1).data());
  auto [h, h_shape, h_accessor] = GetInputStore<double, 3>(context.input(2).data());
  auto num_features = X_shape.hi[1] - X_shape.lo[1] + 1;
  auto num_rows     = std::max<int64_t>(X_shape.hi[0] - X_shape.lo[0] + 1, 0);
  auto num_outputs  = g_shape.hi[2] - g_shape.lo[2] + 1;
  auto max_depth         = context.scalars().at(0).value<int>();
  auto max_nodes         = context.scalars().at(1).value<int>();
  auto split_samples     = context.scalars().at(2).value<int>();
  auto seed              = context.scalars().at(3).value<int>();
  auto dataset_rows      = context.scalars().at(4).value<int64_t>();
  auto l1_regularization = context.scalars().at(5).value<double>();
  auto l2_regularization = context.scalars().at(6).value<double>();
  auto min_split_gain    = context.scalars().at(7).value<double>();
  std::optional<legate::AccessorRO<bool, 1>> optional_feature_set;
  if (context.inputs().size() == 4) {
    auto [feature_set, feature_set_shape, feature_set_accessor] = GetInputStore<bool, 1>(context.input(3).data());
    optional_feature_set = feature_set_accessor;
  }
  auto* stream            = context.get_task_stream();
  auto thrust_alloc       = ThrustAllocator(legate::Memory::GPU_FB_MEM);
  auto thrust_exec_policy = DEFAULT_POLICY(thrust_alloc).on(stream);
  Tree tree(max_nodes, num_outputs, stream, thrust_exec_policy);
  SparseSplitProposals<T> const split_proposals =
    SelectSplitSamples(context, X_accessor, X_shape, split_samples, seed, dataset_rows, stream);
  GradientQuantiser const quantiser(context, g_accessor, h_accessor, g_shape, stream);
  TreeBuilder<T> builder(num_rows, num_features, num_outputs, stream, tree.max_nodes, max_depth, split_proposals, quantiser);
  builder.InitialiseRoot(context, tree, g_accessor, h_accessor, g_shape, l2_regularization, l1_regularization, seed);
  const int64_t B = split_proposals.HistogramSize();
  if (total_bins) *total_bins = static_cast<int32_t>(B);
  for (int depth = 0; depth < max_depth; ++depth) {
    auto batches = builder.PrepareBatches(depth);
    for (auto batch : batches) {
      auto histogram = builder.GetHistogram(batch);
      builder.ComputeHistogram(histogram, context, tree, X_accessor, X_shape, g_accessor, h_accessor, batch, seed);
      if (trace_hist) {
        const int nb = batch.node_idx_begin, ne = std::min<int>(batch.node_idx_end, trace_nodes);
        if (ne > nb) {
          DRV_CUDA(cudaStreamSynchronize(stream));
          DRV_CUDA(cudaMemcpy(trace_hist + static_cast<int64_t>(nb) * num_outputs * B * 2, histogram.Ptr(nb),
                              sizeof(int64_t) * 2 * (ne - nb) * num_outputs * B, cudaMemcpyDeviceToHost));
        }
      }
      builder.PerformBestSplit(tree, histogram, batch, l1_regularization, l2_regularization, min_split_gain,
                               optional_feature_set);
    }
    if (depth < max_depth - 1) { builder.UpdatePositions(tree, X_accessor, X_shape); }
  }
  tree.WriteTreeOutput(context, thrust_exec_policy, quantiser);
  CHECK_CUDA(cudaStreamSynchronize(stream));
  if (trace_node_sums)
    DRV_CUDA(cudaMemcpy(trace_node_sums, tree.node_sums.ptr({0, 0}), sizeof(int64_t) * 2 * max_nodes * num_outputs,
                        cudaMemcpyDeviceToHost));
}

}  // namespace

extern "C" {

int ref_gpu_device_count()
{
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
  return n;
}

int ref_gpu_build_tree(int x_is_f64, const void* X, const double* g, const double* h, const uint8_t* feature_set,
                       int64_t N, int F, int K, int max_depth, int split_samples, int seed, double l1, double l2,
                       double min_split_gain, double* leaf_value, int32_t* feature, double* split_value, double* gain,
                       double* hessian)
{
  try {
    TreeCall c;
    setup_tree_call(c, x_is_f64, X, g, h, feature_set, N, F, K, max_depth, split_samples, seed, l1, l2, min_split_gain);
    legateboost::BuildTreeTask::gpu_variant(c.ctx);
    fetch_tree(c, K, leaf_value, feature, split_value, gain, hessian);
    legate::detail::release_task_buffers();
    return 0;
  } catch (const std::exception& e) {
    legate::detail::release_task_buffers();
    std::fprintf(stderr, "reference gpu build_tree raised: %s\n", e.what());
    return 1;
  }
}

// trace_hist: [trace_nodes, K, B, 2] int64 (B is only known after the call: give room for
// F * split_samples bins per node and output; the rows are packed with the B written to
// total_bins); trace_node_sums: [max_nodes, K, 2] int64.
int ref_gpu_build_tree_trace(int x_is_f64, const void* X, const double* g, const double* h, const uint8_t* feature_set,
                             int64_t N, int F, int K, int max_depth, int split_samples, int seed, double l1, double l2,
                             double min_split_gain, double* leaf_value, int32_t* feature, double* split_value,
                             double* gain, double* hessian, int64_t* trace_hist, int trace_nodes,
                             int64_t* trace_node_sums, int32_t* total_bins)
{
  try {
    TreeCall c;
    setup_tree_call(c, x_is_f64, X, g, h, feature_set, N, F, K, max_depth, split_samples, seed, l1, l2, min_split_gain);
    if (x_is_f64)
      traced_build<double>(c.ctx, trace_hist, trace_nodes, trace_node_sums, total_bins);
    else
      traced_build<float>(c.ctx, trace_hist, trace_nodes, trace_node_sums, total_bins);
    fetch_tree(c, K, leaf_value, feature, split_value, gain, hessian);
    legate::detail::release_task_buffers();
    return 0;
  } catch (const std::exception& e) {
    legate::detail::release_task_buffers();
    std::fprintf(stderr, "reference gpu build_tree (traced) raised: %s\n", e.what());
    return 1;
  }
}

// PREDICT task (legateboost/models/tree.py:252-277): X (N,F,K) stride 0 in dim 2, then
// (leaf_value, feature, split_value) per tree, output pred (N,F,K) stride 0 in dim 1.
int ref_gpu_predict(int x_is_f64, const void* X, int64_t N, int F, int K, int n_trees, const int32_t* max_nodes,
                    const double* const* leaf, const int32_t* const* feat, const double* const* split, double* pred)
{
  try {
    DeviceArrays dev;
    legate::TaskContext ctx;
    cudaStream_t stream = nullptr;
    DRV_CUDA(cudaStreamCreate(&stream));
    ctx.st->stream        = stream;
    const size_t xsz      = x_is_f64 ? 8 : 4;
    const long long e3[3] = {N, F, K};
    const long long sx[3] = {F, 1, 0};
    const long long sp[3] = {K, 0, 1};
    ctx.st->inputs.push_back(
      make_array(dev.upload(X, xsz * N * F), x_is_f64 ? Type::Code::FLOAT64 : Type::Code::FLOAT32, 3, e3, sx));
    for (int t = 0; t < n_trees; ++t) {
      const long long e2[2] = {max_nodes[t], K};
      const long long s2[2] = {K, 1};
      const long long e1[1] = {max_nodes[t]};
      const long long s1[1] = {1};
      ctx.st->inputs.push_back(make_array(dev.upload(leaf[t], sizeof(double) * max_nodes[t] * K), Type::Code::FLOAT64, 2, e2, s2));
      ctx.st->inputs.push_back(make_array(dev.upload(feat[t], sizeof(int32_t) * max_nodes[t]), Type::Code::INT32, 1, e1, s1));
      ctx.st->inputs.push_back(make_array(dev.upload(split[t], sizeof(double) * max_nodes[t]), Type::Code::FLOAT64, 1, e1, s1));
    }
    double* d_pred = static_cast<double*>(dev.zeros(sizeof(double) * N * K));
    ctx.st->outputs.push_back(make_array(d_pred, Type::Code::FLOAT64, 3, e3, sp));
    legateboost::PredictTask::gpu_variant(ctx);
    DRV_CUDA(cudaStreamSynchronize(stream));
    DRV_CUDA(cudaMemcpy(pred, d_pred, sizeof(double) * N * K, cudaMemcpyDeviceToHost));
    cudaStreamDestroy(stream);
    legate::detail::release_task_buffers();
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "reference gpu predict raised: %s\n", e.what());
    return 1;
  }
}
}
