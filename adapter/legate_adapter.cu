// The bodies of legate-boost's two tree task variants on top of liblbk.so.
//
// The reference keeps its Python (legateboost/models/tree.py), its opcodes (src/legateboost.h:20-24)
// and its registration symbol (src/legate_library.cc:38-43); only the bodies of
// BuildTreeTask::gpu_variant (src/models/tree/build_tree.cu:1361-1365) and PredictTask::gpu_variant
// (src/models/tree/predict.cu:86-90) change: they become one-line calls of the functions below,
//
//   /*static*/ void BuildTreeTask::gpu_variant(legate::TaskContext context) { lbk_legate::BuildTree(context); }
//   /*static*/ void PredictTask::gpu_variant(legate::TaskContext context)   { lbk_legate::Predict(context); }
//
// which unpack the task's stores into the argument structs of include/lbk.h in the order the Python
// launcher adds them (legateboost/models/tree.py:117-183, 252-277).  Written against the legate
// C++ API the reference uses (TaskContext, PhysicalStore, accessors, create_buffer); this repository
// compiles it against its stand-in of those headers to keep it honest, a build of the reference
// compiles it against legate itself.
#include <cstdint>
#include <stdexcept>
#include <vector>

#include <cuda_runtime.h>

#include "legate.h"
#include "lbk.h"

#if __has_include(<nccl.h>)
#include <nccl.h>
#else
typedef struct ncclComm* ncclComm_t;
#endif

namespace lbk_legate {
namespace {

// Scratch of the library from the runtime's own pool (what the reference's task bodies do with
// legate::create_buffer, e.g. build_tree.cu:785-809): the buffers live until the task ends, so
// giving one back is a no-op.
void* AllocFromRuntime(void* /*user*/, size_t bytes, void* /*stream*/)
{
  auto buffer = legate::create_buffer<int8_t, 1>(legate::Point<1>(static_cast<legate::coord_t>(bytes)));
  return buffer.ptr(legate::Point<1>(0));
}
void ReleaseToRuntime(void* /*user*/, void* /*ptr*/, void* /*stream*/) {}

// One context per GPU, created on first use: the runtime calls a variant from one thread per GPU.
lbk_context* ContextForThisDevice()
{
  static thread_local lbk_context* ctx = nullptr;
  if (ctx == nullptr) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw std::runtime_error("no current CUDA device");
    if (lbk_context_create(dev, &ctx) != LBK_OK) throw std::runtime_error(lbk_last_error(nullptr));
    if (lbk_context_set_allocator(ctx, AllocFromRuntime, ReleaseToRuntime, nullptr) != LBK_OK)
      throw std::runtime_error(lbk_last_error(ctx));
  }
  return ctx;
}

}  // namespace

void BuildTree(legate::TaskContext context)
{
  const auto& X = context.input(0).data();
  auto X_shape  = X.shape<3>();
  auto g_store  = context.input(1).data();
  auto g_shape  = g_store.shape<3>();
  lbk_build_tree_args a{};
  a.x_dtype      = X.code() == legate::Type::Code::FLOAT32 ? LBK_F32 : LBK_F64;
  a.n_local_rows = X_shape.hi[0] - X_shape.lo[0] + 1 > 0 ? X_shape.hi[0] - X_shape.lo[0] + 1 : 0;
  a.row_offset   = X_shape.lo[0];
  a.n_features   = static_cast<int32_t>(X_shape.hi[1] - X_shape.lo[1] + 1);
  a.n_outputs    = static_cast<int32_t>(g_shape.hi[2] - g_shape.lo[2] + 1);
  // X is (N,F,K) with stride 0 in dim 2; g and h are (N,F,K) with stride 0 in dim 1
  size_t sx[3], sg[3], sh[3];
  if (a.x_dtype == LBK_F32) {
    a.X = X.read_accessor<float, 3>().ptr(X_shape, sx);
  } else {
    a.X = X.read_accessor<double, 3>().ptr(X_shape, sx);
  }
  a.ldx = static_cast<int64_t>(sx[0]);
  a.g   = g_store.read_accessor<double, 3>().ptr(g_shape, sg);
  a.h   = context.input(2).data().read_accessor<double, 3>().ptr(g_shape, sh);
  a.ldg = static_cast<int64_t>(sg[0]);
  if (context.inputs().size() == 4) {
    auto fs       = context.input(3).data();
    a.feature_set = reinterpret_cast<const uint8_t*>(fs.read_accessor<bool, 1>().ptr(fs.shape<1>().lo));
  }
  a.max_depth         = context.scalars().at(0).value<int>();
  a.max_nodes         = context.scalars().at(1).value<int>();
  a.split_samples     = context.scalars().at(2).value<int>();
  a.seed              = context.scalars().at(3).value<int>();
  a.dataset_rows      = context.scalars().at(4).value<int64_t>();
  a.l1_regularization = context.scalars().at(5).value<double>();
  a.l2_regularization = context.scalars().at(6).value<double>();
  a.min_split_gain    = context.scalars().at(7).value<double>();
  a.leaf_value  = context.output(0).data().write_accessor<double, 2>().ptr(legate::Point<2>(0, 0));
  a.feature     = context.output(1).data().write_accessor<int32_t, 1>().ptr(legate::Point<1>(0));
  a.split_value = context.output(2).data().write_accessor<double, 1>().ptr(legate::Point<1>(0));
  a.gain        = context.output(3).data().write_accessor<double, 1>().ptr(legate::Point<1>(0));
  a.hessian     = context.output(4).data().write_accessor<double, 2>().ptr(legate::Point<2>(0, 0));
  a.stream      = context.get_task_stream();

  lbk_context* ctx = ContextForThisDevice();
  if (context.num_communicators() > 0) {  // the test of cpp_utils.cuh:107-112
    auto* nccl       = context.communicator(0).get<ncclComm_t*>();
    const int rank   = static_cast<int>(context.get_task_index()[0]);
    const int ranks  = static_cast<int>(context.get_launch_domain().get_volume());
    if (nccl != nullptr && lbk_comm_attach_nccl(ctx, *nccl, rank, ranks) != LBK_OK)
      throw legate::TaskException{lbk_last_error(ctx)};
  }
  if (lbk_build_tree(ctx, &a) != LBK_OK) throw legate::TaskException{lbk_last_error(ctx)};
}

void Predict(legate::TaskContext context)
{
  const auto& X = context.input(0).data();
  auto X_shape  = X.shape<3>();
  auto pred     = context.output(0).data();
  auto p_shape  = pred.shape<3>();
  lbk_predict_args a{};
  a.n_rows = X_shape.hi[0] - X_shape.lo[0] + 1;
  if (a.n_rows < 1) return;  // predict.cu:35
  a.x_dtype    = X.code() == legate::Type::Code::FLOAT32 ? LBK_F32 : LBK_F64;
  a.n_features = static_cast<int32_t>(X_shape.hi[1] - X_shape.lo[1] + 1);
  a.n_outputs  = static_cast<int32_t>(p_shape.hi[2] - p_shape.lo[2] + 1);
  size_t sx[3], sp[3];
  if (a.x_dtype == LBK_F32) {
    a.X = X.read_accessor<float, 3>().ptr(X_shape, sx);
  } else {
    a.X = X.read_accessor<double, 3>().ptr(X_shape, sx);
  }
  a.ldx  = static_cast<int64_t>(sx[0]);
  a.pred = pred.write_accessor<double, 3>().ptr(p_shape, sp);
  a.ldp  = static_cast<int64_t>(sp[0]);
  const int n_trees = static_cast<int>((context.inputs().size() - 1) / 3);  // predict.cu:56
  std::vector<const double*> leaf(n_trees), split(n_trees);
  std::vector<const int32_t*> feat(n_trees);
  std::vector<int32_t> max_nodes(n_trees);
  for (int t = 0; t < n_trees; ++t) {
    auto f       = context.input(2 + 3 * t).data();
    leaf[t]      = context.input(1 + 3 * t).data().read_accessor<double, 2>().ptr(legate::Point<2>(0, 0));
    feat[t]      = f.read_accessor<int32_t, 1>().ptr(legate::Point<1>(0));
    split[t]     = context.input(3 + 3 * t).data().read_accessor<double, 1>().ptr(legate::Point<1>(0));
    max_nodes[t] = static_cast<int32_t>(f.shape<1>().hi[0] + 1);
  }
  a.n_trees     = n_trees;
  a.leaf_value  = leaf.data();
  a.feature     = feat.data();
  a.split_value = split.data();
  a.max_nodes   = max_nodes.data();
  a.stream      = context.get_task_stream();
  lbk_context* ctx = ContextForThisDevice();
  if (lbk_predict(ctx, &a) != LBK_OK) throw legate::TaskException{lbk_last_error(ctx)};
}

}  // namespace lbk_legate
