// UPDATE_TREE: the structure of a tree stays, its leaf values and hessians are recomputed from new
// gradients.
//
// Reference behaviour restated here: update_tree_fn, src/models/tree/update_tree.cc:36-134 (the
// reference has a CPU variant only) - every row walks from the root and adds its (g, h) to every
// node it visits, the two arrays are summed over the ranks, then
// leaf = H > 0 ? CalculateLeafValue(G, H, l1, l2) : 0 and hessian = H for every node.
//
// Design for B200: a row only adds its pair where its walk ENDS; the sums of the inner nodes are
// the sums of their children, added bottom-up afterwards (one small block), so the hot kernel does
// K pairs of float64 atomics per row instead of K * depth, and none of them on the root.  The
// per-node sums of a block are kept in shared memory when the tree is small enough, so that the
// global atomics are one pair per (block, node that rows of the block reached).  Float64 sums in a
// different order than the reference's row loop: equal to it within rounding (about 1e-15
// relative), not bit for bit.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

constexpr int kUpdThreads   = 256;
constexpr int kUpdSmemBytes = 64 * 1024;  // block-private sums up to this size

template <typename T>
__device__ inline int WalkToEnd(const T* __restrict__ xr, const int32_t* __restrict__ feature,
                                const double* __restrict__ split_value, int max_nodes, int F)
{
  int pos = 0;
  for (int depth = 0; depth < 100; ++depth) {  // reference: at most 100 levels
    const int f = __ldg(feature + pos);
    if (f < 0 || f >= F) break;  // a leaf (-1); an id outside the matrix also ends the walk
    const int next = static_cast<double>(xr[f]) <= __ldg(split_value + pos) ? 2 * pos + 1 : 2 * pos + 2;
    if (next >= max_nodes) break;  // a split on the last level of the arrays: the walk cannot go on
    pos = next;
  }
  return pos;
}

// sums[node][k] = (G, H) of the rows whose walk ends in `node`
template <typename T, bool kSmem>
__global__ void __launch_bounds__(kUpdThreads)
  k_update_ends(const T* __restrict__ X, int64_t ldx, int64_t n_rows, const double* __restrict__ g,
                const double* __restrict__ h, int64_t ldg, int F, int K, int max_nodes, const int32_t* __restrict__ feature,
                const double* __restrict__ split_value, double* __restrict__ sums /* [max_nodes][K][2] */)
{
  extern __shared__ double s_sums[];
  const int words = max_nodes * K * 2;
  if (kSmem) {
    for (int i = threadIdx.x; i < words; i += blockDim.x) s_sums[i] = 0.0;
    __syncthreads();
  }
  for (int64_t row = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; row < n_rows;
       row += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int pos = WalkToEnd(X + row * ldx, feature, split_value, max_nodes, F);
    double* dst   = (kSmem ? s_sums : sums) + static_cast<int64_t>(pos) * K * 2;
    for (int k = 0; k < K; ++k) {
      atomicAdd(dst + 2 * k, g[row * ldg + k]);
      atomicAdd(dst + 2 * k + 1, h[row * ldg + k]);
    }
  }
  if (kSmem) {
    __syncthreads();
    for (int i = threadIdx.x; i < words; i += blockDim.x)
      if (s_sums[i] != 0.0) atomicAdd(sums + i, s_sums[i]);
  }
}

// Bottom-up: an inner node's sums are its own (rows that ended there: none, unless its children
// fall outside the arrays) plus its children's, left first.  One block, level by level.
__global__ void __launch_bounds__(1024)
  k_update_ascend(double* __restrict__ sums, int K, int max_nodes, int F, const int32_t* __restrict__ feature)
{
  int top = 0;
  while ((2 << top) - 1 <= max_nodes) ++top;  // levels 0..top-1 are complete; level `top` may be cut
  for (int level = top; level >= 0; --level) {
    const int begin = (1 << level) - 1;
    const int end   = min(max_nodes, (2 << level) - 1);
    for (int i = begin * K + threadIdx.x; i < end * K; i += blockDim.x) {
      const int node = i / K, k = i - node * K;
      const int l = 2 * node + 1, r = 2 * node + 2;
      if (feature[node] >= 0 && feature[node] < F && r < max_nodes) {
        sums[2 * i] += sums[(static_cast<int64_t>(l) * K + k) * 2] + sums[(static_cast<int64_t>(r) * K + k) * 2];
        sums[2 * i + 1] += sums[(static_cast<int64_t>(l) * K + k) * 2 + 1] + sums[(static_cast<int64_t>(r) * K + k) * 2 + 1];
      }
    }
    __syncthreads();
  }
}

__global__ void k_update_finish(const double* __restrict__ sums, int64_t n, double l1, double l2,
                                double* __restrict__ leaf_value, double* __restrict__ hessian)
{
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const double G = sums[2 * i], H = sums[2 * i + 1];
  leaf_value[i] = H > 0.0 ? CalculateLeafValue(G, H, l1, l2) : 0.0;
  hessian[i]    = H;
}

template <typename T>
void UpdateTreeImpl(lbk_context* ctx, const lbk_update_tree_args& a, cudaStream_t stream)
{
  Scratch s(ctx, stream);
  const int64_t N = a.n_local_rows;
  const int K = a.n_outputs, M = a.max_nodes;
  const int64_t words = static_cast<int64_t>(M) * K * 2;
  double* sums        = s.alloc<double>(static_cast<size_t>(words));
  LBK_CUDA(cudaMemsetAsync(sums, 0, sizeof(double) * words, stream));
  if (N > 0) {
    int64_t blocks = (N + kUpdThreads - 1) / kUpdThreads;
    const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    const size_t smem = sizeof(double) * static_cast<size_t>(words);
    const T* X        = static_cast<const T*>(a.X);
    if (smem <= static_cast<size_t>(kUpdSmemBytes)) {
      if (smem > 48 * 1024)
        LBK_CUDA(cudaFuncSetAttribute(k_update_ends<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kUpdSmemBytes));
      k_update_ends<T, true><<<static_cast<unsigned>(blocks), kUpdThreads, smem, stream>>>(
        X, a.ldx, N, a.g, a.h, a.ldg, a.n_features, K, M, a.feature, a.split_value, sums);
    } else {
      k_update_ends<T, false><<<static_cast<unsigned>(blocks), kUpdThreads, 0, stream>>>(
        X, a.ldx, N, a.g, a.h, a.ldg, a.n_features, K, M, a.feature, a.split_value, sums);
    }
    LBK_LAUNCH_CHECK();
  }
  k_update_ascend<<<1, 1024, 0, stream>>>(sums, K, M, a.n_features, a.feature);
  LBK_LAUNCH_CHECK();
  // the reference reduces gradients and hessians with one all-reduce each; they are interleaved here
  AllReduce(ctx, sums, static_cast<size_t>(words), LBK_F64, LBK_SUM, stream);
  const int64_t n = static_cast<int64_t>(M) * K;
  k_update_finish<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(sums, n, a.l1_regularization,
                                                                             a.l2_regularization, a.leaf_value, a.hessian);
  LBK_LAUNCH_CHECK();
  CheckDeviceStatus(ctx, stream);
}

}  // namespace
}  // namespace lbk

extern "C" int lbk_update_tree(lbk_context* ctx, const lbk_update_tree_args* a)
{
  using namespace lbk;
  return Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "context is null");
    LBK_EXPECT(a != nullptr, "null argument");
    LBK_EXPECT(a->x_dtype == LBK_F32 || a->x_dtype == LBK_F64, "X must be float32 or float64");
    LBK_EXPECT(a->n_local_rows >= 0 && a->n_features >= 1 && a->n_outputs >= 1 && a->max_nodes >= 1, "bad shape");
    LBK_EXPECT(a->feature && a->split_value && a->leaf_value && a->hessian, "null argument");
    LBK_EXPECT(a->n_local_rows == 0 || (a->X && a->g && a->h), "null argument");
    LBK_EXPECT(a->n_local_rows == 0 || (a->ldx >= a->n_features && a->ldg >= a->n_outputs),
               "Expected a dense row major store");
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    if (a->x_dtype == LBK_F32) UpdateTreeImpl<float>(ctx, *a, stream);
    else UpdateTreeImpl<double>(ctx, *a, stream);
  });
}
