// Ensemble predict: pred[row, :] = sum over trees of leaf_value[leaf reached by row, :].
//
// Reference behaviour restated here: predict_fn, src/models/tree/predict.cu:26-84 - one kernel
// launch per tree, each re-reading and re-writing pred; rows walk from node 0 while
// feature[pos] != -1 (at most 100 steps), going left iff (double)x <= split_value[pos].
//
// Design for B200: ONE launch for the whole ensemble.  The trees are first packed into one
// array of 16-byte nodes (split, feature) plus one leaf array, so a step of the walk is one
// 16-byte load that stays in L1/L2 (500 depth-8 trees are 4 MB).  A block stages a tile of rows
// of X in shared memory, feature-major, so the lane that owns row r always reads bank r%32
// whatever feature its node asks for; every row is read from HBM exactly once, predictions are
// accumulated in float64 in tree order and written exactly once.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

struct PNode {
  double split;
  int feature;
  int pad;
};

struct TreePtrs {
  const double* leaf;
  const int32_t* feature;
  const double* split;
  int max_nodes;
  int node_off;  // offset of this tree's first node in the packed arrays
};

__global__ void k_pack_trees(const TreePtrs* __restrict__ trees, int K, PNode* __restrict__ nodes,
                             double* __restrict__ leaves)
{
  const TreePtrs t = trees[blockIdx.x];
  for (int i = threadIdx.x; i < t.max_nodes; i += blockDim.x) {
    PNode n;
    n.split   = t.split[i];
    n.feature = t.feature[i];
    n.pad     = 0;
    nodes[t.node_off + i] = n;
  }
  for (int64_t i = threadIdx.x; i < static_cast<int64_t>(t.max_nodes) * K; i += blockDim.x)
    leaves[static_cast<int64_t>(t.node_off) * K + i] = t.leaf[i];
}

template <typename T, bool kStage>
__global__ void __launch_bounds__(128)
  k_predict(const T* __restrict__ X, int64_t ldx, int64_t n_rows, int F, int K, int n_trees,
            const TreePtrs* __restrict__ trees, const PNode* __restrict__ nodes, const double* __restrict__ leaves,
            double* __restrict__ pred, int64_t ldp, int acc_in_smem)
{
  constexpr int RB = 128;  // rows per block = threads per block
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int RBP = RB + 1;  // row pitch of the staged tile: consecutive features fall in consecutive banks
  T* xs        = reinterpret_cast<T*>(smem_raw);                                    // [F][RBP]
  double* accs = reinterpret_cast<double*>(smem_raw + (kStage ? (sizeof(T) * F * RBP + 15) / 16 * 16 : 0));  // [K][RB]
  const int tid        = threadIdx.x;
  const int64_t row0   = static_cast<int64_t>(blockIdx.x) * RB;
  const int64_t row    = row0 + tid;
  const int rows_here  = static_cast<int>((n_rows - row0) < RB ? (n_rows - row0) : RB);
  if (kStage) {
    // a warp stages whole rows: coalesced reads along the features, transposed writes whose
    // pitch of RB+1 elements spreads consecutive features over consecutive banks
    const int lane = tid & 31, warp = tid >> 5;
    constexpr int NW = RB / 32, U = 8;  // eight independent row loads in flight per lane
    for (int rb = warp; rb < rows_here; rb += NW * U) {
      for (int f = lane; f < F; f += 32) {
        T v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int r = rb + u * NW;
          if (r < rows_here) v[u] = __ldcs(X + (row0 + r) * ldx + f);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int r = rb + u * NW;
          if (r < rows_here) xs[f * RBP + r] = v[u];
        }
      }
    }
    __syncthreads();
  }
  if (tid >= rows_here) return;
  const T* xr = X + row * ldx;
  double acc0 = 0.0;
  if (K > 1) {
    if (acc_in_smem) {
      for (int k = 0; k < K; ++k) accs[k * RB + tid] = 0.0;
    } else {
      for (int k = 0; k < K; ++k) pred[row * ldp + k] = 0.0;
    }
  }
  for (int t = 0; t < n_trees; ++t) {
    const int off = trees[t].node_off;
    const int mn  = trees[t].max_nodes;
    int pos       = 0;
    for (int depth = 0; depth < 100; ++depth) {
      const PNode n = nodes[off + pos];
      // a split node on the last level of the arrays has no children to go to: stop there
      if (n.feature == -1 || 2 * pos + 2 >= mn) break;
      const double xv = static_cast<double>(kStage ? xs[n.feature * RBP + tid] : xr[n.feature]);
      pos             = xv <= n.split ? 2 * pos + 1 : 2 * pos + 2;
    }
    const double* lf = leaves + static_cast<int64_t>(off + pos) * K;
    if (K == 1) {
      acc0 += lf[0];
    } else if (acc_in_smem) {
      for (int k = 0; k < K; ++k) accs[k * RB + tid] += lf[k];
    } else {
      for (int k = 0; k < K; ++k) pred[row * ldp + k] += lf[k];
    }
  }
  if (K == 1) {
    pred[row * ldp] = acc0;
  } else if (acc_in_smem) {
    for (int k = 0; k < K; ++k) pred[row * ldp + k] = accs[k * RB + tid];
  }
}

}  // namespace

template <typename T>
void PredictLaunch(lbk_context* ctx, Scratch& s, const T* X, int64_t ldx, int64_t n_rows, int F, int K, int n_trees,
                   const double* const* leaf, const int32_t* const* feat, const double* const* split,
                   const int32_t* max_nodes, double* pred, int64_t ldp, cudaStream_t stream)
{
  if (n_rows < 1) return;  // an empty shard returns at once (reference: predict.cu:35)
  if (n_trees == 0) {
    LBK_CUDA(cudaMemset2DAsync(pred, sizeof(double) * ldp, 0, sizeof(double) * K, n_rows, stream));
    return;
  }
  std::vector<TreePtrs> h(n_trees);
  int64_t total_nodes = 0;
  for (int t = 0; t < n_trees; ++t) {
    LBK_EXPECT(leaf[t] && feat[t] && split[t] && max_nodes[t] >= 1, "bad tree arrays");
    h[t].leaf      = leaf[t];
    h[t].feature   = feat[t];
    h[t].split     = split[t];
    h[t].max_nodes = max_nodes[t];
    LBK_EXPECT(total_nodes + max_nodes[t] < (int64_t{1} << 31), "ensemble too large");
    h[t].node_off = static_cast<int>(total_nodes);
    total_nodes += max_nodes[t];
  }
  TreePtrs* d_trees = s.alloc<TreePtrs>(n_trees);
  PNode* nodes      = s.alloc<PNode>(total_nodes);
  double* leaves    = s.alloc<double>(total_nodes * K);
  LBK_CUDA(cudaMemcpyAsync(d_trees, h.data(), sizeof(TreePtrs) * n_trees, cudaMemcpyHostToDevice, stream));
  LBK_CUDA(cudaStreamSynchronize(stream));  // h is a local; the copy must have read it
  k_pack_trees<<<n_trees, 256, 0, stream>>>(d_trees, K, nodes, leaves);
  LBK_LAUNCH_CHECK();

  constexpr int RB      = 128;
  const size_t x_bytes  = (sizeof(T) * static_cast<size_t>(F) * (RB + 1) + 15) / 16 * 16;
  const size_t a_bytes  = K > 1 ? sizeof(double) * static_cast<size_t>(K) * RB : 0;
  const size_t budget   = static_cast<size_t>(ctx->max_smem_optin) - 1024;
  const bool stage      = x_bytes <= budget;
  const int acc_in_smem = (K > 1 && (stage ? x_bytes : 0) + a_bytes <= budget) ? 1 : 0;
  const size_t smem     = (stage ? x_bytes : 0) + (acc_in_smem ? a_bytes : 0);
  const unsigned grid   = static_cast<unsigned>((n_rows + RB - 1) / RB);
  if (stage) {
    if (smem > 48 * 1024)
      LBK_CUDA(cudaFuncSetAttribute(k_predict<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    k_predict<T, true><<<grid, RB, smem, stream>>>(X, ldx, n_rows, F, K, n_trees, d_trees, nodes, leaves, pred, ldp,
                                                    acc_in_smem);
  } else {
    if (smem > 48 * 1024)
      LBK_CUDA(cudaFuncSetAttribute(k_predict<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    k_predict<T, false><<<grid, RB, smem, stream>>>(X, ldx, n_rows, F, K, n_trees, d_trees, nodes, leaves, pred, ldp,
                                                     acc_in_smem);
  }
  LBK_LAUNCH_CHECK();
}

template void PredictLaunch<float>(lbk_context*, Scratch&, const float*, int64_t, int64_t, int, int, int,
                                   const double* const*, const int32_t* const*, const double* const*, const int32_t*,
                                   double*, int64_t, cudaStream_t);
template void PredictLaunch<double>(lbk_context*, Scratch&, const double*, int64_t, int64_t, int, int, int,
                                    const double* const*, const int32_t* const*, const double* const*, const int32_t*,
                                    double*, int64_t, cudaStream_t);

}  // namespace lbk
