// Node selection, prefix scan with sibling subtraction, and split evaluation.
//
// Reference behaviour restated here (src/models/tree/):
//   SelectHistogramNode / ComputeHistogramBin  build_tree.h:80-104 - only the child with the
//     smaller quantised hessian of output 0 is built (ties: the right child) when the parent's
//     histogram is available;
//   scan_kernel        build_tree.cu:597-668 - inclusive prefix over the bins of each feature; the
//     prefix replaces the bin value only if prefix.grad > 0 or prefix.hess > 0; then
//     sibling = parent - node;
//   perform_best_split build_tree.cu:682-782 - gain of every bin summed over outputs in float64 on
//     dequantised sums, zero if any output has a non-positive hessian on either side, accept if
//     the best gain exceeds 1e-5.  Ties: the reference keeps, per thread t = bin mod 512, the
//     first strict maximum and reduces with op(a,b) = a.gain > b.gain ? a : b where a always
//     comes from lower thread ids, so equal gains resolve to the largest (bin mod 512) and then
//     the smallest bin.  That total order is applied here, independent of the reduction shape.
// Compiled with -fmad=false.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

__global__ void k_plan_built(const GPairI64* __restrict__ node_sums, int K, int node_begin, int n_nodes,
                             bool parent_available, int32_t* __restrict__ slot_of_node)
{
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n_nodes) return;
  const int node = node_begin + j;
  int slot;
  if (node == 0) {
    slot = 0;
  } else if (!parent_available) {
    slot = j;
  } else {
    const int parent = (node - 1) / 2;
    const int l = 2 * parent + 1, r = 2 * parent + 2;
    const int hist_node =
      (node_sums[static_cast<int64_t>(l) * K].hess < node_sums[static_cast<int64_t>(r) * K].hess) ? l : r;
    slot = hist_node == node ? j / 2 : -1;
  }
  slot_of_node[j] = slot;
}

// One warp per (node, feature); blockIdx.y = output.
__global__ void __launch_bounds__(256)
  k_scan(const GPairI64* __restrict__ built, const int32_t* __restrict__ slot_of_node,
         GPairI64* __restrict__ level_hist, const GPairI64* __restrict__ parent_hist, int parent_begin,
         const GPairI64* __restrict__ node_sums, int node_begin, int n_nodes, int K, int f_begin, int n_features,
         int B, const int32_t* __restrict__ row_ptr, bool parent_available)
{
  const int lane    = threadIdx.x & 31;
  const int64_t wid = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  if (wid >= static_cast<int64_t>(n_nodes) * n_features) return;
  const int j    = static_cast<int>(wid / n_features);
  const int f    = f_begin + static_cast<int>(wid % n_features);
  const int k    = blockIdx.y;
  const int node = node_begin + j;
  const int slot = slot_of_node[j];
  if (slot < 0) return;
  const GPairI64* src = built + (static_cast<int64_t>(slot) * K + k) * B;
  GPairI64* dst       = level_hist + (static_cast<int64_t>(j) * K + k) * B;
  const int fb = row_ptr[f], fe = row_ptr[f + 1];
  if (node_sums[static_cast<int64_t>(node) * K + k].hess <= 0) {
    // not scanned: the raw values stay, no sibling is derived
    if (src != dst)
      for (int b = fb + lane; b < fe; b += 32) StorePair(dst + b, LoadPair(src + b));
    return;
  }
  const bool derive = node != 0 && parent_available;
  GPairI64* sib     = nullptr;
  const GPairI64* par = nullptr;
  if (derive) {
    const int js = j ^ 1;  // a level starts at an odd heap index: j even = left child
    sib          = level_hist + (static_cast<int64_t>(js) * K + k) * B;
    par          = parent_hist + (static_cast<int64_t>((node - 1) / 2 - parent_begin) * K + k) * B;
  }
  long long agg_g = 0, agg_h = 0;
  for (int base = fb; base < fe; base += 32) {
    const int b     = base + lane;
    const bool part = b < fe;
    GPairI64 raw{0, 0};
    if (part) raw = LoadPair(src + b);
    long long sg = raw.grad, sh = raw.hess;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const long long ng = __shfl_up_sync(0xffffffffu, sg, off);
      const long long nh = __shfl_up_sync(0xffffffffu, sh, off);
      if (lane >= off) {
        sg += ng;
        sh += nh;
      }
    }
    const long long tile_g = __shfl_sync(0xffffffffu, sg, 31);
    const long long tile_h = __shfl_sync(0xffffffffu, sh, 31);
    sg += agg_g;
    sh += agg_h;
    if (part) {
      const GPairI64 v = (sg > 0 || sh > 0) ? GPairI64{sg, sh} : raw;
      StorePair(dst + b, v);
      if (derive) {
        const GPairI64 pv = LoadPair(par + b);
        StorePair(sib + b, GPairI64{pv.grad - v.grad, pv.hess - v.hess});
      }
    }
    agg_g += tile_g;
    agg_h += tile_h;
  }
}

struct Cand {
  double gain;
  int bin;
};
__device__ inline bool Better(const Cand& a, const Cand& b)
{
  if (a.gain > b.gain) return true;
  if (a.gain < b.gain) return false;
  if (a.bin < 0 || b.bin < 0) return b.bin < 0 && a.bin >= 0;
  const int ta = a.bin & 511, tb = b.bin & 511;
  if (ta != tb) return ta > tb;
  return a.bin < b.bin;
}

constexpr int kSplitThreads = 256;

// Candidate of one slice of a node's bins, as it travels through global memory.
struct SliceBest {
  double gain;
  int bin;
  int pad;
};

// The winner of a node becomes the tree: feature, split value, gain, and the sums and leaf values
// of the two children.  left_sums[k * left_stride] = the sums left of the winning bin, output k.
template <typename T>
__device__ inline void ApplyWinner(const Cand& nb, int node, int K, int F, const int32_t* __restrict__ row_ptr,
                                   const T* __restrict__ proposals, const QuantParams& qp, double l1, double l2,
                                   TreeArrays tree, const GPairI64* __restrict__ left_sums, int64_t left_stride, int tid,
                                   int n_threads)
{
  if (!(nb.gain > 1e-5)) return;
  GPairI64* node_sums = tree.node_sums;
  int lo = 0, hi = F;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (row_ptr[mid] <= nb.bin) lo = mid; else hi = mid;
  }
  const int bf = lo;
  const int l = 2 * node + 1, r = 2 * node + 2;
  for (int k = tid; k < K; k += n_threads) {
    const GPairI64 ns = LoadPair(node_sums + static_cast<int64_t>(node) * K + k);
    const GPairI64 ls = LoadPair(left_sums + static_cast<int64_t>(k) * left_stride);
    const GPairI64 rs{ns.grad - ls.grad, ns.hess - ls.hess};
    StorePair(node_sums + static_cast<int64_t>(l) * K + k, ls);
    StorePair(node_sums + static_cast<int64_t>(r) * K + k, rs);
    const GPairF64 dl = Dequantise(ls, qp), dr = Dequantise(rs, qp);
    tree.leaf_value[static_cast<int64_t>(l) * K + k] = CalculateLeafValue(dl.grad, dl.hess, l1, l2);
    tree.leaf_value[static_cast<int64_t>(r) * K + k] = CalculateLeafValue(dr.grad, dr.hess, l1, l2);
    if (k == 0) {
      tree.feature[node]     = bf;
      tree.split_value[node] = static_cast<double>(proposals[nb.bin]);
      tree.gain[node]        = nb.gain;
      tree.split_bin[node]   = nb.bin - row_ptr[bf];
    }
  }
}

// What a rank knows about its best split of a node when the features are divided among the ranks:
// the candidate and the sums left of it; K pairs follow the header.
struct SplitRecordHeader {
  double gain;
  int bin;
  int pad;
};
__host__ __device__ inline size_t SplitRecordBytes(int K) { return sizeof(SplitRecordHeader) + sizeof(GPairI64) * K; }

// grid = (nodes, slices): a block evaluates one slice of the node's bins (all of them when there is
// one slice).  With several slices every block leaves its best candidate in `slice_best`, and the
// block that arrives last (a counter per node, zeroed once per tree) picks the winner and writes
// the tree.  Better() is a total order, so the winner does not depend on how the bins were cut.
template <typename T>
__global__ void __launch_bounds__(kSplitThreads)
  k_best_split(const GPairI64* __restrict__ level_hist, int node_begin, int K, int F, int B,
               const int32_t* __restrict__ row_ptr, const T* __restrict__ proposals,
               const QuantParams* __restrict__ qp_ptr, double l1, double l2, double msg,
               const uint8_t* __restrict__ feature_set, TreeArrays tree, SliceBest* __restrict__ slice_best,
               unsigned int* __restrict__ arrived, int f_begin, int f_end, unsigned char* __restrict__ records)
{
  const int j      = blockIdx.x;
  const int slices = gridDim.y;
  const int node   = node_begin + j;
  GPairI64* node_sums = tree.node_sums;
  if (LoadPair(node_sums + static_cast<int64_t>(node) * K).hess <= 0) return;
  const QuantParams qp = *qp_ptr;
  const GPairI64* hist = level_hist + static_cast<int64_t>(j) * K * B;
  __shared__ Cand s_c[kSplitThreads / 32];
  __shared__ Cand s_best;
  __shared__ bool s_last;
  const int tid = threadIdx.x;
  // the bins this rank evaluates (all of them unless the features are divided among the ranks)
  const int bin_begin = row_ptr[f_begin], bin_end = row_ptr[f_end];
  const int per = (bin_end - bin_begin + slices - 1) / slices;
  const int b0  = bin_begin + blockIdx.y * per, b1 = min(bin_end, b0 + per);
  Cand best{0.0, -1};
  for (int b = b0 + tid; b < b1; b += kSplitThreads) {
    if (feature_set) {
      int lo = 0, hi = F;  // last f with row_ptr[f] <= b
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (row_ptr[mid] <= b) lo = mid; else hi = mid;
      }
      if (!feature_set[lo]) continue;
    }
    double gain = 0;
    for (int k = 0; k < K; ++k) {
      const GPairI64 ns = LoadPair(node_sums + static_cast<int64_t>(node) * K + k);
      const GPairI64 ls = LoadPair(hist + static_cast<int64_t>(k) * B + b);
      const GPairI64 rs{ns.grad - ls.grad, ns.hess - ls.hess};
      if (ls.hess <= 0 || rs.hess <= 0) {
        gain = 0;
        break;
      }
      gain += CalculateGain(Dequantise(ls, qp), Dequantise(rs, qp), Dequantise(ns, qp), l1, l2, msg);
    }
    const Cand c{gain, b};
    if (gain > 0 && Better(c, best)) best = c;
  }
  auto warp_best = [&]() {
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
      Cand o;
      o.gain = __shfl_down_sync(0xffffffffu, best.gain, off);
      o.bin  = __shfl_down_sync(0xffffffffu, best.bin, off);
      if (Better(o, best)) best = o;
    }
  };
  auto block_best = [&]() {
    warp_best();
    if ((tid & 31) == 0) s_c[tid >> 5] = best;
    __syncthreads();
    if (tid == 0) {
      Cand w0 = s_c[0];
      for (int w = 1; w < kSplitThreads / 32; ++w)
        if (Better(s_c[w], w0)) w0 = s_c[w];
      s_best = w0;
    }
    __syncthreads();
  };
  block_best();
  if (slices > 1) {
    if (tid == 0) {
      SliceBest sb;
      sb.gain = s_best.gain;
      sb.bin  = s_best.bin;
      sb.pad  = 0;
      slice_best[static_cast<int64_t>(j) * slices + blockIdx.y] = sb;
      __threadfence();
      s_last = atomicAdd(arrived + node, 1u) == static_cast<unsigned>(slices - 1);
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    best = Cand{0.0, -1};
    for (int i = tid; i < slices; i += kSplitThreads) {
      const volatile SliceBest* sb = slice_best + static_cast<int64_t>(j) * slices + i;
      const Cand c{sb->gain, sb->bin};
      if (Better(c, best)) best = c;
    }
    __syncthreads();
    block_best();
  }
  const Cand nb = s_best;
  if (records != nullptr) {
    // leave the candidate and its left sums for the exchange among the ranks
    unsigned char* rec = records + static_cast<size_t>(j) * SplitRecordBytes(K);
    if (tid == 0) {
      SplitRecordHeader h;
      h.gain = nb.gain;
      h.bin  = nb.bin;
      h.pad  = 0;
      *reinterpret_cast<SplitRecordHeader*>(rec) = h;
    }
    GPairI64* ls = reinterpret_cast<GPairI64*>(rec + sizeof(SplitRecordHeader));
    for (int k = tid; k < K; k += kSplitThreads)
      StorePair(ls + k, nb.bin >= 0 ? LoadPair(hist + static_cast<int64_t>(k) * B + nb.bin) : GPairI64{0, 0});
    return;
  }
  ApplyWinner<T>(nb, node, K, F, row_ptr, proposals, qp, l1, l2, tree, nb.bin >= 0 ? hist + nb.bin : hist, B, tid,
                 kSplitThreads);
}

// One block per node: the best of the ranks' candidates (the same total order as inside a rank, so
// the winner is the one a single rank would have found over all features) becomes the tree.
template <typename T>
__global__ void __launch_bounds__(64)
  k_apply_records(const unsigned char* __restrict__ all_records, int n_ranks, int n_nodes, int node_begin, int K, int F,
                  const int32_t* __restrict__ row_ptr, const T* __restrict__ proposals,
                  const QuantParams* __restrict__ qp_ptr, double l1, double l2, TreeArrays tree)
{
  const int j    = blockIdx.x;
  const int node = node_begin + j;
  if (LoadPair(tree.node_sums + static_cast<int64_t>(node) * K).hess <= 0) return;
  const size_t rb = SplitRecordBytes(K);
  Cand best{0.0, -1};
  int best_rank = -1;
  for (int r = 0; r < n_ranks; ++r) {
    const SplitRecordHeader* h =
      reinterpret_cast<const SplitRecordHeader*>(all_records + (static_cast<size_t>(r) * n_nodes + j) * rb);
    const Cand c{h->gain, h->bin};
    if (c.gain > 0 && c.bin >= 0 && Better(c, best)) {
      best      = c;
      best_rank = r;
    }
  }
  if (best_rank < 0) return;
  const GPairI64* ls = reinterpret_cast<const GPairI64*>(
    all_records + (static_cast<size_t>(best_rank) * n_nodes + j) * rb + sizeof(SplitRecordHeader));
  ApplyWinner<T>(best, node, K, F, row_ptr, proposals, *qp_ptr, l1, l2, tree, ls, 1, threadIdx.x, blockDim.x);
}

__global__ void k_root_leaf(TreeArrays tree, int K, const QuantParams* __restrict__ qp_ptr, double l1, double l2)
{
  const int k = blockIdx.x * blockDim.x + threadIdx.x;
  if (k >= K) return;
  const GPairF64 s   = Dequantise(tree.node_sums[k], *qp_ptr);
  tree.leaf_value[k] = CalculateLeafValue(s.grad, s.hess, l1, l2);
}

__global__ void k_write_hessian(const GPairI64* __restrict__ node_sums, const QuantParams* __restrict__ qp_ptr,
                                double* __restrict__ hessian, int64_t n)
{
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < n) hessian[i] = static_cast<double>(node_sums[i].hess) * qp_ptr->inv_h;
}

}  // namespace

void PlanBuilt(const GPairI64* node_sums, int K, int node_begin, int n_nodes, bool parent_available,
               int32_t* slot_of_node, cudaStream_t stream)
{
  k_plan_built<<<(n_nodes + 255) / 256, 256, 0, stream>>>(node_sums, K, node_begin, n_nodes, parent_available,
                                                          slot_of_node);
  LBK_LAUNCH_CHECK();
}

void ScanLevel(const GPairI64* built, const int32_t* slot_of_node, GPairI64* level_hist, const GPairI64* parent_hist,
               int parent_begin, const GPairI64* node_sums, int node_begin, int n_nodes, int K, int f_begin, int f_end,
               int B, const int32_t* row_ptr, bool parent_available, cudaStream_t stream)
{
  const int n_features = f_end - f_begin;
  if (n_features <= 0 || n_nodes <= 0) return;
  const int64_t warps  = static_cast<int64_t>(n_nodes) * n_features;
  const int64_t blocks = (warps + 7) / 8;
  dim3 grid(static_cast<unsigned>(blocks), K);
  k_scan<<<grid, 256, 0, stream>>>(built, slot_of_node, level_hist, parent_hist, parent_begin, node_sums, node_begin,
                                   n_nodes, K, f_begin, n_features, B, row_ptr, parent_available);
  LBK_LAUNCH_CHECK();
}

template <typename T>
void BestSplit(lbk_context* ctx, Scratch& s, const GPairI64* level_hist, int node_begin, int n_nodes, int K, int F, int B,
               const int32_t* row_ptr, const T* proposals, const QuantParams* qp, const SplitParams& sp, TreeArrays tree,
               unsigned int* arrived, int f_begin, int f_end, bool exchange_records, cudaStream_t stream)
{
  const int sm_count = ctx->sm_count;
  // the bins of the features [f_begin, f_end): row_ptr lives on the device, so the kernel gets the
  // range through two small reads of its own; here only an upper bound of its length matters
  const int n_bins_bound = exchange_records ? (B + ctx->n_ranks - 1) / ctx->n_ranks + 1 : B;
  // enough blocks for two per SM, at least one thread per bin in a block's slice
  int slices = (2 * sm_count + n_nodes - 1) / n_nodes;
  const int most = (n_bins_bound + kSplitThreads - 1) / kSplitThreads;
  if (slices > most) slices = most;
  if (slices > kSplitThreads) slices = kSplitThreads;
  if (slices < 1) slices = 1;
  SliceBest* slice_best = slices > 1 ? s.alloc<SliceBest>(static_cast<size_t>(n_nodes) * slices) : nullptr;
  if (!exchange_records) {
    k_best_split<T><<<dim3(n_nodes, slices), kSplitThreads, 0, stream>>>(
      level_hist, node_begin, K, F, B, row_ptr, proposals, qp, sp.l1, sp.l2, sp.min_split_gain, sp.feature_set, tree,
      slice_best, arrived, f_begin, f_end, nullptr);
    LBK_LAUNCH_CHECK();
    if (slice_best) s.free_one(slice_best);
    return;
  }
  // every rank searches its own features, then the candidates of all ranks meet on every rank
  const size_t rb   = SplitRecordBytes(K);
  const int R       = ctx->n_ranks;
  unsigned char* mine = s.alloc<unsigned char>(rb * n_nodes);
  unsigned char* all  = s.alloc<unsigned char>(rb * n_nodes * R);
  LBK_CUDA(cudaMemsetAsync(mine, 0, rb * n_nodes, stream));
  k_best_split<T><<<dim3(n_nodes, slices), kSplitThreads, 0, stream>>>(
    level_hist, node_begin, K, F, B, row_ptr, proposals, qp, sp.l1, sp.l2, sp.min_split_gain, sp.feature_set, tree,
    slice_best, arrived, f_begin, f_end, mine);
  LBK_LAUNCH_CHECK();
  if (!AllGatherBytes(ctx, mine, all, rb * n_nodes, stream))
    throw Error(LBK_ERR_COMM, "the split records need an NCCL communicator");
  k_apply_records<T><<<n_nodes, 64, 0, stream>>>(all, R, n_nodes, node_begin, K, F, row_ptr, proposals, qp, sp.l1, sp.l2,
                                                  tree);
  LBK_LAUNCH_CHECK();
  if (slice_best) s.free_one(slice_best);
  s.free_one(mine);
  s.free_one(all);
}

void RootLeaf(TreeArrays tree, int K, const QuantParams* qp, double l1, double l2, cudaStream_t stream)
{
  k_root_leaf<<<(K + 127) / 128, 128, 0, stream>>>(tree, K, qp, l1, l2);
  LBK_LAUNCH_CHECK();
}

void WriteHessian(const GPairI64* node_sums, const QuantParams* qp, double* hessian, int64_t n, cudaStream_t stream)
{
  k_write_hessian<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(node_sums, qp, hessian, n);
  LBK_LAUNCH_CHECK();
}

template void BestSplit<float>(lbk_context*, Scratch&, const GPairI64*, int, int, int, int, int, const int32_t*,
                               const float*, const QuantParams*, const SplitParams&, TreeArrays, unsigned int*, int, int,
                               bool, cudaStream_t);
template void BestSplit<double>(lbk_context*, Scratch&, const GPairI64*, int, int, int, int, int, const int32_t*,
                                const double*, const QuantParams*, const SplitParams&, TreeArrays, unsigned int*, int, int,
                                bool, cudaStream_t);

}  // namespace lbk
