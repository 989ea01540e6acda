// lbk_build_tree and the stage-level entry points: host-side orchestration of one tree.
//
// Reference behaviour restated here: build_tree_fn / TreeBuilder, src/models/tree/build_tree.cu:
//   :1274-1359 task body (argument checks, level loop), :1000-1017 histogram cache rule,
//   :1191-1258 batching of a level when its histograms exceed the cache, :1154-1187 root,
//   :826-845 outputs.
// Differences in how, not in what: bins and quantised pairs are computed once per tree; rows are
// kept grouped by node with a stable partition instead of a radix sort; only the nodes that are
// built are held in the reduction buffer that crosses ranks; the whole level loop is enqueued
// without host synchronisation (the only synchronisation of a call is the read-back of the
// number of bins after the split proposals, which sizes the histograms).
#include <algorithm>
#include <cstring>

#include "internal.h"

namespace lbk {
namespace {

// The node each row ends in, read off the binned matrix: "x <= split value" is "bin <= split bin"
// because a split value is one of the feature's proposals (the repartition relies on the same
// fact), so this is the walk the predict kernel does on X, on a quarter of the bytes (float32 X).
//
// Tiled form (rows of at most kLeafMaxPitch bytes, at most kLeafMaxNodes nodes): the load/store
// pipe spends one pass per distinct 128-byte line of a load, so a thread per row reading its own
// line costs 32 passes per level.  Instead a warp copies its 32 consecutive rows - one contiguous
// piece of the matrix - into shared memory with 16-byte loads (the shared rows are one word longer,
// which spreads equal features of the 32 rows over the banks), and the tree's nodes sit in shared
// memory too, feature + 1 and split bin packed into one word.
constexpr int kLeafMaxPitch = 256;
constexpr int kLeafMaxNodes = 8192;
constexpr int kLeafWarps    = 8;

template <typename BinT>
__global__ void __launch_bounds__(kLeafWarps * 32)
  k_leaf_of_row_tiled(const BinT* __restrict__ bins, int pitch_bytes, int64_t n_rows, const int32_t* __restrict__ feature,
                      const int32_t* __restrict__ split_bin, int max_depth, int n_nodes, int32_t* __restrict__ leaf)
{
  extern __shared__ __align__(16) unsigned char smem_raw[];
  unsigned* s_node = reinterpret_cast<unsigned*>(smem_raw);
  for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) {
    const int f = feature[i];
    s_node[i]   = f < 0 ? 0u : (static_cast<unsigned>(f + 1) << 16) | static_cast<unsigned>(split_bin[i] & 0xffff);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int spitch = pitch_bytes + 4;  // bytes of a row in shared memory
  unsigned char* tile = smem_raw + (static_cast<size_t>(n_nodes) * 4 + 15) / 16 * 16 + static_cast<size_t>(warp) * 32 * spitch;
  const int vec_per_row  = pitch_bytes / 16;
  const int64_t n_chunks = (n_rows + 31) / 32;
  for (int64_t chunk = blockIdx.x * static_cast<int64_t>(kLeafWarps) + warp; chunk < n_chunks;
       chunk += static_cast<int64_t>(gridDim.x) * kLeafWarps) {
    const int64_t row0 = chunk * 32;
    const int rows     = static_cast<int>(n_rows - row0 < 32 ? n_rows - row0 : 32);
    const uint4* src   = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(bins) + row0 * pitch_bytes);
    const int n_vec    = rows * vec_per_row;
    __syncwarp();  // the previous chunk's walks are done with the tile
    for (int v = lane; v < n_vec; v += 32) {
      const uint4 w = __ldcs(src + v);
      const int r = v / vec_per_row, c = v - r * vec_per_row;
      unsigned* dst = reinterpret_cast<unsigned*>(tile + r * spitch + c * 16);
      dst[0] = w.x;
      dst[1] = w.y;
      dst[2] = w.z;
      dst[3] = w.w;
    }
    __syncwarp();
    if (lane < rows) {
      const BinT* b = reinterpret_cast<const BinT*>(tile + lane * spitch);
      int node      = 0;
      for (int d = 0; d < max_depth; ++d) {
        // a node without children in the arrays is a leaf (its feature is -1 by construction)
        const unsigned nd = node < n_nodes ? s_node[node] : 0u;
        if (nd == 0u) break;
        node = 2 * node + 1 + (static_cast<unsigned>(b[(nd >> 16) - 1]) > (nd & 0xffffu) ? 1 : 0);
      }
      leaf[row0 + lane] = node;
    }
  }
}

// One thread per row, everything from global memory: wide rows and very deep trees.
template <typename BinT>
__global__ void __launch_bounds__(256)
  k_leaf_of_row(const BinT* __restrict__ bins, int64_t pitch, int64_t n_rows, const int32_t* __restrict__ feature,
                const int32_t* __restrict__ split_bin, int max_depth, int32_t* __restrict__ leaf)
{
  const int64_t row = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (row >= n_rows) return;
  const BinT* b = bins + row * pitch;
  int node      = 0;
  for (int d = 0; d < max_depth; ++d) {
    const int f = __ldg(feature + node);
    if (f < 0) break;
    node = 2 * node + 1 + (static_cast<int>(b[f]) > __ldg(split_bin + node) ? 1 : 0);
  }
  leaf[row] = node;
}

template <typename BinT>
void LeafOfRow(lbk_context* ctx, const void* bins, int64_t pitch, int64_t N, int F, const int32_t* feature,
               const int32_t* split_bin, int D, int M, int32_t* leaf, cudaStream_t stream)
{
  const int64_t pitch_bytes = pitch * static_cast<int64_t>(sizeof(BinT));
  const bool aligned        = (reinterpret_cast<uintptr_t>(bins) & 15) == 0;
  if (pitch_bytes <= kLeafMaxPitch && M <= kLeafMaxNodes && F < 65535 && aligned) {
    const size_t smem = (static_cast<size_t>(M) * 4 + 15) / 16 * 16 + static_cast<size_t>(kLeafWarps) * 32 * (pitch_bytes + 4);
    auto fn           = k_leaf_of_row_tiled<BinT>;
    if (smem > 48 * 1024)
      LBK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    int per_sm = 0;
    LBK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kLeafWarps * 32, smem));
    const int64_t chunks = (N + 31) / 32;
    int64_t blocks       = static_cast<int64_t>(ctx->sm_count) * (per_sm > 0 ? per_sm : 1);
    blocks               = std::min<int64_t>(blocks, (chunks + kLeafWarps - 1) / kLeafWarps);
    fn<<<static_cast<unsigned>(std::max<int64_t>(blocks, 1)), kLeafWarps * 32, smem, stream>>>(
      static_cast<const BinT*>(bins), static_cast<int>(pitch_bytes), N, feature, split_bin, D, M, leaf);
  } else {
    const unsigned blocks = static_cast<unsigned>((N + 255) / 256);
    k_leaf_of_row<BinT><<<blocks, 256, 0, stream>>>(static_cast<const BinT*>(bins), pitch, N, feature, split_bin, D, leaf);
  }
  LBK_LAUNCH_CHECK();
}

// out[i, :] = table[index[i], :]: the leaf values of the nodes a set of rows ended in.
__global__ void __launch_bounds__(256)
  k_gather_rows(const double* __restrict__ table, const int32_t* __restrict__ index, int64_t n, int K,
                double* __restrict__ out)
{
  const int64_t e = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (e >= n * K) return;
  const int64_t i = e / K;
  const int k     = static_cast<int>(e - i * K);
  out[e]          = __ldg(table + static_cast<int64_t>(__ldg(index + i)) * K + k);
}

// The caller's sketch buffer: a header, then the split proposals, their row pointers, the binned
// matrix and its feature-major copy, each on a 512-byte boundary and sized for the widest case
// (two-byte bins when a feature can have more than 256 proposals).
constexpr int32_t kSketchMagic = 0x4c424b53;
struct SketchHeader {
  int32_t magic, total_bins, max_bins_per_feature, n_features, split_samples, elem_bytes, has_feature_major, pad;
  int64_t n_rows;
};
struct SketchLayout {
  size_t proposals, row_ptr, bins, bins_t, bytes;
};
SketchLayout SketchLayoutOf(int64_t N, int F, int S, size_t elem_bytes)
{
  auto up = [](size_t v) { return (v + 511) / 512 * 512; };
  const int bin_bytes   = S <= 256 ? 1 : 2;
  const int64_t pitch_t = (N + 31) / 32 * 32;
  SketchLayout l;
  l.proposals = up(sizeof(SketchHeader));
  l.row_ptr   = l.proposals + up(static_cast<size_t>(F) * S * elem_bytes);
  l.bins      = l.row_ptr + up(sizeof(int32_t) * (static_cast<size_t>(F) + 1));
  l.bins_t    = l.bins + up(lbk_bin_matrix_bytes(N, F, bin_bytes));
  l.bytes     = l.bins_t + up(static_cast<size_t>(F) * pitch_t * bin_bytes + 16);
  return l;
}

template <typename T>
void BuildTreeImpl(lbk_context* ctx, const lbk_build_tree_args& a, cudaStream_t stream)
{
  const int F = a.n_features, K = a.n_outputs, D = a.max_depth;
  const int64_t N = a.n_local_rows;
  const int M     = a.max_nodes;
  Scratch s(ctx, stream);

  const T* X      = static_cast<const T*>(a.X);
  const double* g = a.g;
  const double* h = a.h;
  const uint8_t* fset = a.feature_set;
  int64_t ldx = a.ldx, ldg = a.ldg;
  double *leaf_value = a.leaf_value, *split_value = a.split_value, *gain = a.gain, *hessian = a.hessian;
  int32_t* feature = a.feature;
  if (a.host_buffers) {
    // stage host inputs; outputs are produced on the device and copied back at the end
    T* dX = s.alloc<T>(static_cast<size_t>(N) * F);
    LBK_CUDA(cudaMemcpy2DAsync(dX, sizeof(T) * F, X, sizeof(T) * ldx, sizeof(T) * F, N > 0 ? N : 0, cudaMemcpyHostToDevice, stream));
    double* dg = s.alloc<double>(static_cast<size_t>(N) * K);
    double* dh = s.alloc<double>(static_cast<size_t>(N) * K);
    LBK_CUDA(cudaMemcpy2DAsync(dg, sizeof(double) * K, g, sizeof(double) * ldg, sizeof(double) * K, N > 0 ? N : 0, cudaMemcpyHostToDevice, stream));
    LBK_CUDA(cudaMemcpy2DAsync(dh, sizeof(double) * K, h, sizeof(double) * ldg, sizeof(double) * K, N > 0 ? N : 0, cudaMemcpyHostToDevice, stream));
    X   = dX;
    g   = dg;
    h   = dh;
    ldx = F;
    ldg = K;
    if (fset) {
      uint8_t* df = s.alloc<uint8_t>(F);
      LBK_CUDA(cudaMemcpyAsync(df, fset, F, cudaMemcpyHostToDevice, stream));
      fset = df;
    }
    leaf_value  = s.alloc<double>(static_cast<size_t>(M) * K);
    hessian     = s.alloc<double>(static_cast<size_t>(M) * K);
    split_value = s.alloc<double>(M);
    gain        = s.alloc<double>(M);
    feature     = s.alloc<int32_t>(M);
  }

  // Tree (reference: struct Tree, build_tree.cu:785-809)
  TreeArrays tree;
  tree.leaf_value  = leaf_value;
  tree.feature     = feature;
  tree.split_value = split_value;
  tree.gain        = gain;
  tree.node_sums   = s.alloc<GPairI64>(static_cast<size_t>(M) * K);
  tree.split_bin   = s.alloc<int32_t>(M);
  tree.max_nodes   = M;
  LBK_CUDA(cudaMemsetAsync(leaf_value, 0, sizeof(double) * M * K, stream));
  LBK_CUDA(cudaMemsetAsync(feature, 0xFF, sizeof(int32_t) * M, stream));
  LBK_CUDA(cudaMemsetAsync(split_value, 0, sizeof(double) * M, stream));
  LBK_CUDA(cudaMemsetAsync(gain, 0, sizeof(double) * M, stream));
  LBK_CUDA(cudaMemsetAsync(tree.node_sums, 0, sizeof(GPairI64) * M * K, stream));
  unsigned int* split_arrived = s.alloc<unsigned int>(M);  // see BestSplit
  LBK_CUDA(cudaMemsetAsync(split_arrived, 0, sizeof(unsigned int) * M, stream));

  // split proposals -> B (one host synchronisation); with a sketch buffer they and the binned
  // matrix live in the caller's buffer and may come from an earlier call
  const bool sketch_save = a.sketch_mode == LBK_SKETCH_SAVE, sketch_reuse = a.sketch_mode == LBK_SKETCH_REUSE;
  const SketchLayout sk  = SketchLayoutOf(N, F, a.split_samples, sizeof(T));
  unsigned char* skb     = static_cast<unsigned char*>(a.sketch);
  const bool in_sketch   = sketch_save || sketch_reuse;
  T* proposals     = in_sketch ? reinterpret_cast<T*>(skb + sk.proposals) : s.alloc<T>(static_cast<size_t>(F) * a.split_samples);
  int32_t* row_ptr = in_sketch ? reinterpret_cast<int32_t*>(skb + sk.row_ptr) : s.alloc<int32_t>(F + 1);
  ProposalInfo pi;
  SketchHeader head{};
  if (sketch_reuse) {
    LBK_CUDA(cudaMemcpyAsync(&head, skb, sizeof(head), cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaStreamSynchronize(stream));
    LBK_EXPECT(head.magic == kSketchMagic, "the sketch buffer holds no saved sketch");
    LBK_EXPECT(head.n_rows == N && head.n_features == F && head.split_samples == a.split_samples &&
                 head.elem_bytes == static_cast<int32_t>(sizeof(T)),
               "the sketch was saved for a matrix of another shape or type");
    LBK_EXPECT(D <= 1 || head.has_feature_major, "the sketch was saved without the feature-major copy");
    pi.total_bins           = head.total_bins;
    pi.max_bins_per_feature = head.max_bins_per_feature;
  } else {
    pi = SplitProposals<T>(ctx, s, X, ldx, a.row_offset, N, F, a.split_samples, a.seed, a.dataset_rows, proposals,
                           row_ptr, stream);
  }
  const int B = pi.total_bins;
  if (a.out_total_bins) *a.out_total_bins = B;
  LBK_EXPECT(B >= F, "every feature must have at least one proposal");

  // binned matrix, once per tree
  const int bin_bytes = pi.max_bins_per_feature <= 256 ? 1 : 2;
  void* bins          = in_sketch ? static_cast<void*>(skb + sk.bins) : s.alloc_bytes(lbk_bin_matrix_bytes(N, F, bin_bytes));
  // feature-major copy for the repartition (no copy for a stump: nothing is repartitioned; a saved
  // sketch always has it, later trees may be deeper)
  const int64_t pitch_t = (N + 31) / 32 * 32;
  void* bins_t          = in_sketch ? static_cast<void*>(skb + sk.bins_t)
                          : D > 1   ? s.alloc_bytes(static_cast<size_t>(F) * pitch_t * bin_bytes + 16)
                                    : nullptr;
  if (!sketch_reuse)
    BinMatrix<T>(X, ldx, N, F, proposals, row_ptr, bins, bins_t, pitch_t, bin_bytes, pi.max_bins_per_feature, stream);
  if (sketch_save) {
    head.magic                = kSketchMagic;
    head.total_bins           = pi.total_bins;
    head.max_bins_per_feature = pi.max_bins_per_feature;
    head.n_features           = F;
    head.split_samples        = a.split_samples;
    head.elem_bytes           = static_cast<int32_t>(sizeof(T));
    head.has_feature_major    = 1;
    head.n_rows               = N;
    LBK_CUDA(cudaMemcpyAsync(skb, &head, sizeof(head), cudaMemcpyHostToDevice, stream));
    LBK_CUDA(cudaStreamSynchronize(stream));  // `head` is on this frame
  }

  // quantised pairs and root sums
  QuantParams* qp = s.alloc<QuantParams>(1);
  int2* gpair     = s.alloc<int2>(static_cast<size_t>(N) * K);
  int* max_abs    = s.alloc<int>(2);
  Quantise(ctx, s, g, h, ldg, a.row_offset, N, K, a.seed, gpair, tree.node_sums, qp, max_abs, stream);
  RootLeaf(tree, K, qp, a.l1_regularization, a.l2_regularization, stream);

  // histogram cache rule (reference: build_tree.cu:1000-1017); identical on every rank
  const size_t bytes_per_node      = static_cast<size_t>(K) * B * sizeof(GPairI64);
  const size_t max_histogram_nodes = std::max<size_t>(1, size_t{1000000000} / bytes_per_node);
  int cdepth                       = 0;
  while (static_cast<size_t>(LevelEnd(cdepth + 1)) <= max_histogram_nodes && cdepth <= D) cdepth++;
  // levels >= D are never evaluated; no need to hold them
  const int cache_levels  = std::min(cdepth, std::max(D - 1, 0));
  const int cache_nodes   = LevelEnd(cache_levels);
  const int cache_end_ref = LevelEnd(cdepth);  // extent of the reference's cached histogram
  const int64_t max_batch = static_cast<int>(max_histogram_nodes);
  const size_t node_elems = static_cast<size_t>(K) * B;
  GPairI64* cache         = s.alloc<GPairI64>(static_cast<size_t>(cache_nodes) * node_elems);

  // rows grouped by node, ping-pong
  int32_t* rows_a = s.alloc<int32_t>(N);
  int32_t* rows_b = s.alloc<int32_t>(N);
  const size_t max_level_nodes = D > 0 ? (size_t{1} << (D - 1)) : 1;
  int32_t* seg_a  = s.alloc<int32_t>(2 * max_level_nodes + 2);
  int32_t* seg_b  = s.alloc<int32_t>(2 * max_level_nodes + 2);
  InitRows(rows_a, seg_a, N, stream);
  // With few outputs the quantised pairs are kept in row_index order: at the root that is the order
  // they are in already, and every repartition moves them together with the row ids (8 K bytes read
  // and written per row and level, as streams), so that the histogram kernel reads the pairs of a
  // node as a stream instead of gathering 8 bytes per row from all over the array.
  constexpr int kMaxStreamedOutputs = 4;
  const bool stream_pairs = K <= kMaxStreamedOutputs && D > 0;
  int2* pairs_a = gpair;
  int2* pairs_b = stream_pairs && D > 1 ? s.alloc<int2>(static_cast<size_t>(N) * K) : nullptr;

  SplitParams sp{a.l1_regularization, a.l2_regularization, a.min_split_gain, fset};

  // reduction buffer for the built nodes of a batch; grown on demand
  GPairI64* built    = nullptr;
  size_t built_nodes = 0;
  GPairI64* fresh    = nullptr;  // histogram of a batch that lies outside the cache
  size_t fresh_nodes = 0;
  // the most recently replaced "cache" of the reference, to decide parent availability
  int ref_hist_begin = 0, ref_hist_end = cache_end_ref;

  // the exchange buffers of a multi-rank call, sized once for the largest batch of the tree (the
  // receive form needs up to twice a batch: see BuildHistogramSummed)
  const size_t exchange_bytes =
    2 * sizeof(GPairI64) * node_elems * static_cast<size_t>(std::min<int64_t>(max_batch, static_cast<int64_t>(max_level_nodes))) +
    (size_t{1} << 20);

  for (int depth = 0; depth < D; ++depth) {
    const int level_begin = LevelBegin(depth), level_end = LevelEnd(depth);
    const int level_nodes = level_end - level_begin;
    // batches (reference: PrepareBatches, :1207-1258)
    std::vector<std::pair<int, int>> batches;
    if (level_nodes <= max_batch) {
      batches.push_back({level_begin, level_end});
    } else {
      const int64_t nb = (level_nodes + max_batch - 1) / max_batch;
      for (int64_t b = 0; b < nb; ++b) {
        const int64_t bb = level_begin + b * max_batch;
        batches.push_back({static_cast<int>(bb), static_cast<int>(std::min<int64_t>(bb + max_batch, level_end))});
      }
    }
    for (auto [nb, ne] : batches) {
      const int n_nodes = ne - nb;
      // GetHistogram (:1191-1205): a batch outside the current histogram replaces it
      const bool in_ref_hist = nb >= ref_hist_begin && ne <= ref_hist_end;
      if (!in_ref_hist) {
        ref_hist_begin = nb;
        ref_hist_end   = ne;
      }
      const bool parent_available = nb > 0 && ((nb - 1) / 2) >= ref_hist_begin && ((nb - 1) / 2) < ref_hist_end;
      const bool in_cache         = ne <= cache_nodes;
      // where this batch's histograms live
      GPairI64* level_hist;
      if (in_cache) {
        level_hist = cache + static_cast<size_t>(nb) * node_elems;
      } else {
        if (fresh_nodes < static_cast<size_t>(n_nodes)) {
          if (fresh) s.free_one(fresh);
          fresh       = s.alloc<GPairI64>(static_cast<size_t>(n_nodes) * node_elems);
          fresh_nodes = n_nodes;
        }
        level_hist = fresh;
      }
      const int n_slots = (parent_available && nb > 0) ? n_nodes / 2 : n_nodes;
      // With several ranks the level is built into a buffer the other ranks' GPUs can read, and
      // every rank sums, scans and searches only the features it owns (see exchange.cu); where the
      // peers cannot be mapped the whole buffer is all-reduced and every rank does everything.
      const bool owned = ctx->n_ranks > 1 && EnsureExchange(ctx, exchange_bytes, stream);
      const int f_begin = owned ? OwnedBegin(ctx->rank, ctx->n_ranks, F) : 0;
      const int f_end   = owned ? OwnedBegin(ctx->rank + 1, ctx->n_ranks, F) : F;
      // built buffer: when nothing is derived the level histogram itself is the target
      GPairI64* target;
      if (n_slots == n_nodes) {
        target = level_hist;
      } else {
        if (built_nodes < static_cast<size_t>(n_slots)) {
          if (built) s.free_one(built);
          built       = s.alloc<GPairI64>(static_cast<size_t>(n_slots) * node_elems);
          built_nodes = n_slots;
        }
        target = built;
        LBK_CUDA(cudaMemsetAsync(level_hist, 0, sizeof(GPairI64) * n_nodes * node_elems, stream));
      }
      // (the build zeroes the target where it needs it zeroed)

      int32_t* slot_of_node = s.alloc<int32_t>(n_nodes);
      PlanBuilt(tree.node_sums, K, nb, n_nodes, parent_available, slot_of_node, stream);

      HistLevel lv;
      lv.bins                 = bins;
      lv.bin_bytes            = bin_bytes;
      lv.n_rows               = N;
      lv.F                    = F;
      lv.K                    = K;
      lv.B                    = B;
      lv.max_bins_per_feature = pi.max_bins_per_feature;
      lv.row_ptr              = row_ptr;
      lv.gpair                = stream_pairs ? pairs_a : gpair;
      lv.pairs_by_position    = stream_pairs;
      lv.gpair_f              = nullptr;
      lv.max_abs              = max_abs;
      lv.row_index            = rows_a;
      lv.seg                  = seg_a;
      lv.n_nodes              = n_nodes;
      lv.seg_node_offset      = nb - level_begin;
      lv.slot_of_node         = slot_of_node;
      lv.out                  = target;
      lv.float_mode           = false;
      // build + sum over ranks (reference: :1107-1113 reduces the whole batch; only built nodes here)
      const GPairI64* summed = static_cast<const GPairI64*>(
        BuildHistogramSummed(ctx, s, lv, n_slots, HistSum::kSumOwned, false, true, stream));

      const GPairI64* parent_hist = nullptr;
      int parent_begin            = 0;
      if (parent_available) {
        parent_begin = LevelBegin(depth - 1);
        parent_hist  = cache + static_cast<size_t>(parent_begin) * node_elems;
      }
      ScanLevel(summed, slot_of_node, level_hist, parent_hist, parent_begin, tree.node_sums, nb, n_nodes, K, f_begin,
                f_end, B, row_ptr, parent_available, stream);
      if (a.trace_hist && nb < a.trace_nodes) {
        const int cnt = std::min(ne, a.trace_nodes) - nb;
        LBK_CUDA(cudaMemcpyAsync(a.trace_hist + static_cast<size_t>(nb) * node_elems * 2, level_hist,
                                 sizeof(GPairI64) * cnt * node_elems, cudaMemcpyDeviceToDevice, stream));
      }
      BestSplit<T>(ctx, s, level_hist, nb, n_nodes, K, F, B, row_ptr, proposals, qp, sp, tree, split_arrived, f_begin,
                   f_end, owned, stream);
      s.free_one(slot_of_node);
    }
    if (depth < D - 1) {
      PartitionLevel pl;
      pl.bins          = bins_t;
      pl.bin_bytes     = bin_bytes;
      pl.bin_pitch     = pitch_t;
      pl.n_rows        = N;
      pl.row_index_in  = rows_a;
      pl.seg_in        = seg_a;
      pl.row_index_out = rows_b;
      pl.seg_out       = seg_b;
      pl.node_begin    = level_begin;
      pl.n_nodes       = level_nodes;
      pl.feature       = tree.feature;
      pl.split_bin     = tree.split_bin;
      if (stream_pairs) {
        pl.pairs_in  = pairs_a;
        pl.pairs_out = pairs_b;
        pl.K         = K;
      }
      PartitionRows(ctx, s, pl, stream);
      std::swap(rows_a, rows_b);
      std::swap(seg_a, seg_b);
      std::swap(pairs_a, pairs_b);
    }
  }

  WriteHessian(tree.node_sums, qp, hessian, static_cast<int64_t>(M) * K, stream);
  if (a.out_leaf != nullptr && N > 0) {
    int32_t* d_leaf = a.host_buffers ? s.alloc<int32_t>(static_cast<size_t>(N)) : a.out_leaf;
    const int64_t pitch = static_cast<int64_t>((F + kGroup - 1) / kGroup) * kGroup;
    if (bin_bytes == 1) LeafOfRow<uint8_t>(ctx, bins, pitch, N, F, tree.feature, tree.split_bin, D, M, d_leaf, stream);
    else LeafOfRow<uint16_t>(ctx, bins, pitch, N, F, tree.feature, tree.split_bin, D, M, d_leaf, stream);
    if (a.host_buffers)
      LBK_CUDA(cudaMemcpyAsync(a.out_leaf, d_leaf, sizeof(int32_t) * N, cudaMemcpyDeviceToHost, stream));
  }
  if (a.trace_node_sums)
    LBK_CUDA(cudaMemcpyAsync(a.trace_node_sums, tree.node_sums, sizeof(GPairI64) * M * K, cudaMemcpyDeviceToDevice, stream));
  if (a.host_buffers) {
    LBK_CUDA(cudaMemcpyAsync(a.leaf_value, leaf_value, sizeof(double) * M * K, cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaMemcpyAsync(a.feature, feature, sizeof(int32_t) * M, cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaMemcpyAsync(a.split_value, split_value, sizeof(double) * M, cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaMemcpyAsync(a.gain, gain, sizeof(double) * M, cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaMemcpyAsync(a.hessian, hessian, sizeof(double) * M * K, cudaMemcpyDeviceToHost, stream));
  }
  CheckDeviceStatus(ctx, stream);  // synchronises, as the reference's task does (:1356)
}

}  // namespace
}  // namespace lbk

extern "C" {

size_t lbk_sketch_bytes(int64_t n_local_rows, int n_features, int split_samples, int x_dtype)
{
  if (n_local_rows < 0 || n_features < 1 || split_samples < 1) return 0;
  return lbk::SketchLayoutOf(n_local_rows, n_features, split_samples, x_dtype == LBK_F64 ? 8 : 4).bytes;
}

size_t lbk_bin_matrix_bytes(int64_t n_rows, int n_features, int bin_bytes)
{
  const int64_t G = (n_features + lbk::kGroup - 1) / lbk::kGroup;
  return static_cast<size_t>(G) * static_cast<size_t>(n_rows > 0 ? n_rows : 0) * lbk::kGroup * bin_bytes + 16;
}

int lbk_build_tree(lbk_context* ctx, const lbk_build_tree_args* a)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && a, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_EXPECT(a->x_dtype == LBK_F32 || a->x_dtype == LBK_F64, "X must be float32 or float64");
    LBK_EXPECT(a->n_features >= 1 && a->n_outputs >= 1, "need at least one feature and one output");
    LBK_EXPECT(a->n_local_rows >= 0 && a->n_local_rows < (int64_t{1} << 31), "rows per rank must fit 31 bits");
    LBK_EXPECT(a->dataset_rows >= 1, "dataset_rows must be positive");
    LBK_EXPECT(a->max_depth >= 0 && a->max_depth <= 29, "max_depth out of range");
    LBK_EXPECT(a->max_nodes == (1 << (a->max_depth + 1)) - 1, "max_nodes must be 2^(max_depth+1)-1");
    LBK_EXPECT(a->split_samples >= 1 && a->split_samples <= 2048, "split_samples must be in [1, 2048]");
    LBK_EXPECT(a->sketch_mode == LBK_SKETCH_OFF || a->sketch_mode == LBK_SKETCH_SAVE || a->sketch_mode == LBK_SKETCH_REUSE,
               "unknown sketch mode");
    LBK_EXPECT(a->sketch_mode == LBK_SKETCH_OFF || a->sketch != nullptr, "sketch mode without a sketch buffer");
    LBK_EXPECT(a->n_local_rows == 0 || ((a->X || a->sketch_mode == LBK_SKETCH_REUSE) && a->g && a->h), "null input");
    LBK_EXPECT(a->n_local_rows == 0 || (a->ldx >= a->n_features && a->ldg >= a->n_outputs), "Expected a dense row major store");
    LBK_EXPECT(a->leaf_value && a->feature && a->split_value && a->gain && a->hessian, "null output");
    LBK_EXPECT(a->row_offset >= 0 && a->row_offset + a->n_local_rows <= a->dataset_rows, "row range outside the data set");
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    if (a->x_dtype == LBK_F32)
      lbk::BuildTreeImpl<float>(ctx, *a, stream);
    else
      lbk::BuildTreeImpl<double>(ctx, *a, stream);
  });
}

int lbk_predict(lbk_context* ctx, const lbk_predict_args* a)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && a, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_EXPECT(a->x_dtype == LBK_F32 || a->x_dtype == LBK_F64, "X must be float32 or float64");
    if (a->n_rows < 1) return;
    LBK_EXPECT(a->X && a->pred, "null argument");
    LBK_EXPECT(a->n_features >= 1 && a->n_outputs >= 1 && a->n_trees >= 0, "bad shape");
    LBK_EXPECT(a->n_trees == 0 || (a->leaf_value && a->feature && a->split_value && a->max_nodes), "null tree arrays");
    LBK_EXPECT(a->ldx >= a->n_features && a->ldp >= a->n_outputs, "Expected a dense row major store");
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    lbk::Scratch s(ctx, stream);
    const int F = a->n_features, K = a->n_outputs;
    const int64_t N = a->n_rows;
    const void* X   = a->X;
    double* pred    = a->pred;
    int64_t ldx = a->ldx, ldp = a->ldp;
    std::vector<const double*> leaf(a->n_trees), split(a->n_trees);
    std::vector<const int32_t*> feat(a->n_trees);
    for (int t = 0; t < a->n_trees; ++t) {
      leaf[t]  = a->leaf_value[t];
      feat[t]  = a->feature[t];
      split[t] = a->split_value[t];
    }
    const size_t esz = a->x_dtype == LBK_F32 ? 4 : 8;
    if (a->host_buffers) {
      void* dX = s.alloc_bytes(esz * N * F);
      LBK_CUDA(cudaMemcpy2DAsync(dX, esz * F, X, esz * ldx, esz * F, N, cudaMemcpyHostToDevice, stream));
      X   = dX;
      ldx = F;
      pred = s.alloc<double>(static_cast<size_t>(N) * K);
      ldp  = K;
      for (int t = 0; t < a->n_trees; ++t) {
        const int m = a->max_nodes[t];
        double* dl  = s.alloc<double>(static_cast<size_t>(m) * K);
        double* ds  = s.alloc<double>(m);
        int32_t* df = s.alloc<int32_t>(m);
        LBK_CUDA(cudaMemcpyAsync(dl, leaf[t], sizeof(double) * m * K, cudaMemcpyHostToDevice, stream));
        LBK_CUDA(cudaMemcpyAsync(ds, split[t], sizeof(double) * m, cudaMemcpyHostToDevice, stream));
        LBK_CUDA(cudaMemcpyAsync(df, feat[t], sizeof(int32_t) * m, cudaMemcpyHostToDevice, stream));
        leaf[t]  = dl;
        split[t] = ds;
        feat[t]  = df;
      }
    }
    if (a->x_dtype == LBK_F32)
      lbk::PredictLaunch<float>(ctx, s, static_cast<const float*>(X), ldx, N, F, K, a->n_trees, leaf.data(), feat.data(),
                                split.data(), a->max_nodes, pred, ldp, stream);
    else
      lbk::PredictLaunch<double>(ctx, s, static_cast<const double*>(X), ldx, N, F, K, a->n_trees, leaf.data(),
                                 feat.data(), split.data(), a->max_nodes, pred, ldp, stream);
    if (a->host_buffers)
      LBK_CUDA(cudaMemcpy2DAsync(a->pred, sizeof(double) * a->ldp, pred, sizeof(double) * K, sizeof(double) * K, N,
                                 cudaMemcpyDeviceToHost, stream));
    lbk::CheckDeviceStatus(ctx, stream);
  });
}

int lbk_split_proposals(lbk_context* ctx, const void* X, int x_dtype, int64_t ldx, int64_t row_offset,
                        int64_t n_local_rows, int n_features, int split_samples, int seed, int64_t dataset_rows,
                        void* proposals, int32_t* row_ptr, int32_t* total_bins, void* stream_)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && proposals && row_ptr, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_EXPECT(x_dtype == LBK_F32 || x_dtype == LBK_F64, "X must be float32 or float64");
    LBK_EXPECT(split_samples >= 1 && split_samples <= 2048, "split_samples must be in [1, 2048]");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    lbk::Scratch s(ctx, stream);
    lbk::ProposalInfo pi;
    if (x_dtype == LBK_F32)
      pi = lbk::SplitProposals<float>(ctx, s, static_cast<const float*>(X), ldx, row_offset, n_local_rows, n_features,
                                      split_samples, seed, dataset_rows, static_cast<float*>(proposals), row_ptr, stream);
    else
      pi = lbk::SplitProposals<double>(ctx, s, static_cast<const double*>(X), ldx, row_offset, n_local_rows, n_features,
                                       split_samples, seed, dataset_rows, static_cast<double*>(proposals), row_ptr, stream);
    if (total_bins) *total_bins = pi.total_bins;
  });
}

int lbk_bin_matrix(lbk_context* ctx, const void* X, int x_dtype, int64_t ldx, int64_t n_rows, int n_features,
                   const void* proposals, const int32_t* row_ptr, void* bins, int bin_bytes, void* stream_)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && X && proposals && row_ptr && bins, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_EXPECT(bin_bytes == 1 || bin_bytes == 2, "bin_bytes must be 1 or 2");
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    // the largest feature decides whether the proposals of a feature group fit shared memory
    std::vector<int32_t> rp(n_features + 1);
    LBK_CUDA(cudaMemcpyAsync(rp.data(), row_ptr, sizeof(int32_t) * (n_features + 1), cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaStreamSynchronize(stream));
    int mb = 1;
    for (int f = 0; f < n_features; ++f) mb = std::max(mb, rp[f + 1] - rp[f]);
    LBK_EXPECT(bin_bytes == 2 || mb <= 256, "one-byte bins need <= 256 proposals per feature");
    if (x_dtype == LBK_F32)
      lbk::BinMatrix<float>(static_cast<const float*>(X), ldx, n_rows, n_features, static_cast<const float*>(proposals),
                            row_ptr, bins, nullptr, 0, bin_bytes, mb, stream);
    else
      lbk::BinMatrix<double>(static_cast<const double*>(X), ldx, n_rows, n_features,
                             static_cast<const double*>(proposals), row_ptr, bins, nullptr, 0, bin_bytes, mb, stream);
  });
}

int lbk_quantise(lbk_context* ctx, const double* g, const double* h, int64_t ldg, int64_t row_offset,
                 int64_t n_local_rows, int n_outputs, int seed, int32_t* gpair, int64_t* root_sums, double* scale,
                 int32_t* max_abs, void* stream_)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && gpair && root_sums && scale, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    lbk::Scratch s(ctx, stream);
    lbk::Quantise(ctx, s, g, h, ldg, row_offset, n_local_rows, n_outputs, seed, reinterpret_cast<int2*>(gpair),
                  reinterpret_cast<lbk::GPairI64*>(root_sums), reinterpret_cast<lbk::QuantParams*>(scale),
                  max_abs ? max_abs : s.alloc<int>(2), stream);
  });
}

int lbk_histogram(lbk_context* ctx, const lbk_histogram_args* a)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && a, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_EXPECT(a->bins && a->row_ptr && a->row_index && a->seg && a->hist, "null argument");
    LBK_EXPECT(a->mode == 0 || a->mode == 1, "mode must be 0 or 1");
    LBK_EXPECT(a->mode == 0 ? a->gpair != nullptr : a->gpair_f32 != nullptr, "missing gradient pairs");
    LBK_EXPECT(a->bin_bytes == 1 || a->bin_bytes == 2, "bin_bytes must be 1 or 2");
    LBK_EXPECT(a->n_nodes >= 1 && a->n_features >= 1 && a->n_outputs >= 1 && a->total_bins >= a->n_features, "bad shape");
    LBK_EXPECT(a->all_reduce >= 0 && a->all_reduce <= 2, "all_reduce must be 0, 1 or 2");
    LBK_EXPECT(!a->pairs_by_position || !a->host_buffers, "pairs stored by position are for device buffers");
    LBK_EXPECT(!a->pairs_by_position || a->mode == 1 || a->max_abs != nullptr,
               "pairs stored by position need max_abs (the library cannot know how many entries the array has)");
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    lbk::Scratch s(ctx, stream);
    const int F = a->n_features, K = a->n_outputs, B = a->total_bins;
    const int64_t N = a->n_rows;
    const void* bins         = a->bins;
    const int32_t* row_ptr   = a->row_ptr;
    const void* gp           = a->mode == 0 ? static_cast<const void*>(a->gpair) : static_cast<const void*>(a->gpair_f32);
    const int32_t* row_index = a->row_index;
    const int32_t* seg       = a->seg;
    void* hist               = a->hist;
    const size_t hist_bytes  = sizeof(lbk::GPairI64) * a->n_nodes * K * B;
    std::vector<int32_t> rp(F + 1);
    if (a->host_buffers) {
      std::memcpy(rp.data(), a->row_ptr, sizeof(int32_t) * (F + 1));
      const int32_t n_idx = a->seg[a->n_nodes];
      const size_t bb     = lbk_bin_matrix_bytes(N, F, a->bin_bytes) - 16;
      void* d_bins        = s.alloc_bytes(bb + 16);
      int32_t* d_rp       = s.alloc<int32_t>(F + 1);
      void* d_gp          = s.alloc_bytes(sizeof(int2) * N * K);
      int32_t* d_idx      = s.alloc<int32_t>(n_idx);
      int32_t* d_seg      = s.alloc<int32_t>(a->n_nodes + 1);
      void* d_hist        = s.alloc_bytes(hist_bytes);
      LBK_CUDA(cudaMemcpyAsync(d_bins, bins, bb, cudaMemcpyHostToDevice, stream));
      LBK_CUDA(cudaMemcpyAsync(d_rp, row_ptr, sizeof(int32_t) * (F + 1), cudaMemcpyHostToDevice, stream));
      LBK_CUDA(cudaMemcpyAsync(d_gp, gp, sizeof(int2) * N * K, cudaMemcpyHostToDevice, stream));
      LBK_CUDA(cudaMemcpyAsync(d_idx, row_index, sizeof(int32_t) * n_idx, cudaMemcpyHostToDevice, stream));
      LBK_CUDA(cudaMemcpyAsync(d_seg, seg, sizeof(int32_t) * (a->n_nodes + 1), cudaMemcpyHostToDevice, stream));
      bins = d_bins; row_ptr = d_rp; gp = d_gp; row_index = d_idx; seg = d_seg; hist = d_hist;
    } else if (a->max_bins <= 0) {
      LBK_CUDA(cudaMemcpyAsync(rp.data(), row_ptr, sizeof(int32_t) * (F + 1), cudaMemcpyDeviceToHost, stream));
      LBK_CUDA(cudaStreamSynchronize(stream));
    }
    int mb = 1;
    if (!a->host_buffers && a->max_bins > 0) {
      mb = a->max_bins;  // the caller vouches for it: row_ptr stays on the device, no wait before the launch
    } else {
      LBK_EXPECT(rp[F] == B, "total_bins does not match row_ptr");
      for (int f = 0; f < F; ++f) mb = std::max(mb, rp[f + 1] - rp[f]);
    }
    LBK_EXPECT(a->bin_bytes == 2 || mb <= 256, "one-byte bins need <= 256 proposals per feature");
    // (the summed forms zero what they need themselves; the staging copy of a host buffer is fresh
    // scratch and must not return what it held before)
    if (a->all_reduce == 0 || a->host_buffers) LBK_CUDA(cudaMemsetAsync(hist, 0, hist_bytes, stream));
    lbk::HistLevel lv;
    lv.bins                 = bins;
    lv.bin_bytes            = a->bin_bytes;
    lv.n_rows               = N;
    lv.F                    = F;
    lv.K                    = K;
    lv.B                    = B;
    lv.max_bins_per_feature = mb;
    lv.row_ptr              = row_ptr;
    lv.gpair                = a->mode == 0 ? static_cast<const int2*>(gp) : nullptr;
    lv.gpair_f              = a->mode == 1 ? static_cast<const float2*>(gp) : nullptr;
    lv.max_abs              = a->host_buffers ? nullptr : reinterpret_cast<const int*>(a->max_abs);
    lv.pairs_by_position    = a->pairs_by_position != 0;
    lv.row_index            = row_index;
    lv.seg                  = seg;
    lv.n_nodes              = a->n_nodes;
    lv.seg_node_offset      = 0;
    lv.slot_of_node         = nullptr;
    lv.out                  = hist;
    lv.float_mode           = a->mode == 1;
    if (a->all_reduce == 1) lbk::BuildHistogramSummed(ctx, s, lv, a->n_nodes, lbk::HistSum::kSumEverywhere, true, true, stream);
    else if (a->all_reduce == 2) lbk::BuildHistogramSummed(ctx, s, lv, a->n_nodes, lbk::HistSum::kSumOwned, true, true, stream);
    else lbk::BuildHistogram(ctx, s, lv, stream);
    // host buffers: the histogram has to be back before the call returns; device buffers: the call
    // is one more piece of work on the caller's stream
    if (a->host_buffers) {
      LBK_CUDA(cudaMemcpyAsync(a->hist, hist, hist_bytes, cudaMemcpyDeviceToHost, stream));
      lbk::CheckDeviceStatus(ctx, stream);
    }
  });
}

int lbk_group_rows(lbk_context* ctx, const int32_t* node_of_row, int64_t n_rows, int node_begin, int n_nodes,
                   int32_t* row_index, int32_t* seg, void* stream_)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && node_of_row && row_index && seg, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    lbk::Scratch s(ctx, stream);
    lbk::GroupRows(ctx, s, node_of_row, n_rows, node_begin, n_nodes, row_index, seg, stream);
    LBK_CUDA(cudaStreamSynchronize(stream));
  });
}

int lbk_leaf_values(lbk_context* ctx, const double* leaf_value, const int32_t* leaf, int64_t n_rows, int n_outputs,
                    double* out, void* stream_)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "context is null");
    LBK_EXPECT(n_rows >= 0 && n_outputs >= 1, "bad shape");
    if (n_rows == 0) return;
    LBK_EXPECT(leaf_value && leaf && out, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream  = static_cast<cudaStream_t>(stream_);
    const int64_t total  = n_rows * n_outputs;
    const int64_t blocks = (total + 255) / 256;
    LBK_EXPECT(blocks <= 2147483647ll, "too many elements for one launch");
    lbk::k_gather_rows<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(leaf_value, leaf, n_rows, n_outputs, out);
    LBK_LAUNCH_CHECK();
  });
}

}  // extern "C"
