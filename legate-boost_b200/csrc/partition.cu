// Row-to-node repartition: after a level's splits are chosen, every split node's row segment is
// divided, stably, into the segments of its two children; rows of nodes that stay leaves drop out.
//
// Reference behaviour restated here: UpdatePositions, src/models/tree/build_tree.cu:1026-1080 -
// position := -1 for rows in leaves, else left child iff (double)x <= split_value, followed by a
// full radix sort of all (node,row) pairs by node.  Because a split value is one of the feature's
// proposals, "x <= split_value" is the same as "bin(x) <= bin(split)", so the decision needs one
// byte of the binned matrix instead of the raw feature value, and because the rows are already
// grouped by parent the sort reduces to a stable two-way partition inside each segment.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

constexpr int kPartThreads = 256;
constexpr int kPartItems   = 8;
constexpr int kPartTile    = kPartThreads * kPartItems;  // rows per chunk

__global__ void k_init_rows(int32_t* __restrict__ row_index, int32_t* __restrict__ seg, int64_t n_rows)
{
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < n_rows) row_index[i] = static_cast<int32_t>(i);
  if (i == 0) {
    seg[0] = 0;
    seg[1] = static_cast<int32_t>(n_rows);
  }
}

// Generic single-block exclusive scan helper: out[i+1] = sum_{j<=i} f(j), out[0] = 0.
template <typename F>
__device__ void BlockScanToArray(int n, F f, int32_t* out, int* carry_s, int* wsum)
{
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    *carry_s = 0;
    out[0]   = 0;
  }
  __syncthreads();
  for (int base = 0; base < n; base += blockDim.x) {
    const int i = base + tid;
    const int c = i < n ? f(i) : 0;
    int incl    = c;
    for (int off = 1; off < 32; off <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w  = lane < (blockDim.x >> 5) ? wsum[lane] : 0;
      int wi = w;
      for (int off = 1; off < 32; off <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += v;
      }
      wsum[lane] = wi - w;
    }
    __syncthreads();
    const int before = *carry_s + wsum[warp];
    if (i < n) out[i + 1] = before + incl;
    __syncthreads();
    if (tid == blockDim.x - 1) *carry_s = before + incl;
    __syncthreads();
  }
}

// chunk offsets of the split nodes of the level
__global__ void __launch_bounds__(1024)
  k_part_plan(const int32_t* __restrict__ seg, const int32_t* __restrict__ feature, int node_begin, int n_nodes,
              int32_t* __restrict__ chunk_off)
{
  __shared__ int carry, wsum[32];
  BlockScanToArray(
    n_nodes,
    [&](int j) {
      const int rows = seg[j + 1] - seg[j];
      return (feature[node_begin + j] != -1 && rows > 0) ? (rows + kPartTile - 1) / kPartTile : 0;
    },
    chunk_off, &carry, wsum);
}

__device__ inline int FindOwner(const int32_t* __restrict__ off, int n, int c)
{
  int lo = 0, hi = n;  // last j with off[j] <= c
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (off[mid] <= c) lo = mid; else hi = mid;
  }
  return lo;
}

// One block per chunk: every thread owns kPartItems consecutive rows; bit i of its mask says row
// i goes left.  Writes the masks and the chunk's left count.
template <typename BinT>
__global__ void __launch_bounds__(kPartThreads)
  k_part_count(const BinT* __restrict__ bins, int64_t pitch, const int32_t* __restrict__ row_index,
               const int32_t* __restrict__ seg, const int32_t* __restrict__ chunk_off, int n_nodes, int node_begin,
               const int32_t* __restrict__ feature, const int32_t* __restrict__ split_bin,
               uint8_t* __restrict__ masks, int32_t* __restrict__ chunk_left)
{
  const int c = blockIdx.x;
  if (c >= chunk_off[n_nodes]) return;
  const int j    = FindOwner(chunk_off, n_nodes, c);
  const int node = node_begin + j;
  const int f    = feature[node];
  const int sb   = split_bin[node];
  const int rb   = seg[j] + (c - chunk_off[j]) * kPartTile;
  const int re   = min(seg[j + 1], rb + kPartTile);
  const BinT* col = bins + static_cast<int64_t>(f) * pitch;  // feature-major copy: the rows of a node are neighbours
  const int tid  = threadIdx.x;
  const int r0   = rb + tid * kPartItems;
  unsigned mask  = 0;
#pragma unroll
  for (int i = 0; i < kPartItems; ++i) {
    const int r = r0 + i;
    if (r < re) {
      const int ridx = row_index[r];
      const int bin  = col[ridx];
      if (bin <= sb) mask |= 1u << i;
    }
  }
  masks[static_cast<int64_t>(c) * kPartThreads + tid] = static_cast<uint8_t>(mask);
  int cnt = __popc(mask);
  __shared__ int wsum[kPartThreads / 32];
  for (int off = 16; off >= 1; off >>= 1) cnt += __shfl_down_sync(0xffffffffu, cnt, off);
  if ((tid & 31) == 0) wsum[tid >> 5] = cnt;
  __syncthreads();
  if (tid == 0) {
    int t = 0;
    for (int w = 0; w < kPartThreads / 32; ++w) t += wsum[w];
    chunk_left[c] = t;
  }
}

// left_prefix[c+1] = lefts in chunks 0..c
__global__ void __launch_bounds__(1024)
  k_part_scan_chunks(const int32_t* __restrict__ chunk_left, const int32_t* __restrict__ chunk_off, int n_nodes,
                     int32_t* __restrict__ left_prefix)
{
  __shared__ int carry, wsum[32];
  BlockScanToArray(chunk_off[n_nodes], [&](int c) { return chunk_left[c]; }, left_prefix, &carry, wsum);
}

// seg_out for the next level: children of node j start at new_base[j] (left) and new_base[j] +
// lefts(j) (right); a node that was not split contributes two empty segments.
__global__ void __launch_bounds__(1024)
  k_part_scan_nodes(const int32_t* __restrict__ seg, const int32_t* __restrict__ feature, int node_begin, int n_nodes,
                    const int32_t* __restrict__ chunk_off, const int32_t* __restrict__ left_prefix,
                    int32_t* __restrict__ node_base /* [n_nodes+1] */, int32_t* __restrict__ seg_out /* [2n+1] */)
{
  __shared__ int carry, wsum[32];
  BlockScanToArray(
    n_nodes,
    [&](int j) {
      const int rows = seg[j + 1] - seg[j];
      return (feature[node_begin + j] != -1) ? rows : 0;
    },
    node_base, &carry, wsum);
  __syncthreads();
  for (int j = threadIdx.x; j < n_nodes; j += blockDim.x) {
    const int base  = node_base[j];
    const int lefts = left_prefix[chunk_off[j + 1]] - left_prefix[chunk_off[j]];
    seg_out[2 * j]     = base;
    seg_out[2 * j + 1] = base + lefts;
  }
  if (threadIdx.x == 0) seg_out[2 * n_nodes] = node_base[n_nodes];
}

// One block per chunk.  The rows that go left leave the chunk as one contiguous run of the left
// child's segment and the rows that go right as one run of the right child's, so the block first
// orders its rows (and, if the gradient pairs travel with them, the pairs) in shared memory and then
// copies the two runs out with coalesced stores.
__global__ void __launch_bounds__(kPartThreads)
  k_part_scatter(const int32_t* __restrict__ row_index, const int32_t* __restrict__ seg,
                 const int32_t* __restrict__ chunk_off, int n_nodes, const uint8_t* __restrict__ masks,
                 const int32_t* __restrict__ left_prefix, const int32_t* __restrict__ seg_out,
                 int32_t* __restrict__ row_index_out, const int2* __restrict__ pairs_in, int2* __restrict__ pairs_out,
                 int K)
{
  __shared__ int32_t s_rows[kPartTile];
  __shared__ int2 s_pairs[kPartTile];
  __shared__ int wsum[kPartThreads / 32];
  const int c = blockIdx.x;
  if (c >= chunk_off[n_nodes]) return;
  const int j      = FindOwner(chunk_off, n_nodes, c);
  const int lc     = c - chunk_off[j];
  const int rb     = seg[j] + lc * kPartTile;
  const int re     = min(seg[j + 1], rb + kPartTile);
  const int n_here = re - rb;
  const int lefts_before  = left_prefix[c] - left_prefix[chunk_off[j]];
  const int rights_before = lc * kPartTile - lefts_before;
  const int block_lefts   = left_prefix[c + 1] - left_prefix[c];
  const int tid    = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r0     = rb + tid * kPartItems;
  const int nvalid = max(0, min(kPartItems, re - r0));
  const unsigned mask = masks[static_cast<int64_t>(c) * kPartThreads + tid];
  const int my_left   = __popc(mask);
  int incl = my_left;
  for (int off = 1; off < 32; off <<= 1) {
    int v = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += v;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  int wbefore = 0;
  for (int w = 0; w < warp; ++w) wbefore += wsum[w];
  const int left_rank  = wbefore + incl - my_left;        // lefts before this thread in the chunk
  const int right_rank = tid * kPartItems - left_rank;    // rights before this thread
  // place inside the chunk: the lefts first, then the rights, each in row order
  int local[kPartItems];
  {
    int lp = left_rank, rp = block_lefts + right_rank;
#pragma unroll
    for (int i = 0; i < kPartItems; ++i) local[i] = (mask & (1u << i)) ? lp++ : rp++;
  }
#pragma unroll
  for (int i = 0; i < kPartItems; ++i)
    if (i < nvalid) s_rows[local[i]] = row_index[r0 + i];
  __syncthreads();
  const int lbase = seg_out[2 * j] + lefts_before;
  const int rbase = seg_out[2 * j + 1] + rights_before - block_lefts;  // + t for t >= block_lefts
  for (int t = tid; t < n_here; t += kPartThreads) row_index_out[(t < block_lefts ? lbase : rbase) + t] = s_rows[t];
  // the gradient pairs travel with the row ids, so that the histogram kernel reads them as a stream
  if (pairs_in != nullptr) {
    for (int k = 0; k < K; ++k) {
      __syncthreads();
#pragma unroll
      for (int i = 0; i < kPartItems; ++i)
        if (i < nvalid) s_pairs[local[i]] = pairs_in[static_cast<int64_t>(r0 + i) * K + k];
      __syncthreads();
      for (int t = tid; t < n_here; t += kPartThreads)
        pairs_out[static_cast<int64_t>((t < block_lefts ? lbase : rbase) + t) * K + k] = s_pairs[t];
    }
  }
}

}  // namespace

void InitRows(int32_t* row_index, int32_t* seg, int64_t n_rows, cudaStream_t stream)
{
  const int64_t blocks = (n_rows + 255) / 256;
  k_init_rows<<<static_cast<unsigned>(blocks > 0 ? blocks : 1), 256, 0, stream>>>(row_index, seg, n_rows);
  LBK_LAUNCH_CHECK();
}

void PartitionRows(lbk_context* ctx, Scratch& s, const PartitionLevel& pl, cudaStream_t stream)
{
  (void)ctx;
  const int n = pl.n_nodes;
  // upper bound of the number of chunks, known on the host
  const int64_t max_chunks = pl.n_rows / kPartTile + n + 1;
  int32_t* chunk_off   = s.alloc<int32_t>(static_cast<size_t>(n) + 1);
  int32_t* chunk_left  = s.alloc<int32_t>(max_chunks);
  int32_t* left_prefix = s.alloc<int32_t>(max_chunks + 1);
  int32_t* node_base   = s.alloc<int32_t>(static_cast<size_t>(n) + 1);
  uint8_t* masks       = s.alloc<uint8_t>(static_cast<size_t>(max_chunks) * kPartThreads);
  k_part_plan<<<1, 1024, 0, stream>>>(pl.seg_in, pl.feature, pl.node_begin, n, chunk_off);
  LBK_LAUNCH_CHECK();
  const unsigned grid = static_cast<unsigned>(max_chunks);
  if (pl.bin_bytes == 1) {
    k_part_count<uint8_t><<<grid, kPartThreads, 0, stream>>>(static_cast<const uint8_t*>(pl.bins), pl.bin_pitch,
                                                              pl.row_index_in, pl.seg_in, chunk_off, n, pl.node_begin,
                                                              pl.feature, pl.split_bin, masks, chunk_left);
  } else {
    k_part_count<uint16_t><<<grid, kPartThreads, 0, stream>>>(static_cast<const uint16_t*>(pl.bins), pl.bin_pitch,
                                                               pl.row_index_in, pl.seg_in, chunk_off, n, pl.node_begin,
                                                               pl.feature, pl.split_bin, masks, chunk_left);
  }
  LBK_LAUNCH_CHECK();
  k_part_scan_chunks<<<1, 1024, 0, stream>>>(chunk_left, chunk_off, n, left_prefix);
  LBK_LAUNCH_CHECK();
  k_part_scan_nodes<<<1, 1024, 0, stream>>>(pl.seg_in, pl.feature, pl.node_begin, n, chunk_off, left_prefix, node_base,
                                            pl.seg_out);
  LBK_LAUNCH_CHECK();
  k_part_scatter<<<grid, kPartThreads, 0, stream>>>(pl.row_index_in, pl.seg_in, chunk_off, n, masks, left_prefix,
                                                    pl.seg_out, pl.row_index_out, pl.pairs_in, pl.pairs_out, pl.K);
  LBK_LAUNCH_CHECK();
}

}  // namespace lbk
