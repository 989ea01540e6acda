// Histogram construction: hist[node][output][bin] += (grad, hess) for the rows of the nodes that
// have to be built on this level.
//
// Reference behaviour restated here: fill_histogram_shared / HistogramAgent,
// src/models/tree/build_tree.cu:213-577 (shared-memory int32 pairs per block flushed with 64-bit
// global atomics, impure tiles straight to global atomics).
//
// Design for B200:
//   * rows arrive grouped by node (an index array plus per-node offsets), so a thread block only
//     ever accumulates one node at a time and its private histogram lives in shared memory;
//   * bins are one byte per element, row-major with rows padded to whole 32-feature groups (see
//     proposals.cu): the pieces of a row that different tickets need share DRAM bursts and L2 lines;
//   * the kernel is bound by the load/store data pipe of the SM, not by HBM: the two shared-memory
//     reductions a warp issues per 32 updates are unavoidable (64-bit shared atomics are
//     compare-and-swap loops on this part), and a gather costs the pipe one pass per distinct
//     128-byte line.  So a ticket covers two feature groups (one pass per row for 64 bin bytes),
//     the rows of a batch go straight from global memory into registers with one 16-byte load per
//     lane, and the lanes of a row walk their bytes in an xor-skewed order that keeps the 32
//     reductions of a warp on 32 different banks whatever the bins are (k_hist_smem);
//   * every warp runs its own pipeline over batches of rows (no block barrier in the main loop, no
//     staging in shared memory): the rows of the next two batches and the row ids of the two after
//     are in flight in registers;
//   * accumulation is in int32 like the reference, but guarded: with m = the largest |q| of the
//     call, at most floor((2^31-1)/m) rows are accumulated between flushes, so no partial sum can
//     wrap whatever the bins are;
//   * the planner on the device (k_hist_plan) hands the rows of the level to the resident blocks
//     in equal static ranges (a block walks through the nodes its range touches) or, for small
//     levels, as tickets drawn from a counter;
//   * a node built in one piece owns its output region and flushes with plain stores, turned in
//     shared memory so that the bins of a feature leave as whole 128-byte lines; the pieces of a
//     node that reaches over a range boundary meet in a merge tree of arrival counters in which
//     nobody waits (k_hist_smem); without scratch for the tree: 64-bit global atomics; chunks of
//     <= 128 rows skip shared memory.
#include <mutex>
#include <string>

#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

constexpr int kHistThreads = 512;
constexpr int kTileRows    = 32;    // chunk sizes are multiples of this
constexpr int kDirectRows  = 128;   // chunks up to this size go straight to global atomics
constexpr int kMinChunk    = 2048;
constexpr int kSmemBins    = 256;   // bins per feature held by the private histogram
constexpr int kFaultHistLayout = 31;  // status word: shared memory did not start where the kernel needs it
constexpr int kTreeFanIn   = 4;     // partial sums that meet in one step of the merge tree

struct HistParams {
  const void* bins;
  int64_t n_rows;
  int F, K, B, G, mb;
  const int32_t* row_ptr;
  const void* gpair;
  const int32_t* row_index;
  const int32_t* seg;
  const int32_t* slot_of_node;  // may be null = identity
  int n_nodes;
  const int32_t* chunk_off;  // [n_nodes+1] chunks before each node (tickets drawn from a counter)
  const int32_t* wpre;       // [n_nodes+1] built rows before each node (static ranges); may be null
  const int32_t* plan;       // [0] rows per chunk, [1] total chunks, [3] rows between flushes, [4] rows per
                             // range (0 = tickets from the counter), [7] ranges
  unsigned int* ticket;
  unsigned int* arrive;      // counters of the merge trees (zeroed by the planner); may be null
  void* partial;             // partial-sum slots of the merge trees: [slot][2][mb * 32 W] of the
                             // accumulator type; may be null
  int pairs_by_position;     // 1: gpair is stored in row_index order (pair i belongs to row_index[i]): a stream
  int* status;               // the context's status word; may be null
  void* out;
  // Several ranks, features divided among them: the histogram of a feature goes straight into the
  // memory of the rank that owns the feature (a peer store over NVLink), into that rank's receive
  // slot for this rank: recv[owner][this rank][slot * K + k][bins of the owner's features].
  void* const* push_recv;    // [push_ranks] receive buffers as this device addresses them; null = `out`
  int push_rank, push_ranks;
  long long push_slot_pairs; // pairs per (source rank) block of a receive buffer: segments x push_len
  int push_len;              // pairs per segment in a receive buffer (bound of the owned bins)
};

// Where the bins of feature `f` of segment (slot * K + k) go: the base to which the bin is added.
template <typename out_t>
__device__ inline out_t* FeatureBase(const HistParams& p, int f, int seg)
{
  if (p.push_recv == nullptr) return static_cast<out_t*>(p.out) + static_cast<int64_t>(seg) * p.B + p.row_ptr[f];
  // owner of f: the largest r with r * F / R <= f
  int o = static_cast<int>((static_cast<long long>(f + 1) * p.push_ranks - 1) / p.F);
  if (o > p.push_ranks - 1) o = p.push_ranks - 1;
  const int lo = p.row_ptr[OwnedBegin(o, p.push_ranks, p.F)];
  return static_cast<out_t*>(p.push_recv[o]) + static_cast<long long>(p.push_rank) * p.push_slot_pairs +
         static_cast<long long>(seg) * p.push_len + (p.row_ptr[f] - lo);
}

__device__ inline unsigned SmemAddr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

// largest |grad| and |hess| of a set of quantised pairs (for the stage-level entry point; the
// tree builder gets them from the quantiser)
__global__ void k_max_abs(const int2* __restrict__ gpair, int64_t n, int* __restrict__ max_abs)
{
  int mg = 0, mh = 0;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int2 v = gpair[i];
    // |INT32_MIN| does not fit: saturate
    mg = max(mg, v.x == INT32_MIN ? INT32_MAX : abs(v.x));
    mh = max(mh, v.y == INT32_MIN ? INT32_MAX : abs(v.y));
  }
  for (int off = 16; off >= 1; off >>= 1) {
    mg = max(mg, __shfl_down_sync(0xffffffffu, mg, off));
    mh = max(mh, __shfl_down_sync(0xffffffffu, mh, off));
  }
  if ((threadIdx.x & 31) == 0) {
    atomicMax(max_abs, mg);
    atomicMax(max_abs + 1, mh);
  }
}

// Single block: how the rows of the built nodes are handed to the resident blocks on this level.
//
// A unit of work is (rows, group set, output), GK = group sets x outputs per row.
//
// Static ranges (needs `wpre`, the merge-tree counters and slots): the built rows of the level, laid
// end to end in node order, are cut into resident / GK equal ranges; block b takes range b / GK
// for (group set, output) b % GK and walks through the nodes its range touches.  Every block gets the
// same number of rows whatever the node sizes are (256 equal tickets on 148 blocks would otherwise
// take two rounds, the second one partly empty).  A node that reaches over a range boundary is
// built in pieces whose partial sums meet in a merge tree (see k_hist_smem).  Chosen when every
// range gets at least 2 * kMinChunk rows.
//
// Tickets (everything else): one chunk per node when there are at least as many non-empty nodes as
// resident blocks, else equal chunks of about total / resident rows whose sums are added to the
// histogram with 64-bit atomics; blocks draw (chunk, group set, output) tickets from a counter.
__global__ void __launch_bounds__(1024)
  k_hist_plan(const int32_t* __restrict__ seg, const int32_t* __restrict__ slot_of_node, int n_nodes, int GK,
              int resident, const int* __restrict__ max_abs, long long slot_capacity, int32_t* __restrict__ chunk_off,
              int32_t* __restrict__ wpre, unsigned int* __restrict__ arrive, int n_arrive,
              int32_t* __restrict__ plan, unsigned int* __restrict__ ticket)
{
  __shared__ long long red[32];
  __shared__ long long wsum[32];
  __shared__ long long carry;
  __shared__ long long total_s;
  __shared__ int ch_s, nodes_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  auto rows_of = [&](int j) -> int {
    const bool built = slot_of_node == nullptr || slot_of_node[j] >= 0;
    const int r      = seg[j + 1] - seg[j];
    return built ? r : 0;
  };
  for (int i = tid; i < n_arrive; i += blockDim.x) arrive[i] = 0u;
  long long rows = 0, nonempty = 0;
  for (int j = tid; j < n_nodes; j += blockDim.x) {
    const int r = rows_of(j);
    rows += r;
    nonempty += r > 0;
  }
  rows += nonempty << 40;
  for (int off = 16; off >= 1; off >>= 1) rows += __shfl_down_sync(0xffffffffu, rows, off);
  if (lane == 0) red[warp] = rows;
  __syncthreads();
  if (tid == 0) {
    long long total = 0;
    for (int w = 0; w < n_warps; ++w) total += red[w];
    nodes_s = static_cast<int>(total >> 40);
    total_s = total & ((1ll << 40) - 1);
    int m   = 1;
    if (max_abs) m = max(1, max(max_abs[0], max_abs[1]));
    plan[3] = max_abs ? 2147483647 / m : 2147483647;
  }
  __syncthreads();
  const long long total = total_s;

  // exclusive scan over the nodes: store(j, sum of value(0..j)); 1024 nodes per step
  auto scan_nodes = [&](auto value, auto store) {
    __syncthreads();
    if (tid == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < n_nodes; base += blockDim.x) {
      const int j       = base + tid;
      const long long c = j < n_nodes ? value(j) : 0;
      long long incl    = c;
      for (int off = 1; off < 32; off <<= 1) {
        const long long n = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += n;
      }
      if (lane == 31) wsum[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        const long long w = lane < n_warps ? wsum[lane] : 0;
        long long wi      = w;
        for (int off = 1; off < 32; off <<= 1) {
          const long long n = __shfl_up_sync(0xffffffffu, wi, off);
          if (lane >= off) wi += n;
        }
        wsum[lane] = wi - w;
      }
      __syncthreads();
      const long long before = carry + wsum[warp];
      if (j < n_nodes) store(j, before + incl);
      __syncthreads();
      if (tid == blockDim.x - 1) carry = before + incl;
      __syncthreads();
    }
  };

  // static ranges
  int range_rows = 0, ranges = 0;
  if (wpre != nullptr && arrive != nullptr && GK <= resident && total < (1ll << 31)) {
    ranges      = resident / GK;
    long long q = (total + ranges - 1) / ranges;
    q           = (q + kTileRows - 1) / kTileRows * kTileRows;
    if (q >= 2 * kMinChunk) {
      ranges = static_cast<int>((total + q - 1) / q);
      if (static_cast<long long>(kTreeFanIn) * (ranges - 1) * GK <= slot_capacity &&
          static_cast<long long>(kTreeFanIn) * (ranges - 1) * GK <= n_arrive)
        range_rows = static_cast<int>(q);
    }
  }
  if (wpre != nullptr) {
    scan_nodes([&](int j) -> long long { return rows_of(j); },
               [&](int j, long long incl) { wpre[j + 1] = static_cast<int>(incl); });
    if (tid == 0) wpre[0] = 0;
  }

  // tickets
  if (tid == 0) {
    long long ch = (total * GK + resident - 1) / resident;
    if (static_cast<long long>(nodes_s) * GK >= resident) ch = 1ll << 30;
    if (ch < kMinChunk) ch = kMinChunk;
    ch = (ch + kTileRows - 1) / kTileRows * kTileRows;
    if (ch > (1ll << 30)) ch = 1ll << 30;
    ch_s = static_cast<int>(ch);
  }
  __syncthreads();
  const int ch = ch_s;
  scan_nodes(
    [&](int j) -> long long {
      const int r = rows_of(j);
      return r > 0 ? (r + ch - 1) / ch : 0;
    },
    [&](int j, long long incl) { chunk_off[j + 1] = static_cast<int>(incl); });
  if (tid == 0) {
    chunk_off[0] = 0;
    plan[0]      = ch;
    plan[1]      = static_cast<int>(carry);
    plan[4]      = range_rows;
    plan[7]      = range_rows > 0 ? ranges : 0;
    *ticket      = 0;
  }
}

template <bool kFloat>
struct Acc;
template <>
struct Acc<false> {
  using smem_t = int;
  using in_t   = int2;
  using out_t  = GPairI64;
  __device__ static void add_global(out_t* dst, int g, int h)
  {
    atomicAdd(reinterpret_cast<unsigned long long*>(&dst->grad), static_cast<unsigned long long>(static_cast<long long>(g)));
    atomicAdd(reinterpret_cast<unsigned long long*>(&dst->hess), static_cast<unsigned long long>(static_cast<long long>(h)));
  }
  __device__ static void store_global(out_t* dst, int g, int h)
  {
    *reinterpret_cast<longlong2*>(dst) = make_longlong2(g, h);
  }
  __device__ static bool nonzero(int g, int h) { return (g | h) != 0; }
  __device__ static int4 add4(int4 a, int4 b) { return make_int4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }
  __device__ static void red_shared(unsigned addr, int bits)
  {
    asm volatile("red.shared.add.s32 [%0], %1;\n" ::"r"(addr), "r"(bits) : "memory");
  }
  template <int kOffset>
  __device__ static void red_shared_at(unsigned addr, int bits)
  {
    asm volatile("red.shared.add.s32 [%0+%2], %1;\n" ::"r"(addr), "r"(bits), "n"(kOffset) : "memory");
  }
};
template <>
struct Acc<true> {
  using smem_t = float;
  using in_t   = float2;
  using out_t  = GPairF64;
  __device__ static void add_global(out_t* dst, float g, float h)
  {
    atomicAdd(&dst->grad, static_cast<double>(g));
    atomicAdd(&dst->hess, static_cast<double>(h));
  }
  __device__ static void store_global(out_t* dst, float g, float h)
  {
    *reinterpret_cast<double2*>(dst) = make_double2(g, h);
  }
  __device__ static bool nonzero(float g, float h) { return g != 0.f || h != 0.f; }
  __device__ static int4 add4(int4 a, int4 b)
  {
    return make_int4(__float_as_int(__int_as_float(a.x) + __int_as_float(b.x)),
                     __float_as_int(__int_as_float(a.y) + __int_as_float(b.y)),
                     __float_as_int(__int_as_float(a.z) + __int_as_float(b.z)),
                     __float_as_int(__int_as_float(a.w) + __int_as_float(b.w)));
  }
  __device__ static void red_shared(unsigned addr, int bits)
  {
    asm volatile("red.shared.add.f32 [%0], %1;\n" ::"r"(addr), "f"(__int_as_float(bits)) : "memory");
  }
  template <int kOffset>
  __device__ static void red_shared_at(unsigned addr, int bits)
  {
    asm volatile("red.shared.add.f32 [%0+%2], %1;\n" ::"r"(addr), "f"(__int_as_float(bits)), "n"(kOffset) : "memory");
  }
};

// One piece of work of a block: rows [rb, re) of row_index, all of one node.
struct Piece {
  int j;          // node of the batch
  int slot;       // the node's histogram in `out`
  int rb, re;
  int index;      // which piece of its node this is, 0 .. pieces-1
  int pieces;     // pieces the node is built in
  int tree_base;  // first slot / counter of the node's merge tree (pieces > 1, static ranges)
  int node_rows;  // rows of the whole node
};

__device__ inline Piece DecodeChunk(const HistParams& p, int c)
{
  // node that owns chunk c: last j with chunk_off[j] <= c
  int lo = 0, hi = p.n_nodes;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.chunk_off[mid] <= c) lo = mid; else hi = mid;
  }
  Piece pc;
  pc.j         = lo;
  pc.pieces    = p.chunk_off[lo + 1] - p.chunk_off[lo];
  pc.slot      = p.slot_of_node ? p.slot_of_node[lo] : lo;
  pc.index     = c - p.chunk_off[lo];
  pc.tree_base = -1;
  // the chunks of a node are equal in size (a multiple of 32 rows, the last one takes the rest)
  const int nrows = p.seg[lo + 1] - p.seg[lo];
  pc.node_rows    = nrows;
  const int size  = pc.pieces > 1 ? ((nrows + pc.pieces - 1) / pc.pieces + kTileRows - 1) / kTileRows * kTileRows : nrows;
  pc.rb = min(p.seg[lo + 1], p.seg[lo] + pc.index * size);
  pc.re = min(p.seg[lo + 1], pc.rb + size);
  return pc;
}

// Rows [b, e) of one node, features [f0, f0 + 32 * groups): one lane per feature, the warps of the
// block stride over the rows, every update is a pair of 64-bit global atomics.
template <typename BinT, typename A>
__device__ inline void DirectRows(const HistParams& p, int b, int e, int f0, int groups, int k,
                                  int seg, int warp, int n_warps, int lane)
{
  using in_t          = typename A::in_t;
  const BinT* bins    = static_cast<const BinT*>(p.bins);
  const in_t* gpair   = static_cast<const in_t*>(p.gpair);
  const int64_t pitch = static_cast<int64_t>(p.G) * kGroup;
  for (int u = 0; u < groups; ++u) {
    const int feat = f0 + u * kGroup + lane;
    if (feat >= p.F) continue;
    typename A::out_t* obase = FeatureBase<typename A::out_t>(p, feat, seg);
    for (int r = b + warp; r < e; r += n_warps) {
      const int ridx = p.row_index[r];
      const in_t v   = gpair[static_cast<int64_t>(p.pairs_by_position ? r : ridx) * p.K + k];
      const int bin  = bins[static_cast<int64_t>(ridx) * pitch + feat];
      A::add_global(obase + bin, v.x, v.y);
    }
  }
}

// Bins of two bytes, or more than 256 bins in a feature: every ticket goes straight to global atomics.
template <typename BinT, bool kFloat>
__global__ void __launch_bounds__(kHistThreads)
  k_hist_direct(const HistParams p)
{
  using A = Acc<kFloat>;
  __shared__ unsigned int s_ticket;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long total = static_cast<long long>(p.plan[1]) * p.G * p.K;
  while (true) {
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
    __syncthreads();
    const long long t = s_ticket;
    if (t >= total) break;
    const int k    = static_cast<int>(t % p.K);
    const int g    = static_cast<int>((t / p.K) % p.G);
    const Piece pc = DecodeChunk(p, static_cast<int>(t / (static_cast<long long>(p.K) * p.G)));
    DirectRows<BinT, A>(p, pc.rb, pc.re, g * kGroup, 1, k, pc.slot * p.K + k, warp, kHistThreads / 32, lane);
  }
}

// One update step of a lane: byte J of its 16 bin bytes (already permuted so that step J reads
// the static byte J), both words of the pair.  `lane_word` is the shared-memory address of the
// lane's word in bin row 0 of the gradient histogram.
template <typename A, int W, int J>
__device__ inline void HistStep(const unsigned (&x)[4], unsigned lane_word, const int2& v)
{
  constexpr int kHistBytes = kSmemBins * kGroup * W * 4;
  if (W == 2) {
    // the histogram starts on a multiple of its own size (64 KB), a bin row is 256 bytes: the
    // address is (bin << 8) | (lane_word ^ skew), one byte permute and one three-input logic op
    constexpr unsigned cj = ((J & 7u) << 2) | ((J >> 3) << 7);
    const unsigned b8     = __byte_perm(x[J >> 2], 0u, 0x4404u | ((J & 3) << 4));
    unsigned addr;
    asm("lop3.b32 %0, %1, %2, %3, 0xF6;\n" : "=r"(addr) : "r"(b8), "r"(lane_word), "n"(cj));
    A::red_shared(addr, v.x);
    A::template red_shared_at<kHistBytes>(addr, v.y);
  } else {
    constexpr unsigned cj = 4u * J;
    const unsigned bin    = __byte_perm(x[J >> 2], 0u, 0x4440u | (J & 3));
    const unsigned addr   = (bin * (kGroup * 4) + lane_word) ^ cj;
    A::red_shared(addr, v.x);
    A::template red_shared_at<kHistBytes>(addr, v.y);
  }
}

// The rows [sb, se) of row_index, all of one node, added to the block's private histograms: the
// main loop of k_hist_smem for one warp.  The warps of the block take the batches of 32 / (2 W)
// rows in turn.  Every load of the loop is unconditional: batch numbers beyond the warp's last one
// are clamped to it (the rows are fetched again and dropped), lanes whose feature group does not
// exist read the group that does and add zero pairs, and the last, partial batch of the range is
// handled after the loop.  In flight per warp: the rows of the next two batches and the row ids of
// the two after; the loop is unrolled three times so that the three row buffers rotate by name.
// The row's bin bytes come with a plain load that bypasses L1 and asks L2 for the whole 128-byte
// line (the other half of the row is wanted soon by the block that builds the neighbouring
// groups).  kByPosition: the pairs are stored in row_index order and read as a stream; else they are
// gathered by row id.
template <typename A, int W, bool kByPosition>
__device__ __forceinline__ void HistRows(const HistParams& p, int sb, int se, int g0, int groups, int k, int warp,
                                         int lane, unsigned lane_word)
{
  using in_t = typename A::in_t;
  constexpr int kWarps        = kHistThreads * W / 32;
  constexpr int kLanesPerRow  = 2 * W;
  constexpr int kRowsPerBatch = 32 / kLanesPerRow;
  const unsigned rslot = lane / kLanesPerRow, q = lane % kLanesPerRow;
  const unsigned wsel = rslot >> 2, bsel = rslot & 3;
  const unsigned perm = bsel == 0 ? 0x3210u : bsel == 1 ? 0x2301u : bsel == 2 ? 0x1032u : 0x0123u;
  const unsigned sel0 = perm + ((wsel & 1) ? 0x4444u : 0u), sel1 = perm + ((wsel & 1) ? 0u : 0x4444u);
  const bool lane_on  = static_cast<int>(q >> 1) < groups;  // the group this lane's 16 bytes belong to exists
  const unsigned q_eff = lane_on ? q : (q & 1u);
  const int pair_mask  = lane_on ? -1 : 0;
  const int64_t pitch  = static_cast<int64_t>(p.G) * kGroup;
  const unsigned char* gb = static_cast<const unsigned char*>(p.bins) + g0 * kGroup + q_eff * 16;
  const in_t* gpair    = static_cast<const in_t*>(p.gpair);
  const int pos0       = sb + static_cast<int>(rslot);  // the lane's row of batch 0, as a position in row_index
  const int32_t* rp    = p.row_index + pos0;            // + batch * kRowsPerBatch

  // rid: the row; pos: its position in row_index (only used for pairs stored by position)
  auto load = [&](int rid, int pos, int4& w, int2& v) {
    const int4* ap = reinterpret_cast<const int4*>(gb + static_cast<int64_t>(rid) * pitch);
    asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(w.x), "=r"(w.y), "=r"(w.z), "=r"(w.w)
                 : "l"(ap));
    if (kByPosition) v = __ldcs(reinterpret_cast<const int2*>(gpair + static_cast<int64_t>(pos) * p.K + k));
    else v = __ldcg(reinterpret_cast<const int2*>(gpair + static_cast<int64_t>(rid) * p.K + k));
    if (W == 2) {
      v.x &= pair_mask;
      v.y &= pair_mask;
    }
  };
  auto consume = [&](const int4& w, const int2& v) {
    unsigned x[4];
    if (W == 2) {
      x[0] = __byte_perm(w.x, w.y, sel0);
      x[1] = __byte_perm(w.x, w.y, sel1);
      x[2] = __byte_perm(w.z, w.w, sel0);
      x[3] = __byte_perm(w.z, w.w, sel1);
    } else {
      const unsigned a0 = (wsel & 2) ? w.z : w.x, a1 = (wsel & 2) ? w.w : w.y;
      const unsigned b0 = (wsel & 2) ? w.x : w.z, b1 = (wsel & 2) ? w.y : w.w;
      x[0] = __byte_perm(a0, a1, sel0);
      x[1] = __byte_perm(a0, a1, sel1);
      x[2] = __byte_perm(b0, b1, sel0);
      x[3] = __byte_perm(b0, b1, sel1);
    }
    HistStep<A, W, 0>(x, lane_word, v);
    HistStep<A, W, 1>(x, lane_word, v);
    HistStep<A, W, 2>(x, lane_word, v);
    HistStep<A, W, 3>(x, lane_word, v);
    HistStep<A, W, 4>(x, lane_word, v);
    HistStep<A, W, 5>(x, lane_word, v);
    HistStep<A, W, 6>(x, lane_word, v);
    HistStep<A, W, 7>(x, lane_word, v);
    HistStep<A, W, 8>(x, lane_word, v);
    HistStep<A, W, 9>(x, lane_word, v);
    HistStep<A, W, 10>(x, lane_word, v);
    HistStep<A, W, 11>(x, lane_word, v);
    HistStep<A, W, 12>(x, lane_word, v);
    HistStep<A, W, 13>(x, lane_word, v);
    HistStep<A, W, 14>(x, lane_word, v);
    HistStep<A, W, 15>(x, lane_word, v);
  };

  const int n_here  = se - sb;
  const int nb_full = n_here / kRowsPerBatch;
  int cnt           = nb_full > warp ? (nb_full - warp + kWarps - 1) / kWarps : 0;  // this warp's whole batches
  if (cnt > 0) {
    const int bl = warp + (cnt - 1) * kWarps;  // the warp's last batch
    auto rid_at  = [&](int bb) -> int { return __ldcg(rp + bb * kRowsPerBatch); };
    int b = warp;
    int4 wa, wb, wc;
    int2 va, vb, vc;
    {
      const int b1 = min(b + kWarps, bl);
      load(rid_at(b), pos0 + b * kRowsPerBatch, wa, va);
      load(rid_at(b1), pos0 + b1 * kRowsPerBatch, wb, vb);
    }
    int ba = min(b + 2 * kWarps, bl), bb = min(b + 3 * kWarps, bl);
    int ra = rid_at(ba), rb = rid_at(bb);
#pragma unroll 1
    while (cnt >= 3) {
      load(ra, pos0 + ba * kRowsPerBatch, wc, vc);
      ba = min(b + 4 * kWarps, bl);
      ra = rid_at(ba);
      consume(wa, va);
      load(rb, pos0 + bb * kRowsPerBatch, wa, va);
      bb = min(b + 5 * kWarps, bl);
      rb = rid_at(bb);
      consume(wb, vb);
      load(ra, pos0 + ba * kRowsPerBatch, wb, vb);
      ba = min(b + 6 * kWarps, bl);
      ra = rid_at(ba);
      consume(wc, vc);
      // now the buffers hold batches b + 3, b + 4 (in units of kWarps) and the ids b + 5 (rb), b + 6 (ra)
      int t = ra; ra = rb; rb = t;
      t = ba; ba = bb; bb = t;
      b += 3 * kWarps;
      cnt -= 3;
    }
    if (cnt >= 1) consume(wa, va);
    if (cnt >= 2) consume(wb, vb);
  }
  // the partial batch at the end of the range
  const int tail = n_here - nb_full * kRowsPerBatch;
  if (tail > 0 && warp == nb_full % kWarps) {
    const bool valid = static_cast<int>(rslot) < tail;
    // lanes without a row read the first row of the range (it exists) and add nothing
    const int pos    = valid ? pos0 + nb_full * kRowsPerBatch : sb;
    const int rid    = __ldcg(p.row_index + pos);
    int4 w;
    int2 v;
    load(rid, pos, w, v);
    if (!valid) v = make_int2(0, 0);
    consume(w, v);
  }
}

// One-byte bins, at most 256 per feature: private histograms in shared memory.
//
// W = 1: a unit covers one 32-feature group, 512 threads, two blocks per SM.
// W = 2: a unit covers two neighbouring groups (64 features), 1024 threads, one block per SM.
// The wide form exists because the load/store pipe of the SM spends one pass per distinct
// 128-byte line a gather touches, however few bytes it takes from it: with 64 bin bytes per row
// the row gather costs half as many passes per update, and the row ids and gradient pairs are
// fetched once for two groups.
//
// Shared memory: the gradient histogram [256 bins][32 W words] sits at shared address H = its own
// size (64 KB for W = 2), the hessian histogram at 2 H, so that the bits of (bin << 8), of the word
// inside a bin row and of the base never overlap; what lies below H is the staging area of the
// flush.  Every warp runs its own pipeline over batches of 32 / (2 W) rows (no block barrier
// inside).  2 W lanes own one row of the batch and load its bin bytes straight from global memory
// into registers, 16 bytes per lane.  In step j of 16 the lanes of row slot r handle byte (j xor r)
// of their 16, and the histogram words of a bin are laid out so that the 32 lanes of a warp always
// update 32 different banks, whatever the bins:
//   W = 1 (r < 16, quarter q < 2):  word = 16 q + byte                   (bank = word)
//   W = 2 (r < 8,  quarter q < 4):  word = 32 (byte / 8) + 8 q + byte % 8 (bank = 8 q + byte % 8)
// The bytes are permuted once per batch (a word swap and one byte permute per word) so that step
// j reads the static byte j.  Per 32 updates that leaves the two reductions on the pipe.
//
// Flush: a warp takes a tile of 8 bins x 32 words, turns it in its staging area (a skewed 8 x 32
// array, conflict free both ways) and writes, per word, the 8 bins of a feature as 128 contiguous
// bytes of the output.
//
// Merge tree (static ranges): the P pieces of a node that reaches over range boundaries are summed
// without waits.  A piece writes its 32-bit partial sums to its slot and adds one to the counter
// of its group of four; the last one to arrive adds the others' slots to its own sums and goes on
// as one member of the next level, until one block holds the node's total and writes the
// histogram.  Nobody waits for anybody: whoever arrives first leaves.
template <bool kFloat, int W>
__global__ void __launch_bounds__(kHistThreads * W, W == 1 ? 2 : 1)
  k_hist_smem(const HistParams p)
{
  using A      = Acc<kFloat>;
  using smem_t = typename A::smem_t;
  using in_t   = typename A::in_t;
  using out_t  = typename A::out_t;
  constexpr int kThreads      = kHistThreads * W;
  constexpr int kWarps        = kThreads / 32;
  constexpr int kCols         = kGroup * W;   // histogram words per bin
  constexpr int kHistBytes    = kSmemBins * kCols * 4;
  constexpr int kLanesPerRow  = 2 * W;
  constexpr int kRowsPerBatch = 32 / kLanesPerRow;
  constexpr int kStageWords   = 256;  // per warp: 8 bins x 32 words
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ unsigned int s_ticket;
  __shared__ int s_rp[kCols + 1];  // row_ptr of the unit's features (clamped at F)
  __shared__ typename Acc<kFloat>::out_t* s_base[kCols];  // where bin 0 of each of them goes, for the piece at hand

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned base = SmemAddr(smem_raw);
  unsigned dyn_bytes;
  asm("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn_bytes));
  const unsigned hg_addr = static_cast<unsigned>(kHistBytes);
  // the staging area has to end before the histograms begin, and they inside what was asked for
  if (base + kWarps * kStageWords * 4 > hg_addr || hg_addr + 2u * kHistBytes > base + dyn_bytes) {
    if (tid == 0 && p.status != nullptr) atomicExch(p.status, kFaultHistLayout);
    return;
  }
  smem_t* stage_all = reinterpret_cast<smem_t*>(smem_raw);
  smem_t* hg        = reinterpret_cast<smem_t*>(smem_raw + (hg_addr - base));
  smem_t* hh        = hg + kSmemBins * kCols;

  const int rows_safe   = p.plan[3];
  const int GP          = (p.G + W - 1) / W;  // group sets per row
  const int range_rows  = p.wpre != nullptr ? p.plan[4] : 0;
  const in_t* gpair     = static_cast<const in_t*>(p.gpair);
  const int hist_words  = p.mb * kCols;
  const int64_t pitch   = static_cast<int64_t>(p.G) * kGroup;  // bins are row-major, rows padded to whole groups
  // chunks that merge through slots never flush in the middle: they stay below the safe count
  const int cap_rows    = rows_safe >= (1 << 30) ? (1 << 30) : (rows_safe & ~(kTileRows - 1));
  // feature (relative to the unit's first) of histogram word w
  auto feature_of_word = [](int w) -> int { return W == 1 ? w : 16 * ((w >> 3) & 3) + 8 * (w >> 5) + (w & 7); };

  const unsigned rslot    = lane / kLanesPerRow, q = lane % kLanesPerRow;
  const unsigned wsel     = rslot >> 2, bsel = rslot & 3;
  const unsigned perm     = bsel == 0 ? 0x3210u : bsel == 1 ? 0x2301u : bsel == 2 ? 0x1032u : 0x0123u;
  const unsigned lane_word = hg_addr + (W == 1 ? 16 * q + rslot : 8 * q + rslot) * 4;

  auto zero = [&]() {
    int4* g4 = reinterpret_cast<int4*>(hg);
    int4* h4 = reinterpret_cast<int4*>(hh);
    for (int e = tid; e < (hist_words >> 2); e += kThreads) {
      g4[e] = make_int4(0, 0, 0, 0);
      h4[e] = make_int4(0, 0, 0, 0);
    }
  };

  // One piece: accumulate its rows, then flush / merge.
  auto process = [&](const Piece& pc, int gp, int k) {
    const int g0     = gp * W;
    const int groups = min(W, p.G - g0);
    const int seg    = pc.slot * p.K + k;
    // the merge tree adds 32-bit images: a piece (at most range_rows rows) has to stay below the safe
    // count, and the tree is climbed only as far as the merged images do (see below)
    const bool tree  = pc.pieces > 1 && pc.tree_base >= 0 && p.partial != nullptr && range_rows <= cap_rows &&
                      rows_safe >= kTileRows;
    if (rows_safe < kTileRows || (pc.re - pc.rb <= kDirectRows && !tree)) {
      DirectRows<uint8_t, A>(p, pc.rb, pc.re, g0 * kGroup, groups, k, seg, warp, kWarps, lane);
      return;
    }
    __syncthreads();  // whoever still reads the histogram or s_rp of the piece before
    for (int i = tid; i <= kCols; i += kThreads) {
      const int f = g0 * kGroup + i;
      s_rp[i]     = p.row_ptr[min(p.F, f)];
      if (i < kCols) s_base[i] = f < p.F ? FeatureBase<out_t>(p, f, seg) : nullptr;
    }
    zero();
    __syncthreads();

    // the flush: tiles of 8 bins x 32 words, turned in the warp's staging area
    auto flush = [&](bool atomics) {
      smem_t* stage      = stage_all + warp * kStageWords;
      const int n_btiles = (p.mb + 7) >> 3;
      const int a = lane >> 3, b = lane & 7;
      for (int t = warp; t < n_btiles * W; t += kWarps) {
        const int half = t / n_btiles, bin0 = (t - half * n_btiles) << 3;
        smem_t gv[8];
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const smem_t* src = (pass == 0 ? hg : hh) + half * 32 + lane;
#pragma unroll
          for (int bb = 0; bb < 8; ++bb) {
            const int bin = bin0 + bb;
            stage[bb * 32 + ((lane + 4 * bb) & 31)] = bin < p.mb ? src[bin * kCols] : smem_t(0);
          }
          __syncwarp();
          if (pass == 0) {
#pragma unroll
            for (int i = 0; i < 8; ++i) gv[i] = stage[b * 32 + ((4 * i + a + 4 * b) & 31)];
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const smem_t hv = stage[b * 32 + ((4 * i + a + 4 * b) & 31)];
              const int f     = feature_of_word(half * 32 + 4 * i + a);
              const int bin   = bin0 + b;
              if (bin < s_rp[f + 1] - s_rp[f] && A::nonzero(gv[i], hv)) {
                if (atomics) A::add_global(s_base[f] + bin, gv[i], hv);
                else A::store_global(s_base[f] + bin, gv[i], hv);
              }
            }
          }
          __syncwarp();
        }
      }
    };

    bool use_atomics   = pc.pieces > 1 && !tree;
    const int seg_rows = rows_safe >= (1 << 30) ? (1 << 30) : (rows_safe & ~31);
    for (int sb = pc.rb; sb < pc.re; sb += seg_rows) {
      const int se = min(pc.re, sb + seg_rows);
      if (sb > pc.rb) {
        __syncthreads();
        flush(true);
        use_atomics = true;
        __syncthreads();
        zero();
        __syncthreads();
      }
      if (p.pairs_by_position != 0) HistRows<A, W, true>(p, sb, se, g0, groups, k, warp, lane, lane_word);
      else HistRows<A, W, false>(p, sb, se, g0, groups, k, warp, lane, lane_word);
    }
    __syncthreads();
    if (!tree) {
      flush(use_atomics);
      return;
    }
    // merge tree
    const int GK          = GP * p.K;
    const int gk          = gp * p.K + k;
    const size_t stride   = static_cast<size_t>(hist_words) * 2;  // words per slot
    smem_t* slots         = static_cast<smem_t*>(p.partial);
    const int n4          = hist_words >> 2;
    int idx = pc.index, members = pc.pieces, soff = 0, coff = 0;
    long long image_rows = range_rows;  // rows an image of this tree level holds at most
    while (true) {
      const int n_groups = (members + kTreeFanIn - 1) / kTreeFanIn;
      const int grp      = idx / kTreeFanIn;
      const int gsize    = min(kTreeFanIn, members - grp * kTreeFanIn);
      // A node with more rows than 32-bit sums are safe for: its images are merged as far as they
      // stay below that count, and what is left (a handful instead of one per piece) is added into
      // the output with 64-bit atomics.  Every holder of an image of this level decides alike.
      if (min(static_cast<long long>(pc.node_rows), image_rows * kTreeFanIn) > cap_rows) {
        flush(true);
        return;
      }
      if (gsize > 1) {
        // leave my sums where the last one of the group finds them, then count myself in
        smem_t* mine = slots + (static_cast<size_t>(pc.tree_base + soff + idx) * GK + gk) * stride;
        for (int e4 = tid; e4 < n4; e4 += kThreads) {
          __stcg(reinterpret_cast<int4*>(mine) + e4, reinterpret_cast<const int4*>(hg)[e4]);
          __stcg(reinterpret_cast<int4*>(mine + hist_words) + e4, reinterpret_cast<const int4*>(hh)[e4]);
        }
        __threadfence();
        __syncthreads();
        if (tid == 0) s_ticket = atomicAdd(p.arrive + static_cast<size_t>(pc.tree_base + coff + grp) * GK + gk, 1u);
        __syncthreads();
        const int arrived = static_cast<int>(s_ticket);
        if (arrived != gsize - 1) return;  // somebody else carries the group on
        __threadfence();
        for (int m = grp * kTreeFanIn; m < grp * kTreeFanIn + gsize; ++m) {
          if (m == idx) continue;
          const smem_t* other = slots + (static_cast<size_t>(pc.tree_base + soff + m) * GK + gk) * stride;
          for (int e4 = tid; e4 < n4; e4 += kThreads) {
            int4* mg = reinterpret_cast<int4*>(hg) + e4;
            int4* mh = reinterpret_cast<int4*>(hh) + e4;
            *mg = A::add4(*mg, __ldcg(reinterpret_cast<const int4*>(other) + e4));
            *mh = A::add4(*mh, __ldcg(reinterpret_cast<const int4*>(other + hist_words) + e4));
          }
        }
        __syncthreads();
      }
      if (n_groups == 1) break;  // this block holds the node's total
      soff += members;
      coff += n_groups;
      idx     = grp;
      members = n_groups;
      image_rows *= kTreeFanIn;
    }
    flush(false);
  };

  // The pieces of this block: the nodes its static range touches, or the chunks it draws as
  // tickets; one loop so that the piece code exists once.
  const int GK = GP * p.K;
  int gp = 0, k = 0, bj = 0;
  long long lo = 0, hi = 0;
  if (range_rows > 0) {
    // static ranges: block b = (range, group set, output)
    const int c = static_cast<int>(blockIdx.x) / GK;
    if (c >= p.plan[7]) return;
    const int gk = static_cast<int>(blockIdx.x) - c * GK;
    gp = gk / p.K;
    k  = gk - gp * p.K;
    const long long all = p.wpre[p.n_nodes];
    lo = static_cast<long long>(c) * range_rows;
    hi = lo + range_rows < all ? lo + range_rows : all;
    int a = 0, b = p.n_nodes;  // last node whose rows begin at or before lo
    while (b - a > 1) {
      const int m = (a + b) >> 1;
      if (p.wpre[m] <= lo) a = m; else b = m;
    }
    bj = a;
  }
  const long long total = static_cast<long long>(p.plan[1]) * GK;
  while (true) {
    Piece pc;
    if (range_rows > 0) {
      if (lo >= hi) break;
      const int c = static_cast<int>(blockIdx.x) / GK;
      while (p.wpre[bj + 1] <= lo) ++bj;  // nodes without built rows
      const long long ws = p.wpre[bj], we = p.wpre[bj + 1];
      const long long pe = we < hi ? we : hi;
      const int first_c  = static_cast<int>(ws / range_rows);        // range that holds the node's first row
      const int last_c   = static_cast<int>((we - 1) / range_rows);  // ... and its last one
      pc.j         = bj;
      pc.slot      = p.slot_of_node ? p.slot_of_node[bj] : bj;
      pc.pieces    = last_c - first_c + 1;
      pc.index     = c - first_c;
      pc.tree_base = kTreeFanIn * first_c;  // the node owns the boundaries first_c+1 .. last_c
      pc.node_rows = static_cast<int>(we - ws);
      pc.rb        = p.seg[bj] + static_cast<int>(lo - ws);
      pc.re        = p.seg[bj] + static_cast<int>(pe - ws);
      lo           = pe;
    } else {
      __syncthreads();
      if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
      __syncthreads();
      const long long t = s_ticket;
      if (t >= total) break;
      k  = static_cast<int>(t % p.K);
      gp = static_cast<int>((t / p.K) % GP);
      pc = DecodeChunk(p, static_cast<int>(t / GK));
    }
    process(pc, gp, k);
  }
}

// ---- row grouping (utility for the stage-level API) -------------------------------------------
constexpr int kGroupTile = 4096;

// Kernel, dynamic shared memory and persistent grid (resident blocks of the whole device, from the
// occupancy calculator) for one combination of bin width, pair type and path.
struct HistLaunch {
  void (*fn)(HistParams);
  size_t smem;
  int threads;
  int grid;
  int width;  // feature groups per unit of work
};

HistLaunch PickHistKernel(bool smem_path, int bin_bytes, bool float_mode, int n_groups, int sm_count)
{
  HistLaunch h;
  h.width   = smem_path && n_groups >= 2 ? 2 : 1;
  h.threads = kHistThreads * h.width;
  // staging below H, the two histograms at H and 2 H (H = 256 bins x 32 W words x 4 bytes)
  h.smem    = smem_path ? static_cast<size_t>(kSmemBins) * kGroup * h.width * 4 * 3 : 0;
  if (smem_path && h.width == 2) h.fn = float_mode ? k_hist_smem<true, 2> : k_hist_smem<false, 2>;
  else if (smem_path) h.fn = float_mode ? k_hist_smem<true, 1> : k_hist_smem<false, 1>;
  else if (bin_bytes == 1) h.fn = float_mode ? k_hist_direct<uint8_t, true> : k_hist_direct<uint8_t, false>;
  else h.fn = float_mode ? k_hist_direct<uint16_t, true> : k_hist_direct<uint16_t, false>;
  if (h.smem > 48 * 1024)
    LBK_CUDA(cudaFuncSetAttribute(h.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(h.smem)));
  int per_sm = 0;
  LBK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, h.fn, h.threads, h.smem));
  if (per_sm < 1) per_sm = 1;
  if (!smem_path && per_sm > 4) per_sm = 4;
  h.grid = sm_count * per_sm;
  return h;
}

__global__ void k_group_count(const int32_t* __restrict__ node_of_row, int64_t n_rows, int node_begin, int n_nodes,
                              int32_t* __restrict__ counts /* [blocks][n_nodes] */)
{
  extern __shared__ int cnt[];
  for (int i = threadIdx.x; i < n_nodes; i += blockDim.x) cnt[i] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kGroupTile;
  for (int i = threadIdx.x; i < kGroupTile; i += blockDim.x) {
    const int64_t r = base + i;
    if (r < n_rows) {
      const int nd = node_of_row[r] - node_begin;
      if (nd >= 0 && nd < n_nodes) atomicAdd(&cnt[nd], 1);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_nodes; i += blockDim.x)
    counts[static_cast<int64_t>(blockIdx.x) * n_nodes + i] = cnt[i];
}

// counts[b][nd] -> exclusive offset of (nd, b) in node-major order; seg[nd] = start of node nd
__global__ void k_group_scan(int32_t* __restrict__ counts, int n_blocks, int n_nodes, int32_t* __restrict__ seg)
{
  // one thread per node sums its column, then a serial scan over nodes by thread 0
  extern __shared__ int tot[];
  for (int nd = threadIdx.x; nd < n_nodes; nd += blockDim.x) {
    int s = 0;
    for (int b = 0; b < n_blocks; ++b) s += counts[static_cast<int64_t>(b) * n_nodes + nd];
    tot[nd] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int nd = 0; nd < n_nodes; ++nd) {
      seg[nd] = run;
      run += tot[nd];
    }
    seg[n_nodes] = run;
  }
  __syncthreads();
  for (int nd = threadIdx.x; nd < n_nodes; nd += blockDim.x) {
    int run = seg[nd];
    for (int b = 0; b < n_blocks; ++b) {
      const int c = counts[static_cast<int64_t>(b) * n_nodes + nd];
      counts[static_cast<int64_t>(b) * n_nodes + nd] = run;
      run += c;
    }
  }
}

// one warp per tile walks its rows in order so that rows keep their relative order inside a node
__global__ void k_group_scatter(const int32_t* __restrict__ node_of_row, int64_t n_rows, int node_begin, int n_nodes,
                                const int32_t* __restrict__ offsets, int32_t* __restrict__ row_index)
{
  extern __shared__ int cur[];
  const int lane = threadIdx.x;
  for (int i = lane; i < n_nodes; i += 32) cur[i] = offsets[static_cast<int64_t>(blockIdx.x) * n_nodes + i];
  __syncwarp();
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kGroupTile;
  for (int i = 0; i < kGroupTile; i += 32) {
    const int64_t r = base + i + lane;
    int nd          = -1;
    if (r < n_rows) {
      nd = node_of_row[r] - node_begin;
      if (nd < 0 || nd >= n_nodes) nd = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, nd);
    const int rank       = __popc(peers & ((1u << lane) - 1u));
    int start            = 0;
    if (nd >= 0) start = cur[nd];
    __syncwarp();
    if (nd >= 0) {
      row_index[start + rank] = static_cast<int32_t>(r);
      if (rank == __popc(peers) - 1) cur[nd] = start + rank + 1;
    }
    __syncwarp();
  }
}

}  // namespace

void BuildHistogram(lbk_context* ctx, Scratch& s, const HistLevel& lv, cudaStream_t stream)
{
  if (lv.n_nodes <= 0) return;
  HistParams p;
  p.bins         = lv.bins;
  p.n_rows       = lv.n_rows;
  p.F            = lv.F;
  p.K            = lv.K;
  p.B            = lv.B;
  p.G            = (lv.F + kGroup - 1) / kGroup;
  p.row_ptr      = lv.row_ptr;
  p.gpair        = lv.float_mode ? static_cast<const void*>(lv.gpair_f) : static_cast<const void*>(lv.gpair);
  p.row_index    = lv.row_index;
  p.seg          = lv.seg + lv.seg_node_offset;
  p.slot_of_node = lv.slot_of_node;
  p.n_nodes      = lv.n_nodes;
  int32_t* chunk_off = s.alloc<int32_t>(static_cast<size_t>(lv.n_nodes) + 1);
  int32_t* plan      = s.alloc<int32_t>(8);
  p.chunk_off        = chunk_off;
  p.plan             = plan;
  p.ticket           = reinterpret_cast<unsigned int*>(plan + 2);
  p.status           = ctx->d_status;
  p.pairs_by_position = lv.pairs_by_position ? 1 : 0;
  p.out              = lv.out;
  p.push_recv        = lv.push_recv;
  p.push_rank        = ctx->rank;
  p.push_ranks       = ctx->n_ranks;
  p.push_slot_pairs  = lv.push_slot_pairs;
  p.push_len         = lv.push_len;

  const bool smem_path = lv.bin_bytes == 1 && lv.max_bins_per_feature <= kSmemBins;
  p.mb                 = smem_path ? lv.max_bins_per_feature : 0;
  const HistLaunch hl  = PickHistKernel(smem_path, lv.bin_bytes, lv.float_mode, p.G, ctx->sm_count);

  const int* max_abs = lv.max_abs;
  if (!lv.float_mode && max_abs == nullptr) {
    // the caller gave quantised pairs without their largest magnitude: find it
    int* m = s.alloc<int>(2);
    LBK_CUDA(cudaMemsetAsync(m, 0, 2 * sizeof(int), stream));
    const int64_t n = lv.n_rows * lv.K;
    if (n > 0) {
      k_max_abs<<<ctx->sm_count * 8, 256, 0, stream>>>(lv.gpair, n, m);
      LBK_LAUNCH_CHECK();
    }
    max_abs = m;
  }
  const int units_per_row = (p.G + hl.width - 1) / hl.width * p.K;
  // static ranges need the rows before each node, and slots and counters for the merge trees of
  // the nodes that reach over a range boundary: kTreeFanIn per resident block covers every cut
  long long slot_capacity = 0;
  int n_arrive            = 0;
  p.wpre    = nullptr;
  p.arrive  = nullptr;
  p.partial = nullptr;
  int32_t* wpre = nullptr;
  if (smem_path) {
    slot_capacity           = static_cast<long long>(kTreeFanIn) * hl.grid;
    n_arrive                = kTreeFanIn * hl.grid;
    const size_t slot_bytes = static_cast<size_t>(p.mb) * kGroup * hl.width * 8;
    wpre                    = s.alloc<int32_t>(static_cast<size_t>(lv.n_nodes) + 1);
    p.wpre                  = wpre;
    p.arrive                = s.alloc<unsigned int>(static_cast<size_t>(n_arrive));
    p.partial               = s.alloc<unsigned char>(slot_bytes * slot_capacity);
  }
  k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, p.slot_of_node, p.n_nodes, units_per_row, hl.grid,
                                      lv.float_mode ? nullptr : max_abs, slot_capacity, chunk_off, wpre, p.arrive,
                                      n_arrive, plan, p.ticket);
  LBK_LAUNCH_CHECK();
  std::pair<cudaEvent_t, cudaEvent_t> ev{nullptr, nullptr};
  if (ctx->profile) {
    ev = NextProfileEvents(ctx);
    LBK_CUDA(cudaEventRecord(ev.first, stream));
  }
  hl.fn<<<hl.grid, hl.threads, hl.smem, stream>>>(p);
  LBK_LAUNCH_CHECK();
  if (ctx->profile) LBK_CUDA(cudaEventRecord(ev.second, stream));
  // stream ordered: the slots go back to the pool once the kernel has run
  if (p.partial) s.free_one(p.partial);
}

void* BuildHistogramSummed(lbk_context* ctx, Scratch& s, const HistLevel& lv, int n_slots, HistSum mode,
                           bool result_in_out, bool zero_out, cudaStream_t stream)
{
  const size_t slot_words = static_cast<size_t>(lv.K) * lv.B * 2;  // 64-bit words per slot
  const size_t bytes      = static_cast<size_t>(n_slots) * slot_words * 8;
  if (ctx->n_ranks <= 1) {
    if (zero_out) LBK_CUDA(cudaMemsetAsync(lv.out, 0, bytes, stream));
    if (lv.n_rows > 0) BuildHistogram(ctx, s, lv, stream);
    return lv.out;
  }
  // every decision below depends only on what is equal on every rank (the shapes, the kind of
  // communicator, the collective answer of EnsureExchange): all ranks issue the same collectives
  // The owned sums by push: every rank's kernel stores the histogram of a feature straight into
  // the owner's receive slot while it runs, a barrier, then the owner adds up its slots locally.
  // The receive buffers hold ranks x segments x (a bound of the owned bins): where the features'
  // bin counts are so uneven that the bound is far above the real size, the pull form below is used.
  if (mode == HistSum::kSumOwned) {
    const int R          = ctx->n_ranks;
    const long long fo   = (lv.F + R - 1) / R;  // features of the largest owner
    long long push_len   = fo * (lv.max_bins_per_feature > 0 ? lv.max_bins_per_feature : lv.B);
    if (push_len > lv.B) push_len = lv.B;
    const int n_seg      = n_slots * lv.K;
    const size_t push_bytes = static_cast<size_t>(R) * n_seg * static_cast<size_t>(push_len) * 16;
    if (push_bytes <= 2 * bytes + (size_t{1} << 20) && EnsureExchange(ctx, push_bytes, stream)) {
      void* dst = lv.out;  // every owned bin is written below; the others are not touched
      HistLevel sub       = lv;
      sub.push_recv       = NextPushBuffers(ctx, stream);
      sub.push_slot_pairs = static_cast<long long>(n_seg) * push_len;
      sub.push_len        = static_cast<int>(push_len);
      if (lv.n_rows > 0) BuildHistogram(ctx, s, sub, stream);
      ExchangeReducePushed(ctx, dst, n_seg, static_cast<int>(push_len), lv.B, lv.F, lv.row_ptr, lv.float_mode, stream);
      return dst;
    }
  }
  if (EnsureExchange(ctx, bytes, stream)) {
    void* buf = NextExchangeBuffer(ctx, bytes, stream);
    HistLevel sub = lv;
    sub.out       = buf;
    if (lv.n_rows > 0) BuildHistogram(ctx, s, sub, stream);
    const int n_seg = n_slots * lv.K;
    if (mode == HistSum::kSumOwned) {
      void* dst = result_in_out ? lv.out : buf;
      ExchangeReduceOwned(ctx, buf, dst, n_seg, lv.B, lv.F, lv.row_ptr, lv.float_mode, stream);
      return dst;
    }
    ExchangeReduceOwned(ctx, buf, buf, n_seg, lv.B, lv.F, lv.row_ptr, lv.float_mode, stream);
    ExchangeGatherAll(ctx, buf, lv.out, n_seg, lv.B, lv.F, lv.row_ptr, stream);
    return lv.out;
  }
  if (zero_out) LBK_CUDA(cudaMemsetAsync(lv.out, 0, bytes, stream));
  if (lv.n_rows > 0) BuildHistogram(ctx, s, lv, stream);
  AllReduce(ctx, lv.out, static_cast<size_t>(n_slots) * slot_words, lv.float_mode ? LBK_F64 : LBK_I64, LBK_SUM, stream);
  return lv.out;
}

void GroupRows(lbk_context* ctx, Scratch& s, const int32_t* node_of_row, int64_t n_rows, int node_begin,
               int n_nodes, int32_t* row_index, int32_t* seg, cudaStream_t stream)
{
  LBK_EXPECT(n_nodes >= 1 && n_nodes <= 8192, "group_rows supports 1..8192 nodes");
  const int64_t n_blocks = (n_rows + kGroupTile - 1) / kGroupTile;
  if (n_blocks == 0) {
    LBK_CUDA(cudaMemsetAsync(seg, 0, sizeof(int32_t) * (n_nodes + 1), stream));
    return;
  }
  int32_t* counts   = s.alloc<int32_t>(static_cast<size_t>(n_blocks) * n_nodes);
  const size_t smem = sizeof(int) * n_nodes;
  k_group_count<<<static_cast<unsigned>(n_blocks), 256, smem, stream>>>(node_of_row, n_rows, node_begin, n_nodes, counts);
  LBK_LAUNCH_CHECK();
  k_group_scan<<<1, 1024, smem, stream>>>(counts, static_cast<int>(n_blocks), n_nodes, seg);
  LBK_LAUNCH_CHECK();
  k_group_scatter<<<static_cast<unsigned>(n_blocks), 32, smem, stream>>>(node_of_row, n_rows, node_begin, n_nodes, counts,
                                                                         row_index);
  LBK_LAUNCH_CHECK();
  (void)ctx;
}

}  // namespace lbk

// ---------------------------------------------------------------------------------------------
// lbk_histogram_noalloc: the histogram build for callers that must not allocate device memory.
//
// Who needs it: code that runs under a memory budget that a runtime has already handed out
// completely (a task variant registered without the right to allocate: any cudaMalloc there fails or
// takes memory the runtime believes it owns), or a process that wants its device footprint fixed
// after start-up so that no later call can fail for lack of memory.  lbk_histogram takes its
// per-call scratch (chunk offsets, the level plan, the largest magnitudes) from the context's
// pool; this entry point keeps that scratch in a fixed array inside the library image instead
// and needs no context at all.
//
// Limits and rules
//   * at most LBK_NOALLOC_MAX_NODES nodes and LBK_NOALLOC_MAX_FEATURES features per call,
//     device pointers only (host_buffers must be 0), one rank (all_reduce must be 0: there is no
//     context and so no communicator); larger or other calls are rejected with LBK_ERR_ARGUMENT
//     before anything is launched;
//   * the array (about 16 KB) exists once per GPU that loads the library, until the process ends;
//   * the first call on a device looks the array's device address up (the array's name is only a
//     host-side handle; kernels get the address found here).  Make that first call before any
//     stream capture begins;
//   * the call blocks: it reads row_ptr back and synchronises `stream` before it returns (so it is
//     not something to issue from a host callback of a stream); it makes `device` current for the
//     duration of the call and restores the caller's device before it returns;
//   * all calls on a device share the array: what has to start at zero is cleared by each call, and
//     two calls whose kernels overlap on the GPU (different streams, different threads) race -
//     serialise them on one stream.
namespace lbk {
namespace {

constexpr int kNoAllocMaxNodes    = LBK_NOALLOC_MAX_NODES;
constexpr int kNoAllocMaxFeatures = LBK_NOALLOC_MAX_FEATURES;
constexpr int kNoAllocPlanOffset  = kNoAllocMaxNodes + 4;   // chunk offsets first, then plan[8], max_abs[2]
constexpr int kNoAllocInts        = kNoAllocPlanOffset + 12;

static __device__ __align__(256) int32_t g_hist_scratch[kNoAllocInts];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
int32_t* g_scratch_addr[kMaxDevices] = {};

// Device address of the scratch array on `device`, which must be the current device.
int32_t* HistScratchAddress(int device)
{
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[device] == nullptr) {
    void* ptr = nullptr;
    LBK_CUDA(cudaGetSymbolAddress(&ptr, g_hist_scratch));
    g_scratch_addr[device] = static_cast<int32_t*>(ptr);
  }
  return g_scratch_addr[device];
}

}  // namespace
}  // namespace lbk

extern "C" int lbk_histogram_noalloc(int device, const lbk_histogram_args* a)
{
  using namespace lbk;
  return Guard(nullptr, [&] {
    LBK_EXPECT(a != nullptr, "null argument");
    LBK_EXPECT(device >= 0 && device < kMaxDevices, "device index out of range");
    LBK_EXPECT(a->host_buffers == 0, "lbk_histogram_noalloc takes device pointers only");
    LBK_EXPECT(a->all_reduce == 0, "lbk_histogram_noalloc has no communicator: all_reduce must be 0");
    LBK_EXPECT(!a->pairs_by_position || a->mode == 1 || a->max_abs != nullptr,
               "pairs stored by position need max_abs (the library cannot know how many entries the array has)");
    LBK_EXPECT(a->bins && a->row_ptr && a->row_index && a->seg && a->hist, "null argument");
    LBK_EXPECT(a->mode == 0 || a->mode == 1, "mode must be 0 or 1");
    LBK_EXPECT(a->mode == 0 ? a->gpair != nullptr : a->gpair_f32 != nullptr, "missing gradient pairs");
    LBK_EXPECT(a->bin_bytes == 1 || a->bin_bytes == 2, "bin_bytes must be 1 or 2");
    LBK_EXPECT(a->n_features >= 1 && a->n_outputs >= 1 && a->total_bins >= a->n_features, "bad shape");
    LBK_EXPECT(a->n_nodes >= 1 && a->n_nodes <= kNoAllocMaxNodes,
               "lbk_histogram_noalloc handles at most " + std::to_string(kNoAllocMaxNodes) + " nodes per call");
    LBK_EXPECT(a->n_features <= kNoAllocMaxFeatures,
               "lbk_histogram_noalloc handles at most " + std::to_string(kNoAllocMaxFeatures) + " features per call");
    int caller_device = -1;
    LBK_CUDA(cudaGetDevice(&caller_device));
    struct RestoreDevice {
      int d;
      ~RestoreDevice() { cudaSetDevice(d); }
    } restore{caller_device};
    LBK_CUDA(cudaSetDevice(device));
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    int32_t* scratch    = HistScratchAddress(device);
    int32_t* chunk_off  = scratch;
    int32_t* plan       = scratch + kNoAllocPlanOffset;
    int* max_abs        = reinterpret_cast<int*>(plan + 8);

    const int F = a->n_features, K = a->n_outputs, B = a->total_bins;
    int32_t rp[kNoAllocMaxFeatures + 1];
    LBK_CUDA(cudaMemcpyAsync(rp, a->row_ptr, sizeof(int32_t) * (F + 1), cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaStreamSynchronize(stream));
    LBK_EXPECT(rp[F] == B, "total_bins does not match row_ptr");
    int mb = 1;  // (max_bins is not needed here: row_ptr has been read back anyway)
    for (int f = 0; f < F; ++f) mb = rp[f + 1] - rp[f] > mb ? rp[f + 1] - rp[f] : mb;
    LBK_EXPECT(a->bin_bytes == 2 || mb <= 256, "one-byte bins need <= 256 proposals per feature");

    int sm_count = 0;
    LBK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));

    const bool float_mode = a->mode == 1;
    HistParams p;
    p.bins         = a->bins;
    p.n_rows       = a->n_rows;
    p.F            = F;
    p.K            = K;
    p.B            = B;
    p.G            = (F + kGroup - 1) / kGroup;
    p.row_ptr      = a->row_ptr;
    p.gpair        = float_mode ? static_cast<const void*>(a->gpair_f32) : static_cast<const void*>(a->gpair);
    p.row_index    = a->row_index;
    p.seg          = a->seg;
    p.slot_of_node = nullptr;
    p.n_nodes      = a->n_nodes;
    p.chunk_off    = chunk_off;
    p.plan         = plan;
    p.ticket       = reinterpret_cast<unsigned int*>(plan + 2);
    p.out          = a->hist;
    const bool smem_path = a->bin_bytes == 1 && mb <= kSmemBins;
    p.mb                 = smem_path ? mb : 0;
    const HistLaunch hl  = PickHistKernel(smem_path, a->bin_bytes, float_mode, p.G, sm_count);

    // the array keeps what the previous call left: clear the words that accumulate
    LBK_CUDA(cudaMemsetAsync(plan, 0, sizeof(int32_t) * 12, stream));
    LBK_CUDA(cudaMemsetAsync(a->hist, 0, sizeof(GPairI64) * a->n_nodes * K * B, stream));
    if (!float_mode && a->max_abs != nullptr) {
      max_abs = const_cast<int*>(reinterpret_cast<const int*>(a->max_abs));
    } else if (!float_mode) {
      const int64_t n = a->n_rows * K;
      if (n > 0) {
        k_max_abs<<<sm_count * 8, 256, 0, stream>>>(static_cast<const int2*>(p.gpair), n, max_abs);
        LBK_LAUNCH_CHECK();
      }
    }
    // no merge-tree slots here (they would have to be allocated): nodes cut into chunks flush with atomics
    p.wpre      = nullptr;
    p.arrive    = nullptr;
    p.partial   = nullptr;
    p.status    = nullptr;
    p.push_recv = nullptr;
    p.push_rank = 0;
    p.push_ranks = 1;
    p.push_slot_pairs = 0;
    p.push_len  = 0;
    p.pairs_by_position = a->pairs_by_position != 0 ? 1 : 0;
    k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, nullptr, p.n_nodes, (p.G + hl.width - 1) / hl.width * p.K, hl.grid,
                                        float_mode ? nullptr : max_abs, 0, chunk_off, nullptr, nullptr, 0, plan,
                                        p.ticket);
    LBK_LAUNCH_CHECK();
    hl.fn<<<hl.grid, hl.threads, hl.smem, stream>>>(p);
    LBK_LAUNCH_CHECK();
    LBK_CUDA(cudaStreamSynchronize(stream));
  });
}
