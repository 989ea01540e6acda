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
//   * work is cut into (node chunk, feature groups, output) tickets by a planner on the device
//     (k_hist_plan); blocks draw tickets from an atomic counter (persistent grid);
//   * a node in one chunk owns its output region and flushes with plain stores; a node cut into
//     several chunks leaves int32 partial sums in slots and k_hist_sum adds them up afterwards
//     (without slot memory: 64-bit global atomics); chunks of <= 128 rows skip shared memory.
#include <mutex>
#include <string>

#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

constexpr int kHistThreads = 512;
constexpr int kHistWarps   = kHistThreads / 32;
constexpr int kTileRows    = 32;    // chunk sizes are multiples of this
constexpr int kBatchRows   = 16;    // rows a warp takes per step of its pipeline (one per lane pair)
constexpr int kDirectRows  = 128;   // chunks up to this size go straight to global atomics
constexpr int kMinChunk    = 2048;
constexpr int kSmemBins    = 256;   // bins per feature held by the private histogram

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
  const int32_t* chunk_off;  // [n_nodes+1]
  const int32_t* part_off;   // [n_nodes+1] partial-sum slots before each node (nodes with > 1 chunk); may be null
  const int32_t* multi;      // [plan[5]] the nodes that were cut into several chunks; may be null
  const int32_t* plan;       // [0] rows per chunk, [1] total chunks, [3] rows between flushes, [5] nodes in
                             // `multi`, [6] slots usable
  unsigned int* ticket;
  cudaTextureObject_t tex_bins;   // the bin matrix as 16-byte texels, the pairs as 8-byte texels: the row
  cudaTextureObject_t tex_pairs;  // gathers then go through the texture data pipe; 0 = plain loads
  void* partial;             // partial-sum slots: [slot][2][mb * 32] of the accumulator type; may be null
  void* out;
};

__device__ inline unsigned SmemAddr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ inline void RedShared(unsigned addr, int v)
{
  asm volatile("red.shared.add.s32 [%0], %1;\n" ::"r"(addr), "r"(v) : "memory");
}
__device__ inline void RedShared(unsigned addr, float v)
{
  asm volatile("red.shared.add.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}

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

// Single block: how the rows of every built node are cut into chunks on this level.
//
// A ticket is (node chunk, feature group, output).  Resident blocks draw tickets from a counter, so
// the level takes about ceil(tickets / resident) rounds of the largest ticket, or (list scheduling)
// total work / resident + the largest ticket, whichever is smaller.  The planner evaluates that
// bound for "one chunk per node" and for a geometric ladder of chunk sizes, with a per-ticket
// overhead (clear, flush, partial sums) expressed in rows, and keeps the cheapest.  Chunks of a node
// are equal in size.  A node with several chunks needs one partial-sum slot per chunk and (feature
// group, output); candidates that need more slots than `slot_capacity` are not considered, and
// plan[6] says whether the chosen cut can use the slots (1) or has to flush with atomics (0).
constexpr int kPlanCandidates = 64;
constexpr int kPlanCachedNodes = 4096;
constexpr int kOverheadSingle = 2000;  // rows a block could have processed while it clears and flushes with stores
constexpr int kOverheadMulti  = 5000;  // the same for clear + partial store + its share of the final sum (measured)

__global__ void __launch_bounds__(1024)
  k_hist_plan(const int32_t* __restrict__ seg, const int32_t* __restrict__ slot_of_node, int n_nodes, int GK,
              int resident, const int* __restrict__ max_abs, long long slot_capacity, int32_t* __restrict__ chunk_off,
              int32_t* __restrict__ part_off, int32_t* __restrict__ multi, int32_t* __restrict__ plan,
              unsigned int* __restrict__ ticket)
{
  __shared__ long long red[32];
  __shared__ long long wsum[32];
  __shared__ long long carry;
  __shared__ long long total_s;
  __shared__ int ch_s, cap_s, mode_s, multi_s;
  __shared__ double cand_cost[kPlanCandidates];
  __shared__ int cand_ch[kPlanCandidates];
  __shared__ int cand_fit[kPlanCandidates];
  __shared__ int rows_s[kPlanCachedNodes];  // rows of the first nodes (0 for nodes that are not built)
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
  auto rows_global = [&](int j) -> int {
    const bool built = slot_of_node == nullptr || slot_of_node[j] >= 0;
    const int r      = seg[j + 1] - seg[j];
    return built ? r : 0;
  };
  // every later pass reads the node sizes many times: from shared memory where they fit
  auto rows_of = [&](int j) -> int { return j < kPlanCachedNodes ? rows_s[j] : rows_global(j); };
  long long rows = 0;
  for (int j = tid; j < n_nodes; j += blockDim.x) {
    const int r = rows_global(j);
    if (j < kPlanCachedNodes) rows_s[j] = r;
    rows += r;
  }
  for (int off = 16; off >= 1; off >>= 1) rows += __shfl_down_sync(0xffffffffu, rows, off);
  if (lane == 0) red[warp] = rows;
  __syncthreads();
  if (tid == 0) {
    long long total = 0;
    for (int w = 0; w < n_warps; ++w) total += red[w];
    total_s = total;
    int m   = 1;
    if (max_abs) m = max(1, max(max_abs[0], max_abs[1]));
    const int safe = max_abs ? 2147483647 / m : 2147483647;
    plan[3]        = safe;
    // chunks that can use partial-sum slots never need a flush in the middle
    cap_s = safe >= (1 << 30) ? (1 << 30) : (safe & ~(kTileRows - 1));
    carry = 0;
    multi_s = 0;
    chunk_off[0] = 0;
    if (part_off) part_off[0] = 0;
  }
  __syncthreads();
  const long long total = total_s;
  const int cap         = cap_s;

  // candidate 0: one chunk per node; candidate c > 0: total work / (resident * 2^(c / 16)) rows
  for (int c = warp; c < kPlanCandidates; c += n_warps) {
    long long ch = 1ll << 30;
    if (c > 0) {
      const double f = exp2(static_cast<double>(c - 1) / 16.0);
      ch             = static_cast<long long>(static_cast<double>(total) * GK / (static_cast<double>(resident) * f)) + 1;
      if (ch < kMinChunk) ch = kMinChunk;
      ch = (ch + kTileRows - 1) / kTileRows * kTileRows;
      if (ch > (1ll << 30)) ch = 1ll << 30;
    }
    const long long chs = cap >= kTileRows && ch > cap ? cap : ch;  // with slots: never beyond the safe count
    long long tickets = 0, multi = 0, cost = 0;
    int biggest = 0;
    for (int j = lane; j < n_nodes; j += 32) {
      const int r = rows_of(j);
      if (r <= 0) continue;
      const int nch  = static_cast<int>((r + chs - 1) / chs);
      const int size = (r + nch - 1) / nch + (nch > 1 ? kOverheadMulti : kOverheadSingle);
      tickets += nch;
      if (nch > 1) multi += nch;
      cost += static_cast<long long>(size) * nch;
      biggest = max(biggest, size);
    }
    for (int off = 16; off >= 1; off >>= 1) {
      tickets += __shfl_down_sync(0xffffffffu, tickets, off);
      multi += __shfl_down_sync(0xffffffffu, multi, off);
      cost += __shfl_down_sync(0xffffffffu, cost, off);
      biggest = max(biggest, __shfl_down_sync(0xffffffffu, biggest, off));
    }
    if (lane == 0) {
      const double T      = static_cast<double>(tickets) * GK;
      const double rounds = ceil(T / resident) * biggest;
      const double list   = static_cast<double>(cost) * GK / resident + biggest;
      cand_cost[c]        = rounds < list ? rounds : list;
      cand_ch[c]          = static_cast<int>(chs);
      cand_fit[c]         = multi * GK <= slot_capacity;
    }
  }
  __syncthreads();
  if (tid == 0) {
    int best = -1;
    for (int c = 0; c < kPlanCandidates; ++c)
      if (slot_capacity > 0 && cap >= kTileRows && cand_fit[c] && (best < 0 || cand_cost[c] < cand_cost[best] * 0.98)) best = c;
    if (best >= 0) {
      ch_s   = cand_ch[best];
      mode_s = 1;
    } else {
      // no slots (or too few even for one chunk per node): the cut of the first candidates that
      // gives every resident block about one ticket, flushed with atomics
      long long ch = (total * GK + resident - 1) / resident;
      long long nodes = 0;
      for (int j = 0; j < n_nodes; ++j) nodes += rows_of(j) > 0;
      if (nodes * GK >= resident) ch = 1ll << 30;
      if (ch < kMinChunk) ch = kMinChunk;
      ch = (ch + kTileRows - 1) / kTileRows * kTileRows;
      if (ch > (1ll << 30)) ch = 1ll << 30;
      ch_s   = static_cast<int>(ch);
      mode_s = 0;
    }
  }
  __syncthreads();
  const int ch = ch_s;
  // exclusive scans over the nodes: chunks (low word) and partial-sum slots (high word)
  for (int base = 0; base < n_nodes; base += blockDim.x) {
    const int j = base + tid;
    long long c = 0;
    if (j < n_nodes) {
      const int r   = rows_of(j);
      const int nch = r > 0 ? (r + ch - 1) / ch : 0;
      c             = nch + (nch > 1 ? (static_cast<long long>(nch) << 32) : 0);
      if (nch > 1 && multi) multi[atomicAdd(&multi_s, 1)] = j;
    }
    long long incl = c;
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
    if (j < n_nodes) {
      chunk_off[j + 1] = static_cast<int>((before + incl) & 0xffffffffll);
      if (part_off) part_off[j + 1] = static_cast<int>((before + incl) >> 32);
    }
    __syncthreads();
    if (tid == blockDim.x - 1) carry = before + incl;
    __syncthreads();
  }
  if (tid == 0) {
    plan[0] = ch;
    plan[1] = static_cast<int>(carry & 0xffffffffll);
    plan[5] = multi_s;
    plan[6] = mode_s;
    *ticket = 0;
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
  using wide_t = long long;
  __device__ static long long widen(int bits) { return bits; }
  __device__ static void add_wide(out_t* dst, long long g, long long h)
  {
    atomicAdd(reinterpret_cast<unsigned long long*>(&dst->grad), static_cast<unsigned long long>(g));
    atomicAdd(reinterpret_cast<unsigned long long*>(&dst->hess), static_cast<unsigned long long>(h));
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
  using wide_t = double;
  __device__ static double widen(int bits) { return static_cast<double>(__int_as_float(bits)); }
  __device__ static void add_wide(out_t* dst, double g, double h)
  {
    atomicAdd(&dst->grad, g);
    atomicAdd(&dst->hess, h);
  }
};

// What a chunk index means: the node, the chunk's place in it, the rows.
struct Chunk {
  int j, ci, nchunks, slot, rb, re;
};

__device__ inline Chunk DecodeChunk(const HistParams& p, int c)
{
  // node that owns chunk c: last j with chunk_off[j] <= c
  int lo = 0, hi = p.n_nodes;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (p.chunk_off[mid] <= c) lo = mid; else hi = mid;
  }
  Chunk ch;
  ch.j       = lo;
  ch.nchunks = p.chunk_off[lo + 1] - p.chunk_off[lo];
  ch.slot    = p.slot_of_node ? p.slot_of_node[lo] : lo;
  ch.ci      = c - p.chunk_off[lo];
  // the chunks of a node are equal in size (a multiple of 32 rows, the last one takes the rest)
  const int nrows = p.seg[lo + 1] - p.seg[lo];
  const int size  = ch.nchunks > 1 ? ((nrows + ch.nchunks - 1) / ch.nchunks + kTileRows - 1) / kTileRows * kTileRows : nrows;
  ch.rb = min(p.seg[lo + 1], p.seg[lo] + ch.ci * size);
  ch.re = min(p.seg[lo + 1], ch.rb + size);
  return ch;
}

// Rows [b, e) of one node, features [f0, f0 + 32 * groups): one lane per feature, the warps of the
// block stride over the rows, every update is a pair of 64-bit global atomics.
template <typename BinT, typename A>
__device__ inline void DirectRows(const HistParams& p, int b, int e, int f0, int groups, int k,
                                  typename A::out_t* onode, int warp, int n_warps, int lane)
{
  using in_t          = typename A::in_t;
  const BinT* bins    = static_cast<const BinT*>(p.bins);
  const in_t* gpair   = static_cast<const in_t*>(p.gpair);
  const int64_t pitch = static_cast<int64_t>(p.G) * kGroup;
  for (int u = 0; u < groups; ++u) {
    const int feat = f0 + u * kGroup + lane;
    if (feat >= p.F) continue;
    typename A::out_t* obase = onode + p.row_ptr[feat];
    for (int r = b + warp; r < e; r += n_warps) {
      const int ridx = p.row_index[r];
      const in_t v   = gpair[static_cast<int64_t>(ridx) * p.K + k];
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
    const Chunk ch = DecodeChunk(p, static_cast<int>(t / (static_cast<long long>(p.K) * p.G)));
    typename A::out_t* onode = static_cast<typename A::out_t*>(p.out) + (static_cast<int64_t>(ch.slot) * p.K + k) * p.B;
    DirectRows<BinT, A>(p, ch.rb, ch.re, g * kGroup, 1, k, onode, warp, kHistWarps, lane);
  }
}

// One-byte bins, at most 256 per feature: private histograms in shared memory.
//
// W = 1: a ticket covers one 32-feature group, 512 threads, two blocks per SM.
// W = 2: a ticket covers two neighbouring groups (64 features), 1024 threads, one block per SM.
// The wide form exists because the load/store pipe of the SM spends one pass per distinct
// 128-byte line a gather touches, however few bytes it takes from it: with 64 bin bytes per row
// the row gather costs half as many passes per update, and the row ids and gradient pairs are
// fetched once for two groups.
//
// Every warp runs its own pipeline over batches of 32 / (2 W) rows (no block barrier inside, no
// staging in shared memory).  2 W lanes own one row of the batch and load its bin bytes straight
// from global memory into registers, 16 bytes per lane.  In step j of 16 the lanes of row slot r
// handle byte (j xor r) of their 16, and the histogram words of a bin are laid out so that the 32
// lanes of a warp always update 32 different banks, whatever the bins:
//   W = 1 (r < 16, quarter q < 2):  word = 16 q + byte                   (bank = word)
//   W = 2 (r < 8,  quarter q < 4):  word = 32 (byte / 8) + 8 q + byte % 8 (bank = 8 q + byte % 8)
// The bytes are permuted once per batch (a word swap and one byte permute per word) so that step
// j reads the static byte j.  Per 32 updates that leaves the two reductions on the pipe.
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
  constexpr int kLanesPerRow  = 2 * W;
  constexpr int kRowsPerBatch = 32 / kLanesPerRow;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // the column arithmetic of the main loop needs the histogram on a 256-byte boundary
  smem_t* hg = reinterpret_cast<smem_t*>(smem_raw + ((256u - (SmemAddr(smem_raw) & 255u)) & 255u));
  smem_t* hh = hg + kSmemBins * kCols;  // every byte value is a valid bin row
  __shared__ unsigned int s_ticket;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int total_chunks = p.plan[1];
  const int rows_safe    = p.plan[3];
  const bool use_slots   = p.plan[6] != 0 && p.partial != nullptr;
  const int GP           = (p.G + W - 1) / W;  // tickets per chunk and output
  const long long total  = static_cast<long long>(total_chunks) * GP * p.K;
  const in_t* gpair      = static_cast<const in_t*>(p.gpair);
  const int hist_words   = p.mb * kCols;
  const int64_t pitch    = static_cast<int64_t>(p.G) * kGroup;  // bins are row-major, rows padded to whole groups
  // feature (relative to the ticket's first) of histogram word w
  auto feature_of_word = [](int w) -> int { return W == 1 ? w : 16 * ((w >> 3) & 3) + 8 * (w >> 5) + (w & 7); };

  while (true) {
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
    __syncthreads();
    const long long t = s_ticket;
    if (t >= total) break;
    const int k    = static_cast<int>(t % p.K);
    const int gp   = static_cast<int>((t / p.K) % GP);
    const Chunk ch = DecodeChunk(p, static_cast<int>(t / (static_cast<long long>(p.K) * GP)));
    const int g0   = gp * W;
    const int groups = min(W, p.G - g0);
    out_t* onode   = static_cast<out_t*>(p.out) + (static_cast<int64_t>(ch.slot) * p.K + k) * p.B;

    // a chunk that will leave partial sums in a slot cannot take the direct path: the last
    // chunk of its node stores the total and would overwrite what the atomics added
    const bool slots = use_slots && ch.nchunks > 1 && rows_safe >= kTileRows;
    if (rows_safe < kTileRows || (ch.re - ch.rb <= kDirectRows && !slots)) {
      DirectRows<uint8_t, A>(p, ch.rb, ch.re, g0 * kGroup, groups, k, onode, warp, kWarps, lane);
      continue;
    }

    // the word a thread meets in the strided loops below is always the same one
    const int my_word  = tid % kCols;
    const int my_feat  = g0 * kGroup + feature_of_word(my_word);
    const int my_fbeg  = my_feat < p.F ? p.row_ptr[my_feat] : 0;
    const int my_fbins = my_feat < p.F ? p.row_ptr[my_feat + 1] - my_fbeg : 0;
    bool use_atomics   = ch.nchunks > 1 && !slots;
    auto flush = [&](bool atomics) {
      out_t* obase = onode + my_fbeg;
      for (int e = tid; e < hist_words; e += kThreads) {  // e % kCols == my_word for every e of a thread
        const int bin = e / kCols;
        if (bin < my_fbins) {
          const smem_t vg = hg[e], vh = hh[e];
          if (A::nonzero(vg, vh)) {
            if (atomics) A::add_global(obase + bin, vg, vh); else A::store_global(obase + bin, vg, vh);
          }
        }
      }
    };
    auto zero = [&]() {
      for (int e = tid; e < hist_words; e += kThreads) {
        hg[e] = smem_t(0);
        hh[e] = smem_t(0);
      }
    };
    zero();
    __syncthreads();

    const unsigned rslot    = lane / kLanesPerRow, q = lane % kLanesPerRow;
    const bool lane_on      = static_cast<int>(q >> 1) < groups;  // the group this lane's 16 bytes belong to exists
    const unsigned wsel     = rslot >> 2, bsel = rslot & 3;
    const unsigned perm     = bsel == 0 ? 0x3210u : bsel == 1 ? 0x2301u : bsel == 2 ? 0x1032u : 0x0123u;
    const unsigned lanebase = SmemAddr(hg) + (W == 1 ? 16 * q + rslot : 8 * q + rslot) * 4;
    const unsigned hh_off   = static_cast<unsigned>(kSmemBins) * kCols * 4;
    const unsigned char* gb = static_cast<const unsigned char*>(p.bins) + g0 * kGroup + q * 16;
    const int seg_rows = rows_safe >= (1 << 30) ? (1 << 30) : (rows_safe & ~31);
    for (int sb = ch.rb; sb < ch.re; sb += seg_rows) {
      const int se = min(ch.re, sb + seg_rows);
      if (sb > ch.rb) {
        __syncthreads();
        flush(true);
        use_atomics = true;
        __syncthreads();
        zero();
        __syncthreads();
      }
      const int nb = (se - sb + kRowsPerBatch - 1) / kRowsPerBatch;
      auto load_rid = [&](int batch) -> int {
        const int r = sb + batch * kRowsPerBatch + static_cast<int>(rslot);
        return (batch < nb && r < se && lane_on) ? __ldcg(p.row_index + r) : -1;
      };
      // rows beyond the end carry zero pairs and bin 0: they add nothing
      auto load_row = [&](int rid, int4& w, int2& v) {
        if (rid >= 0) {
          // through the texture pipe where the buffers have texture objects: the load/store pipe,
          // which the reductions saturate, is spared the gathers
          if (p.tex_bins != 0) {
            w = tex1Dfetch<int4>(p.tex_bins, static_cast<int>((static_cast<int64_t>(rid) * pitch + g0 * kGroup + q * 16) >> 4));
          } else {
            w = __ldcs(reinterpret_cast<const int4*>(gb + static_cast<int64_t>(rid) * pitch));
          }
          if (p.tex_pairs != 0) {
            v = tex1Dfetch<int2>(p.tex_pairs, static_cast<int>(static_cast<int64_t>(rid) * p.K + k));
          } else {
            v = __ldcg(reinterpret_cast<const int2*>(gpair + static_cast<int64_t>(rid) * p.K + k));
          }
        } else {
          w = make_int4(0, 0, 0, 0);
          v = make_int2(0, 0);
        }
      };
      auto consume = [&](const int4& w, const int2& v) {
        unsigned x[4];
        x[0] = (wsel & 1) ? w.y : w.x;
        x[1] = (wsel & 1) ? w.x : w.y;
        x[2] = (wsel & 1) ? w.w : w.z;
        x[3] = (wsel & 1) ? w.z : w.w;
        if (W == 1 && (wsel & 2)) {
          unsigned t2 = x[0]; x[0] = x[2]; x[2] = t2;
          t2 = x[1]; x[1] = x[3]; x[3] = t2;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = __byte_perm(x[i], 0u, perm);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const unsigned bin  = __byte_perm(x[j >> 2], 0u, 0x4440u | (j & 3));
          const unsigned cj   = W == 1 ? 4u * j : (((j & 7u) << 2) | ((j >> 3) << 7));
          const unsigned addr = (bin * (kCols * 4) + lanebase) ^ cj;
          if (kFloat) {
            RedShared(addr, __int_as_float(v.x));
            RedShared(addr + hh_off, __int_as_float(v.y));
          } else {
            RedShared(addr, v.x);
            RedShared(addr + hh_off, v.y);
          }
        }
      };
      // in flight per warp: the rows of the next two batches and the row ids of the two after
      int4 w0, w1, w2;
      int2 v0, v1, v2;
      load_row(load_rid(warp), w0, v0);
      load_row(load_rid(warp + kWarps), w1, v1);
      int rid_a = load_rid(warp + 2 * kWarps);
      int rid_b = load_rid(warp + 3 * kWarps);
      for (int b = warp; b < nb; b += kWarps) {
        load_row(rid_a, w2, v2);  // batch b + 2 * kWarps
        rid_a = rid_b;
        rid_b = load_rid(b + 4 * kWarps);
        consume(w0, v0);
        w0 = w1; v0 = v1;
        w1 = w2; v1 = v2;
      }
    }
    __syncthreads();
    if (!slots) {
      flush(use_atomics);
      continue;
    }
    // Several chunks of this node: every chunk leaves its sums in a slot; k_hist_sum adds the slots
    // up afterwards and stores the total (no atomics on the histogram itself).
    smem_t* part        = static_cast<smem_t*>(p.partial);
    const size_t stride = static_cast<size_t>(hist_words) * 2;
    const size_t first  = ((static_cast<size_t>(p.part_off[ch.j]) * p.K + k) * GP + gp);  // slot of chunk 0
    const size_t step   = static_cast<size_t>(p.K) * GP;                                  // slot distance between chunks
    smem_t* mine        = part + (first + ch.ci * step) * stride;
    const int n4        = hist_words >> 2;  // 16-byte pieces: four neighbouring features of one bin
    for (int e4 = tid; e4 < n4; e4 += kThreads) {
      __stcg(reinterpret_cast<int4*>(mine) + e4, reinterpret_cast<const int4*>(hg)[e4]);
      __stcg(reinterpret_cast<int4*>(mine + hist_words) + e4, reinterpret_cast<const int4*>(hh)[e4]);
    }
  }
}

// Adds up the partial-sum slots of every node that was cut into several chunks and adds the
// totals to the (zeroed) histogram.  A work item is one (node of the `multi` list, group set,
// output), 1/kSumSplits of its histogram words and 1/kSumParts of its slots; the blocks of a
// fixed-size grid take items in turn (no items, no work).  A thread reads 16 bytes of every slot of
// the item's part (four neighbouring features of one bin), four slots in flight, and finishes with
// one pair of 64-bit atomics per feature (kSumParts items meet in every word).
constexpr int kSumSplits  = 16;
constexpr int kSumParts   = 8;
constexpr int kSumThreads = 256;

template <bool kFloat, int W>
__global__ void __launch_bounds__(kSumThreads)
  k_hist_sum(const HistParams p)
{
  using A      = Acc<kFloat>;
  using smem_t = typename A::smem_t;
  using out_t  = typename A::out_t;
  constexpr int kCols = kGroup * W;
  if (p.plan[6] == 0) return;
  const int GP         = (p.G + W - 1) / W;
  const long long items = static_cast<long long>(p.plan[5]) * GP * p.K * kSumSplits * kSumParts;
  const int hist_words = p.mb * kCols;
  const int n4         = hist_words >> 2;
  const smem_t* part   = static_cast<const smem_t*>(p.partial);
  const size_t stride  = static_cast<size_t>(hist_words) * 2;
  const size_t step    = static_cast<size_t>(p.K) * GP;
  for (long long item = blockIdx.x; item < items; item += gridDim.x) {
    const int zpart = static_cast<int>(item % kSumParts);
    const int split = static_cast<int>((item / kSumParts) % kSumSplits);
    const long long t = item / (kSumParts * kSumSplits);
    const int k  = static_cast<int>(t % p.K);
    const int gp = static_cast<int>((t / p.K) % GP);
    const int j  = p.multi[t / (static_cast<long long>(p.K) * GP)];
    const int nchunks = p.chunk_off[j + 1] - p.chunk_off[j];
    const int per = (nchunks + kSumParts - 1) / kSumParts;
    const int qb  = zpart * per, qe = min(nchunks, qb + per);
    if (qb >= qe) continue;
    const int slot     = p.slot_of_node ? p.slot_of_node[j] : j;
    const size_t first = (static_cast<size_t>(p.part_off[j]) * p.K + k) * GP + gp;
    out_t* onode       = static_cast<out_t*>(p.out) + (static_cast<int64_t>(slot) * p.K + k) * p.B;
    for (int e4 = split * kSumThreads + threadIdx.x; e4 < n4; e4 += kSumSplits * kSumThreads) {
      typename A::wide_t sg[4], sh[4];
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) sg[c4] = sh[c4] = 0;
      for (int q0 = qb; q0 < qe; q0 += 4) {
        int4 vg[4], vh[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (q0 + u < qe) {
            const smem_t* src = part + (first + (q0 + u) * step) * stride;
            vg[u] = __ldcg(reinterpret_cast<const int4*>(src) + e4);
            vh[u] = __ldcg(reinterpret_cast<const int4*>(src + hist_words) + e4);
          } else {
            vg[u] = vh[u] = make_int4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          sg[0] += A::widen(vg[u].x); sg[1] += A::widen(vg[u].y); sg[2] += A::widen(vg[u].z); sg[3] += A::widen(vg[u].w);
          sh[0] += A::widen(vh[u].x); sh[1] += A::widen(vh[u].y); sh[2] += A::widen(vh[u].z); sh[3] += A::widen(vh[u].w);
        }
      }
      const int bin = (e4 * 4) / kCols, w0 = (e4 * 4) % kCols;
      const int f0  = (gp * W) * kGroup + (W == 1 ? w0 : 16 * ((w0 >> 3) & 3) + 8 * (w0 >> 5) + (w0 & 7));
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const int f = f0 + c4;
        if (f >= p.F) continue;
        const int fbeg = p.row_ptr[f];
        if (bin < p.row_ptr[f + 1] - fbeg && (sg[c4] != 0 || sh[c4] != 0)) A::add_wide(onode + fbeg + bin, sg[c4], sh[c4]);
      }
    }
  }
}

// ---- row grouping (utility for the stage-level API) -------------------------------------------
constexpr int kGroupTile = 4096;

// Kernel, dynamic shared memory and persistent grid (resident blocks of the whole device, from the
// occupancy calculator) for one combination of bin width, pair type and path.
struct HistLaunch {
  void (*fn)(HistParams);
  void (*sum)(HistParams);  // adds up partial-sum slots; null for the kernels that have none
  size_t smem;
  int threads;
  int grid;
  int width;  // feature groups per ticket
};

HistLaunch PickHistKernel(bool smem_path, int bin_bytes, bool float_mode, int n_groups, int sm_count)
{
  HistLaunch h;
  h.width   = smem_path && n_groups >= 2 ? 2 : 1;
  h.threads = kHistThreads * h.width;
  h.smem    = smem_path ? static_cast<size_t>(kSmemBins) * kGroup * h.width * 8 + 256 : 0;
  h.sum = nullptr;
  if (smem_path && h.width == 2) {
    h.fn  = float_mode ? k_hist_smem<true, 2> : k_hist_smem<false, 2>;
    h.sum = float_mode ? k_hist_sum<true, 2> : k_hist_sum<false, 2>;
  } else if (smem_path) {
    h.fn  = float_mode ? k_hist_smem<true, 1> : k_hist_smem<false, 1>;
    h.sum = float_mode ? k_hist_sum<true, 1> : k_hist_sum<false, 1>;
  }
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
  p.out              = lv.out;

  const bool smem_path = lv.bin_bytes == 1 && lv.max_bins_per_feature <= kSmemBins;
  p.mb                 = smem_path ? lv.max_bins_per_feature : 0;
  p.tex_bins           = 0;
  p.tex_pairs          = 0;
  // (measured: the float path, bound by its float reductions, is slower with the texture fetches)
  if (smem_path && lv.n_rows > 0 && !lv.float_mode) {
    p.tex_bins  = LinearTexture(ctx, lv.bins, static_cast<size_t>(lv.n_rows) * p.G * kGroup, 16);
    p.tex_pairs = LinearTexture(ctx, p.gpair, static_cast<size_t>(lv.n_rows) * lv.K * 8, 8);
  }
  const HistLaunch hl  = PickHistKernel(smem_path, lv.bin_bytes, lv.float_mode, p.G, ctx->sm_count - (lv.reserve_sms < ctx->sm_count ? lv.reserve_sms : 0));

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
  const int tickets_per_chunk = (p.G + hl.width - 1) / hl.width * p.K;
  // partial-sum slots for nodes that are cut into several chunks: ten per resident block
  long long slot_capacity = 0;
  p.part_off = nullptr;
  p.multi    = nullptr;
  p.partial  = nullptr;
  if (smem_path) {
    slot_capacity           = 10ll * hl.grid;
    const size_t slot_bytes = static_cast<size_t>(p.mb) * kGroup * hl.width * 8;
    int32_t* part_off       = s.alloc<int32_t>(static_cast<size_t>(lv.n_nodes) + 1);
    int32_t* multi          = s.alloc<int32_t>(static_cast<size_t>(lv.n_nodes));
    p.part_off              = part_off;
    p.multi                 = multi;
    p.partial               = s.alloc<unsigned char>(slot_bytes * slot_capacity);
    k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, p.slot_of_node, p.n_nodes, tickets_per_chunk, hl.grid,
                                        lv.float_mode ? nullptr : max_abs, slot_capacity, chunk_off, part_off,
                                        multi, plan, p.ticket);
  } else {
    k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, p.slot_of_node, p.n_nodes, tickets_per_chunk, hl.grid,
                                        lv.float_mode ? nullptr : max_abs, 0, chunk_off, nullptr, nullptr, plan,
                                        p.ticket);
  }
  LBK_LAUNCH_CHECK();
  if (ctx->profile) LBK_CUDA(cudaEventRecord(ctx->ev_start, stream));
  hl.fn<<<hl.grid, hl.threads, hl.smem, stream>>>(p);
  LBK_LAUNCH_CHECK();
  if (p.partial) {
    hl.sum<<<ctx->sm_count * 8, kSumThreads, 0, stream>>>(p);
    LBK_LAUNCH_CHECK();
  }
  if (ctx->profile) {
    LBK_CUDA(cudaEventRecord(ctx->ev_stop, stream));
    ctx->profile_recorded = true;
  }
  // stream ordered: the slots go back to the pool once the kernel has run
  if (p.partial) s.free_one(p.partial);
}

void BuildHistogramAllReduce(lbk_context* ctx, Scratch& s, const HistLevel& lv, int n_slots, bool pairs,
                             cudaStream_t stream)
{
  const size_t slot_words = static_cast<size_t>(lv.K) * lv.B * 2;  // 64-bit words per slot
  const lbk_dtype dtype   = lv.float_mode ? LBK_F64 : LBK_I64;
  if (ctx->n_ranks <= 1) {
    if (lv.n_rows > 0) BuildHistogram(ctx, s, lv, stream);
    return;
  }
  // Parts: only with NCCL (a callback communicator is not known to be stream-safe), only when every
  // part still has a ticket for every resident block, and only when there is something to hide.
  constexpr int kReserve = 20;  // SMs left to the all-reduce kernel
  const int G            = (lv.F + kGroup - 1) / kGroup;
  const bool smem_path   = lv.bin_bytes == 1 && lv.max_bins_per_feature <= kSmemBins;
  const int width        = smem_path && G >= 2 ? 2 : 1;
  const long long tickets = static_cast<long long>(lv.n_nodes) / (pairs ? 2 : 1) * ((G + width - 1) / width) * lv.K;
  const int resident     = (ctx->sm_count - kReserve) * (width == 2 ? 1 : 2);
  int parts              = static_cast<int>(tickets / (resident > 0 ? resident : 1));
  if (parts > 4) parts = 4;
  if (ctx->cb != nullptr || ctx->nccl_comm == nullptr || !smem_path || lv.n_rows <= 0 ||
      static_cast<size_t>(n_slots) * slot_words * 8 < (size_t{8} << 20))
    parts = 1;
  if (parts <= 1) {
    if (lv.n_rows > 0) BuildHistogram(ctx, s, lv, stream);
    AllReduce(ctx, lv.out, static_cast<size_t>(n_slots) * slot_words, dtype, LBK_SUM, stream);
    return;
  }
  if (ctx->comm_stream == nullptr) {
    int lo = 0, hi = 0;
    LBK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    LBK_CUDA(cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking, hi));
    for (cudaEvent_t& e : ctx->ev_part) LBK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    LBK_CUDA(cudaEventCreateWithFlags(&ctx->ev_comm_done, cudaEventDisableTiming));
  }
  const int unit = pairs ? 2 : 1;  // nodes per slot
  // the optional timing covers the histogram kernels of all parts (they run back to back)
  const bool timed = ctx->profile;
  ctx->profile     = false;
  if (timed) LBK_CUDA(cudaEventRecord(ctx->ev_start, stream));
  for (int i = 0; i < parts; ++i) {
    // node range of the part, on slot boundaries
    const int s0 = static_cast<int>(static_cast<long long>(n_slots) * i / parts);
    const int s1 = static_cast<int>(static_cast<long long>(n_slots) * (i + 1) / parts);
    if (s1 <= s0) continue;
    HistLevel sub       = lv;
    sub.seg_node_offset = lv.seg_node_offset + s0 * unit;
    sub.n_nodes         = (s1 - s0) * unit;
    sub.reserve_sms     = kReserve;
    if (lv.slot_of_node != nullptr) {
      sub.slot_of_node = lv.slot_of_node + s0 * unit;  // absolute slots: `out` stays the base
    } else {
      sub.out = static_cast<unsigned char*>(lv.out) + static_cast<size_t>(s0) * slot_words * 8;
    }
    BuildHistogram(ctx, s, sub, stream);
    if (timed && i == parts - 1) {
      LBK_CUDA(cudaEventRecord(ctx->ev_stop, stream));
      ctx->profile_recorded = true;
    }
    LBK_CUDA(cudaEventRecord(ctx->ev_part[i], stream));
    LBK_CUDA(cudaStreamWaitEvent(ctx->comm_stream, ctx->ev_part[i], 0));
    // every part but the last has the next part's kernel beside it
    AllReduce(ctx, static_cast<unsigned char*>(lv.out) + static_cast<size_t>(s0) * slot_words * 8,
              static_cast<size_t>(s1 - s0) * slot_words, dtype, LBK_SUM, ctx->comm_stream, i + 1 < parts);
  }
  ctx->profile = timed;
  LBK_CUDA(cudaEventRecord(ctx->ev_comm_done, ctx->comm_stream));
  LBK_CUDA(cudaStreamWaitEvent(stream, ctx->ev_comm_done, 0));
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
// Who needs it: code that runs where cudaMalloc / cudaFree are off limits - inside a stream
// callback or another thread's critical section where the allocator's implicit device
// synchronisation would deadlock or stall every stream, under a memory budget that a runtime
// has already handed out completely (a task variant registered without the right to allocate),
// or in a process that wants its device footprint fixed after start-up.  lbk_histogram takes its
// per-call scratch (chunk offsets, the level plan, the largest magnitudes) from the context's
// pool; this entry point keeps that scratch in a fixed array inside the library image instead
// and needs no context at all.
//
// Limits and rules
//   * at most LBK_NOALLOC_MAX_NODES nodes and LBK_NOALLOC_MAX_FEATURES features per call,
//     device pointers only (host_buffers must be 0); larger calls are rejected with
//     LBK_ERR_ARGUMENT before anything is launched;
//   * the array (about 16 KB) exists once per GPU that loads the library, until the process ends;
//   * the first call on a device looks the array's device address up (the array's name is only a
//     host-side handle; kernels get the address found here).  Make that first call before any
//     stream capture;
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
    LBK_EXPECT(a->bins && a->row_ptr && a->row_index && a->seg && a->hist, "null argument");
    LBK_EXPECT(a->mode == 0 || a->mode == 1, "mode must be 0 or 1");
    LBK_EXPECT(a->mode == 0 ? a->gpair != nullptr : a->gpair_f32 != nullptr, "missing gradient pairs");
    LBK_EXPECT(a->bin_bytes == 1 || a->bin_bytes == 2, "bin_bytes must be 1 or 2");
    LBK_EXPECT(a->n_features >= 1 && a->n_outputs >= 1 && a->total_bins >= a->n_features, "bad shape");
    LBK_EXPECT(a->n_nodes >= 1 && a->n_nodes <= kNoAllocMaxNodes,
               "lbk_histogram_noalloc handles at most " + std::to_string(kNoAllocMaxNodes) + " nodes per call");
    LBK_EXPECT(a->n_features <= kNoAllocMaxFeatures,
               "lbk_histogram_noalloc handles at most " + std::to_string(kNoAllocMaxFeatures) + " features per call");
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
    int mb = 1;
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
    // no partial-sum slots here (they would have to be allocated): nodes cut into chunks flush with atomics
    p.part_off  = nullptr;
    p.multi     = nullptr;
    p.partial   = nullptr;
    p.tex_bins  = 0;  // texture objects belong to a context; this entry point has none
    p.tex_pairs = 0;
    k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, nullptr, p.n_nodes, (p.G + hl.width - 1) / hl.width * p.K, hl.grid,
                                        float_mode ? nullptr : max_abs, 0, chunk_off, nullptr, nullptr, plan, p.ticket);
    LBK_LAUNCH_CHECK();
    hl.fn<<<hl.grid, hl.threads, hl.smem, stream>>>(p);
    LBK_LAUNCH_CHECK();
    LBK_CUDA(cudaStreamSynchronize(stream));
  });
}
