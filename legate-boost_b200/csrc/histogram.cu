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
//   * bins are one byte per element in groups of 32 features (see proposals.cu); a warp handles
//     one row at a time with ONE LANE PER FEATURE, and the private histogram is laid out
//     [bin][lane]: lane l always hits shared-memory bank l, so the two atomics a warp issues per
//     row are conflict free whatever the bins are, and no two lanes of a warp share an address;
//   * the kernel is bound by the load/store pipe of the SM, not by HBM: the two reductions a warp
//     issues per row are unavoidable (64-bit shared atomics are compare-and-swap loops on this
//     part), so everything else is kept small: per row one byte load (the lane's bin) and half a
//     broadcast 16-byte load (the pairs of two rows);
//   * every warp runs its own pipeline over 32-row batches (no block barrier in the main loop):
//     the rows of a node are scattered, so each 32-byte row of a group is its own gather; the bins
//     of the warp's next batch travel global -> shared asynchronously (cp.async.cg, 16 bytes per
//     lane, one instruction moves 16 rows and bypasses the small L1 left beside the histograms)
//     into a two-deep per-warp ring, the pairs of that batch wait in one register pair per lane,
//     and the row ids of the batch after that are being loaded; with 32 warps per SM that keeps
//     64 KB per SM in flight;
//   * accumulation is in int32 like the reference, but guarded: with m = the largest |q| of the
//     call, at most floor((2^31-1)/m) rows are accumulated between flushes, so no partial sum can
//     wrap whatever the bins are;
//   * work is cut into (node, row chunk, feature group, output) tickets sized on the device:
//     one chunk per node when the level has at least as many (node, group, output) triples as
//     resident blocks, else chunks that give every resident block about one ticket; blocks draw
//     tickets from an atomic counter (persistent grid, two 512-thread blocks per SM);
//   * a node whose rows fit one chunk owns its output region and flushes with plain stores;
//     otherwise the flush uses 64-bit global atomics; chunks of <= 128 rows skip shared memory.
#include <cstdlib>
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
  const int32_t* plan;       // [0] rows per chunk, [1] total chunks, [3] rows between flushes
  unsigned int* ticket;
  void* out;
};

__device__ inline void CpAsync16(unsigned smem_dst, const void* gsrc)
{
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ inline void CpAsyncCommit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ inline void CpAsyncWait()
{
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ inline unsigned LdsU8(unsigned addr)
{
  unsigned v;
  asm volatile("ld.shared.u8 %0, [%1];\n" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ inline int2 LdsV2(unsigned addr)
{
  int2 v;
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr) : "memory");
  return v;
}
__device__ inline void StsV2(unsigned addr, int2 v)
{
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(addr), "r"(v.x), "r"(v.y) : "memory");
}
__device__ inline unsigned SmemAddr(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }
__device__ inline int4 LdsV4(unsigned addr)
{
  int4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
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

// Single block: rows per chunk for this level and the chunk offsets of every built node.
__global__ void __launch_bounds__(1024)
  k_hist_plan(const int32_t* __restrict__ seg, const int32_t* __restrict__ slot_of_node, int n_nodes, int GK,
              int target_tickets, const int* __restrict__ max_abs, int32_t* __restrict__ chunk_off,
              int32_t* __restrict__ plan, unsigned int* __restrict__ ticket)
{
  __shared__ long long red[32];
  __shared__ int wsum[32];
  __shared__ int carry;
  __shared__ int ch_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // rows to process, with the number of non-empty built nodes in the top 20 bits
  long long rows = 0;
  for (int j = tid; j < n_nodes; j += blockDim.x) {
    const bool built = slot_of_node == nullptr || slot_of_node[j] >= 0;
    const int r      = seg[j + 1] - seg[j];
    if (built && r > 0) rows += r + (1ll << 40);
  }
  for (int off = 16; off >= 1; off >>= 1) rows += __shfl_down_sync(0xffffffffu, rows, off);
  if (lane == 0) red[warp] = rows;
  __syncthreads();
  if (tid == 0) {
    long long total = 0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) total += red[w];
    const long long nodes = total >> 40;
    total &= (1ll << 40) - 1;
    long long ch = (total * GK + target_tickets - 1) / target_tickets;
    // enough nodes to fill the machine: one chunk per node, so that every node is flushed
    // once, with plain stores
    if (nodes * GK >= target_tickets) ch = 1ll << 30;
    if (ch < kMinChunk) ch = kMinChunk;
    ch = (ch + kTileRows - 1) / kTileRows * kTileRows;
    if (ch > (1ll << 30)) ch = 1ll << 30;
    ch_s  = static_cast<int>(ch);
    carry = 0;
    chunk_off[0] = 0;
  }
  __syncthreads();
  const int ch = ch_s;
  for (int base = 0; base < n_nodes; base += blockDim.x) {
    const int j = base + tid;
    int c       = 0;
    if (j < n_nodes) {
      const bool built = slot_of_node == nullptr || slot_of_node[j] >= 0;
      const int r      = seg[j + 1] - seg[j];
      c                = (built && r > 0) ? (r + ch - 1) / ch : 0;
    }
    int incl = c;
    for (int off = 1; off < 32; off <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += n;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w  = lane < (blockDim.x >> 5) ? wsum[lane] : 0;
      int wi = w;
      for (int off = 1; off < 32; off <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += n;
      }
      wsum[lane] = wi - w;
    }
    __syncthreads();
    const int before = carry + wsum[warp];
    if (j < n_nodes) chunk_off[j + 1] = before + incl;
    __syncthreads();
    if (tid == blockDim.x - 1) carry = before + incl;
    __syncthreads();
  }
  if (tid == 0) {
    plan[0] = ch;
    plan[1] = carry;
    int m   = 1;
    if (max_abs) m = max(1, max(max_abs[0], max_abs[1]));
    plan[3] = max_abs ? 2147483647 / m : 2147483647;
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
};

template <typename BinT, bool kFloat, bool kSmem>
__global__ void __launch_bounds__(kHistThreads, 2)
  k_hist(const HistParams p)
{
  using A      = Acc<kFloat>;
  using smem_t = typename A::smem_t;
  using in_t   = typename A::in_t;
  using out_t  = typename A::out_t;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  // the column arithmetic of the main loop needs the histogram on a 128-byte boundary
  smem_t* hg = reinterpret_cast<smem_t*>(smem_raw + ((128u - (SmemAddr(smem_raw) & 127u)) & 127u));
  constexpr int hist_rows = kSmem ? kSmemBins : 0;  // every byte value is a valid row
  smem_t* hh           = hg + hist_rows * kGroup;
  __shared__ unsigned int s_ticket;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int CH           = p.plan[0];
  const int total_chunks = p.plan[1];
  const int rows_safe    = p.plan[3];
  const long long total  = static_cast<long long>(total_chunks) * p.G * p.K;
  const BinT* bins       = static_cast<const BinT*>(p.bins);
  const in_t* gpair      = static_cast<const in_t*>(p.gpair);
  out_t* out             = static_cast<out_t*>(p.out);
  const int hist_words   = p.mb * kGroup;

  while (true) {
    __syncthreads();
    if (tid == 0) s_ticket = atomicAdd(p.ticket, 1u);
    __syncthreads();
    const long long t = s_ticket;
    if (t >= total) break;
    const int k = static_cast<int>(t % p.K);
    const int g = static_cast<int>((t / p.K) % p.G);
    const int c = static_cast<int>(t / (static_cast<long long>(p.K) * p.G));
    // node that owns chunk c: last j with chunk_off[j] <= c
    int lo = 0, hi = p.n_nodes;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.chunk_off[mid] <= c) lo = mid; else hi = mid;
    }
    const int j       = lo;
    const int nchunks = p.chunk_off[j + 1] - p.chunk_off[j];
    const int slot    = p.slot_of_node ? p.slot_of_node[j] : j;
    const int rb      = p.seg[j] + (c - p.chunk_off[j]) * CH;
    const int re      = min(p.seg[j + 1], rb + CH);
    const int feat    = g * kGroup + lane;
    const bool active = feat < p.F;
    const int fbeg    = active ? p.row_ptr[feat] : 0;
    const int fbins   = active ? p.row_ptr[feat + 1] - fbeg : 0;
    out_t* obase      = out + (static_cast<int64_t>(slot) * p.K + k) * p.B + fbeg;
    const BinT* gbins = bins + static_cast<int64_t>(g) * p.n_rows * kGroup;

    auto direct_rows = [&](int b, int e) {
      for (int r = b + warp; r < e; r += kHistWarps) {
        const int ridx = p.row_index[r];
        const in_t v   = gpair[static_cast<int64_t>(ridx) * p.K + k];
        if (active) {
          const int bin = gbins[static_cast<int64_t>(ridx) * kGroup + lane];
          A::add_global(obase + bin, v.x, v.y);
        }
      }
    };

    if (!kSmem || re - rb <= kDirectRows || rows_safe < kTileRows) {
      direct_rows(rb, re);
      continue;
    }

    bool use_atomics = nchunks > 1;
    auto flush = [&](bool atomics) {
      for (int e = tid; e < hist_words; e += kHistThreads) {  // e & 31 == lane for every e of a thread
        const int bin = e >> 5;
        if (bin < fbins) {
          const smem_t vg = hg[e], vh = hh[e];
          if (A::nonzero(vg, vh)) {
            if (atomics) A::add_global(obase + bin, vg, vh); else A::store_global(obase + bin, vg, vh);
          }
        }
      }
    };
    auto zero = [&]() {
      for (int e = tid; e < hist_words; e += kHistThreads) {
        hg[e] = smem_t(0);
        hh[e] = smem_t(0);
      }
    };
    zero();
    __syncthreads();

    // Every warp runs its own pipeline over 16-row batches of the chunk (no block barrier inside,
    // no staging in shared memory).  A lane PAIR owns one row of the batch: the even lane loads the
    // first 16 bin bytes of the row's 32, the odd lane the other 16, straight from global memory
    // into registers (one 16-byte load per lane, 16 rows = 16 full sectors per instruction).  In
    // step j of 16 the pair with row slot s handles feature (j xor s) of its half, so that the 32
    // lanes of a warp always update 32 different columns = 32 different banks, whatever the bins.
    // The bytes are permuted once per batch (word swaps + one byte permute per word) so that step
    // j reads the static byte j.  Per 32 updates that leaves the two reductions and nothing else on
    // the load/store pipe.
    const unsigned slot16   = lane >> 1, half = lane & 1;
    const unsigned wsel     = slot16 >> 2, bsel = slot16 & 3;
    const unsigned perm     = bsel == 0 ? 0x3210u : bsel == 1 ? 0x2301u : bsel == 2 ? 0x1032u : 0x0123u;
    const unsigned lanebase = SmemAddr(hg) + half * 64 + slot16 * 4;  // hg is 128-byte aligned
    const unsigned hh_off   = static_cast<unsigned>(hist_rows) * kGroup * 4;
    const unsigned char* gb = reinterpret_cast<const unsigned char*>(gbins) + half * 16;
    const int seg_rows = rows_safe >= (1 << 30) ? (1 << 30) : (rows_safe & ~31);
    for (int sb = rb; sb < re; sb += seg_rows) {
      const int se = min(re, sb + seg_rows);
      if (sb > rb) {
        __syncthreads();
        flush(true);
        use_atomics = true;
        __syncthreads();
        zero();
        __syncthreads();
      }
      const int nb = (se - sb + kBatchRows - 1) / kBatchRows;
      auto load_rid = [&](int batch) -> int {
        const int r = sb + batch * kBatchRows + static_cast<int>(slot16);
        return (batch < nb && r < se) ? __ldcg(p.row_index + r) : -1;
      };
      // rows beyond the end carry zero pairs and bin 0: they add nothing
      auto load_row = [&](int rid, int4& w, int2& v) {
        if (rid >= 0) {
          w = __ldcs(reinterpret_cast<const int4*>(gb + static_cast<int64_t>(rid) * kGroup));
          v = __ldcg(reinterpret_cast<const int2*>(gpair + static_cast<int64_t>(rid) * p.K + k));
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
        if (wsel & 2) {
          unsigned t = x[0]; x[0] = x[2]; x[2] = t;
          t = x[1]; x[1] = x[3]; x[3] = t;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = __byte_perm(x[i], 0u, perm);
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const unsigned bin  = __byte_perm(x[j >> 2], 0u, 0x4440u | (j & 3));
          const unsigned addr = (bin * (kGroup * 4) + lanebase) ^ (4u * j);
          if (kFloat) {
            RedShared(addr, __int_as_float(v.x));
            RedShared(addr + hh_off, __int_as_float(v.y));
          } else {
            RedShared(addr, v.x);
            RedShared(addr + hh_off, v.y);
          }
        }
      };
      int4 w0, w1, w2;
      int2 v0, v1, v2;
      load_row(load_rid(warp), w0, v0);
      load_row(load_rid(warp + kHistWarps), w1, v1);
      int rid_next = load_rid(warp + 2 * kHistWarps);
      for (int b = warp; b < nb; b += kHistWarps) {
        load_row(rid_next, w2, v2);  // batch b + 2 * kHistWarps
        rid_next = load_rid(b + 3 * kHistWarps);
        consume(w0, v0);
        w0 = w1; v0 = v1;
        w1 = w2; v1 = v2;
      }
    }
    __syncthreads();
    flush(use_atomics);
  }
}

// ---- row grouping (utility for the stage-level API) -------------------------------------------
constexpr int kGroupTile = 4096;

// Kernel, dynamic shared memory and persistent grid (resident blocks of the whole device, from the
// occupancy calculator) for one combination of bin width, pair type and path.
struct HistLaunch {
  void (*fn)(HistParams);
  size_t smem;
  int grid;
};

HistLaunch PickHistKernel(bool smem_path, int bin_bytes, bool float_mode, int sm_count)
{
  HistLaunch h;
  h.smem = smem_path ? static_cast<size_t>(kSmemBins) * kGroup * 8 + 128 : 0;
  if (smem_path) h.fn = float_mode ? k_hist<uint8_t, true, true> : k_hist<uint8_t, false, true>;
  else if (bin_bytes == 1) h.fn = float_mode ? k_hist<uint8_t, true, false> : k_hist<uint8_t, false, false>;
  else h.fn = float_mode ? k_hist<uint16_t, true, false> : k_hist<uint16_t, false, false>;
  if (h.smem > 48 * 1024)
    LBK_CUDA(cudaFuncSetAttribute(h.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(h.smem)));
  int per_sm = 0;
  LBK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, h.fn, kHistThreads, h.smem));
  if (per_sm < 1) per_sm = 1;
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
  int32_t* plan      = s.alloc<int32_t>(4);
  p.chunk_off        = chunk_off;
  p.plan             = plan;
  p.ticket           = reinterpret_cast<unsigned int*>(plan + 2);
  p.out              = lv.out;

  const bool smem_path = lv.bin_bytes == 1 && lv.max_bins_per_feature <= kSmemBins;
  p.mb                 = smem_path ? lv.max_bins_per_feature : 0;
  const HistLaunch hl  = PickHistKernel(smem_path, lv.bin_bytes, lv.float_mode, ctx->sm_count);

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
  double mult = 1.0;
  if (const char* e = getenv("LBK_HIST_TICKETS_PER_BLOCK")) mult = atof(e);
  k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, p.slot_of_node, p.n_nodes, p.G * p.K, static_cast<int>(hl.grid * mult) + 1,
                                      lv.float_mode ? nullptr : max_abs, chunk_off, plan, p.ticket);
  LBK_LAUNCH_CHECK();
  if (ctx->profile) LBK_CUDA(cudaEventRecord(ctx->ev_start, stream));
  hl.fn<<<hl.grid, kHistThreads, hl.smem, stream>>>(p);
  LBK_LAUNCH_CHECK();
  if (ctx->profile) {
    LBK_CUDA(cudaEventRecord(ctx->ev_stop, stream));
    ctx->profile_recorded = true;
  }
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
constexpr int kNoAllocPlanOffset  = kNoAllocMaxNodes + 4;   // chunk offsets first, then plan[4], max_abs[2]
constexpr int kNoAllocInts        = kNoAllocPlanOffset + 8;

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
    int* max_abs        = reinterpret_cast<int*>(plan + 4);

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
    const HistLaunch hl  = PickHistKernel(smem_path, a->bin_bytes, float_mode, sm_count);

    // the array keeps what the previous call left: clear the words that accumulate
    LBK_CUDA(cudaMemsetAsync(plan, 0, sizeof(int32_t) * 8, stream));
    LBK_CUDA(cudaMemsetAsync(a->hist, 0, sizeof(GPairI64) * a->n_nodes * K * B, stream));
    if (!float_mode) {
      const int64_t n = a->n_rows * K;
      if (n > 0) {
        k_max_abs<<<sm_count * 8, 256, 0, stream>>>(static_cast<const int2*>(p.gpair), n, max_abs);
        LBK_LAUNCH_CHECK();
      }
    }
    k_hist_plan<<<1, 1024, 0, stream>>>(p.seg, nullptr, p.n_nodes, p.G * p.K, hl.grid + 1, float_mode ? nullptr : max_abs,
                                        chunk_off, plan, p.ticket);
    LBK_LAUNCH_CHECK();
    hl.fn<<<hl.grid, kHistThreads, hl.smem, stream>>>(p);
    LBK_LAUNCH_CHECK();
    LBK_CUDA(cudaStreamSynchronize(stream));
  });
}
