// Split proposals and the binned matrix.
//
// Reference behaviour restated here:
//   SelectSplitSamples  src/models/tree/build_tree.cu:867-964 - draw split_samples row ids from
//     the seed, gather those rows (zeros where another rank owns the row), sum over ranks, keep
//     the sorted unique values per feature as a CSR, overwrite each feature's largest value
//     with +inf.
//   FindBin             src/models/tree/build_tree.h:178-185 - bin = first proposal >= x.
// The reference re-runs the search for every element on every tree level; here it runs once per
// tree and the result is kept as one byte (or two) per element, grouped 32 features at a time
// so that a warp reads one 32-byte sector per row with one lane per feature.
#include <cfloat>
#include <cmath>
#include <limits>

#include "device_utils.cuh"
#include <type_traits>

#include "internal.h"

namespace lbk {
namespace {

constexpr int kSortThreads = 256;

template <typename T>
__global__ void k_gather_samples(const T* __restrict__ X, int64_t ldx, int64_t row_offset, int64_t n_local,
                                 int F, int S, int seed, int64_t dataset_rows, T* __restrict__ draft)
{
  // draft is feature-major [F][S]
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= static_cast<int64_t>(F) * S) return;
  const int i = static_cast<int>(idx / F);
  const int f = static_cast<int>(idx % F);
  MinStd eng(static_cast<uint32_t>(seed));
  eng.discard(static_cast<unsigned long long>(i));
  const long long row = eng.uniform_int(0, dataset_rows - 1);
  const bool has      = row >= row_offset && row < row_offset + n_local;
  draft[static_cast<int64_t>(f) * S + i] = has ? X[(row - row_offset) * ldx + f] : T(0);
}

// One block per feature: bitonic sort of the S samples in shared memory, then unique.
template <typename T>
__global__ void __launch_bounds__(kSortThreads)
  k_sort_unique(const T* __restrict__ draft, int S, int S_pad, T* __restrict__ uniq, int32_t* __restrict__ counts)
{
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* vals        = reinterpret_cast<T*>(smem_raw);
  int* scan_tmp  = reinterpret_cast<int*>(vals + S_pad);
  const int f    = blockIdx.x;
  const int tid  = threadIdx.x;
  for (int i = tid; i < S_pad; i += kSortThreads)
    vals[i] = i < S ? draft[static_cast<int64_t>(f) * S + i] : static_cast<T>(INFINITY);
  __syncthreads();
  for (int k = 2; k <= S_pad; k <<= 1) {
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < S_pad; i += kSortThreads) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const T a = vals[i], b = vals[ixj];
          const bool up = (i & k) == 0;
          if (up ? (b < a) : (a < b)) {
            vals[i]   = b;
            vals[ixj] = a;
          }
        }
      }
      __syncthreads();
    }
  }
  // unique over the first S sorted entries; each thread owns a contiguous run
  const int per   = (S + kSortThreads - 1) / kSortThreads;
  const int begin = min(tid * per, S), end = min(begin + per, S);
  int local = 0;
  for (int i = begin; i < end; ++i) local += (i == 0 || vals[i] != vals[i - 1]) ? 1 : 0;
  scan_tmp[tid] = local;
  __syncthreads();
  // exclusive scan of 256 counts by a single warp (8 per lane)
  if (tid < 32) {
    int v[kSortThreads / 32];
    int sum = 0;
#pragma unroll
    for (int j = 0; j < kSortThreads / 32; ++j) {
      v[j] = scan_tmp[tid * (kSortThreads / 32) + j];
      sum += v[j];
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, incl, off);
      if (tid >= off) incl += n;
    }
    int run = incl - sum;
#pragma unroll
    for (int j = 0; j < kSortThreads / 32; ++j) {
      scan_tmp[tid * (kSortThreads / 32) + j] = run;
      run += v[j];
    }
    if (tid == 31) counts[f] = incl;
  }
  __syncthreads();
  int pos = scan_tmp[tid];
  for (int i = begin; i < end; ++i) {
    if (i == 0 || vals[i] != vals[i - 1]) uniq[static_cast<int64_t>(f) * S + pos++] = vals[i];
  }
}

// row_ptr = exclusive scan of counts (single block)
__global__ void k_scan_counts(const int32_t* __restrict__ counts, int F, int32_t* __restrict__ row_ptr,
                              int32_t* __restrict__ max_bins)
{
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  __shared__ int max_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    carry_s = 0;
    max_s   = 0;
    row_ptr[0] = 0;
  }
  __syncthreads();
  for (int base = 0; base < F; base += blockDim.x) {
    const int i = base + tid;
    const int c = i < F ? counts[i] : 0;
    int incl    = c;
    for (int off = 1; off < 32; off <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += n;
    }
    if (lane == 31) warp_sums[warp] = incl;
    atomicMax(&max_s, c);
    __syncthreads();
    if (warp == 0) {
      int w = lane < (blockDim.x >> 5) ? warp_sums[lane] : 0;
      int wi = w;
      for (int off = 1; off < 32; off <<= 1) {
        int n = __shfl_up_sync(0xffffffffu, wi, off);
        if (lane >= off) wi += n;
      }
      warp_sums[lane] = wi - w;  // exclusive
    }
    __syncthreads();
    const int total_before = carry_s + warp_sums[warp];
    if (i < F) row_ptr[i + 1] = total_before + incl;
    __syncthreads();
    if (tid == blockDim.x - 1) carry_s = total_before + incl;
    __syncthreads();
  }
  if (tid == 0) *max_bins = max_s;
}

template <typename T>
__global__ void k_write_proposals(const T* __restrict__ uniq, int S, const int32_t* __restrict__ row_ptr,
                                  T* __restrict__ proposals)
{
  const int f     = blockIdx.x;
  const int begin = row_ptr[f], end = row_ptr[f + 1];
  for (int j = threadIdx.x; j < end - begin; j += blockDim.x) {
    T v = uniq[static_cast<int64_t>(f) * S + j];
    if (j == end - begin - 1) v = static_cast<T>(INFINITY);
    proposals[begin + j] = v;
  }
}

// Streaming global loads as volatile asm: they stay where they are written, ahead of the search
// of the previous rows (the compiler otherwise sinks them to their first use).
__device__ inline float LdgStream(const float* p)
{
  float v;
  asm volatile("ld.global.cs.f32 %0, [%1];\n" : "=f"(v) : "l"(p));
  return v;
}
__device__ inline double LdgStream(const double* p)
{
  double v;
  asm volatile("ld.global.cs.f64 %0, [%1];\n" : "=d"(v) : "l"(p));
  return v;
}

template <int kOffset>
__device__ inline float LdsT(unsigned addr, float)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];\n" : "=f"(v) : "r"(addr), "n"(kOffset));
  return v;
}
template <int kOffset>
__device__ inline double LdsT(unsigned addr, double)
{
  double v;
  asm volatile("ld.shared.f64 %0, [%1+%2];\n" : "=d"(v) : "r"(addr), "n"(kOffset));
  return v;
}

// One lower_bound step for U rows at once: "advance by 2^kLevel proposals if the proposal just
// before that point is below x".  The probe offset is an immediate of the load; what remains per
// row and step is one shared-memory load, one compare and one predicated add.
template <typename T, int U, int kLevel, unsigned kPitch>
struct SearchLevels {
  __device__ static void run(unsigned (&pos)[U], const T (&x)[U])
  {
    constexpr int step = 1 << kLevel;
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (LdsT<(step - 1) * static_cast<int>(kPitch)>(pos[u], T()) < x[u]) pos[u] += step * kPitch;
    SearchLevels<T, U, kLevel - 1, kPitch>::run(pos, x);
  }
};
template <typename T, int U, unsigned kPitch>
struct SearchLevels<T, U, -1, kPitch> {
  __device__ static void run(unsigned (&)[U], const T (&)[U]) {}
};

// One warp per row, one lane per feature of the group.
//
// Shared-memory variant: the proposals of the group are kept transposed and padded, sp[j][lane] =
// proposal j of the lane's feature (+inf beyond the feature's last one and for the lanes beyond
// the last feature, P = 2^kLog2P rows), so that every probe of lane l goes to bank l: the probes
// of a lower_bound are conflict-free passes whatever the values.  The search is the branchless
// form "pos += step while sp[pos+step-1] < x" on the shared-memory address of the lane's column,
// fully unrolled; it returns the number of proposals below x, i.e. the index of the first
// proposal >= x.  The pivots of the first two levels are kept in registers.
//
// A warp takes kTileRows consecutive rows per turn, eight at a time.  What bounds the kernel is
// the load/store pipe (one pass per distinct 128-byte line of an instruction) and the issue slots,
// so: the turns that lie wholly inside the matrix run without row checks; and the feature-major
// copy of one-byte ids goes through a per-warp tile in shared memory, [32 features][kTileRows
// bytes], from which the warp writes kTileRows contiguous bytes per feature (two features per
// store instruction) instead of one 16-byte piece per lane and line.
constexpr int kBinTileRows  = 64;
constexpr int kBinTilePitch = kBinTileRows + 8;  // bytes; 18 words: 8-byte stores of 16 lanes fall on distinct banks

template <typename T, typename BinT, int kLog2P, bool kCopyT>
__global__ void __launch_bounds__(256, sizeof(T) == 4 ? 4 : 2)
  k_bin_smem(const T* __restrict__ X, int64_t ldx, int64_t n_rows, int F, const T* __restrict__ proposals,
             const int32_t* __restrict__ row_ptr, BinT* __restrict__ bins, BinT* __restrict__ bins_t, int64_t pitch_t)
{
  constexpr int P = 1 << kLog2P;
  constexpr bool kTile = kCopyT && sizeof(BinT) == 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* sp          = reinterpret_cast<T*>(smem_raw);
  const int g    = blockIdx.y;
  const int f0   = g * kGroup;
  const int lane = threadIdx.x & 31;
  for (int idx = threadIdx.x; idx < P * kGroup; idx += blockDim.x) {
    const int j = idx >> 5, f = f0 + (idx & 31);
    T v = static_cast<T>(INFINITY);
    if (f < F) {
      const int b = row_ptr[f];
      if (j < row_ptr[f + 1] - b) v = proposals[b + j];
    }
    sp[idx] = v;
  }
  __syncthreads();
  // Lanes beyond the last feature read the last feature's values (in bounds); their column of the
  // table is all +inf, so their ids are 0.
  const bool active = f0 + lane < F;
  constexpr unsigned kPitch = kGroup * sizeof(T);  // bytes from one proposal of a feature to the next
  const unsigned col_s      = static_cast<unsigned>(__cvta_generic_to_shared(sp + lane));
  unsigned char* tile = smem_raw + sizeof(T) * P * kGroup + (threadIdx.x >> 5) * (kGroup * kBinTilePitch);
  const unsigned tile_s = static_cast<unsigned>(__cvta_generic_to_shared(tile));
  // rows are counted in 32 bits (row indices are 32-bit everywhere in this library)
  const int pitch   = static_cast<int>(gridDim.y) * kGroup;  // bins are row-major, rows padded to groups
  constexpr int U   = 8;  // rows per warp in flight
  const int n       = static_cast<int>(n_rows);
  const int ld      = static_cast<int>(ldx);
  constexpr int kSubs = kBinTileRows / U;
  constexpr int kTurn = kBinTileRows;
  const int hop     = static_cast<int>(gridDim.x) * (blockDim.x >> 5) * kTurn;  // rows from one turn of a warp to the next
  int turn          = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * kTurn;
  const T* xcol     = X + (active ? f0 + lane : F - 1);
  BinT* ocol        = bins + f0 + lane;
  BinT* tcol        = kCopyT ? bins_t + static_cast<int64_t>(active ? f0 + lane : F - 1) * pitch_t : nullptr;
  // pivots of the first two levels
  T piv_h = T(), piv_q1 = T(), piv_q3 = T();
  if (kLog2P >= 2) {
    piv_h  = sp[(P / 2 - 1) * kGroup + lane];
    piv_q1 = sp[(P / 4 - 1) * kGroup + lane];
    piv_q3 = sp[(3 * P / 4 - 1) * kGroup + lane];
  }
  // the values of the warp's next eight rows are loaded while the current eight are searched
  auto load_rows = [&](int first, T (&x)[U]) {
    const T* src = xcol + static_cast<int64_t>(first) * ld;
#pragma unroll
    for (int u = 0; u < U; ++u) x[u] = LdgStream(src + u * ld);
  };
  auto load_rows_checked = [&](int first, T (&x)[U]) {
    const T* src = xcol + static_cast<int64_t>(first) * ld;
#pragma unroll
    for (int u = 0; u < U; ++u) x[u] = first + u < n ? LdgStream(src + u * ld) : static_cast<T>(-INFINITY);
  };
  T xn[U];
  if (turn < n) load_rows_checked(turn, xn);
  // one turn; kChecked: the turn may reach beyond the last row
  auto do_turn = [&](auto checked) {
    constexpr bool kChecked = decltype(checked)::value;
#pragma unroll 2
    for (int sub = 0; sub < kSubs; ++sub) {
      const int base = turn + sub * U;
      T x[U];
      unsigned pos[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = xn[u];
      {
        const int nb = sub + 1 < kSubs ? base + U : turn + hop;
        if (sub + 1 < kSubs && !kChecked) load_rows(nb, xn);
        else if (nb < n) load_rows_checked(nb, xn);
      }
      if (kLog2P >= 2) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const bool c1 = piv_h < x[u];
          pos[u]        = c1 ? col_s + (P / 2) * kPitch : col_s;
          const T piv   = c1 ? piv_q3 : piv_q1;
          if (piv < x[u]) pos[u] += (P / 4) * kPitch;
        }
        SearchLevels<T, U, kLog2P - 3, kPitch>::run(pos, x);
      } else {
#pragma unroll
        for (int u = 0; u < U; ++u) pos[u] = col_s;
        SearchLevels<T, U, kLog2P - 1, kPitch>::run(pos, x);
      }
      unsigned id[U];
#pragma unroll
      for (int u = 0; u < U; ++u) id[u] = (pos[u] - col_s) / kPitch;
      BinT* orow = ocol + static_cast<int64_t>(base) * pitch;
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (!kChecked || base + u < n) orow[u * pitch] = static_cast<BinT>(id[u]);
      if (kCopyT) {
        if (kTile) {
          const unsigned lo = id[0] | (id[1] << 8) | (id[2] << 16) | (id[3] << 24);
          const unsigned hi = id[4] | (id[5] << 8) | (id[6] << 16) | (id[7] << 24);
          asm volatile("st.shared.v2.b32 [%0], {%1, %2};\n" ::"r"(tile_s + lane * kBinTilePitch + sub * U), "r"(lo), "r"(hi)
                       : "memory");
        } else if (active && base < n) {
          uint4 pk;
          pk.x = id[0] | (id[1] << 16);
          pk.y = id[2] | (id[3] << 16);
          pk.z = id[4] | (id[5] << 16);
          pk.w = id[6] | (id[7] << 16);
          *reinterpret_cast<uint4*>(tcol + base) = pk;
        }
      }
    }
    if (kTile) {
      // the tile leaves feature by feature: lanes 0-15 write the 64 bytes of one feature, lanes
      // 16-31 those of the next (rows up to the padded end of a feature's row of the copy; the ids
      // of rows beyond the last one are 0)
      __syncwarp();
      const int w    = lane & 15;
      const bool in  = turn + 4 * w < pitch_t;
#pragma unroll 4
      for (int i = 0; i < kGroup / 2; ++i) {
        const int fl = 2 * i + (lane >> 4);
        unsigned v;
        asm volatile("ld.shared.b32 %0, [%1];\n" : "=r"(v) : "r"(tile_s + fl * kBinTilePitch + 4 * w));
        if (in && f0 + fl < F)
          *reinterpret_cast<unsigned*>(bins_t + static_cast<int64_t>(f0 + fl) * pitch_t + turn + 4 * w) = v;
      }
      __syncwarp();
    }
  };
  for (; turn + kTurn <= n; turn += hop) do_turn(std::false_type());
  if (turn < n) do_turn(std::true_type());
}

// Global-memory variant for features with more proposals than shared memory holds.
template <typename T, typename BinT>
__global__ void __launch_bounds__(256)
  k_bin_global(const T* __restrict__ X, int64_t ldx, int64_t n_rows, int F, const T* __restrict__ proposals,
               const int32_t* __restrict__ row_ptr, BinT* __restrict__ bins, BinT* __restrict__ bins_t, int64_t pitch_t)
{
  const int g    = blockIdx.y;
  const int f0   = g * kGroup;
  const int lane = threadIdx.x & 31;
  const int f    = f0 + lane;
  const bool active = f < F;
  int begin = 0, n = 0;
  if (active) {
    begin = row_ptr[f];
    n     = row_ptr[f + 1] - begin;
  }
  const T* p = proposals + begin;
  const int64_t pitch = static_cast<int64_t>(gridDim.y) * kGroup;
  BinT* out  = bins + f0;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t row = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + (threadIdx.x >> 5); row < n_rows;
       row += warps_total) {
    int bin = 0;
    if (active) {
      const T x = X[row * ldx + f];
      int len = n, base = 0;
      while (len > 1) {
        const int half = len >> 1;
        base           = (p[base + half] < x) ? base + half : base;
        len -= half;
      }
      bin = base + ((p[base] < x) ? 1 : 0);
    }
    out[row * pitch + lane] = static_cast<BinT>(bin);
    if (bins_t != nullptr && active) bins_t[static_cast<int64_t>(f) * pitch_t + row] = static_cast<BinT>(bin);
  }
}

int NextPow2(int v)
{
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

template <typename T>
ProposalInfo SplitProposals(lbk_context* ctx, Scratch& s, const T* X, int64_t ldx, int64_t row_offset, int64_t n_local,
                   int F, int S, int seed, int64_t dataset_rows, T* proposals, int32_t* row_ptr,
                   cudaStream_t stream)
{
  const int64_t FS = static_cast<int64_t>(F) * S;
  T* draft         = s.alloc<T>(FS);
  T* uniq          = s.alloc<T>(FS);
  int32_t* counts  = s.alloc<int32_t>(F + 1);
  {
    const int threads = 256;
    const int64_t blocks = (FS + threads - 1) / threads;
    k_gather_samples<T><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(X, ldx, row_offset, n_local, F, S, seed,
                                                                               dataset_rows, draft);
    LBK_LAUNCH_CHECK();
  }
  AllReduce(ctx, draft, static_cast<size_t>(FS), sizeof(T) == 4 ? LBK_F32 : LBK_F64, LBK_SUM, stream);
  const int S_pad   = NextPow2(S);
  const size_t smem = sizeof(T) * S_pad + sizeof(int) * kSortThreads;
  k_sort_unique<T><<<F, kSortThreads, smem, stream>>>(draft, S, S_pad, uniq, counts);
  LBK_LAUNCH_CHECK();
  k_scan_counts<<<1, 1024, 0, stream>>>(counts, F, row_ptr, counts + F);
  LBK_LAUNCH_CHECK();
  k_write_proposals<T><<<F, 128, 0, stream>>>(uniq, S, row_ptr, proposals);
  LBK_LAUNCH_CHECK();
  int32_t h[2] = {0, 0};
  LBK_CUDA(cudaMemcpyAsync(&h[0], row_ptr + F, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  LBK_CUDA(cudaMemcpyAsync(&h[1], counts + F, sizeof(int32_t), cudaMemcpyDeviceToHost, stream));
  LBK_CUDA(cudaStreamSynchronize(stream));
  s.free_one(draft);
  s.free_one(uniq);
  return ProposalInfo{h[0], h[1]};
}

template <typename T>
void BinMatrix(const T* X, int64_t ldx, int64_t n_rows, int F, const T* proposals, const int32_t* row_ptr,
               void* bins, void* bins_t, int64_t pitch_t, int bin_bytes, int max_bins_per_feature, cudaStream_t stream)
{
  if (n_rows <= 0) return;
  LBK_EXPECT(n_rows <= 2000000000ll && ldx <= (1 << 27), "bin_matrix: at most 2e9 rows per rank and a row pitch of 2^27 elements");
  const int G           = (F + kGroup - 1) / kGroup;
  // the shared-memory table is padded to one of a few sizes (each is its own fully unrolled kernel)
  const int need   = NextPow2(max_bins_per_feature);
  const int log2p  = need <= 16 ? 4 : need <= 64 ? 6 : need <= 256 ? 8 : 9;
  // the table, and one tile per warp for the feature-major copy of one-byte ids
  const size_t table    = sizeof(T) * static_cast<size_t>(kGroup) * (size_t{1} << log2p);
  const size_t smem     = table + (bins_t != nullptr && bin_bytes == 1 ? size_t{8} * kGroup * kBinTilePitch : 0);
  const bool use_smem   = need <= 512 && table <= 96 * 1024;
  // a block fills its table once and then walks the rows with a grid stride: the grid is what is
  // resident at once (from the occupancy calculator), spread over the feature groups
  auto make_grid = [&](int blocks_per_sm) {
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t blocks_x = (static_cast<int64_t>(sms) * (blocks_per_sm > 0 ? blocks_per_sm : 1) + G - 1) / G;
    const int64_t most = (n_rows + 63) / 64;
    if (blocks_x > most) blocks_x = most;
    if (blocks_x < 1) blocks_x = 1;
    return dim3(static_cast<unsigned>(blocks_x), G);
  };
#define LBK_BIN_SMEM2(BinT, L, CT)                                                                        \
  do {                                                                                                    \
    auto fn_ = k_bin_smem<T, BinT, L, CT>;                                                                \
    if (smem > 48 * 1024)                                                                                 \
      LBK_CUDA(cudaFuncSetAttribute(fn_, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem))); \
    int per_sm_ = 0;                                                                                      \
    LBK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm_, fn_, 256, smem));                    \
    fn_<<<make_grid(per_sm_), 256, smem, stream>>>(X, ldx, n_rows, F, proposals, row_ptr,                 \
                                                   static_cast<BinT*>(bins), static_cast<BinT*>(bins_t), pitch_t); \
  } while (0)
#define LBK_BIN_SMEM(BinT, L)                                                                             \
  do {                                                                                                    \
    if (bins_t != nullptr) LBK_BIN_SMEM2(BinT, L, true); else LBK_BIN_SMEM2(BinT, L, false);              \
  } while (0)
#define LBK_BIN_LAUNCH(BinT)                                                                              \
  do {                                                                                                    \
    if (use_smem) {                                                                                       \
      if (log2p == 4) LBK_BIN_SMEM(BinT, 4);                                                              \
      else if (log2p == 6) LBK_BIN_SMEM(BinT, 6);                                                         \
      else if (log2p == 8) LBK_BIN_SMEM(BinT, 8);                                                         \
      else LBK_BIN_SMEM(BinT, 9);                                                                         \
    } else {                                                                                              \
      k_bin_global<T, BinT><<<make_grid(8), 256, 0, stream>>>(X, ldx, n_rows, F, proposals, row_ptr,     \
                                                       static_cast<BinT*>(bins), static_cast<BinT*>(bins_t), \
                                                       pitch_t);                                          \
    }                                                                                                     \
  } while (0)
  if (bin_bytes == 1) {
    LBK_BIN_LAUNCH(uint8_t);
  } else {
    LBK_BIN_LAUNCH(uint16_t);
  }
#undef LBK_BIN_SMEM
#undef LBK_BIN_SMEM2
#undef LBK_BIN_LAUNCH
  LBK_LAUNCH_CHECK();
}

template ProposalInfo SplitProposals<float>(lbk_context*, Scratch&, const float*, int64_t, int64_t, int64_t, int, int, int,
                                   int64_t, float*, int32_t*, cudaStream_t);
template ProposalInfo SplitProposals<double>(lbk_context*, Scratch&, const double*, int64_t, int64_t, int64_t, int, int, int,
                                    int64_t, double*, int32_t*, cudaStream_t);
template void BinMatrix<float>(const float*, int64_t, int64_t, int, const float*, const int32_t*, void*, void*, int64_t,
                               int, int, cudaStream_t);
template void BinMatrix<double>(const double*, int64_t, int64_t, int, const double*, const int32_t*, void*, void*,
                                int64_t, int, int, cudaStream_t);

}  // namespace lbk
