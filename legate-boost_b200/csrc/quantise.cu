// Gradient quantiser: scale from the local |g|,|h| sums, one stochastic-rounded int32 pair per
// (row, output), and the root node sums.
//
// Reference behaviour restated here:
//   GradientQuantiser ctor   src/models/tree/build_tree.cu:69-104  - scale = INT32_MAX / max over
//     ranks of the local sum of |g| (resp. |h|), 1 if that sum is 0.
//   QuantiseStochasticRounding  :112-129, hash_combine :143-165.
//   reduce_base_sums            :168-204 - node_sums[0,k] = sum of the quantised pairs.
// The reference recomputes the quantised pair of a row for every feature group on every level;
// its value depends only on (seed, global row, output), so it is computed once here.
//
// Order of the floating-point |g| sum (the reference leaves it to thrust::reduce): blocks of
// 4096 elements; thread t of 256 adds elements t, t+256, ... in order; groups of 32 threads fold
// with offsets 16,8,4,2,1; the 8 group sums are added left to right; block sums are reduced the
// same way until one value is left.  The CPU oracle uses the same order.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

constexpr int kSumThreads = 256;
constexpr int kSumItems   = 16;
constexpr int kSumBlock   = kSumThreads * kSumItems;  // 4096

// level 0 reads |g|,|h| from the strided [n_rows, K] inputs; higher levels read partial sums
template <bool kFirst>
__global__ void __launch_bounds__(kSumThreads)
  k_abs_sum(const double* __restrict__ g, const double* __restrict__ h, int64_t ldg, int K, int64_t n,
            double* __restrict__ out_g, double* __restrict__ out_h)
{
  __shared__ double wg[kSumThreads / 32], wh[kSumThreads / 32];
  const int tid      = threadIdx.x;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * kSumBlock;
  double sg = 0.0, sh = 0.0;
#pragma unroll
  for (int j = 0; j < kSumItems; ++j) {
    const int64_t idx = base + static_cast<int64_t>(j) * kSumThreads + tid;
    double vg = 0.0, vh = 0.0;
    if (idx < n) {
      if (kFirst) {
        const int64_t row = idx / K;
        const int k       = static_cast<int>(idx - row * K);
        vg                = fabs(g[row * ldg + k]);
        vh                = fabs(h[row * ldg + k]);
      } else {
        vg = g[idx];
        vh = h[idx];
      }
    }
    sg += vg;
    sh += vh;
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    sg += __shfl_down_sync(0xffffffffu, sg, off);
    sh += __shfl_down_sync(0xffffffffu, sh, off);
  }
  if ((tid & 31) == 0) {
    wg[tid >> 5] = sg;
    wh[tid >> 5] = sh;
  }
  __syncthreads();
  if (tid == 0) {
    double tg = wg[0], th = wh[0];
#pragma unroll
    for (int w = 1; w < kSumThreads / 32; ++w) {
      tg += wg[w];
      th += wh[w];
    }
    out_g[blockIdx.x] = tg;
    out_h[blockIdx.x] = th;
  }
}

__global__ void k_make_scale(const double* __restrict__ sums /* g,h */, QuantParams* __restrict__ qp)
{
  const double max_int = 2147483647.0;
  const double sg = sums[0], sh = sums[1];
  QuantParams p;
  p.scale_g = sg == 0 ? 1.0 : max_int / sg;
  p.scale_h = sh == 0 ? 1.0 : max_int / sh;
  p.inv_g   = 1.0 / p.scale_g;
  p.inv_h   = 1.0 / p.scale_h;
  *qp       = p;
}

// Per-output block sums go to node_sums[0,k] with one 64-bit atomic pair per block and output;
// blocks walk the elements with a grid stride so that the number of atomics stays small.
// Element (row, k) = flat index row * K + k; a thread keeps one k (the grid's stride is a multiple
// of K), so the loads and stores of a warp are contiguous whatever K is.
__global__ void __launch_bounds__(256)
  k_quantise(const double* __restrict__ g, const double* __restrict__ h, int64_t ldg, int64_t row_offset,
             int64_t n_local, int K, long long seed, const QuantParams* __restrict__ qp_ptr,
             int2* __restrict__ gpair, GPairI64* __restrict__ root_sums, int* __restrict__ max_abs)
{
  extern __shared__ unsigned long long s_sum[];  // [K][2]
  const QuantParams qp = *qp_ptr;
  const int tid        = threadIdx.x;
  for (int i = tid; i < 2 * K; i += blockDim.x) s_sum[i] = 0ull;
  __syncthreads();
  const int64_t threads = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int64_t rows_per_turn = threads / K;  // >= 1: the launcher gives at least K threads
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + tid;
  int mg = 0, mh = 0;
  if (t < rows_per_turn * K) {
    const int k = static_cast<int>(t % K);
    long long sg = 0, sh = 0;
    for (int64_t row = t / K; row < n_local; row += rows_per_turn) {
      const double gv = g[row * ldg + k];
      const double hv = h[row * ldg + k];
      const int2 q    = QuantisePair(gv, hv, qp, HashCombine(seed, row_offset + row, k));
      gpair[row * K + k] = q;
      sg += q.x;
      sh += q.y;
      mg = max(mg, q.x == INT32_MIN ? INT32_MAX : abs(q.x));
      mh = max(mh, q.y == INT32_MIN ? INT32_MAX : abs(q.y));
    }
    if (K == 1) {
      // every lane holds the same output: one pair of shared-memory atomics per warp
      for (int off = 16; off >= 1; off >>= 1) {
        sg += __shfl_down_sync(0xffffffffu, sg, off);
        sh += __shfl_down_sync(0xffffffffu, sh, off);
      }
      if ((tid & 31) == 0) {
        atomicAdd(&s_sum[0], static_cast<unsigned long long>(sg));
        atomicAdd(&s_sum[1], static_cast<unsigned long long>(sh));
      }
    } else {
      atomicAdd(&s_sum[2 * k], static_cast<unsigned long long>(sg));
      atomicAdd(&s_sum[2 * k + 1], static_cast<unsigned long long>(sh));
    }
  }
  __syncthreads();
  for (int i = tid; i < 2 * K; i += blockDim.x) {
    unsigned long long* dst = reinterpret_cast<unsigned long long*>(root_sums) + i;  // grad, hess of k = i / 2
    if (s_sum[i] != 0ull) atomicAdd(dst, s_sum[i]);
  }
  for (int off = 16; off >= 1; off >>= 1) {
    mg = max(mg, __shfl_down_sync(0xffffffffu, mg, off));
    mh = max(mh, __shfl_down_sync(0xffffffffu, mh, off));
  }
  if ((tid & 31) == 0) {
    atomicMax(max_abs, mg);
    atomicMax(max_abs + 1, mh);
  }
}

}  // namespace

void Quantise(lbk_context* ctx, Scratch& s, const double* g, const double* h, int64_t ldg, int64_t row_offset,
              int64_t n_local, int K, int seed, int2* gpair, GPairI64* root_sums, QuantParams* params,
              int* max_abs, cudaStream_t stream)
{
  // canonical |g|,|h| sums
  int64_t n        = n_local * K;
  double* sums     = s.alloc<double>(2);
  if (n == 0) {
    LBK_CUDA(cudaMemsetAsync(sums, 0, 2 * sizeof(double), stream));
  } else {
    const double* in_g = g;
    const double* in_h = h;
    bool first         = true;
    while (true) {
      const int64_t nblocks = (n + kSumBlock - 1) / kSumBlock;
      double* out_g;
      double* out_h;
      if (nblocks == 1) {
        out_g = sums;
        out_h = sums + 1;
      } else {
        out_g = s.alloc<double>(nblocks);
        out_h = s.alloc<double>(nblocks);
      }
      if (first)
        k_abs_sum<true><<<static_cast<unsigned>(nblocks), kSumThreads, 0, stream>>>(in_g, in_h, ldg, K, n, out_g, out_h);
      else
        k_abs_sum<false><<<static_cast<unsigned>(nblocks), kSumThreads, 0, stream>>>(in_g, in_h, 0, 1, n, out_g, out_h);
      LBK_LAUNCH_CHECK();
      if (nblocks == 1) break;
      in_g  = out_g;
      in_h  = out_h;
      n     = nblocks;
      first = false;
    }
  }
  AllReduce(ctx, sums, 2, LBK_F64, LBK_MAX, stream);
  k_make_scale<<<1, 1, 0, stream>>>(sums, params);
  LBK_LAUNCH_CHECK();
  LBK_CUDA(cudaMemsetAsync(root_sums, 0, sizeof(GPairI64) * K, stream));
  LBK_CUDA(cudaMemsetAsync(max_abs, 0, 2 * sizeof(int), stream));
  if (n_local > 0) {
    int64_t blocks = (n_local * K + 255) / 256;
    const int64_t cap = static_cast<int64_t>(ctx->sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks * 256 < K) blocks = (K + 255) / 256;  // a thread keeps one output: at least K threads
    const size_t smem = sizeof(unsigned long long) * 2 * K;
    LBK_EXPECT(smem <= 48 * 1024, "too many outputs for the quantiser's block sums");
    k_quantise<<<static_cast<unsigned>(blocks), 256, smem, stream>>>(g, h, ldg, row_offset, n_local, K,
                                                                  static_cast<long long>(seed), params, gpair, root_sums, max_abs);
    LBK_LAUNCH_CHECK();
  }
  AllReduce(ctx, root_sums, static_cast<size_t>(2) * K, LBK_I64, LBK_SUM, stream);
}

}  // namespace lbk
