// Ensemble predict: pred[row, :] = sum over trees of leaf_value[leaf reached by row, :].
//
// Reference behaviour restated here: predict_fn, src/models/tree/predict.cu:26-84 - one kernel
// launch per tree, each re-reading and re-writing pred; rows walk from node 0 while
// feature[pos] != -1 (at most 100 steps), going left iff (double)x <= split_value[pos].
//
// Design for B200: ONE launch for the whole ensemble, everything a step of the walk touches lives
// in shared memory.
//   * A block owns a tile of rows (one thread per row); every thread stages its own row,
//     feature-major with a pitch of one element per thread, so thread t only ever touches bank
//     t mod 32 whatever feature a tree asks for: the x lookups of a walk never conflict.  Every row
//     of X is read from HBM exactly once (16-byte loads, the rest of a sector comes from L1).
//   * The trees are first packed into one array of small nodes: for float32 X a node is 8 bytes
//     (float split, int feature) - "x <= split" with x a float is the same test as
//     "x <= the largest float not above split", so the split is rounded down once at packing time
//     and the walk compares floats; for float64 X a node is 16 bytes.
//   * At packing time every tree is completed to the depth S of the deepest one: below a leaf
//     the nodes become pass-through nodes (split = +inf) and the leaf's value is copied to the
//     bottom level.  A walk is then exactly S steps of "load node, load x, compare, descend" with
//     no leaf test, and only the bottom level of leaf values is kept.
//   * Trees are brought into shared memory in groups of up to eight (bulk async copies, double buffered)
//     together with their bottom-level leaf values; a thread walks the trees of a group as
//     independent chains, which hides the shared-memory latency that one dependent chain exposes.
//   * Predictions are accumulated in float64 in tree order (bit-identical to the reference's
//     tree-by-tree accumulation) and written once.
// A fallback kernel with the nodes in global memory covers shapes whose tile or trees do not fit.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

// `foff` = feature index times a caller-chosen multiplier (the byte pitch of the staged tile for
// the tiled kernel, 1 for the fallback), or -1 for a leaf
struct Node8 {
  float split;
  int foff;
};
struct Node16 {
  double split;
  int foff;
  int pad;
};
template <typename T>
struct NodeOf {
  using type = Node16;
};
template <>
struct NodeOf<float> {
  using type = Node8;
};

struct TreePtrs {
  const double* leaf;
  const int32_t* feature;
  const double* split;
  int max_nodes;
  int node_off;  // offset of this tree's first node in the packed arrays
};

__device__ inline void MakeNode(Node8& n, double split, int foff)
{
  n.split = __double2float_rd(split);  // x <= split  <=>  x <= round-down(split) for float x
  n.foff  = foff;
}
__device__ inline void MakeNode(Node16& n, double split, int foff)
{
  n.split = split;
  n.foff  = foff;
  n.pad   = 0;
}

// A split node whose children would fall outside the arrays is treated as a leaf, so a walk can
// never leave the tree whatever the input arrays hold.
template <typename NodeT>
__global__ void k_pack_trees(const TreePtrs* __restrict__ trees, int K, int F, int xmul, NodeT* __restrict__ nodes,
                             double* __restrict__ leaves)
{
  const TreePtrs t = trees[blockIdx.x];
  for (int i = threadIdx.x; i < t.max_nodes; i += blockDim.x) {
    int f = t.feature[i];
    if (2 * i + 2 >= t.max_nodes || f < 0 || f >= F) f = -1;
    NodeT n;
    MakeNode(n, t.split[i], f < 0 ? -1 : f * xmul);
    nodes[t.node_off + i] = n;
  }
  for (int64_t i = threadIdx.x; i < static_cast<int64_t>(t.max_nodes) * K; i += blockDim.x)
    leaves[static_cast<int64_t>(t.node_off) * K + i] = t.leaf[i];
}

// Bulk asynchronous copy global -> shared (the copy engine moves whole lines; nothing passes
// through the load/store pipe), completion counted in bytes on an mbarrier; a plain copy into this block only.
__device__ inline void MbarInit(unsigned bar, unsigned count)
{
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ inline void MbarExpectTx(unsigned bar, unsigned bytes)
{
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ inline void BulkCopy(unsigned smem_dst, const void* gsrc, unsigned bytes, unsigned bar)
{
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(smem_dst),
               "l"(gsrc), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ inline bool MbarTryWait(unsigned bar, unsigned parity)
{
  unsigned ok;
  asm volatile(
    "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
    : "=r"(ok)
    : "r"(bar), "r"(parity)
    : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about a second, reports through the context's status word and lets
// the block finish (with wrong sums, which the host then refuses) instead of spinning for ever.
constexpr int kFaultPredictStaging = 21;
__device__ inline bool MbarWait(unsigned bar, unsigned parity, int* status)
{
  for (unsigned spin = 0; spin < (1u << 22); ++spin) {
    if (MbarTryWait(bar, parity)) return true;
    if (spin > 64) __nanosleep(256);
  }
  atomicExch(status, kFaultPredictStaging);
  return false;
}

__device__ inline void LdsNode(unsigned addr, float& split, int& foff)
{
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];\n" : "=f"(split), "=r"(foff) : "r"(addr));
}
__device__ inline void LdsNode(unsigned addr, double& split, int& foff)
{
  int pad;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n"
               : "=r"(reinterpret_cast<int2&>(split).x), "=r"(reinterpret_cast<int2&>(split).y), "=r"(foff), "=r"(pad)
               : "r"(addr));
}
__device__ inline float LdsX(unsigned addr, float)
{
  float v;
  asm volatile("ld.shared.f32 %0, [%1];\n" : "=f"(v) : "r"(addr));
  return v;
}
__device__ inline double LdsX(unsigned addr, double)
{
  double v;
  asm volatile("ld.shared.f64 %0, [%1];\n" : "=d"(v) : "r"(addr));
  return v;
}
__device__ inline double LdsF64(unsigned addr)
{
  double v;
  asm volatile("ld.shared.f64 %0, [%1];\n" : "=d"(v) : "r"(addr));
  return v;
}

// Completed-tree packing for the tiled kernel.  For tree t: nodes_c[t*NI + i], i < 2^S - 1, are the
// internal levels of a complete tree of depth S; leaves_c[(t*NL + j)*K + k], j < 2^S, the values of
// its bottom level.  A node whose children would fall outside the input arrays, or whose feature
// id is outside [0, F), counts as a leaf, so a walk can never leave the arrays.
template <typename NodeT>
__global__ void k_pack_complete(const TreePtrs* __restrict__ trees, int K, int F, int xmul, int S, int NI, int NL,
                                NodeT* __restrict__ nodes_c, double* __restrict__ leaves_c)
{
  const TreePtrs t = trees[blockIdx.x];
  const int M      = t.max_nodes;
  const int total  = (2 << S) - 1;  // nodes of the complete tree
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int L = 31 - __clz(i + 1);
    int cover   = -1;  // first leaf on the path root -> i
    for (int l = 0; l <= L; ++l) {
      const int a   = ((i + 1) >> (L - l)) - 1;
      const int f   = a < M ? t.feature[a] : -1;
      if (a >= M || f < 0 || f >= F || 2 * a + 2 >= M) {
        cover = a;
        break;
      }
    }
    if (L < S) {
      NodeT n;
      if (cover >= 0) {
        MakeNode(n, static_cast<double>(INFINITY), 0);  // pass-through: always descends left
      } else {
        MakeNode(n, t.split[i], t.feature[i] * xmul);
      }
      nodes_c[static_cast<int64_t>(blockIdx.x) * NI + i] = n;
    } else {
      const int j = i - ((1 << S) - 1);
      for (int k = 0; k < K; ++k)
        leaves_c[(static_cast<int64_t>(blockIdx.x) * NL + j) * K + k] = t.leaf[static_cast<int64_t>(cover) * K + k];
    }
  }
}

// Tiled kernel.  Shared memory: X tile [F][RB] | accumulators [K][RB] (K > 1) |
// NBUF x TG x slot, slot = NI nodes (+ NL leaf values when K == 1).
template <typename T, int RB, int TG, bool kLeafShared>
__global__ void __launch_bounds__(RB)
  k_predict_tiled(const T* __restrict__ X, int64_t ldx, int64_t n_rows, int F, int K, int n_trees,
                  const typename NodeOf<T>::type* __restrict__ nodes_c, const double* __restrict__ leaves_c,
                  double* __restrict__ pred, int64_t ldp, int S, int NI, int NL, int* __restrict__ status)
{
  using NodeT = typename NodeOf<T>::type;
  __shared__ __align__(8) unsigned long long s_bar[2];
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* xs = reinterpret_cast<T*>(smem_raw);
  size_t off = (sizeof(T) * static_cast<size_t>(F) * RB + 15) / 16 * 16;
  double* accs = reinterpret_cast<double*>(smem_raw + off);
  off += K > 1 ? sizeof(double) * static_cast<size_t>(K) * RB : 0;
  // a group buffer: the nodes of its TG trees, then (K == 1) their bottom-level values
  const unsigned node_bytes = static_cast<unsigned>(NI * sizeof(NodeT));
  const unsigned leaf_bytes = kLeafShared ? static_cast<unsigned>(NL * sizeof(double)) : 0u;
  const unsigned buf_bytes  = TG * (node_bytes + leaf_bytes);
  unsigned char* tree_s     = smem_raw + off;

  const int tid       = threadIdx.x;
  const int64_t row0  = static_cast<int64_t>(blockIdx.x) * RB;
  const int rows_here = static_cast<int>((n_rows - row0) < RB ? (n_rows - row0) : RB);
  const unsigned tree0 = static_cast<unsigned>(__cvta_generic_to_shared(tree_s));
  const unsigned bar0  = static_cast<unsigned>(__cvta_generic_to_shared(&s_bar[0]));
  const int n_groups   = (n_trees + TG - 1) / TG;
  if (tid == 0) {
    MbarInit(bar0, 1);
    MbarInit(bar0 + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  // group of trees -> shared memory: two bulk copies (the trees of a group are neighbours in the
  // packed arrays), issued by one thread
  auto stage_group = [&](int group, int buf) {
    if (tid != 0) return;
    const int t0       = group * TG;
    const unsigned nt  = static_cast<unsigned>(min(TG, n_trees - t0));
    const unsigned bar = bar0 + 8u * buf;
    const unsigned dst = tree0 + static_cast<unsigned>(buf) * buf_bytes;
    MbarExpectTx(bar, nt * (node_bytes + leaf_bytes));
    BulkCopy(dst, nodes_c + static_cast<int64_t>(t0) * NI, nt * node_bytes, bar);
    if (kLeafShared) BulkCopy(dst + TG * node_bytes, leaves_c + static_cast<int64_t>(t0) * NL, nt * leaf_bytes, bar);
  };
  stage_group(0, 0);

  // Stage the X tile: every thread copies its own row, feature-major with a pitch of RB elements,
  // so that thread t only ever touches bank t mod 32 (x 2 for float64) - on the way in and in every
  // step of every walk, whatever features the trees ask for.  16-byte loads when the rows allow it;
  // the sectors of a row are reused from L1 by the following loads of the same thread.
  if (tid < rows_here) {
    const T* xr     = X + (row0 + tid) * ldx;
    constexpr int V = 16 / sizeof(T);
    int f           = 0;
    if ((reinterpret_cast<uintptr_t>(X) & 15) == 0 && ldx % V == 0) {
#pragma unroll 4
      for (; f + V <= F; f += V) {
        const int4 v = *reinterpret_cast<const int4*>(xr + f);
#pragma unroll
        for (int i = 0; i < V; ++i) xs[(f + i) * RB + tid] = reinterpret_cast<const T*>(&v)[i];
      }
    }
    for (; f < F; ++f) xs[f * RB + tid] = xr[f];
  }
  if (K > 1)
    for (int k = 0; k < K; ++k) accs[k * RB + tid] = 0.0;

  // The walk works on 32-bit shared addresses.  `p8` is the heap index of the current node times 8
  // (times sizeof(NodeT)/8 it is the node's byte offset); after S steps it points into the bottom
  // level, whose values start at heap index 2^S - 1.
  constexpr unsigned kNodeShift = sizeof(NodeT) == 16 ? 1 : 0;
  const unsigned xcol_s   = static_cast<unsigned>(__cvta_generic_to_shared(xs + tid));
  const unsigned leaf_adj = TG * node_bytes - 8u * ((1u << S) - 1u);  // from a bottom-level p8 to the value, tree 0
  const bool one_buffer   = n_groups == 1;
  double acc0             = 0.0;
  __syncthreads();  // the X tile is in place
  for (int g = 0; g < n_groups; ++g) {
    const int buf = one_buffer ? 0 : (g & 1);
    // buffer `buf` is filled for the (g / 2)-th time (every time when there is one buffer)
    const unsigned parity = one_buffer ? (g & 1) : ((g >> 1) & 1);
    // group g has landed - or every thread of the block gives up together
    if (!__syncthreads_and(MbarWait(bar0 + 8u * buf, parity, status) ? 1 : 0)) break;
    if (g + 1 < n_groups && !one_buffer) stage_group(g + 1, buf ^ 1);
    const unsigned gbase = tree0 + static_cast<unsigned>(buf) * buf_bytes;
    const int nt         = min(TG, n_trees - g * TG);
    if (tid < rows_here) {
      unsigned p8[TG];
#pragma unroll
      for (int j = 0; j < TG; ++j) p8[j] = 0;
      if (nt == TG) {
        // a step of all TG walks: first every node load, then every x load, then the compares, so
        // that the loads of the independent walks are in flight together (the loads are volatile
        // and keep their order: interleaved per walk they would run one after the other)
        for (int step = 0; step < S; ++step) {
          T split[TG];
          int foff[TG];
          T x[TG];
#pragma unroll
          for (int j = 0; j < TG; ++j) LdsNode(gbase + j * node_bytes + (p8[j] << kNodeShift), split[j], foff[j]);
#pragma unroll
          for (int j = 0; j < TG; ++j) x[j] = LdsX(xcol_s + foff[j], T());
#pragma unroll
          for (int j = 0; j < TG; ++j) p8[j] = 2 * p8[j] + (x[j] <= split[j] ? 8u : 16u);
        }
      } else {
        // (the last, partial group: the same unrolled steps under a predicate, so that p8 stays in
        // registers)
        for (int step = 0; step < S; ++step) {
          T split[TG];
          int foff[TG];
          T x[TG];
#pragma unroll
          for (int j = 0; j < TG; ++j)
            if (j < nt) LdsNode(gbase + j * node_bytes + (p8[j] << kNodeShift), split[j], foff[j]);
#pragma unroll
          for (int j = 0; j < TG; ++j)
            if (j < nt) x[j] = LdsX(xcol_s + foff[j], T());
#pragma unroll
          for (int j = 0; j < TG; ++j)
            if (j < nt) p8[j] = 2 * p8[j] + (x[j] <= split[j] ? 8u : 16u);
        }
      }
#pragma unroll
      for (int j = 0; j < TG; ++j) {
        if (j < nt) {
          if (kLeafShared) {
            acc0 += LdsF64(gbase + j * leaf_bytes + leaf_adj + p8[j]);
          } else {
            const int64_t lj = static_cast<int64_t>(g * TG + j) * NL + ((p8[j] >> 3) - ((1u << S) - 1u));
            const double* lf = leaves_c + lj * K;
            for (int k = 0; k < K; ++k) accs[k * RB + tid] += lf[k];
          }
        }
      }
    }
    __syncthreads();  // everyone is done with buffer `buf` before it is refilled
    if (g + 1 < n_groups && one_buffer) stage_group(g + 1, 0);
  }
  if (tid < rows_here) {
    const int64_t row = row0 + tid;
    if (K == 1) {
      pred[row * ldp] = acc0;
    } else {
      for (int k = 0; k < K; ++k) pred[row * ldp + k] = accs[k * RB + tid];
    }
  }
}

// Fallback: original (uncompleted) trees, nodes and leaves in global memory, X read directly.
template <typename T>
__global__ void __launch_bounds__(128)
  k_predict_global(const T* __restrict__ X, int64_t ldx, int64_t n_rows, int K, int n_trees,
                   const TreePtrs* __restrict__ trees, const typename NodeOf<T>::type* __restrict__ nodes,
                   const double* __restrict__ leaves, double* __restrict__ pred, int64_t ldp)
{
  using NodeT       = typename NodeOf<T>::type;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (row >= n_rows) return;
  const T* xr = X + row * ldx;
  for (int k = 0; k < K; ++k) pred[row * ldp + k] = 0.0;
  for (int t = 0; t < n_trees; ++t) {
    const int off = trees[t].node_off;
    int pos       = 0;
    for (int depth = 0; depth < 100; ++depth) {
      const NodeT n = nodes[off + pos];
      if (n.foff < 0) break;
      pos = 2 * pos + 1 + (xr[n.foff] <= n.split ? 0 : 1);
    }
    const double* lf = leaves + static_cast<int64_t>(off + pos) * K;
    for (int k = 0; k < K; ++k) pred[row * ldp + k] += lf[k];
  }
}

template <typename T>
size_t TiledSmem(int rb, int tg, int nbuf, int F, int K, int NI, int NL, bool leaf_shared)
{
  using NodeT = typename NodeOf<T>::type;
  const size_t x_bytes    = (sizeof(T) * static_cast<size_t>(F) * rb + 15) / 16 * 16;
  const size_t a_bytes    = K > 1 ? sizeof(double) * static_cast<size_t>(K) * rb : 0;
  const size_t slot_bytes = static_cast<size_t>(NI) * sizeof(NodeT) + (leaf_shared ? static_cast<size_t>(NL) * sizeof(double) : 0);
  return x_bytes + a_bytes + static_cast<size_t>(nbuf) * tg * slot_bytes;
}

template <typename T, int RB, int TG, bool kLeafShared>
void LaunchTiled(const T* X, int64_t ldx, int64_t n_rows, int F, int K, int n_trees,
                 const typename NodeOf<T>::type* nodes_c, const double* leaves_c, double* pred, int64_t ldp, int S,
                 int NI, int NL, size_t smem, int* status, cudaStream_t stream)
{
  if (smem > 48 * 1024)
    LBK_CUDA(cudaFuncSetAttribute(k_predict_tiled<T, RB, TG, kLeafShared>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  static_cast<int>(smem)));
  const unsigned grid = static_cast<unsigned>((n_rows + RB - 1) / RB);
  k_predict_tiled<T, RB, TG, kLeafShared><<<grid, RB, smem, stream>>>(X, ldx, n_rows, F, K, n_trees, nodes_c, leaves_c, pred, ldp, S,
                                                          NI, NL, status);
  LBK_LAUNCH_CHECK();
}

}  // namespace

template <typename T>
void PredictLaunch(lbk_context* ctx, Scratch& s, const T* X, int64_t ldx, int64_t n_rows, int F, int K, int n_trees,
                   const double* const* leaf, const int32_t* const* feat, const double* const* split,
                   const int32_t* max_nodes, double* pred, int64_t ldp, cudaStream_t stream)
{
  using NodeT = typename NodeOf<T>::type;
  if (n_rows < 1) return;  // an empty shard returns at once (reference: predict.cu:35)
  if (n_trees == 0) {
    LBK_CUDA(cudaMemset2DAsync(pred, sizeof(double) * ldp, 0, sizeof(double) * K, n_rows, stream));
    return;
  }
  std::vector<TreePtrs> h(n_trees);
  int64_t total_nodes = 0;
  int m_max           = 1;
  for (int t = 0; t < n_trees; ++t) {
    LBK_EXPECT(leaf[t] && feat[t] && split[t] && max_nodes[t] >= 1, "bad tree arrays");
    h[t].leaf      = leaf[t];
    h[t].feature   = feat[t];
    h[t].split     = split[t];
    h[t].max_nodes = max_nodes[t];
    LBK_EXPECT(total_nodes + max_nodes[t] < (int64_t{1} << 31), "ensemble too large");
    h[t].node_off = static_cast<int>(total_nodes);
    total_nodes += max_nodes[t];
    m_max = max_nodes[t] > m_max ? max_nodes[t] : m_max;
  }
  // a walk through M heap-ordered nodes takes at most S = floor(log2(M)) steps
  int S = 0;
  while ((2 << S) <= m_max) ++S;
  const int NI = (1 << S) > 2 ? (1 << S) : 2;  // internal nodes 2^S - 1, padded to a 16-byte multiple
  const int NL = NI;                           // bottom level 2^S values, same padding

  // tile shape: rows per block RB, trees per group TG, one or two group buffers.  (Measured at 5 M x
  // 100, 500 trees of depth 8: groups of 8 trees 14.8 ms; groups of 16 with the bottom-level values
  // left in global memory 29.8 ms; groups of 4 27.3 ms.)
  const size_t budget = static_cast<size_t>(ctx->max_smem_optin) - 1024;
  int rb = 0, tg = 0;
  const bool leaf_shared = K == 1;
  size_t smem = 0;
  if (S <= 14) {
    const int rbs[4] = {256, 128, 64, 32};
    const int tgs[4] = {8, 4, 2, 1};
    for (int ri = 0; ri < 4 && rb == 0; ++ri) {
      if (static_cast<int64_t>(F) * rbs[ri] * static_cast<int64_t>(sizeof(T)) >= (int64_t{1} << 30)) continue;
      for (int ti = 0; ti < 4 && rb == 0; ++ti) {
        if (tgs[ti] > n_trees && tgs[ti] > 1) continue;  // no wider than the ensemble
        const int nbuf = n_trees > tgs[ti] ? 2 : 1;
        const size_t need = TiledSmem<T>(rbs[ri], tgs[ti], nbuf, F, K, NI, NL, leaf_shared);
        if (need <= budget) {
          rb   = rbs[ri];
          tg   = tgs[ti];
          smem = need;
        }
      }
    }
  }

  TreePtrs* d_trees = s.alloc<TreePtrs>(n_trees);
  LBK_CUDA(cudaMemcpyAsync(d_trees, h.data(), sizeof(TreePtrs) * n_trees, cudaMemcpyHostToDevice, stream));
  LBK_CUDA(cudaStreamSynchronize(stream));  // h is a local; the copy must have read it

  if (rb == 0) {
    NodeT* nodes   = s.alloc<NodeT>(total_nodes);
    double* leaves = s.alloc<double>(total_nodes * K);
    k_pack_trees<NodeT><<<n_trees, 256, 0, stream>>>(d_trees, K, F, 1, nodes, leaves);
    LBK_LAUNCH_CHECK();
    const unsigned grid = static_cast<unsigned>((n_rows + 127) / 128);
    k_predict_global<T><<<grid, 128, 0, stream>>>(X, ldx, n_rows, K, n_trees, d_trees, nodes, leaves, pred, ldp);
    LBK_LAUNCH_CHECK();
    return;
  }
  NodeT* nodes_c   = s.alloc<NodeT>(static_cast<size_t>(n_trees) * NI);
  double* leaves_c = s.alloc<double>(static_cast<size_t>(n_trees) * NL * K);
  k_pack_complete<NodeT><<<n_trees, 256, 0, stream>>>(d_trees, K, F, rb * static_cast<int>(sizeof(T)), S, NI, NL,
                                                      nodes_c, leaves_c);
  LBK_LAUNCH_CHECK();
#define LBK_PREDICT_CASE(RB_, TG_, LS_)                                                                             \
  if (rb == RB_ && tg == TG_ && leaf_shared == LS_) {                                                               \
    LaunchTiled<T, RB_, TG_, LS_>(X, ldx, n_rows, F, K, n_trees, nodes_c, leaves_c, pred, ldp, S, NI, NL, smem,     \
                                  ctx->d_status, stream);                                                           \
    return;                                                                                                         \
  }
#define LBK_PREDICT_ROW(RB_)                                                                                        \
  LBK_PREDICT_CASE(RB_, 8, true) LBK_PREDICT_CASE(RB_, 4, true) LBK_PREDICT_CASE(RB_, 2, true) LBK_PREDICT_CASE(RB_, 1, true) \
  LBK_PREDICT_CASE(RB_, 8, false) LBK_PREDICT_CASE(RB_, 4, false) LBK_PREDICT_CASE(RB_, 2, false) LBK_PREDICT_CASE(RB_, 1, false)
  LBK_PREDICT_ROW(256)
  LBK_PREDICT_ROW(128)
  LBK_PREDICT_ROW(64)
  LBK_PREDICT_ROW(32)
#undef LBK_PREDICT_ROW
#undef LBK_PREDICT_CASE
  throw Error(LBK_ERR_ARGUMENT, "predict: no kernel for the chosen tile");
}

template void PredictLaunch<float>(lbk_context*, Scratch&, const float*, int64_t, int64_t, int, int, int,
                                   const double* const*, const int32_t* const*, const double* const*, const int32_t*,
                                   double*, int64_t, cudaStream_t);
template void PredictLaunch<double>(lbk_context*, Scratch&, const double*, int64_t, int64_t, int, int, int,
                                    const double* const*, const int32_t* const*, const double* const*, const int32_t*,
                                    double*, int64_t, cudaStream_t);

}  // namespace lbk
