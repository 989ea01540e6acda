// CPU oracle for the tree-building hot path of legate-boost (BUILD_TREE and PREDICT tasks).
//
// TEST INFRASTRUCTURE ONLY.  This file restates, in plain single-threaded C++17, the algorithm
// of the reference's tree builder so the CUDA library can be checked against it.  It is
// never linked into, imported by or called from the product library; only the test-suite,
// the smoke check and the CPU-baseline leg of the benchmark load it.
//
// Two modes are restated, each citing the reference file (paths relative to the reference
// project root) it follows:
//   Mode Q ("quantised") = semantics of the GPU variant  src/models/tree/build_tree.cu
//   Mode D ("double")    = semantics of the CPU variant  src/models/tree/build_tree.cc
// plus the ensemble predict of src/models/tree/predict.cc / predict.cu.
//
// Pinning: Mode D and predict are checked bit-for-bit against the reference's own
// unmodified build_tree.cc / predict.cc compiled against a host-only stand-in for the
// runtime headers (see ref_stub/ and the Makefile target `ref`).  The random-number
// restatement is checked against the CUDA toolkit's thrust headers (check_rng.cpp).  Mode Q
// follows a GPU-only source file that cannot run on a machine without a GPU; it is pinned
// by construction (shared code with Mode D for every stage the two variants have in
// common) and by the reference's known-answer tests.
//
// Floating point: compile with -ffp-contract=off.  Products that feed comparisons are not
// fused with the following add/subtract.
//
// Canonical |g|,|h| summation order (the reference uses thrust::reduce, whose order is
// unspecified): see canonical_abs_sum() below.  The CUDA library implements the same order.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <random>
#include <set>
#include <tuple>
#include <vector>

namespace {

constexpr double kEps = 1e-5;  // build_tree.h:31

struct GPairD {
  double grad = 0.0, hess = 0.0;
};
struct GPairI {
  int64_t grad = 0, hess = 0;
};

// ---------------------------------------------------------------------------------------
// Binary-tree helpers, build_tree.h:63-73
inline int Parent(int i) { return (i - 1) / 2; }
inline int LeftChild(int i) { return 2 * i + 1; }
inline int RightChild(int i) { return 2 * i + 2; }
inline int Sibling(int i) { return (i % 2 == 0) ? i - 1 : i + 1; }
inline int64_t LevelBegin(int level) { return (int64_t{1} << level) - 1; }
inline int64_t LevelEnd(int level) { return (int64_t{1} << (level + 1)) - 1; }
inline int64_t NodesInLevel(int level) { return int64_t{1} << level; }

// ---------------------------------------------------------------------------------------
// thrust::default_random_engine = minstd_rand: x <- 48271 x mod (2^31-1); a seed congruent
// to 0 becomes 1 (thrust/random/detail/linear_congruential_engine.inl, seed()).  The seed
// argument is converted to the engine's 32-bit unsigned result type first.
struct MinStd {
  static constexpr uint64_t kA = 48271, kM = 2147483647;
  uint32_t x;
  explicit MinStd(uint32_t s)
  {
    uint32_t r = static_cast<uint32_t>(s % kM);
    x          = r == 0 ? 1u : r;
  }
  uint32_t next()
  {
    x = static_cast<uint32_t>((kA * x) % kM);
    return x;
  }
  void discard(uint64_t z)
  {  // modular exponentiation, linear_congruential_engine_discard.h
    uint64_t mult = kA, mult_z = 1;
    while (z > 0) {
      if (z & 1) mult_z = (mult_z * mult) % kM;
      z >>= 1;
      mult = (mult * mult) % kM;
    }
    x = static_cast<uint32_t>((mult_z * x) % kM);
  }
  // thrust::uniform_real_distribution<double>(a,b): (urng()-min)/(1+(max-min)) * (b-a) + a
  // with min = 1, max = 2^31-2.
  double uniform_real(double a, double b)
  {
    double r = static_cast<double>(next() - 1u);
    r /= (1.0 + static_cast<double>(2147483646u - 1u));
    return (r * (b - a)) + a;
  }
  // thrust::uniform_int_distribution<int64_t>(a,b): truncation of a real draw from [a,b+1)
  int64_t uniform_int(int64_t a, int64_t b)
  {
    const double real_min = static_cast<double>(a);
    const double real_max = static_cast<double>(b);
    return static_cast<int64_t>(uniform_real(real_min, real_max + 1.0));
  }
};

// build_tree.cu:143-165  (MurmurHash3 fmix64 on a signed 64-bit value; boost hash_combine)
inline int64_t hash64(int64_t k)
{
  k ^= k >> 33;
  k = static_cast<int64_t>(static_cast<uint64_t>(k) * 0xff51afd7ed558ccdULL);
  k ^= k >> 33;
  k = static_cast<int64_t>(static_cast<uint64_t>(k) * 0xc4ceb9fe1a85ec53ULL);
  k ^= k >> 33;
  return k;
}
inline int64_t hash_combine1(int64_t seed, int64_t v)
{
  uint64_t add = static_cast<uint64_t>(hash64(v)) + 0x9e3779b9ULL +
                 (static_cast<uint64_t>(seed) << 6) + static_cast<uint64_t>(seed >> 2);
  return seed ^ static_cast<int64_t>(add);
}
inline int64_t hash_combine(int64_t seed, int64_t a, int64_t b)
{
  return hash_combine1(hash_combine1(seed, a), b);
}

// ---------------------------------------------------------------------------------------
// Canonical summation order for the local sum of |v| that fixes the quantiser scale
// (build_tree.cu:77-83 uses thrust::reduce; its order is unspecified, this fixes one).
//   * elements are cut into blocks of 4096;
//   * inside a block, "thread" t in [0,256) adds elements t, t+256, ..., t+15*256 in that
//     order starting from +0.0 (missing elements count as +0.0);
//   * every group of 32 consecutive threads is folded with offsets 16,8,4,2,1
//     (s[l] += s[l+offset] for l < offset);
//   * the eight group sums are added left to right;
//   * the block sums form a new array which is reduced the same way until one value is left.
double canonical_sum(std::vector<double> v)
{
  if (v.empty()) return 0.0;
  while (true) {
    const size_t n       = v.size();
    const size_t nblocks = (n + 4095) / 4096;
    std::vector<double> out(nblocks);
    for (size_t b = 0; b < nblocks; ++b) {
      double s[256];
      for (int t = 0; t < 256; ++t) {
        double acc = 0.0;
        for (int j = 0; j < 16; ++j) {
          size_t idx = b * 4096 + static_cast<size_t>(j) * 256 + t;
          acc += idx < n ? v[idx] : 0.0;
        }
        s[t] = acc;
      }
      double total = 0.0;
      for (int w = 0; w < 8; ++w) {
        double* l = s + w * 32;
        for (int off = 16; off >= 1; off >>= 1)
          for (int i = 0; i < off; ++i) l[i] += l[i + off];
        total = (w == 0) ? l[0] : total + l[0];
      }
      out[b] = total;
    }
    if (nblocks == 1) return out[0];
    v.swap(out);
  }
}

// ---------------------------------------------------------------------------------------
// CalculateGain / CalculateLeafValue, build_tree.h:106-152
inline double LeafGain(GPairD s, double l1, double l2)
{
  double z = 0.0;
  if (s.grad > l1) {
    z = s.grad - l1;
  } else if (s.grad < -l1) {
    z = s.grad + l1;
  }
  return (z * z) / (s.hess + l2);
}
inline double CalculateGain(GPairD l, GPairD r, GPairD p, double l1, double l2, double msg)
{
  const double reg = std::max(kEps, l2);
  return (0.5 * (LeafGain(l, l1, reg) + LeafGain(r, l1, reg) - LeafGain(p, l1, reg))) - msg;
}
inline double CalculateLeafValue(double G, double H, double l1, double l2)
{
  double z = 0.0;
  if (G > l1) {
    z = G - l1;
  } else if (G < -l1) {
    z = G + l1;
  }
  return -z / (H + l2);
}

// ---------------------------------------------------------------------------------------
// Split proposals.  Mode Q: build_tree.cu:867-964.  Mode D: build_tree.cc:171-226.
template <typename T>
struct Proposals {
  std::vector<T> values;         // CSR values, length B
  std::vector<int32_t> row_ptr;  // F+1
  int FindBin(T x, int f) const
  {  // lower_bound, build_tree.h:178-213
    const T* b = values.data() + row_ptr[f];
    const T* e = values.data() + row_ptr[f + 1];
    return static_cast<int>(std::lower_bound(b, e, x) - values.data());
  }
};

template <typename T>
Proposals<T> SelectSplitSamples(int mode,
                                const T* X,
                                int64_t n_rows,
                                int F,
                                int S,
                                int seed,
                                int n_ranks,
                                const int64_t* rank_off)
{
  std::vector<int64_t> rows(S);
  if (mode == 0) {
    for (int i = 0; i < S; ++i) {
      MinStd eng(static_cast<uint32_t>(seed));
      eng.discard(static_cast<uint64_t>(i));
      rows[i] = eng.uniform_int(0, n_rows - 1);
    }
  } else {
    std::default_random_engine eng(seed);
    std::uniform_int_distribution<int64_t> dist(0, n_rows - 1);
    for (int i = 0; i < S; ++i) rows[i] = dist(eng);
  }
  // draft[f][i]: the owning rank contributes the value, every other rank 0; summed in rank
  // order as an allreduce would.
  std::vector<T> draft(static_cast<size_t>(F) * S);
  for (int i = 0; i < S; ++i) {
    for (int f = 0; f < F; ++f) {
      T acc = T(0);
      for (int r = 0; r < n_ranks; ++r) {
        bool has = rows[i] >= rank_off[r] && rows[i] < rank_off[r + 1];
        T v      = has ? X[rows[i] * F + f] : T(0);
        acc      = (r == 0) ? v : acc + v;
      }
      draft[static_cast<size_t>(f) * S + i] = acc;
    }
  }
  Proposals<T> p;
  p.row_ptr.assign(F + 1, 0);
  for (int f = 0; f < F; ++f) {
    std::vector<T> col(draft.begin() + static_cast<size_t>(f) * S,
                       draft.begin() + static_cast<size_t>(f + 1) * S);
    std::sort(col.begin(), col.end());
    col.erase(std::unique(col.begin(), col.end()), col.end());
    p.values.insert(p.values.end(), col.begin(), col.end());
    p.row_ptr[f + 1] = static_cast<int32_t>(p.values.size());
    p.values.back()  = std::numeric_limits<T>::infinity();
  }
  return p;
}

// ---------------------------------------------------------------------------------------
// Gradient quantiser, build_tree.cu:51-140.
struct Quantiser {
  GPairD scale, inv;
  void Init(const double* g,
            const double* h,
            int K,
            int n_ranks,
            const int64_t* rank_off)
  {
    double mg = 0.0, mh = 0.0;
    for (int r = 0; r < n_ranks; ++r) {
      const int64_t b = rank_off[r] * K, e = rank_off[r + 1] * K;
      std::vector<double> ag(e - b), ah(e - b);
      for (int64_t i = b; i < e; ++i) {
        ag[i - b] = std::fabs(g[i]);
        ah[i - b] = std::fabs(h[i]);
      }
      double sg = canonical_sum(std::move(ag));
      double sh = canonical_sum(std::move(ah));
      mg        = (r == 0) ? sg : std::max(mg, sg);  // ncclMax over ranks
      mh        = (r == 0) ? sh : std::max(mh, sh);
    }
    const double max_int = 2147483647.0;
    scale.grad           = mg == 0 ? 1 : max_int / mg;
    scale.hess           = mh == 0 ? 1 : max_int / mh;
    inv.grad             = 1.0 / scale.grad;
    inv.hess             = 1.0 / scale.hess;
  }
  GPairI Quantise(double gv, double hv, int64_t seed) const
  {
    MinStd eng(static_cast<uint32_t>(static_cast<uint64_t>(seed)));
    const double sg = gv * scale.grad;
    const double sh = hv * scale.hess;
    const double rg = sg - std::floor(sg);
    const double rh = sh - std::floor(sh);
    GPairI q;
    q.grad = static_cast<int64_t>(std::floor(sg) + static_cast<double>(eng.uniform_real(0, 1) < rg));
    q.hess = static_cast<int64_t>(std::floor(sh) + static_cast<double>(eng.uniform_real(0, 1) < rh));
    return q;
  }
  GPairD Dequantise(GPairI v) const
  {
    GPairD r;
    r.grad = static_cast<double>(v.grad) * inv.grad;
    r.hess = static_cast<double>(v.hess) * inv.hess;
    return r;
  }
};

// SelectHistogramNode / ComputeHistogramBin, build_tree.h:80-104
template <typename SumT>
inline bool ComputeHistogramBin(int node, const std::vector<SumT>& node_sums, int K, bool parent_exists)
{
  if (node == 0) return true;
  if (node < 0) return false;
  if (!parent_exists) return true;
  const int parent = Parent(node);
  const int l = LeftChild(parent), r = RightChild(parent);
  const int hist_node =
    (node_sums[static_cast<size_t>(l) * K].hess < node_sums[static_cast<size_t>(r) * K].hess) ? l : r;
  return hist_node == node;
}

// Histogram over a node range, [node][output][bin]; build_tree.h:231-306
template <typename P>
struct Hist {
  std::vector<P> data;
  int node_begin = 0, node_end = 0, K = 0, B = 0;
  void Reset(int nb, int ne, int K_, int B_)
  {
    node_begin = nb;
    node_end   = ne;
    K          = K_;
    B          = B_;
    data.assign(static_cast<size_t>(ne - nb) * K * B, P{});
  }
  bool ContainsBatch(int nb, int ne) const { return nb >= node_begin && ne <= node_end; }
  bool ContainsNode(int n) const { return n >= node_begin && n < node_end; }
  P& at(int node, int k, int bin)
  {
    return data[(static_cast<size_t>(node - node_begin) * K + k) * B + bin];
  }
};

}  // namespace

// =======================================================================================
// C interface
extern "C" {

struct lbo_tree_args {
  int32_t mode;       // 0 = Q (GPU-variant semantics), 1 = D (CPU-variant semantics)
  int32_t x_is_f64;   // 0: X is float32, 1: float64
  const void* X;      // [n_rows, F] row-major, the whole (global) matrix
  const double* g;    // [n_rows, K]
  const double* h;    // [n_rows, K]
  const uint8_t* feature_set;  // optional bool[F]
  int64_t n_rows;
  int32_t F, K;
  int32_t max_depth, split_samples, seed;
  double l1, l2, min_split_gain;
  int32_t n_ranks;            // simulated row shards
  const int64_t* rank_off;    // [n_ranks+1] row offsets
  // outputs, M = 2^(max_depth+1)-1
  double* leaf_value;   // [M,K]
  int32_t* feature;     // [M]
  double* split_value;  // [M]
  double* gain;         // [M]
  double* hessian;      // [M,K]
  // optional traces (may be null)
  int32_t* out_B;         // total bins
  int32_t* out_row_ptr;   // [F+1]
  void* out_proposals;    // T[F*S] (first B valid)
  int64_t* out_q;         // mode Q: [n_rows,K,2] quantised pairs
  double* out_scale;      // mode Q: scale.g, scale.h, inv.g, inv.h
  int64_t* out_node_sums; // mode Q: [M,K,2] integers; mode D: doubles bit-cast
  int32_t trace_nodes;    // number of leading nodes whose final histogram is copied out
  void* trace_hist;       // [trace_nodes,K,B,2] (int64 in mode Q, double in mode D); the
                          // state each node's histogram had when its split was evaluated
  int32_t* out_positions; // [n_rows] node id of every row after the last position update
};

}  // extern "C"

namespace {

template <typename T>
int BuildTreeQ(const lbo_tree_args& a)
{
  const T* X        = static_cast<const T*>(a.X);
  const int F = a.F, K = a.K;
  const int64_t N   = a.n_rows;
  const int max_nodes = static_cast<int>(LevelEnd(a.max_depth));
  std::vector<int64_t> one_rank = {0, N};
  const int n_ranks       = a.n_ranks > 0 ? a.n_ranks : 1;
  const int64_t* rank_off = a.n_ranks > 0 ? a.rank_off : one_rank.data();

  // Tree, build_tree.cu:785-809
  std::vector<double> leaf_value(static_cast<size_t>(max_nodes) * K, 0.0);
  std::vector<int32_t> feature(max_nodes, -1);
  std::vector<double> split_value(max_nodes, 0.0), gain(max_nodes, 0.0);
  std::vector<GPairI> node_sums(static_cast<size_t>(max_nodes) * K);

  auto prop   = SelectSplitSamples<T>(0, X, N, F, a.split_samples, a.seed, n_ranks, rank_off);
  const int B = static_cast<int>(prop.values.size());
  if (a.out_B) *a.out_B = B;
  if (a.out_row_ptr) std::copy(prop.row_ptr.begin(), prop.row_ptr.end(), a.out_row_ptr);
  if (a.out_proposals) std::memcpy(a.out_proposals, prop.values.data(), sizeof(T) * B);

  // bins once (the GPU variant searches per level; the value is the same)
  std::vector<int32_t> bins(static_cast<size_t>(N) * F);
  for (int64_t i = 0; i < N; ++i)
    for (int f = 0; f < F; ++f) bins[i * F + f] = prop.FindBin(X[i * F + f], f);

  Quantiser quant;
  quant.Init(a.g, a.h, K, n_ranks, rank_off);
  if (a.out_scale) {
    a.out_scale[0] = quant.scale.grad;
    a.out_scale[1] = quant.scale.hess;
    a.out_scale[2] = quant.inv.grad;
    a.out_scale[3] = quant.inv.hess;
  }
  const int64_t seed = a.seed;
  std::vector<GPairI> q(static_cast<size_t>(N) * K);
  for (int64_t i = 0; i < N; ++i)
    for (int k = 0; k < K; ++k)
      q[i * K + k] = quant.Quantise(a.g[i * K + k], a.h[i * K + k], hash_combine(seed, i, k));
  if (a.out_q) std::memcpy(a.out_q, q.data(), sizeof(GPairI) * q.size());

  // InitialiseRoot, build_tree.cu:1154-1187
  for (int64_t i = 0; i < N; ++i)
    for (int k = 0; k < K; ++k) {
      node_sums[k].grad += q[i * K + k].grad;
      node_sums[k].hess += q[i * K + k].hess;
    }
  for (int k = 0; k < K; ++k) {
    GPairD s      = quant.Dequantise(node_sums[k]);
    leaf_value[k] = CalculateLeafValue(s.grad, s.hess, a.l1, a.l2);
  }

  // histogram cache, build_tree.cu:1000-1017
  const size_t max_bytes           = 1000000000;
  const size_t bytes_per_node      = static_cast<size_t>(K) * B * 16;
  const size_t max_histogram_nodes = std::max<size_t>(1, max_bytes / bytes_per_node);
  int cdepth                       = 0;
  while (static_cast<size_t>(LevelEnd(cdepth + 1)) <= max_histogram_nodes && cdepth <= a.max_depth) cdepth++;
  Hist<GPairI> hist;
  hist.Reset(0, static_cast<int>(LevelEnd(cdepth)), K, B);
  const int64_t max_batch_size = static_cast<int>(max_histogram_nodes);  // stored in an int

  std::vector<int32_t> pos(N, 0);
  GPairI* trace = static_cast<GPairI*>(a.trace_hist);

  for (int depth = 0; depth < a.max_depth; ++depth) {
    // PrepareBatches, build_tree.cu:1207-1258
    std::vector<std::pair<int, int>> batches;
    if (NodesInLevel(depth) <= max_batch_size) {
      batches.push_back({static_cast<int>(LevelBegin(depth)), static_cast<int>(LevelEnd(depth))});
    } else {
      const int64_t nb = (NodesInLevel(depth) + max_batch_size - 1) / max_batch_size;
      for (int64_t b = 0; b < nb; ++b) {
        int64_t bb = LevelBegin(depth) + b * max_batch_size;
        int64_t be = std::min(bb + max_batch_size, LevelEnd(depth));
        batches.push_back({static_cast<int>(bb), static_cast<int>(be)});
      }
    }
    for (auto [nb, ne] : batches) {
      if (!hist.ContainsBatch(nb, ne)) hist.Reset(nb, ne, K, B);  // GetHistogram :1191-1205
      // fill_histogram_shared, :363-408 (integer sums: order free)
      for (int64_t i = 0; i < N; ++i) {
        const int p = pos[i];
        if (p < nb || p >= ne) continue;
        if (!ComputeHistogramBin(p, node_sums, K, hist.ContainsNode(Parent(p)))) continue;
        for (int k = 0; k < K; ++k) {
          const GPairI v = q[i * K + k];
          for (int f = 0; f < F; ++f) {
            GPairI& e = hist.at(p, k, bins[i * F + f]);
            e.grad += v.grad;
            e.hess += v.hess;
          }
        }
      }
      // scan_kernel, :597-668
      for (int node = nb; node < ne; ++node) {
        const int parent = Parent(node);
        for (int k = 0; k < K; ++k) {
          if (node_sums[static_cast<size_t>(node) * K + k].hess <= 0) continue;
          if (!ComputeHistogramBin(node, node_sums, K, hist.ContainsNode(parent))) continue;
          for (int f = 0; f < F; ++f) {
            GPairI agg;
            for (int b = prop.row_ptr[f]; b < prop.row_ptr[f + 1]; ++b) {
              GPairI& e = hist.at(node, k, b);
              agg.grad += e.grad;
              agg.hess += e.hess;
              if (agg.grad > 0 || agg.hess > 0) e = agg;  // write skipped when both <= 0
            }
          }
          if (node == 0) continue;
          const int sib = Sibling(node);
          if (!ComputeHistogramBin(sib, node_sums, K, hist.ContainsNode(parent))) {
            for (int b = 0; b < B; ++b) {
              GPairI s = hist.at(node, k, b), p = hist.at(parent, k, b);
              hist.at(sib, k, b) = GPairI{p.grad - s.grad, p.hess - s.hess};
            }
          }
        }
      }
      if (trace) {
        for (int node = nb; node < ne && node < a.trace_nodes; ++node)
          std::memcpy(trace + static_cast<size_t>(node) * K * B, &hist.at(node, 0, 0), sizeof(GPairI) * K * B);
      }
      // perform_best_split, :682-782
      for (int node = nb; node < ne; ++node) {
        if (node_sums[static_cast<size_t>(node) * K].hess <= 0) continue;
        // thread t owns bins t, t+512, ... and keeps its first strict maximum
        constexpr int kThreads = 512;
        double tbest[kThreads];
        int tbin[kThreads];
        for (int t = 0; t < kThreads; ++t) {
          tbest[t] = 0;
          tbin[t]  = -1;
        }
        int f = 0;
        for (int b = 0; b < B; ++b) {
          while (b >= prop.row_ptr[f + 1]) ++f;
          if (a.feature_set && !a.feature_set[f]) continue;
          double gsum = 0;
          for (int k = 0; k < K; ++k) {
            GPairI ns = node_sums[static_cast<size_t>(node) * K + k];
            GPairI ls = hist.at(node, k, b);
            GPairI rs{ns.grad - ls.grad, ns.hess - ls.hess};
            if (ls.hess <= 0 || rs.hess <= 0) {
              gsum = 0;
              break;
            }
            gsum += CalculateGain(quant.Dequantise(ls), quant.Dequantise(rs), quant.Dequantise(ns),
                                  a.l1, a.l2, a.min_split_gain);
          }
          const int t = b % kThreads;
          if (gsum > tbest[t]) {
            tbest[t] = gsum;
            tbin[t]  = b;
          }
        }
        // cub::BlockReduce with op(a,b) = a.gain > b.gain ? a : b, left operand = lower
        // thread ids: equal gains resolve to the higher thread id.
        double best = tbest[0];
        int bbin    = tbin[0];
        for (int t = 1; t < kThreads; ++t) {
          if (!(best > tbest[t])) {
            best = tbest[t];
            bbin = tbin[t];
          }
        }
        if (best > kEps) {
          int bf = 0;
          while (bbin >= prop.row_ptr[bf + 1]) ++bf;
          const int l = LeftChild(node), r = RightChild(node);
          for (int k = 0; k < K; ++k) {
            GPairI ns = node_sums[static_cast<size_t>(node) * K + k];
            GPairI ls = hist.at(node, k, bbin);
            GPairI rs{ns.grad - ls.grad, ns.hess - ls.hess};
            node_sums[static_cast<size_t>(l) * K + k] = ls;
            node_sums[static_cast<size_t>(r) * K + k] = rs;
            GPairD dl = quant.Dequantise(ls), dr = quant.Dequantise(rs);
            leaf_value[static_cast<size_t>(l) * K + k] = CalculateLeafValue(dl.grad, dl.hess, a.l1, a.l2);
            leaf_value[static_cast<size_t>(r) * K + k] = CalculateLeafValue(dr.grad, dr.hess, a.l1, a.l2);
          }
          feature[node]     = bf;
          split_value[node] = static_cast<double>(prop.values[bbin]);
          gain[node]        = best;
        }
      }
    }
    // UpdatePositions, :1026-1047
    if (depth < a.max_depth - 1) {
      for (int64_t i = 0; i < N; ++i) {
        int p = pos[i];
        if (p < 0 || p >= max_nodes || feature[p] == -1) {
          pos[i] = -1;
          continue;
        }
        const double xv = static_cast<double>(X[i * F + feature[p]]);
        pos[i]          = xv <= split_value[p] ? LeftChild(p) : RightChild(p);
      }
    }
  }
  std::copy(leaf_value.begin(), leaf_value.end(), a.leaf_value);
  std::copy(feature.begin(), feature.end(), a.feature);
  std::copy(split_value.begin(), split_value.end(), a.split_value);
  std::copy(gain.begin(), gain.end(), a.gain);
  for (size_t i = 0; i < node_sums.size(); ++i) a.hessian[i] = quant.Dequantise(node_sums[i]).hess;
  if (a.out_node_sums) std::memcpy(a.out_node_sums, node_sums.data(), sizeof(GPairI) * node_sums.size());
  if (a.out_positions) std::copy(pos.begin(), pos.end(), a.out_positions);
  return 0;
}

// Sum over simulated ranks in rank order starting from 0.0, as the CPU allreduce does
// (cpp_utils.h:204-221: partials[j] = 0.0; partials[j] = partials[j] + recv[rank][j]).
inline void RankSum(std::vector<std::vector<GPairD>>& parts, GPairD* out, size_t n)
{
  for (size_t j = 0; j < n; ++j) {
    GPairD s{0.0, 0.0};
    for (auto& p : parts) {
      s.grad += p[j].grad;
      s.hess += p[j].hess;
    }
    out[j] = s;
  }
}

template <typename T>
int BuildTreeD(const lbo_tree_args& a)
{
  const T* X = static_cast<const T*>(a.X);
  const int F = a.F, K = a.K;
  const int64_t N     = a.n_rows;
  const int max_nodes = static_cast<int>(LevelEnd(a.max_depth));
  std::vector<int64_t> one_rank = {0, N};
  const int n_ranks       = a.n_ranks > 0 ? a.n_ranks : 1;
  const int64_t* rank_off = a.n_ranks > 0 ? a.rank_off : one_rank.data();

  std::vector<double> leaf_value(static_cast<size_t>(max_nodes) * K, 0.0);
  std::vector<int32_t> feature(max_nodes, -1);
  std::vector<double> split_value(max_nodes, 0.0), gain(max_nodes, 0.0);
  std::vector<GPairD> node_sums(static_cast<size_t>(max_nodes) * K);

  auto prop   = SelectSplitSamples<T>(1, X, N, F, a.split_samples, a.seed, n_ranks, rank_off);
  const int B = static_cast<int>(prop.values.size());
  if (a.out_B) *a.out_B = B;
  if (a.out_row_ptr) std::copy(prop.row_ptr.begin(), prop.row_ptr.end(), a.out_row_ptr);
  if (a.out_proposals) std::memcpy(a.out_proposals, prop.values.data(), sizeof(T) * B);

  std::vector<int32_t> bins(static_cast<size_t>(N) * F);  // BinnedX, build_tree.cc:32-70
  for (int64_t i = 0; i < N; ++i)
    for (int f = 0; f < F; ++f) bins[i * F + f] = prop.FindBin(X[i * F + f], f);

  // InitialiseRoot, build_tree.cc:471-493
  {
    std::vector<std::vector<GPairD>> parts(n_ranks, std::vector<GPairD>(K));
    for (int r = 0; r < n_ranks; ++r)
      for (int64_t i = rank_off[r]; i < rank_off[r + 1]; ++i)
        for (int k = 0; k < K; ++k) {
          parts[r][k].grad += a.g[i * K + k];
          parts[r][k].hess += a.h[i * K + k];
        }
    if (n_ranks == 1) {
      for (int k = 0; k < K; ++k) node_sums[k] = parts[0][k];
    } else {
      RankSum(parts, node_sums.data(), K);
    }
    for (int k = 0; k < K; ++k)
      leaf_value[k] = CalculateLeafValue(node_sums[k].grad, node_sums[k].hess, a.l1, a.l2);
  }

  const size_t max_bytes           = 1000000000;
  const size_t bytes_per_node      = static_cast<size_t>(K) * B * 16;
  const size_t max_histogram_nodes = std::max<size_t>(1, max_bytes / bytes_per_node);
  int cdepth                       = 0;
  while (static_cast<size_t>(LevelEnd(cdepth + 1)) <= max_histogram_nodes && cdepth <= a.max_depth) cdepth++;
  Hist<GPairD> hist;
  hist.Reset(0, static_cast<int>(LevelEnd(cdepth)), K, B);
  const int64_t max_batch_size = static_cast<int>(max_histogram_nodes);

  // (node,row) pairs per rank; order matters for the double sums
  std::vector<std::vector<std::pair<int32_t, int32_t>>> sorted(n_ranks);
  for (int r = 0; r < n_ranks; ++r)
    for (int64_t i = rank_off[r]; i < rank_off[r + 1]; ++i)
      sorted[r].push_back({0, static_cast<int32_t>(i - rank_off[r])});
  GPairD* trace = static_cast<GPairD*>(a.trace_hist);

  for (int depth = 0; depth < a.max_depth; ++depth) {
    std::vector<std::pair<int, int>> batches;
    const bool single = NodesInLevel(depth) <= max_batch_size;
    if (single) {
      batches.push_back({static_cast<int>(LevelBegin(depth)), static_cast<int>(LevelEnd(depth))});
    } else {
      // build_tree.cc:442-469 sorts by node with std::sort (order inside a node is then
      // unspecified; a stable sort is used here) and drops empty batches per rank.  With
      // one simulated process per rank an empty batch on some ranks only would desynchronise
      // the reference's collectives, so batches are kept whenever any rank has rows.
      for (auto& s : sorted)
        std::stable_sort(s.begin(), s.end(), [](auto& x, auto& y) { return x.first < y.first; });
      const int64_t nb = (NodesInLevel(depth) + max_batch_size - 1) / max_batch_size;
      for (int64_t b = 0; b < nb; ++b) {
        int64_t bb = LevelBegin(depth) + b * max_batch_size;
        int64_t be = std::min(bb + max_batch_size, LevelEnd(depth));
        bool any   = false;
        for (auto& s : sorted)
          for (auto& pr : s)
            if (pr.first >= bb && pr.first < be) {
              any = true;
              break;
            }
        if (any) batches.push_back({static_cast<int>(bb), static_cast<int>(be)});
      }
    }
    for (auto [nb, ne] : batches) {
      if (!hist.ContainsBatch(nb, ne)) hist.Reset(nb, ne, K, B);
      // ComputeHistogram, build_tree.cc:258-289
      const size_t span = static_cast<size_t>(ne - nb) * K * B;
      std::vector<std::vector<GPairD>> parts;
      GPairD* base = &hist.at(nb, 0, 0);
      for (int r = 0; r < n_ranks; ++r) {
        std::vector<GPairD> local;
        GPairD* dst = base;
        if (n_ranks > 1) {
          // every rank starts from the current (shared, already reduced) contents
          local.assign(base, base + span);
          dst = local.data();
        }
        for (auto [p, il] : sorted[r]) {
          if (!single && (p < nb || p >= ne)) continue;
          const bool compute = ComputeHistogramBin(p, node_sums, K, hist.ContainsNode(Parent(p)));
          if (p < 0 || !compute) continue;
          const int64_t ig = il + rank_off[r];
          for (int k = 0; k < K; ++k) {
            const GPairD gp{a.g[ig * K + k], a.h[ig * K + k]};
            for (int f = 0; f < F; ++f) {
              GPairD& e = dst[(static_cast<size_t>(p - nb) * K + k) * B + bins[ig * F + f]];
              e.grad += gp.grad;
              e.hess += gp.hess;
            }
          }
        }
        if (n_ranks > 1) parts.push_back(std::move(local));
      }
      if (n_ranks > 1) RankSum(parts, base, span);
      // Scan, build_tree.cc:291-341
      auto scan_node = [&](int node) {
        for (int f = 0; f < F; ++f)
          for (int k = 0; k < K; ++k) {
            GPairD sum{0.0, 0.0};
            for (int b = prop.row_ptr[f]; b < prop.row_ptr[f + 1]; ++b) {
              GPairD& e = hist.at(node, k, b);
              sum.grad += e.grad;
              sum.hess += e.hess;
              e = sum;
            }
          }
      };
      if (nb == 0 && ne == 1) {
        scan_node(0);
      } else {
        for (int node = nb; node < ne; ++node) {
          const int parent = Parent(node);
          if (!ComputeHistogramBin(node, node_sums, K, hist.ContainsNode(parent))) continue;
          scan_node(node);
          if (node == 0) continue;
          const int sib = Sibling(node);
          if (!ComputeHistogramBin(sib, node_sums, K, hist.ContainsNode(parent))) {
            for (int k = 0; k < K; ++k)
              for (int b = 0; b < B; ++b) {
                GPairD s = hist.at(node, k, b), p = hist.at(parent, k, b);
                hist.at(sib, k, b) = GPairD{p.grad - s.grad, p.hess - s.hess};
              }
          }
        }
      }
      if (trace) {
        for (int node = nb; node < ne && node < a.trace_nodes; ++node)
          std::memcpy(trace + static_cast<size_t>(node) * K * B, &hist.at(node, 0, 0), sizeof(GPairD) * K * B);
      }
      // PerformBestSplit, build_tree.cc:342-401
      for (int node = nb; node < ne; ++node) {
        double best_gain = 0;
        int best_feature = -1, best_bin = -1;
        for (int f = 0; f < F; ++f) {
          if (a.feature_set && !a.feature_set[f]) continue;
          for (int b = prop.row_ptr[f]; b < prop.row_ptr[f + 1]; ++b) {
            double gsum = 0;
            for (int k = 0; k < K; ++k) {
              GPairD left   = hist.at(node, k, b);
              GPairD parent = node_sums[static_cast<size_t>(node) * K + k];
              GPairD right{parent.grad - left.grad, parent.hess - left.hess};
              gsum += CalculateGain(left, right, parent, a.l1, a.l2, a.min_split_gain);
            }
            if (gsum > best_gain) {
              best_gain    = gsum;
              best_feature = f;
              best_bin     = b;
            }
          }
        }
        if (best_gain > kEps) {
          std::vector<double> ll(K), rl(K);
          std::vector<GPairD> ls(K), rs(K);
          for (int k = 0; k < K; ++k) {
            GPairD l = hist.at(node, k, best_bin);
            GPairD p = node_sums[static_cast<size_t>(node) * K + k];
            double GR = p.grad - l.grad, HR = p.hess - l.hess;
            ll[k] = CalculateLeafValue(l.grad, l.hess, a.l1, a.l2);
            rl[k] = CalculateLeafValue(GR, HR, a.l1, a.l2);
            ls[k] = l;
            rs[k] = GPairD{GR, HR};
          }
          if (ls[0].hess <= 0.0 || rs[0].hess <= 0.0) continue;
          feature[node]     = best_feature;
          split_value[node] = static_cast<double>(prop.values[best_bin]);
          gain[node]        = best_gain;
          for (int k = 0; k < K; ++k) {
            node_sums[static_cast<size_t>(LeftChild(node)) * K + k]   = ls[k];
            node_sums[static_cast<size_t>(RightChild(node)) * K + k]  = rs[k];
            leaf_value[static_cast<size_t>(LeftChild(node)) * K + k]  = ll[k];
            leaf_value[static_cast<size_t>(RightChild(node)) * K + k] = rl[k];
          }
        }
      }
    }
    // UpdatePositions, build_tree.cc:402-417 (compares in T, split_value is double)
    if (depth < a.max_depth - 1) {
      for (int r = 0; r < n_ranks; ++r)
        for (auto& pr : sorted[r]) {
          int p = pr.first;
          if (p < 0 || p >= max_nodes || feature[p] == -1) {
            pr.first = -1;
            continue;
          }
          const T xv = X[(pr.second + rank_off[r]) * F + feature[p]];
          pr.first   = xv <= split_value[p] ? LeftChild(p) : RightChild(p);
        }
    }
  }
  std::copy(leaf_value.begin(), leaf_value.end(), a.leaf_value);
  std::copy(feature.begin(), feature.end(), a.feature);
  std::copy(split_value.begin(), split_value.end(), a.split_value);
  std::copy(gain.begin(), gain.end(), a.gain);
  for (size_t i = 0; i < node_sums.size(); ++i) a.hessian[i] = node_sums[i].hess;
  if (a.out_node_sums) std::memcpy(a.out_node_sums, node_sums.data(), sizeof(GPairD) * node_sums.size());
  if (a.out_positions)
    for (int r = 0; r < n_ranks; ++r)
      for (auto& pr : sorted[r]) a.out_positions[pr.second + rank_off[r]] = pr.first;
  return 0;
}

template <typename T>
void Predict(const T* X,
             int64_t n_rows,
             int F,
             int K,
             int n_trees,
             const double* const* leaf,
             const int32_t* const* feat,
             const double* const* split,
             double* pred)
{  // predict.cc:23-67
  for (int64_t i = 0; i < n_rows * K; ++i) pred[i] = 0.0;
  for (int t = 0; t < n_trees; ++t) {
    for (int64_t i = 0; i < n_rows; ++i) {
      int64_t pos = 0;
      for (int depth = 0; depth < 100; ++depth) {
        if (feat[t][pos] == -1) break;
        const double xv = static_cast<double>(X[i * F + feat[t][pos]]);
        pos             = xv <= split[t][pos] ? pos * 2 + 1 : pos * 2 + 2;
      }
      for (int k = 0; k < K; ++k) pred[i * K + k] += leaf[t][pos * K + k];
    }
  }
}

}  // namespace

// UPDATE_TREE (reference: update_tree_fn, src/models/tree/update_tree.cc:36-134): the structure of
// a tree stays, its statistics are recomputed from new gradients.  Every row walks from the root
// (at most 100 levels) and adds its (g, h) to every node it visits, the leaf included; per rank the
// rows are taken in order and the sums are float64; the ranks' sums are added in rank order (the
// reference's two all-reduces); then leaf = H > 0 ? CalculateLeafValue(G, H) : 0, hessian = H.
template <typename T>
void UpdateTree(const T* X, int64_t n_rows, int F, int K, const double* g, const double* h, int max_nodes,
                const int32_t* feature, const double* split_value, double l1, double l2, int n_ranks,
                const int64_t* rank_off, double* leaf_value, double* hessian)
{
  const size_t MK = static_cast<size_t>(max_nodes) * K;
  std::vector<double> G(MK, 0.0), H(MK, 0.0);
  for (int r = 0; r < n_ranks; ++r) {
    std::vector<double> lg(MK, 0.0), lh(MK, 0.0);
    for (int64_t i = rank_off[r]; i < rank_off[r + 1]; ++i) {
      int pos = 0;
      for (int depth = 0; depth < 100; ++depth) {
        for (int k = 0; k < K; ++k) {
          lg[static_cast<size_t>(pos) * K + k] += g[i * K + k];
          lh[static_cast<size_t>(pos) * K + k] += h[i * K + k];
        }
        if (feature[pos] == -1) break;
        const T x = X[i * F + feature[pos]];
        pos       = x <= split_value[pos] ? pos * 2 + 1 : pos * 2 + 2;
      }
    }
    for (size_t e = 0; e < MK; ++e) {
      G[e] += lg[e];
      H[e] += lh[e];
    }
  }
  for (size_t e = 0; e < MK; ++e) {
    leaf_value[e] = H[e] > 0.0 ? CalculateLeafValue(G[e], H[e], l1, l2) : 0.0;
    hessian[e]    = H[e];
  }
}

extern "C" {

int lbo_build_tree(const lbo_tree_args* a)
{
  if (a->mode == 0) return a->x_is_f64 ? BuildTreeQ<double>(*a) : BuildTreeQ<float>(*a);
  return a->x_is_f64 ? BuildTreeD<double>(*a) : BuildTreeD<float>(*a);
}

void lbo_predict(const void* X,
                 int x_is_f64,
                 int64_t n_rows,
                 int F,
                 int K,
                 int n_trees,
                 const double* const* leaf,
                 const int32_t* const* feat,
                 const double* const* split,
                 double* pred)
{
  if (x_is_f64)
    Predict(static_cast<const double*>(X), n_rows, F, K, n_trees, leaf, feat, split, pred);
  else
    Predict(static_cast<const float*>(X), n_rows, F, K, n_trees, leaf, feat, split, pred);
}

void lbo_update_tree(const void* X, int x_is_f64, int64_t n_rows, int F, int K, const double* g, const double* h,
                     int max_nodes, const int32_t* feature, const double* split_value, double l1, double l2,
                     int n_ranks, const int64_t* rank_off, double* leaf_value, double* hessian)
{
  std::vector<int64_t> one = {0, n_rows};
  if (n_ranks <= 0) {
    n_ranks  = 1;
    rank_off = one.data();
  }
  if (x_is_f64)
    UpdateTree(static_cast<const double*>(X), n_rows, F, K, g, h, max_nodes, feature, split_value, l1, l2, n_ranks,
               rank_off, leaf_value, hessian);
  else
    UpdateTree(static_cast<const float*>(X), n_rows, F, K, g, h, max_nodes, feature, split_value, l1, l2, n_ranks,
               rank_off, leaf_value, hessian);
}

// Stage-level entry points ----------------------------------------------------------------

// Returns B; proposals (T[F*S], first B valid) and row_ptr[F+1] are written.
int lbo_split_proposals(int mode,
                        const void* X,
                        int x_is_f64,
                        int64_t n_rows,
                        int F,
                        int S,
                        int seed,
                        int n_ranks,
                        const int64_t* rank_off,
                        void* out_proposals,
                        int32_t* out_row_ptr)
{
  std::vector<int64_t> one = {0, n_rows};
  if (n_ranks <= 0) {
    n_ranks  = 1;
    rank_off = one.data();
  }
  if (x_is_f64) {
    auto p = SelectSplitSamples<double>(mode, static_cast<const double*>(X), n_rows, F, S, seed, n_ranks, rank_off);
    std::memcpy(out_proposals, p.values.data(), sizeof(double) * p.values.size());
    std::copy(p.row_ptr.begin(), p.row_ptr.end(), out_row_ptr);
    return static_cast<int>(p.values.size());
  }
  auto p = SelectSplitSamples<float>(mode, static_cast<const float*>(X), n_rows, F, S, seed, n_ranks, rank_off);
  std::memcpy(out_proposals, p.values.data(), sizeof(float) * p.values.size());
  std::copy(p.row_ptr.begin(), p.row_ptr.end(), out_row_ptr);
  return static_cast<int>(p.values.size());
}

// Sampled row ids of Mode Q (thrust engine, discard(i)) for i in [0,S)
void lbo_sample_rows(int seed, int S, int64_t n_rows, int64_t* out)
{
  for (int i = 0; i < S; ++i) {
    MinStd eng(static_cast<uint32_t>(seed));
    eng.discard(static_cast<uint64_t>(i));
    out[i] = eng.uniform_int(0, n_rows - 1);
  }
}

// Feature-relative bin of every element (index of the first proposal >= x inside its feature)
void lbo_bin_x(const void* X,
               int x_is_f64,
               int64_t n_rows,
               int F,
               const void* proposals,
               const int32_t* row_ptr,
               int16_t* out_bins)
{
  for (int64_t i = 0; i < n_rows; ++i)
    for (int f = 0; f < F; ++f) {
      int rel;
      if (x_is_f64) {
        const double* p = static_cast<const double*>(proposals);
        rel = static_cast<int>(std::lower_bound(p + row_ptr[f], p + row_ptr[f + 1],
                                                static_cast<const double*>(X)[i * F + f]) - (p + row_ptr[f]));
      } else {
        const float* p = static_cast<const float*>(proposals);
        rel = static_cast<int>(std::lower_bound(p + row_ptr[f], p + row_ptr[f + 1],
                                                static_cast<const float*>(X)[i * F + f]) - (p + row_ptr[f]));
      }
      out_bins[i * F + f] = static_cast<int16_t>(rel);
    }
}

double lbo_abs_sum(const double* v, int64_t n)
{
  std::vector<double> a(n);
  for (int64_t i = 0; i < n; ++i) a[i] = std::fabs(v[i]);
  return canonical_sum(std::move(a));
}

// Quantised pairs [n_rows,K,2] and the four scale values
void lbo_quantise(const double* g,
                  const double* h,
                  int64_t n_rows,
                  int K,
                  int seed,
                  int n_ranks,
                  const int64_t* rank_off,
                  int64_t* out_q,
                  double* out_scale)
{
  std::vector<int64_t> one = {0, n_rows};
  if (n_ranks <= 0) {
    n_ranks  = 1;
    rank_off = one.data();
  }
  Quantiser quant;
  quant.Init(g, h, K, n_ranks, rank_off);
  out_scale[0] = quant.scale.grad;
  out_scale[1] = quant.scale.hess;
  out_scale[2] = quant.inv.grad;
  out_scale[3] = quant.inv.hess;
  for (int64_t i = 0; i < n_rows; ++i)
    for (int k = 0; k < K; ++k) {
      GPairI q = quant.Quantise(g[i * K + k], h[i * K + k], hash_combine(static_cast<int64_t>(seed), i, k));
      out_q[(i * K + k) * 2]     = q.grad;
      out_q[(i * K + k) * 2 + 1] = q.hess;
    }
}

// Plain histogram accumulation over rows whose node lies in [node_begin,node_end):
// out[node-node_begin][k][row_ptr[f]+bins[row,f]] += value(row,k).  Integer version takes
// int32 pairs [n_rows,K,2]; double version takes g,h float64 [n_rows,K].
void lbo_histogram_q(const uint8_t* bins_u8,
                     const int16_t* bins_i16,
                     int64_t n_rows,
                     int F,
                     const int32_t* row_ptr,
                     const int32_t* q,
                     int K,
                     const int32_t* node_of_row,
                     int node_begin,
                     int node_end,
                     int64_t* out)
{
  const int B = row_ptr[F];
  for (int64_t i = 0; i < n_rows; ++i) {
    const int p = node_of_row[i];
    if (p < node_begin || p >= node_end) continue;
    for (int k = 0; k < K; ++k) {
      const int64_t gq = q[(i * K + k) * 2], hq = q[(i * K + k) * 2 + 1];
      int64_t* base = out + (static_cast<size_t>(p - node_begin) * K + k) * B * 2;
      for (int f = 0; f < F; ++f) {
        const int b = row_ptr[f] + (bins_u8 ? static_cast<int>(bins_u8[i * F + f]) : static_cast<int>(bins_i16[i * F + f]));
        base[2 * b] += gq;
        base[2 * b + 1] += hq;
      }
    }
  }
}

void lbo_histogram_d(const uint8_t* bins_u8,
                     const int16_t* bins_i16,
                     int64_t n_rows,
                     int F,
                     const int32_t* row_ptr,
                     const float* g32,
                     const float* h32,
                     const double* g64,
                     const double* h64,
                     int K,
                     const int32_t* node_of_row,
                     int node_begin,
                     int node_end,
                     double* out)
{
  const int B = row_ptr[F];
  for (int64_t i = 0; i < n_rows; ++i) {
    const int p = node_of_row[i];
    if (p < node_begin || p >= node_end) continue;
    for (int k = 0; k < K; ++k) {
      const double gv = g64 ? g64[i * K + k] : static_cast<double>(g32[i * K + k]);
      const double hv = h64 ? h64[i * K + k] : static_cast<double>(h32[i * K + k]);
      double* base = out + (static_cast<size_t>(p - node_begin) * K + k) * B * 2;
      for (int f = 0; f < F; ++f) {
        const int b = row_ptr[f] + (bins_u8 ? static_cast<int>(bins_u8[i * F + f]) : static_cast<int>(bins_i16[i * F + f]));
        base[2 * b] += gv;
        base[2 * b + 1] += hv;
      }
    }
  }
}

// RNG pieces exposed for cross-checks against the toolkit's thrust headers
int64_t lbo_hash_combine(int64_t seed, int64_t a, int64_t b) { return hash_combine(seed, a, b); }
void lbo_uniform_pair(int64_t seed, double* out2)
{
  MinStd eng(static_cast<uint32_t>(static_cast<uint64_t>(seed)));
  out2[0] = eng.uniform_real(0, 1);
  out2[1] = eng.uniform_real(0, 1);
}

int lbo_version() { return 1; }

}  // extern "C"
