// Internal declarations shared by the translation units of liblbk.so.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "lbk.h"

namespace lbk {

struct Error : public std::runtime_error {
  int code;
  Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

#define LBK_CUDA(call)                                                                        \
  do {                                                                                        \
    cudaError_t e_ = (call);                                                                  \
    if (e_ != cudaSuccess) {                                                                  \
      throw ::lbk::Error(LBK_ERR_CUDA, std::string(__FILE__) + ":" + std::to_string(__LINE__) + \
                                         ": " #call ": " + cudaGetErrorString(e_));           \
    }                                                                                         \
  } while (0)

#define LBK_EXPECT(cond, msg)                                                                 \
  do {                                                                                        \
    if (!(cond)) {                                                                            \
      throw ::lbk::Error(LBK_ERR_ARGUMENT, std::string(__FILE__) + ":" + std::to_string(__LINE__) + \
                                             ": " + (msg));                                   \
    }                                                                                         \
  } while (0)

#define LBK_LAUNCH_CHECK() LBK_CUDA(cudaGetLastError())

// 16-byte (grad, hess) pairs
struct GPairI64 {
  long long grad, hess;
};
struct GPairF64 {
  double grad, hess;
};

// Quantiser parameters, device resident (reference: GradientQuantiser, build_tree.cu:51-104)
struct QuantParams {
  double scale_g, scale_h, inv_g, inv_h;
};

inline int LevelBegin(int level) { return (1 << level) - 1; }
inline int LevelEnd(int level) { return (1 << (level + 1)) - 1; }

constexpr int kGroup = 32;  // features per feature group (one lane per feature)

}  // namespace lbk

namespace lbk {
struct PeerExchange;
}

// The context is an opaque C struct for callers.
struct lbk_context {
  int device        = 0;
  int sm_count      = 0;
  int max_smem_optin = 0;
  cudaMemPool_t pool = nullptr;
  // the caller's allocator for scratch (both set or both null)
  lbk_alloc_fn alloc_cb     = nullptr;
  lbk_release_fn release_cb = nullptr;
  void* alloc_user          = nullptr;
  std::string err;
  // device status word: 0 = ok, otherwise a kernel wrote a fault code
  int* d_status = nullptr;
  // communicator
  int rank = 0, n_ranks = 1;
  void* nccl_comm     = nullptr;
  bool owns_nccl      = false;
  lbk_allreduce_fn cb = nullptr;
  void* cb_user       = nullptr;
  // buffers that the other ranks' GPUs can read (see exchange.cu); made on first use
  lbk::PeerExchange* xchg = nullptr;
  // optional timing of the histogram kernel alone (events on the caller's stream)
  bool profile            = false;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events;  // one pair per timed launch since the last total
  size_t prof_used        = 0;
};

namespace lbk {

// Stream-ordered scratch allocation from the context's pool (replaces legate::create_buffer).
class Scratch {
 public:
  Scratch(lbk_context* ctx, cudaStream_t stream) : ctx_(ctx), stream_(stream) {}
  ~Scratch();
  Scratch(const Scratch&)            = delete;
  Scratch& operator=(const Scratch&) = delete;
  void* alloc_bytes(size_t bytes);
  template <typename T>
  T* alloc(size_t n)
  {
    return static_cast<T*>(alloc_bytes(sizeof(T) * (n > 0 ? n : 1)));
  }
  void free_one(void* p);

 private:
  lbk_context* ctx_;
  cudaStream_t stream_;
  std::vector<void*> ptrs_;
};

// In-place all-reduce over the context's communicator; no-op for a single rank.
void AllReduce(lbk_context* ctx, void* buf, size_t count, lbk_dtype dtype, lbk_redop op, cudaStream_t stream);
// Every rank contributes `bytes` bytes at `send` and receives all contributions, in rank order, at
// `recv` (device pointers; NCCL communicators only: returns false where the communicator is a
// callback or missing).
bool AllGatherBytes(lbk_context* ctx, const void* send, void* recv, size_t bytes, cudaStream_t stream);

// ---- peer exchange (exchange.cu) ------------------------------------------------------------
// Two buffers per rank that every other rank's GPU can read directly over NVLink (CUDA IPC between
// processes, plain peer access inside one process), used to sum the histograms of a level: every
// rank builds into its own buffer, a barrier, then rank r reads the bins of the features it owns
// from all ranks and adds them up (a reduce-scatter made of peer loads).  The two buffers
// alternate so that one barrier per level is enough.
//
// Collective: every rank calls with the same `bytes`.  Returns false (on every rank alike) where the
// peers cannot be mapped or the communicator is not NCCL; callers then fall back to AllReduce.
bool EnsureExchange(lbk_context* ctx, size_t bytes, cudaStream_t stream);
void DestroyExchange(lbk_context* ctx);
// The buffer the next build goes into (alternates on every call), its first `bytes` bytes zeroed.
void* NextExchangeBuffer(lbk_context* ctx, size_t bytes, cudaStream_t stream);
// Features [OwnedBegin(r), OwnedBegin(r + 1)) belong to rank r.
__host__ __device__ inline int OwnedBegin(int rank, int n_ranks, int F) { return static_cast<int>(static_cast<long long>(rank) * F / n_ranks); }
// After every rank has built [n_seg][B] pairs into `buf` (the buffer NextExchangeBuffer returned):
// dst[seg][b] = sum over ranks of their buf[seg][b] for the bins b of this rank's features; dst may
// be `buf` itself (in place).  Includes the barrier.
void ExchangeReduceOwned(lbk_context* ctx, void* buf, void* dst, int n_seg, int B, int F, const int32_t* row_ptr,
                         bool float_mode, cudaStream_t stream);
// The push form.  NextPushBuffers: the device array of every rank's receive buffer for the next
// build (alternating, all zero when handed out).  ExchangeReducePushed, after every rank has built
// with them: a barrier, then dst[seg][b] = sum over source ranks of this rank's receive slots, for the
// bins b of its features (dst is local memory, [n_seg][B] pairs); the slots are zeroed as they are
// read, so the buffer is clean when its turn comes again.
void* const* NextPushBuffers(lbk_context* ctx, cudaStream_t stream);
void ExchangeReducePushed(lbk_context* ctx, void* dst, int n_seg, int push_len, int B, int F, const int32_t* row_ptr,
                          bool float_mode, cudaStream_t stream);
// After ExchangeReduceOwned in place on every rank: dst[seg][b] = the owner's sum, for all bins.
// Includes a barrier.
void ExchangeGatherAll(lbk_context* ctx, void* buf, void* dst, int n_seg, int B, int F, const int32_t* row_ptr,
                       cudaStream_t stream);
// The event pair that brackets the next timed histogram launch (profile mode): the first that is
// free, made on demand; when kMaxProfiledLaunches are in use the last one is used again.
std::pair<cudaEvent_t, cudaEvent_t> NextProfileEvents(lbk_context* ctx);
// Reads the device status word (synchronises the stream) and throws LBK_ERR_DEVICE if set.
void CheckDeviceStatus(lbk_context* ctx, cudaStream_t stream);

// Runs f, turning exceptions into a status code and an error text (the ABI boundary).
int Guard(lbk_context* ctx, const std::function<void()>& f);

// ---- stage launchers (defined in the .cu files named in the comments) ------------------------
// proposals.cu
struct ProposalInfo {
  int total_bins;            // B
  int max_bins_per_feature;  // largest feature
};
template <typename T>
ProposalInfo SplitProposals(lbk_context* ctx, Scratch& s, const T* X, int64_t ldx, int64_t row_offset,
                            int64_t n_local, int F, int S, int seed, int64_t dataset_rows, T* proposals,
                            int32_t* row_ptr, cudaStream_t stream);  // synchronises the stream
template <typename T>
// bins_t (optional): feature-major copy, bins_t[f * pitch_t + row], pitch_t a multiple of 32 >= n_rows
void BinMatrix(const T* X, int64_t ldx, int64_t n_rows, int F, const T* proposals, const int32_t* row_ptr,
               void* bins, void* bins_t, int64_t pitch_t, int bin_bytes, int max_bins_per_feature,
               cudaStream_t stream);
// quantise.cu
void Quantise(lbk_context* ctx, Scratch& s, const double* g, const double* h, int64_t ldg, int64_t row_offset,
              int64_t n_local, int K, int seed, int2* gpair, GPairI64* root_sums, QuantParams* params,
              int* max_abs /* device [2] */, cudaStream_t stream);
// histogram.cu
struct HistLevel {
  const void* bins;
  int bin_bytes;
  int64_t n_rows;      // rows of the bin matrix (local rows)
  int F, K, B;
  int max_bins_per_feature;
  const int32_t* row_ptr;
  const int2* gpair;       // int path
  const float2* gpair_f;   // float path
  bool pairs_by_position = false;  // gpair / gpair_f are stored in row_index order: entry i belongs to row_index[i]
  const int* max_abs;      // device [2]: largest |grad|, |hess| of gpair (null: computed by the call)
  const int32_t* row_index;
  const int32_t* seg;      // [n_level_nodes+1] offsets for nodes node_begin.. of the level range
  int n_nodes;             // nodes in this batch
  int seg_node_offset;     // index into seg of the batch's first node
  // built-node selection: slot_of_node[j] = slot in `out` for node j of the batch, or -1
  const int32_t* slot_of_node;
  void* out;               // [n_slots, K, B] pairs (int64 or double), already zeroed
  bool float_mode;
  // set by BuildHistogramSummed only: the histograms go into the owners' receive buffers (see
  // HistParams in histogram.cu)
  void* const* push_recv     = nullptr;
  long long push_slot_pairs = 0;
  int push_len              = 0;
};
void BuildHistogram(lbk_context* ctx, Scratch& s, const HistLevel& lv, cudaStream_t stream);
// BuildHistogram followed by the sum over ranks of the n_slots histograms.
//   kSumEverywhere: lv.out holds the sums of all bins on every rank when the call returns.
//   kSumOwned:      only the bins of the features this rank owns are summed (OwnedBegin); the
//                   result is where the returned pointer says: lv.out, or the exchange buffer the
//                   level was built in (which stays valid until the build after the next).
// Through the peer exchange where it is available, else one all-reduce of the whole buffer (then
// every bin is summed on every rank, whatever the mode).  The sequence of collectives depends only
// on values that are equal on every rank; a rank without rows skips the kernel, nothing else.
// zero_out: lv.out has not been zeroed; the call zeroes it where the build goes into it (through the
// exchange it does not: what is not written there stays as it was).
enum class HistSum { kSumEverywhere, kSumOwned };
void* BuildHistogramSummed(lbk_context* ctx, Scratch& s, const HistLevel& lv, int n_slots, HistSum mode,
                           bool result_in_out, bool zero_out, cudaStream_t stream);
void GroupRows(lbk_context* ctx, Scratch& s, const int32_t* node_of_row, int64_t n_rows, int node_begin,
               int n_nodes, int32_t* row_index, int32_t* seg, cudaStream_t stream);
// split.cu
struct TreeArrays {
  double* leaf_value;
  int32_t* feature;
  double* split_value;
  double* gain;
  GPairI64* node_sums;
  int32_t* split_bin;  // feature-relative bin of the chosen split, per node
  int max_nodes;
};
struct SplitParams {
  double l1, l2, min_split_gain;
  const uint8_t* feature_set;
};
// Decide which nodes of the batch are built: slot_of_node[j] (>=0 built, -1 derived/none).
void PlanBuilt(const GPairI64* node_sums, int K, int node_begin, int n_nodes, bool parent_available,
               int32_t* slot_of_node, cudaStream_t stream);
// Scan built histograms into the level histogram, derive siblings from the parent.
// Only the features [f_begin, f_end) are scanned / derived (all of them on one rank; the owned ones
// when the features are divided among the ranks).
void ScanLevel(const GPairI64* built, const int32_t* slot_of_node, GPairI64* level_hist /* node_begin based */,
               const GPairI64* parent_hist /* level above, may be null */, int parent_begin,
               const GPairI64* node_sums, int node_begin, int n_nodes, int K, int f_begin, int f_end, int B,
               const int32_t* row_ptr, bool parent_available, cudaStream_t stream);
// arrived: one counter per tree node, zero before the first call of a tree.  The bins of the features
// [f_begin, f_end) are evaluated; with exchange_records every rank's best candidate of every node
// (and the sums left of it) is gathered on all ranks and the best of them becomes the tree - the same
// total order as within a rank, so the tree is the one a single rank would grow.
template <typename T>
void BestSplit(lbk_context* ctx, Scratch& s, const GPairI64* level_hist, int node_begin, int n_nodes, int K, int F, int B,
               const int32_t* row_ptr, const T* proposals, const QuantParams* qp, const SplitParams& sp,
               TreeArrays tree, unsigned int* arrived, int f_begin, int f_end, bool exchange_records,
               cudaStream_t stream);
void RootLeaf(TreeArrays tree, int K, const QuantParams* qp, double l1, double l2, cudaStream_t stream);
void WriteHessian(const GPairI64* node_sums, const QuantParams* qp, double* hessian, int64_t n, cudaStream_t stream);
// partition.cu
struct PartitionLevel {
  const void* bins;   // feature-major copy of the bin ids: bins[f * bin_pitch + row]
  int bin_bytes;
  int64_t bin_pitch;  // elements per feature
  int64_t n_rows;
  const int32_t* row_index_in;
  const int32_t* seg_in;  // [n_nodes+1] for the level
  int32_t* row_index_out;
  int32_t* seg_out;       // [2*n_nodes+1] for the next level
  int node_begin, n_nodes;
  const int32_t* feature;
  const int32_t* split_bin;
  // optional: the quantised pairs in row_index order, moved together with the row ids
  const int2* pairs_in = nullptr;  // [rows of the level][K]
  int2* pairs_out      = nullptr;
  int K                = 0;
};
void PartitionRows(lbk_context* ctx, Scratch& s, const PartitionLevel& pl, cudaStream_t stream);
void InitRows(int32_t* row_index, int32_t* seg, int64_t n_rows, cudaStream_t stream);
// predict.cu
template <typename T>
void PredictLaunch(lbk_context* ctx, Scratch& s, const T* X, int64_t ldx, int64_t n_rows, int F, int K, int n_trees,
                   const double* const* leaf, const int32_t* const* feat, const double* const* split,
                   const int32_t* max_nodes, double* pred, int64_t ldp, cudaStream_t stream);

}  // namespace lbk
