/* lbk.h - C ABI of the B200 tree-building kernels ("lbk").
 *
 * This is the drop-in boundary for the two tasks of legate-boost's tree model:
 *   BUILD_TREE  (reference: src/models/tree/build_tree.cu:1274-1365, opcode 1 in src/legateboost.h:22)
 *   PREDICT     (reference: src/models/tree/predict.cu:26-91,        opcode 2 in src/legateboost.h:23)
 * A task body that receives a legate::TaskContext unpacks its stores into the argument
 * structs below and calls lbk_build_tree / lbk_predict; nothing else of the reference changes.
 *
 * Conventions
 *   - plain C, no C++/torch types; every pointer is a raw address and every size is explicit;
 *   - data pointers are DEVICE pointers unless the struct's `host_buffers` field is non-zero,
 *     in which case they are host pointers and the library stages the copies itself on `stream`;
 *   - every call returns 0 on success or a negative lbk_status; lbk_last_error() gives the text;
 *   - a context belongs to one device and one host thread at a time; different contexts may be
 *     used concurrently from different threads (one per GPU, as the runtime calls task variants);
 *   - there is no CPU fallback: every entry point fails with LBK_ERR_CUDA when no device is
 *     usable.
 */
#ifndef LBK_H_
#define LBK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum lbk_status {
  LBK_OK            = 0,
  LBK_ERR_ARGUMENT  = -1, /* bad shape / null pointer / unsupported value (reference: EXPECT, cpp_utils.h:85-96) */
  LBK_ERR_CUDA      = -2, /* a CUDA runtime call failed (reference: CHECK_CUDA, cpp_utils.cuh:45-58) */
  LBK_ERR_COMM      = -3, /* a collective failed (reference: CHECK_NCCL, cpp_utils.cuh:35-43) */
  LBK_ERR_DEVICE    = -4, /* a kernel reported a fault through its status word (replaces EXPECT_DEVICE's trap) */
  LBK_ERR_ALLOC     = -5  /* scratch allocation failed */
} lbk_status;

typedef enum lbk_dtype { LBK_F32 = 0, LBK_F64 = 1, LBK_I32 = 2, LBK_I64 = 3 } lbk_dtype;
typedef enum lbk_redop { LBK_SUM = 0, LBK_MAX = 1 } lbk_redop;

typedef struct lbk_context lbk_context;

/* Version of this ABI (major*1000 + minor). */
int lbk_version(void);

/* Context: owns the scratch memory pool, the status word and (optionally) a communicator for
 * one device.  Replaces the per-task state the reference gets from the runtime
 * (legate::create_buffer scratch, context.get_task_stream(), context.communicator(0)). */
int lbk_context_create(int device, lbk_context** out);
void lbk_context_destroy(lbk_context* ctx);
/* Text of the last error on this context (or of the last context-less call on this thread). */
const char* lbk_last_error(const lbk_context* ctx);
/* Release cached scratch memory back to the driver. */
int lbk_context_trim(lbk_context* ctx);

/* Scratch from the caller's allocator instead of the context's own pool (reference: every scratch
 * buffer of the task bodies is a legate::create_buffer, e.g. build_tree.cu:785-809, which is why the
 * variants are registered with_has_allocations(true), build_tree.h:308-317): a runtime that has
 * reserved the GPU's memory wants the binned matrix, the quantised pairs and the row lists of a tree
 * (13 GB at 100M x 64) inside that reservation.
 *   alloc(user, bytes, stream) returns device memory (256-byte aligned) that work queued on `stream`
 *     after the call may use, or NULL (the library then fails with LBK_ERR_ALLOC);
 *   release(user, ptr, stream) is called once per allocation after the library has queued its last
 *     use of it on `stream`: the memory may be handed out again for work that is ordered after what
 *     `stream` holds at that moment (what cudaFreeAsync, torch's caching allocator and a buffer that
 *     lives until the end of the task all provide).
 * Both are called on the thread that calls into the library.  NULL for both restores the pool.  The
 * buffers that other ranks' GPUs map (multi-rank calls, see lbk_histogram_args.all_reduce) are not
 * scratch of one call and stay with the library. */
typedef void* (*lbk_alloc_fn)(void* user, size_t bytes, void* stream);
typedef void (*lbk_release_fn)(void* user, void* ptr, void* stream);
int lbk_context_set_allocator(lbk_context* ctx, lbk_alloc_fn alloc, lbk_release_fn release, void* user);
/* Bytes the context's own pool holds at the moment (reserved from the driver, in use or cached). */
int lbk_context_pool_bytes(lbk_context* ctx, size_t* reserved);

/* Communicator (reference: the ncclComm_t* the runtime hands to the task, cpp_utils.cuh:100-134).
 * Either create one from an id that rank 0 made and every rank received out of band ... */
#define LBK_UNIQUE_ID_BYTES 128
int lbk_comm_unique_id(void* id_out /* LBK_UNIQUE_ID_BYTES */);
int lbk_comm_init(lbk_context* ctx, const void* id, int rank, int n_ranks);
/* ... or attach an existing ncclComm_t (what a legate adapter passes; not destroyed by lbk) ... */
int lbk_comm_attach_nccl(lbk_context* ctx, void* nccl_comm, int rank, int n_ranks);
/* ... or supply the all-reduce as a callback (in place on a device buffer, ordered on `stream`). */
typedef int (*lbk_allreduce_fn)(void* user, void* buf, size_t count, int dtype /* lbk_dtype */,
                                int op /* lbk_redop */, void* stream);
int lbk_comm_set_callback(lbk_context* ctx, lbk_allreduce_fn fn, void* user, int rank, int n_ranks);
int lbk_comm_size(const lbk_context* ctx);
/* The features rank `rank` of `n_ranks` owns when the features are divided among the ranks for the
 * sum of a level's histograms and the split search: [*begin, *end).  Contiguous, in rank order, every
 * feature exactly once; a pure function of its arguments (no device needed).  The reference has no
 * counterpart: all of its ranks reduce and search everything (build_tree.cu:1107-1151). */
int lbk_owned_features(int rank, int n_ranks, int n_features, int* begin, int* end);
/* Failure detection check that needs no second GPU and faults nothing: runs the barrier kernel of the
 * peer exchange for an emulated world of two ranks on this context's device.  With peer_present != 0
 * the other rank's flag is preset and the call returns LBK_OK; with 0 nobody ever sets it, the
 * kernel's wait runs out after about a second, it reports through the context's status word and
 * returns, and the call returns LBK_ERR_DEVICE with the fault code in lbk_last_error.  The context
 * is usable afterwards.  No counterpart in the reference (NCCL's own timeouts play that role). */
int lbk_selftest_peer_barrier(lbk_context* ctx, int peer_present, void* stream);

/* Timing of the histogram kernel alone (no counterpart in the reference, which leaves profiling
 * to external tools): when enabled, every histogram launch is bracketed by CUDA events on the
 * caller's stream; lbk_profile_histogram_ms returns the duration of the most recent one. */
int lbk_profile_enable(lbk_context* ctx, int on);
int lbk_profile_histogram_ms(lbk_context* ctx, float* ms);
/* The sum over all histogram launches since the last call of this function (or since the timing was
 * enabled) and their number; starts a new sum.  Waits for the launches to finish. */
int lbk_profile_histogram_total(lbk_context* ctx, float* ms, int* launches);

/* ------------------------------------------------------------------------------------------
 * BUILD_TREE.  Field order follows the task's argument order (legateboost/models/tree.py:117-183,
 * build_tree.cu:1278-1307): inputs X, g, h, optional feature set; scalars max_depth, max_nodes,
 * split_samples, seed, dataset_rows, l1, l2, min_split_gain; outputs leaf_value, feature,
 * split_value, gain, hessian.  Rows [row_offset, row_offset+n_local_rows) of the global data set
 * live on this rank (the store's shape.lo[0] and extent).
 */
typedef struct lbk_build_tree_args {
  const void* X;      /* [n_local_rows, n_features], element stride 1, row stride ldx elements */
  int32_t x_dtype;    /* LBK_F32 or LBK_F64 */
  int64_t ldx;
  const double* g;    /* [n_local_rows, n_outputs], row stride ldg elements */
  const double* h;
  int64_t ldg;
  const uint8_t* feature_set; /* optional bool[n_features]; NULL = all features */
  int64_t row_offset;
  int64_t n_local_rows;
  int32_t n_features;
  int32_t n_outputs;
  /* scalars 0-7 */
  int32_t max_depth;
  int32_t max_nodes;     /* must equal 2^(max_depth+1)-1 */
  int32_t split_samples; /* <= 2048 */
  int32_t seed;
  int64_t dataset_rows;
  double l1_regularization;
  double l2_regularization;
  double min_split_gain;
  /* outputs 0-4, identical on every rank */
  double* leaf_value;  /* [max_nodes, n_outputs] */
  int32_t* feature;    /* [max_nodes], -1 = leaf */
  double* split_value; /* [max_nodes] */
  double* gain;        /* [max_nodes] */
  double* hessian;     /* [max_nodes, n_outputs] */
  void* stream;        /* cudaStream_t; the call returns after the stream has drained, as the
                          reference does (build_tree.cu:1356) */
  int32_t host_buffers;
  /* Optional device-side traces for tests (NULL to skip): */
  int64_t* trace_node_sums; /* [max_nodes, n_outputs, 2] quantised node sums */
  int64_t* trace_hist;      /* [trace_nodes, n_outputs, B, 2]: each node's histogram as it was when
                               its split was evaluated */
  int32_t trace_nodes;
  int32_t* out_total_bins;  /* host pointer: B */
  /* Optional (NULL to skip): the node in which each local row of X ends, int32 [n_local_rows],
   * device (host if host_buffers).  It is the node lbk_predict's walk of this tree reaches for the
   * row (read off the binned matrix while it still exists), so leaf_value[out_leaf[i]] is the
   * tree's prediction for training row i without a second pass over X.  No counterpart in the
   * reference, whose callers run PREDICT on the training matrix after every BUILD_TREE. */
  int32_t* out_leaf;
  /* Optional fixed sketch.  The reference draws new split proposals and bins X again for every tree,
   * because every tree has its own seed (models/tree.py:125, build_tree.cu:882-956); `sketch` is a
   * device buffer of lbk_sketch_bytes() bytes that keeps the proposals and the binned matrix of one
   * call for later ones.  LBK_SKETCH_OFF ignores it.  LBK_SKETCH_SAVE builds the tree as usual (the
   * same tree as OFF) and leaves its proposals and bins in the buffer.  LBK_SKETCH_REUSE takes them
   * from the buffer instead of sampling and binning X (X is not read and may be NULL): the tree then
   * differs from the reference's, since its proposals are those of the saving call's seed; `seed`
   * still drives the rounding of the gradients.  n_local_rows, n_features, split_samples and x_dtype
   * must be those of the saving call (checked), and X unchanged (the caller's promise). */
  void* sketch;
  int32_t sketch_mode;
} lbk_build_tree_args;

enum { LBK_SKETCH_OFF = 0, LBK_SKETCH_SAVE = 1, LBK_SKETCH_REUSE = 2 };

int lbk_build_tree(lbk_context* ctx, const lbk_build_tree_args* args);

/* Bytes of the sketch buffer for a matrix of this shape (0 for a bad shape). */
size_t lbk_sketch_bytes(int64_t n_local_rows, int n_features, int split_samples, int x_dtype);

/* out[i, :] = leaf_value[leaf[i], :] for the rows of lbk_build_tree_args.out_leaf: the tree's
 * predictions for its training rows (what the reference gets from a PREDICT task on the training
 * matrix, legateboost.py `train_pred += model.predict(X)`).  Device pointers; leaf_value
 * [max_nodes, n_outputs], leaf [n_rows], out [n_rows, n_outputs]; asynchronous on `stream`. */
int lbk_leaf_values(lbk_context* ctx, const double* leaf_value, const int32_t* leaf, int64_t n_rows,
                    int n_outputs, double* out, void* stream);

/* ------------------------------------------------------------------------------------------
 * PREDICT.  Inputs X then (leaf_value, feature, split_value) per tree, output pred
 * (legateboost/models/tree.py:252-277, predict.cu:26-84).  pred is overwritten (zero + sum of
 * leaves in tree order, float64); the caller adds the model's initial prediction.
 */
typedef struct lbk_predict_args {
  const void* X;
  int32_t x_dtype;
  int64_t ldx;
  int64_t n_rows;
  int32_t n_features;
  int32_t n_outputs;
  int32_t n_trees;
  const double* const* leaf_value;  /* host array of n_trees pointers, each [max_nodes[t], n_outputs] */
  const int32_t* const* feature;    /* each [max_nodes[t]] */
  const double* const* split_value; /* each [max_nodes[t]] */
  const int32_t* max_nodes;         /* host array [n_trees] */
  double* pred;                     /* [n_rows, n_outputs], row stride ldp elements */
  int64_t ldp;
  void* stream;
  int32_t host_buffers;
} lbk_predict_args;

int lbk_predict(lbk_context* ctx, const lbk_predict_args* args);

/* ------------------------------------------------------------------------------------------
 * Weighted gradients of a boosting round in one pass (reference: LBBase._get_weighted_gradient,
 * legateboost/legateboost.py:189-224, with unit sample weights and no subsampling, over
 * SquaredErrorObjective / LogLossObjective transform + gradient, legateboost/objectives.py:131-135,
 * 489-512): g = d loss / d raw prediction * learning_rate, h = max(second derivative, 1e-8).
 * raw_pred, g, h: float64 [n_rows, n_outputs]; y: float64 [n_rows, n_outputs] for squared error,
 * class index [n_rows] for log loss (0/1 when n_outputs == 1).  Device pointers, asynchronous on
 * `stream`.
 */
enum { LBK_SQUARED_ERROR = 0, LBK_LOG_LOSS = 1 };
int lbk_gradient(lbk_context* ctx, int objective, const double* raw_pred, const double* y, int64_t n_rows,
                 int n_outputs, double learning_rate, double* g, double* h, void* stream);

/* ------------------------------------------------------------------------------------------
 * UPDATE_TREE: a tree keeps its structure (feature, split_value) and gets new leaf values and
 * hessians from new gradients (reference: update_tree_fn, src/models/tree/update_tree.cc:36-134,
 * launched by Tree.update, legateboost/models/tree.py:197-240; the reference has a CPU variant
 * only).  Every row adds its (g, h) to every node on its path; the sums are added over the ranks of
 * the context's communicator; leaf = H > 0 ? -softthreshold(G, l1) / (H + l2) : 0, hessian = H.
 * Device pointers.  Float64 sums in another order than the reference's row loop: equal within
 * rounding, not bit for bit.
 */
typedef struct lbk_update_tree_args {
  const void* X;       /* [n_local_rows, n_features], row stride ldx elements */
  int32_t x_dtype;
  int64_t ldx;
  const double* g;     /* [n_local_rows, n_outputs], row stride ldg */
  const double* h;
  int64_t ldg;
  int64_t n_local_rows;
  int32_t n_features;
  int32_t n_outputs;
  int32_t max_nodes;
  const int32_t* feature;     /* [max_nodes], -1 = leaf */
  const double* split_value;  /* [max_nodes] */
  double l1_regularization;
  double l2_regularization;
  double* leaf_value;  /* out [max_nodes, n_outputs] */
  double* hessian;     /* out [max_nodes, n_outputs] */
  void* stream;        /* the call returns after the stream has drained */
} lbk_update_tree_args;

int lbk_update_tree(lbk_context* ctx, const lbk_update_tree_args* args);

/* ------------------------------------------------------------------------------------------
 * Stage-level entry points.  They expose the steps of BUILD_TREE separately so each can be
 * checked and timed on its own; lbk_build_tree runs the same kernels.
 */

/* Split proposals (reference: SelectSplitSamples, build_tree.cu:867-964).  Writes the CSR of
 * sorted unique sampled values per feature, last value of every feature = +inf.
 * proposals: [n_features*split_samples] of x_dtype (first B valid), row_ptr: [n_features+1].
 * total_bins is a host pointer. */
int lbk_split_proposals(lbk_context* ctx, const void* X, int x_dtype, int64_t ldx, int64_t row_offset,
                        int64_t n_local_rows, int n_features, int split_samples, int seed,
                        int64_t dataset_rows, void* proposals, int32_t* row_ptr, int32_t* total_bins,
                        void* stream);

/* Bin ids (reference: SparseSplitProposals::FindBin, build_tree.h:178-185, evaluated once per
 * tree instead of once per level).  bins layout: row-major, every row padded with zeros to a
 * whole number of 32-feature groups (pitch = 32 * ceil(n_features / 32) elements):
 *   bins[row*pitch + f] = index of the first proposal >= x inside feature f.
 * With one-byte bins the 32 ids of a (row, group) are one 32-byte sector and a row of up to 128
 * features is one 128-byte line.  bin_bytes = 1 (every feature has <= 256 proposals) or 2. */
int lbk_bin_matrix(lbk_context* ctx, const void* X, int x_dtype, int64_t ldx, int64_t n_rows,
                   int n_features, const void* proposals, const int32_t* row_ptr, void* bins,
                   int bin_bytes, void* stream);
/* Size in bytes of the bins buffer for the layout above. */
size_t lbk_bin_matrix_bytes(int64_t n_rows, int n_features, int bin_bytes);

/* Quantised gradient pairs (reference: GradientQuantiser, build_tree.cu:51-140, and
 * reduce_base_sums, :168-204).  gpair: int32 [n_local_rows, n_outputs, 2]; root_sums: int64
 * [n_outputs, 2] (summed over ranks); scale: double[4] = scale.g, scale.h, 1/scale.g, 1/scale.h;
 * max_abs (optional, may be NULL): device int32[2], the largest |grad| and |hess| among this
 * rank's quantised pairs - what lbk_histogram_args.max_abs takes. */
int lbk_quantise(lbk_context* ctx, const double* g, const double* h, int64_t ldg, int64_t row_offset,
                 int64_t n_local_rows, int n_outputs, int seed, int32_t* gpair, int64_t* root_sums,
                 double* scale, int32_t* max_abs, void* stream);

/* Histogram build over node-grouped rows (reference: fill_histogram_shared, build_tree.cu:213-577).
 * Rows are given as an index array grouped by node: rows of node (node_begin + j) are
 * row_index[seg[j] .. seg[j+1]).  For every listed node, output and feature:
 *   hist[j][k][row_ptr[f] + bin(row,f)] += value(row,k)
 * mode 0: value = int32 pair from gpair, hist = int64 pairs  [n_nodes, n_outputs, B, 2]
 * mode 1: value = float32 pair from gpair_f32, hist = float64 pairs of the same shape.
 * hist is overwritten by the call.  With device buffers the call is asynchronous on `stream` (unless it
 * has to read row_ptr back, see max_bins); with host buffers it returns when hist is filled. */
typedef struct lbk_histogram_args {
  const void* bins;   /* layout of lbk_bin_matrix */
  int32_t bin_bytes;
  int64_t n_rows;     /* rows of the bin matrix */
  int32_t n_features;
  const int32_t* row_ptr;   /* [n_features+1] device (host if host_buffers) */
  int32_t total_bins;       /* B = row_ptr[n_features] */
  const int32_t* gpair;     /* mode 0: [n_rows, n_outputs, 2] int32 */
  const float* gpair_f32;   /* mode 1: [n_rows, n_outputs, 2] float32 */
  int32_t n_outputs;
  const int32_t* row_index; /* [seg[n_nodes]] */
  const int32_t* seg;       /* [n_nodes+1] */
  int32_t n_nodes;
  int32_t mode;
  void* hist;
  void* stream;
  int32_t host_buffers;
  const int32_t* max_abs;   /* mode 0, optional: device int32[2] = largest |grad|, |hess| in gpair (the
                               call bounds its 32-bit partial sums with it); NULL = found by the call */
  int32_t max_bins;         /* optional, device buffers only: an upper bound of the bins of any one
                               feature (max of row_ptr[f+1] - row_ptr[f]); with it the call does not
                               read row_ptr back and nothing waits before the kernels are queued.
                               0 = found by the call.  A bound that is too small gives wrong sums. */
  int32_t all_reduce;       /* 1: hist is summed over the ranks of the context's communicator: every rank
                               ends with the sums of all bins.  2: every rank ends with the sums of the
                               bins of the features it owns (lbk_owned_features) - what the tree builder
                               uses, half of the bytes of 1 on the wire; the other bins of hist are not
                               written (or hold sums too).  Both go through buffers the ranks' GPUs read
                               from each other over NVLink where those can be mapped, else through one
                               all-reduce (then 2 also sums every bin). */
  int32_t pairs_by_position; /* 1: gpair / gpair_f32 are stored in row_index order, [seg[n_nodes], n_outputs, 2]:
                               entry i belongs to row row_index[i].  The pairs of a node are then read as a
                               stream instead of gathered (the tree builder keeps its pairs this way: the
                               repartition moves them together with the row ids).  mode 0 needs max_abs. */
} lbk_histogram_args;

int lbk_histogram(lbk_context* ctx, const lbk_histogram_args* args);

/* The same histogram build for callers that cannot allocate device memory at the time of the
 * call: a task running under a runtime that has already handed out the whole memory budget (a
 * cudaMalloc there fails, or takes memory the runtime believes it owns), or a process whose device
 * footprint must stay fixed after start-up.  It has no counterpart in the reference.  No context
 * is needed and nothing is allocated or freed: the per-call scratch lives in a fixed array of about
 * 16 KB inside the library image, present once on every GPU that loads the library until the
 * process exits.
 * Limits: n_nodes <= LBK_NOALLOC_MAX_NODES, n_features <= LBK_NOALLOC_MAX_FEATURES, device
 * pointers only (host_buffers = 0), all_reduce = 0 (no context, no communicator); anything else is
 * rejected with LBK_ERR_ARGUMENT.  max_bins is ignored (row_ptr is read back).
 * The first call on a device looks up the array's device address; make that call before any
 * stream capture begins.  All calls on a device share the array, so calls that overlap on the GPU
 * race: issue them on one stream.  The call blocks until `stream` has drained (do not issue it from
 * a host callback of a stream); `device` is current during the call and the caller's device is
 * restored afterwards; the error text is read with lbk_last_error(NULL). */
#define LBK_NOALLOC_MAX_NODES 4096
#define LBK_NOALLOC_MAX_FEATURES 4096
int lbk_histogram_noalloc(int device, const lbk_histogram_args* args);

/* Group rows by node id (stable): row_index/seg as lbk_histogram expects.  node_of_row values
 * outside [node_begin, node_begin+n_nodes) are dropped.  (Reference: the radix sort of
 * (node,row) pairs in UpdatePositions, build_tree.cu:1050-1079.) */
int lbk_group_rows(lbk_context* ctx, const int32_t* node_of_row, int64_t n_rows, int node_begin,
                   int n_nodes, int32_t* row_index, int32_t* seg, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LBK_H_ */
