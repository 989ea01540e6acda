// Peer exchange: the sum over ranks of a level's histograms as a reduce-scatter made of peer loads.
//
// Reference behaviour replaced here: the ncclAllReduce of the whole batch of histograms after
// every ComputeHistogram (src/models/tree/build_tree.cu:1107-1113, src/cpp_utils/cpp_utils.cuh:
// 100-134).  All ranks then hold all sums and all of them scan and evaluate every feature.
//
// Design for B200 / NVSwitch: every GPU reaches every peer's memory at full NVLink bandwidth, so
// a rank does not need a library collective to fetch what it owns.  Every rank builds its local
// histograms into a buffer the others can map; after a barrier rank r reads the bins of ITS
// features from all ranks with plain 16-byte loads and adds them up in rank order (exact for the
// integer sums, and the same order on whoever owns a bin for the float ones).  That is
// (R-1)/R of the buffer per GPU on the wire, half of an all-reduce, and the split search that
// follows only runs on the owned features.  Where a caller needs every bin everywhere, a second
// kernel copies the owners' sums (the all-gather half).
//
// The buffers are mapped with CUDA IPC between processes and with plain peer access inside one
// process (the runtime of the reference drives all GPUs of a node from one process).  Only plain
// loads and stores of peer memory are used: no bulk-copy engine, no multicast.  The barrier is a
// one-warp kernel: every rank stores the number of the barrier into its slot of every peer's flag
// array (a system-scope release store over NVLink) and waits until all slots of its own array have
// reached that number; the wait is bounded (about a second), after which the kernel reports
// through the context's status word and returns, so a rank that died cannot hang the others' GPUs.
// While it sums, the reduce kernel also clears the other buffer (which no rank reads any more once
// the barrier has passed), so that the next level finds it zeroed without a pass of its own.
#include <unistd.h>

#include <cstring>

#include "device_utils.cuh"
#include "internal.h"

namespace lbk {

constexpr int kMaxExchangeRanks = 64;

constexpr int kFaultPeerBarrier = 41;  // status word: a peer did not reach the barrier in time

struct PeerExchange {
  bool tried = false;  // the mapping was attempted (and failed if !ok)
  bool ok    = false;
  size_t bytes = 0;                 // per buffer
  // [0], [1]: the two histogram buffers; [2]: the barrier's flag array (one word per rank)
  void* local[3]   = {nullptr, nullptr, nullptr};
  void* peer[3][kMaxExchangeRanks];   // every rank's buffers as this device addresses them
  bool opened[3][kMaxExchangeRanks];  // the address came from cudaIpcOpenMemHandle
  void** d_peer[3] = {nullptr, nullptr, nullptr};  // the same, on the device
  size_t dirty[2]  = {0, 0};   // leading bytes of the histogram buffers that may be non-zero (the rest is zero)
  unsigned epoch   = 0;        // barriers so far
  int* d_word      = nullptr;  // a word for the small all-reduces of the set-up
  int next         = 0;
};

namespace {

struct Blob {
  int pid;
  int device;
  int ok;
  int pad;
  void* ptr[3];
  cudaIpcMemHandle_t handle[3];
};

void CloseMappings(lbk_context* ctx)
{
  PeerExchange* x = ctx->xchg;
  if (x == nullptr) return;
  for (int b = 0; b < 3; ++b) {
    for (int r = 0; r < ctx->n_ranks && r < kMaxExchangeRanks; ++r)
      if (x->opened[b][r] && x->peer[b][r] != nullptr) cudaIpcCloseMemHandle(x->peer[b][r]);
    if (x->local[b]) cudaFree(x->local[b]);
    if (x->d_peer[b]) cudaFree(x->d_peer[b]);
    x->local[b]  = nullptr;
    x->d_peer[b] = nullptr;
  }
  std::memset(x->peer, 0, sizeof(x->peer));
  std::memset(x->opened, 0, sizeof(x->opened));
  x->bytes    = 0;
  x->dirty[0] = x->dirty[1] = 0;
  x->epoch    = 0;
}

constexpr int kPullThreads = 256;

// dst[seg][b] = sum over ranks (in rank order) of peer[r][seg][b] for the bins b in [lo, hi) of
// the calling rank's features; 16 bytes (one pair) per thread and turn, every peer's load in flight
// together.
template <typename PairT, int R_UNROLL>
__global__ void __launch_bounds__(kPullThreads)
  k_pull_reduce(void* const* __restrict__ peers, int n_ranks, int rank, PairT* __restrict__ dst, int n_seg, int B, int F,
                const int32_t* __restrict__ row_ptr, int4* __restrict__ clear, long long clear_int4)
{
  // the other buffer, free since the barrier: zeroed here, beside the loads that wait for NVLink
  for (long long i = blockIdx.x * static_cast<long long>(kPullThreads) + threadIdx.x; i < clear_int4;
       i += static_cast<long long>(gridDim.x) * kPullThreads)
    clear[i] = make_int4(0, 0, 0, 0);
  const int lo  = row_ptr[OwnedBegin(rank, n_ranks, F)];
  const int hi  = row_ptr[OwnedBegin(rank + 1, n_ranks, F)];
  const int len = hi - lo;
  if (len <= 0) return;
  const long long total = static_cast<long long>(n_seg) * len;
  for (long long i = blockIdx.x * static_cast<long long>(kPullThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kPullThreads) {
    const int seg       = static_cast<int>(i / len);
    const int b         = lo + static_cast<int>(i - static_cast<long long>(seg) * len);
    const long long off = static_cast<long long>(seg) * B + b;
    PairT acc{0, 0};
    for (int r0 = 0; r0 < n_ranks; r0 += R_UNROLL) {
      PairT v[R_UNROLL];
#pragma unroll
      for (int u = 0; u < R_UNROLL; ++u)
        if (r0 + u < n_ranks) v[u] = LoadPairStreaming(static_cast<const PairT*>(peers[r0 + u]) + off);
#pragma unroll
      for (int u = 0; u < R_UNROLL; ++u)
        if (r0 + u < n_ranks) {
          acc.grad += v[u].grad;
          acc.hess += v[u].hess;
        }
    }
    StorePair(dst + off, acc);
  }
}

// The push form: this rank's receive buffer holds, per source rank, [n_seg][push_len] pairs of which
// the first `len` of a segment are the bins of this rank's features.  dst[seg][lo + e] = the sum
// over the source ranks, in rank order; every slot is zeroed as it is read.
template <typename PairT, int R_UNROLL>
__global__ void __launch_bounds__(kPullThreads)
  k_reduce_pushed(PairT* __restrict__ recv, int n_ranks, int rank, PairT* __restrict__ dst, int n_seg, int push_len,
                  int B, int F, const int32_t* __restrict__ row_ptr, int4* __restrict__ clear, long long clear_int4)
{
  for (long long i = blockIdx.x * static_cast<long long>(kPullThreads) + threadIdx.x; i < clear_int4;
       i += static_cast<long long>(gridDim.x) * kPullThreads)
    clear[i] = make_int4(0, 0, 0, 0);
  const int lo  = row_ptr[OwnedBegin(rank, n_ranks, F)];
  const int hi  = row_ptr[OwnedBegin(rank + 1, n_ranks, F)];
  const int len = min(hi - lo, push_len);
  if (len <= 0) return;
  const long long total  = static_cast<long long>(n_seg) * len;
  const long long stride = static_cast<long long>(n_seg) * push_len;  // pairs per source rank
  for (long long i = blockIdx.x * static_cast<long long>(kPullThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kPullThreads) {
    const int seg       = static_cast<int>(i / len);
    const int e         = static_cast<int>(i - static_cast<long long>(seg) * len);
    PairT* slot         = recv + static_cast<long long>(seg) * push_len + e;
    PairT acc{0, 0};
    for (int r0 = 0; r0 < n_ranks; r0 += R_UNROLL) {
      PairT v[R_UNROLL];
#pragma unroll
      for (int u = 0; u < R_UNROLL; ++u)
        if (r0 + u < n_ranks) v[u] = LoadPairStreaming(slot + (r0 + u) * stride);
#pragma unroll
      for (int u = 0; u < R_UNROLL; ++u)
        if (r0 + u < n_ranks) {
          acc.grad += v[u].grad;
          acc.hess += v[u].hess;
          StorePair(slot + (r0 + u) * stride, PairT{0, 0});
        }
    }
    StorePair(dst + static_cast<long long>(seg) * B + lo + e, acc);
  }
}

// dst[seg][b] = owner(b)'s buffer[seg][b] for every bin: the all-gather half.
template <typename PairT>
__global__ void __launch_bounds__(kPullThreads)
  k_pull_gather(void* const* __restrict__ peers, int n_ranks, PairT* __restrict__ dst, int n_seg, int B, int F,
                const int32_t* __restrict__ row_ptr)
{
  __shared__ int bounds[kMaxExchangeRanks + 1];
  for (int r = threadIdx.x; r <= n_ranks; r += kPullThreads) bounds[r] = row_ptr[OwnedBegin(r, n_ranks, F)];
  __syncthreads();
  const long long total = static_cast<long long>(n_seg) * B;
  for (long long i = blockIdx.x * static_cast<long long>(kPullThreads) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kPullThreads) {
    const int b = static_cast<int>(i % B);
    int lo = 0, hi = n_ranks;  // last r with bounds[r] <= b
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (bounds[mid] <= b) lo = mid; else hi = mid;
    }
    StorePair(dst + i, LoadPairStreaming(static_cast<const PairT*>(peers[lo]) + i));
  }
}

// One warp, lane r talks to rank r: "I have reached barrier `epoch`" into my slot of its flags, then
// wait for its word in mine.  Everything a rank wrote before (earlier kernels on its stream) is
// visible to whoever has seen its flag.
__global__ void k_peer_barrier(void* const* __restrict__ peer_flags, int n_ranks, int rank, unsigned epoch,
                               int* __restrict__ status)
{
  const int r = threadIdx.x;
  if (r >= n_ranks) return;
  __threadfence_system();
  unsigned* theirs = static_cast<unsigned*>(peer_flags[r]) + rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
  const unsigned* mine = static_cast<const unsigned*>(peer_flags[rank]) + r;
  unsigned seen        = 0;
  // about a second at most: a load over the local memory system takes a few hundred nanoseconds
  for (int spin = 0; spin < 4000000; ++spin) {
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
    if (static_cast<int>(seen - epoch) >= 0) return;
    __nanosleep(100);
  }
  if (status != nullptr) atomicExch(status, kFaultPeerBarrier);
}

void Barrier(lbk_context* ctx, cudaStream_t stream)
{
  PeerExchange* x = ctx->xchg;
  ++x->epoch;
  k_peer_barrier<<<1, 64, 0, stream>>>(x->d_peer[2], ctx->n_ranks, ctx->rank, x->epoch, ctx->d_status);
  LBK_LAUNCH_CHECK();
}

}  // namespace

void DestroyExchange(lbk_context* ctx)
{
  if (ctx->xchg == nullptr) return;
  CloseMappings(ctx);
  if (ctx->xchg->d_word) cudaFree(ctx->xchg->d_word);
  delete ctx->xchg;
  ctx->xchg = nullptr;
}

bool EnsureExchange(lbk_context* ctx, size_t bytes, cudaStream_t stream)
{
  if (ctx->n_ranks <= 1 || ctx->n_ranks > kMaxExchangeRanks || ctx->cb != nullptr || ctx->nccl_comm == nullptr)
    return false;
  if (ctx->xchg == nullptr) {
    ctx->xchg = new PeerExchange();
    std::memset(ctx->xchg->peer, 0, sizeof(ctx->xchg->peer));
    std::memset(ctx->xchg->opened, 0, sizeof(ctx->xchg->opened));
  }
  PeerExchange* x = ctx->xchg;
  if (x->tried && !x->ok) return false;
  if (x->ok && x->bytes >= bytes) return true;

  // (re)build, collectively: the sizes are equal on every rank, so every rank gets here together
  const int R = ctx->n_ranks;
  LBK_CUDA(cudaStreamSynchronize(stream));  // nobody may still read the buffers that go away
  if (x->ok) {
    // every rank has drained its stream only after the barrier below
    int* w = x->d_word;
    AllReduce(ctx, w, 1, LBK_I32, LBK_SUM, stream);
    LBK_CUDA(cudaStreamSynchronize(stream));
  }
  CloseMappings(ctx);
  x->tried = true;
  x->ok    = false;
  if (x->d_word == nullptr) {
    LBK_CUDA(cudaMalloc(&x->d_word, sizeof(int)));
    LBK_CUDA(cudaMemset(x->d_word, 0, sizeof(int)));
  }
  const size_t want = (bytes + (size_t{1} << 21) - 1) >> 21 << 21;  // whole 2 MB pages
  Blob mine;
  std::memset(&mine, 0, sizeof(mine));
  mine.pid    = static_cast<int>(getpid());
  mine.device = ctx->device;
  mine.ok     = 1;
  for (int b = 0; b < 3 && mine.ok; ++b) {
    const size_t sz = b < 2 ? want : sizeof(unsigned) * kMaxExchangeRanks;
    if (cudaMalloc(&x->local[b], sz) != cudaSuccess) {
      cudaGetLastError();
      mine.ok = 0;
      break;
    }
    if (cudaMemset(x->local[b], 0, sz) != cudaSuccess) {
      cudaGetLastError();
      mine.ok = 0;
      break;
    }
    mine.ptr[b] = x->local[b];
    if (cudaIpcGetMemHandle(&mine.handle[b], x->local[b]) != cudaSuccess) {
      cudaGetLastError();
      mine.ok = 0;
    }
  }
  // all ranks' blobs, through the communicator
  Blob* d_blobs = nullptr;
  LBK_CUDA(cudaMalloc(&d_blobs, sizeof(Blob) * (R + 1)));
  LBK_CUDA(cudaMemcpyAsync(d_blobs + R, &mine, sizeof(Blob), cudaMemcpyHostToDevice, stream));
  std::vector<Blob> all(R);
  const bool gathered = AllGatherBytes(ctx, d_blobs + R, d_blobs, sizeof(Blob), stream);
  if (gathered) {
    LBK_CUDA(cudaMemcpyAsync(all.data(), d_blobs, sizeof(Blob) * R, cudaMemcpyDeviceToHost, stream));
    LBK_CUDA(cudaStreamSynchronize(stream));
  }
  cudaFree(d_blobs);
  int good = gathered ? 1 : 0;
  for (int r = 0; r < R && good; ++r) good = all[r].ok;
  // map the peers
  for (int r = 0; r < R && good; ++r) {
    for (int b = 0; b < 3 && good; ++b) {
      if (r == ctx->rank) {
        x->peer[b][r] = x->local[b];
      } else if (all[r].pid == mine.pid) {
        // same process: the pointer is valid here once peer access is on
        cudaError_t e = cudaDeviceEnablePeerAccess(all[r].device, 0);
        if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) good = 0;
        cudaGetLastError();
        x->peer[b][r] = all[r].ptr[b];
      } else {
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[r].handle[b], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
          cudaGetLastError();
          good = 0;
        } else {
          x->peer[b][r]   = p;
          x->opened[b][r] = true;
        }
      }
    }
  }
  // every rank has to come to the same answer
  int* d_flag = x->d_word;
  LBK_CUDA(cudaMemcpyAsync(d_flag, &good, sizeof(int), cudaMemcpyHostToDevice, stream));
  AllReduce(ctx, d_flag, 1, LBK_I32, LBK_SUM, stream);
  int sum = 0;
  LBK_CUDA(cudaMemcpyAsync(&sum, d_flag, sizeof(int), cudaMemcpyDeviceToHost, stream));
  LBK_CUDA(cudaStreamSynchronize(stream));
  LBK_CUDA(cudaMemsetAsync(d_flag, 0, sizeof(int), stream));
  if (sum != R) {
    CloseMappings(ctx);
    return false;
  }
  for (int b = 0; b < 3; ++b) {
    LBK_CUDA(cudaMalloc(&x->d_peer[b], sizeof(void*) * R));
    LBK_CUDA(cudaMemcpyAsync(x->d_peer[b], x->peer[b], sizeof(void*) * R, cudaMemcpyHostToDevice, stream));
  }
  LBK_CUDA(cudaStreamSynchronize(stream));
  x->bytes = want;
  x->ok    = true;
  return true;
}

void* NextExchangeBuffer(lbk_context* ctx, size_t bytes, cudaStream_t stream)
{
  PeerExchange* x = ctx->xchg;
  x->next ^= 1;
  // (normally clean: the reduce kernel of the call before has cleared it)
  if (x->dirty[x->next] > 0) LBK_CUDA(cudaMemsetAsync(x->local[x->next], 0, x->dirty[x->next], stream));
  x->dirty[x->next] = bytes;  // about to be written
  return x->local[x->next];
}

void* const* NextPushBuffers(lbk_context* ctx, cudaStream_t stream)
{
  PeerExchange* x = ctx->xchg;
  x->next ^= 1;
  if (x->dirty[x->next] > 0) {
    // (not reached in the usual sequences.)  The peers are about to store into this buffer: it has to
    // be clean on every rank before any of them starts, hence the collective behind the clearing.
    LBK_CUDA(cudaMemsetAsync(x->local[x->next], 0, x->dirty[x->next], stream));
    AllReduce(ctx, x->d_word, 1, LBK_I32, LBK_SUM, stream);
    x->dirty[x->next] = 0;
  }
  return x->d_peer[x->next];
}

static int BufferIndex(lbk_context* ctx, const void* buf)
{
  PeerExchange* x = ctx->xchg;
  LBK_EXPECT(x != nullptr && x->ok && (buf == x->local[0] || buf == x->local[1]), "not an exchange buffer");
  return buf == x->local[0] ? 0 : 1;
}

void ExchangeReduceOwned(lbk_context* ctx, void* buf, void* dst, int n_seg, int B, int F, const int32_t* row_ptr,
                         bool float_mode, cudaStream_t stream)
{
  const int which = BufferIndex(ctx, buf);
  PeerExchange* x = ctx->xchg;
  // every rank's build of this level is complete - and so is everything of the level before: nobody
  // reads the other buffer any more
  Barrier(ctx, stream);
  const long long per_rank = static_cast<long long>(n_seg) * ((B + ctx->n_ranks - 1) / ctx->n_ranks);
  long long blocks         = (per_rank + kPullThreads - 1) / kPullThreads;
  if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  if (blocks < 1) blocks = 1;
  void* const* peers = x->d_peer[which];
  // the other buffer is cleared, as far as the call before dirtied it
  int4* clear             = static_cast<int4*>(x->local[1 - which]);
  const long long clear_n = static_cast<long long>((x->dirty[1 - which] + 15) / 16);
  if (float_mode)
    k_pull_reduce<GPairF64, 8><<<static_cast<unsigned>(blocks), kPullThreads, 0, stream>>>(
      peers, ctx->n_ranks, ctx->rank, static_cast<GPairF64*>(dst), n_seg, B, F, row_ptr, clear, clear_n);
  else
    k_pull_reduce<GPairI64, 8><<<static_cast<unsigned>(blocks), kPullThreads, 0, stream>>>(
      peers, ctx->n_ranks, ctx->rank, static_cast<GPairI64*>(dst), n_seg, B, F, row_ptr, clear, clear_n);
  LBK_LAUNCH_CHECK();
  x->dirty[1 - which] = 0;
}

void ExchangeReducePushed(lbk_context* ctx, void* dst, int n_seg, int push_len, int B, int F, const int32_t* row_ptr,
                          bool float_mode, cudaStream_t stream)
{
  PeerExchange* x = ctx->xchg;
  const int which = x->next;
  // every rank's kernel has finished storing into everybody's receive slots - and everything of the
  // call before is over: nobody reads the other buffer any more
  Barrier(ctx, stream);
  const long long per_rank = static_cast<long long>(n_seg) * push_len;
  long long blocks         = (per_rank + kPullThreads - 1) / kPullThreads;
  if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  if (blocks < 1) blocks = 1;
  int4* clear             = static_cast<int4*>(x->local[1 - which]);
  const long long clear_n = static_cast<long long>((x->dirty[1 - which] + 15) / 16);
  if (float_mode)
    k_reduce_pushed<GPairF64, 8><<<static_cast<unsigned>(blocks), kPullThreads, 0, stream>>>(
      static_cast<GPairF64*>(x->local[which]), ctx->n_ranks, ctx->rank, static_cast<GPairF64*>(dst), n_seg, push_len, B,
      F, row_ptr, clear, clear_n);
  else
    k_reduce_pushed<GPairI64, 8><<<static_cast<unsigned>(blocks), kPullThreads, 0, stream>>>(
      static_cast<GPairI64*>(x->local[which]), ctx->n_ranks, ctx->rank, static_cast<GPairI64*>(dst), n_seg, push_len, B,
      F, row_ptr, clear, clear_n);
  LBK_LAUNCH_CHECK();
  x->dirty[1 - which] = 0;
}

void ExchangeGatherAll(lbk_context* ctx, void* buf, void* dst, int n_seg, int B, int F, const int32_t* row_ptr,
                       cudaStream_t stream)
{
  const int which = BufferIndex(ctx, buf);
  Barrier(ctx, stream);  // every owner's sums are in place
  const long long total = static_cast<long long>(n_seg) * B;
  long long blocks      = (total + kPullThreads - 1) / kPullThreads;
  if (blocks > ctx->sm_count * 16) blocks = ctx->sm_count * 16;
  if (blocks < 1) blocks = 1;
  // pairs of 16 bytes whatever they hold
  k_pull_gather<GPairI64><<<static_cast<unsigned>(blocks), kPullThreads, 0, stream>>>(
    ctx->xchg->d_peer[which], ctx->n_ranks, static_cast<GPairI64*>(dst), n_seg, B, F, row_ptr);
  LBK_LAUNCH_CHECK();
}

}  // namespace lbk

// The peer barrier's bounded wait, exercised on one GPU: an emulated world of two ranks whose flag
// arrays both live on this device; rank 1 either has arrived already (its flag is preset) or never
// arrives.  In the second case the kernel gives up after its limit (about a second), reports
// through the status word and returns, and this call returns LBK_ERR_DEVICE; the context stays
// usable.  Nothing faults, traps or spins without limit.
extern "C" int lbk_selftest_peer_barrier(lbk_context* ctx, int peer_present, void* stream_)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    lbk::Scratch s(ctx, stream);
    unsigned* flags = s.alloc<unsigned>(4);  // [rank 0's array: slots 0, 1][rank 1's array: slots 0, 1]
    void** table    = s.alloc<void*>(2);
    const unsigned h_flags[4] = {0u, peer_present ? 1u : 0u, 0u, 0u};
    void* h_table[2]          = {flags, flags + 2};
    LBK_CUDA(cudaMemcpyAsync(flags, h_flags, sizeof(h_flags), cudaMemcpyHostToDevice, stream));
    LBK_CUDA(cudaMemcpyAsync(table, h_table, sizeof(h_table), cudaMemcpyHostToDevice, stream));
    lbk::k_peer_barrier<<<1, 64, 0, stream>>>(table, 2, 0, 1u, ctx->d_status);
    LBK_LAUNCH_CHECK();
    lbk::CheckDeviceStatus(ctx, stream);
  });
}

