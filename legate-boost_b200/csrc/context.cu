// Context, scratch pool, status word and communicator of liblbk.so.
//
// Replaces what the reference's task bodies get from the legate runtime: scratch buffers
// (legate::create_buffer), the task stream and the NCCL communicator handed to the task
// (cpp_utils.cuh:100-134).  NCCL is bound at run time with dlopen so that a single-GPU user
// needs no NCCL at all and a multi-GPU user shares the copy already loaded in the process.
#include <dlfcn.h>

#include <cstring>
#include <mutex>

#include "internal.h"

namespace {

thread_local std::string tls_error;

// ---- NCCL, resolved lazily --------------------------------------------------------------------
struct NcclApi {
  void* handle                                                                           = nullptr;
  int (*GetUniqueId)(void*)                                                              = nullptr;
  int (*CommDestroy)(void*)                                                              = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t)            = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t)                 = nullptr;
  const char* (*GetErrorString)(int)                                                     = nullptr;
  void* CommInitRankRaw                                                                  = nullptr;
};

struct UniqueId {
  char bytes[LBK_UNIQUE_ID_BYTES];
};

NcclApi& nccl()
{
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (!api.handle) return;
    api.GetUniqueId     = reinterpret_cast<int (*)(void*)>(dlsym(api.handle, "ncclGetUniqueId"));
    api.CommInitRankRaw = dlsym(api.handle, "ncclCommInitRank");
    api.CommDestroy     = reinterpret_cast<int (*)(void*)>(dlsym(api.handle, "ncclCommDestroy"));
    api.AllReduce       = reinterpret_cast<int (*)(const void*, void*, size_t, int, int, void*, cudaStream_t)>(
      dlsym(api.handle, "ncclAllReduce"));
    api.AllGather = reinterpret_cast<int (*)(const void*, void*, size_t, int, void*, cudaStream_t)>(
      dlsym(api.handle, "ncclAllGather"));
    api.GetErrorString = reinterpret_cast<const char* (*)(int)>(dlsym(api.handle, "ncclGetErrorString"));
  });
  return api;
}

void require_nccl()
{
  auto& a = nccl();
  if (!a.handle || !a.GetUniqueId || !a.CommInitRankRaw || !a.AllReduce)
    throw lbk::Error(LBK_ERR_COMM, "NCCL (libnccl.so.2) could not be loaded");
}

void nccl_check(int rc, const char* what)
{
  if (rc != 0) {
    auto& a        = nccl();
    std::string m  = std::string(what) + ": " + (a.GetErrorString ? a.GetErrorString(rc) : "NCCL error");
    throw lbk::Error(LBK_ERR_COMM, m);
  }
}

// ncclDataType_t / ncclRedOp_t values of the public nccl.h
int nccl_dtype(lbk_dtype t)
{
  switch (t) {
    case LBK_F32: return 7;  // ncclFloat32
    case LBK_F64: return 8;  // ncclFloat64
    case LBK_I32: return 2;  // ncclInt32
    case LBK_I64: return 4;  // ncclInt64
  }
  return -1;
}
int nccl_op(lbk_redop o) { return o == LBK_SUM ? 0 : 2; }  // ncclSum, ncclMax

}  // namespace

namespace lbk {

// An allocation goes back the way it came: the allocator is fixed for the lifetime of a Scratch
// (lbk_context_set_allocator is not to be called while a call is in progress on the context).
static void ReleaseScratch(lbk_context* ctx, void* p, cudaStream_t stream)
{
  if (ctx->release_cb != nullptr) ctx->release_cb(ctx->alloc_user, p, stream);
  else cudaFreeAsync(p, stream);
}

Scratch::~Scratch()
{
  for (void* p : ptrs_)
    if (p) ReleaseScratch(ctx_, p, stream_);
}

void* Scratch::alloc_bytes(size_t bytes)
{
  void* p = nullptr;
  if (ctx_->alloc_cb != nullptr) {
    p = ctx_->alloc_cb(ctx_->alloc_user, bytes > 0 ? bytes : 16, stream_);
    if (p == nullptr)
      throw Error(LBK_ERR_ALLOC, "the caller's allocator returned no memory for " + std::to_string(bytes) + " bytes of scratch");
  } else {
    cudaError_t e = cudaMallocFromPoolAsync(&p, bytes > 0 ? bytes : 16, ctx_->pool, stream_);
    if (e != cudaSuccess) {
      cudaGetLastError();
      throw Error(LBK_ERR_ALLOC, "scratch allocation of " + std::to_string(bytes) + " bytes failed: " + cudaGetErrorString(e));
    }
  }
  ptrs_.push_back(p);
  return p;
}

void Scratch::free_one(void* p)
{
  for (auto& q : ptrs_)
    if (q == p) {
      ReleaseScratch(ctx_, q, stream_);
      q = nullptr;
    }
}

void AllReduce(lbk_context* ctx, void* buf, size_t count, lbk_dtype dtype, lbk_redop op, cudaStream_t stream)
{
  if (ctx->n_ranks <= 1 || count == 0) return;
  if (ctx->cb) {
    int rc = ctx->cb(ctx->cb_user, buf, count, static_cast<int>(dtype), static_cast<int>(op), stream);
    if (rc != 0) throw Error(LBK_ERR_COMM, "all-reduce callback returned " + std::to_string(rc));
    return;
  }
  if (!ctx->nccl_comm) throw Error(LBK_ERR_COMM, "Expected a communicator for a multi-rank call.");
  require_nccl();
  nccl_check(nccl().AllReduce(buf, buf, count, nccl_dtype(dtype), nccl_op(op), ctx->nccl_comm, stream), "ncclAllReduce");
}

bool AllGatherBytes(lbk_context* ctx, const void* send, void* recv, size_t bytes, cudaStream_t stream)
{
  if (ctx->cb != nullptr || ctx->nccl_comm == nullptr) return false;
  require_nccl();
  if (nccl().AllGather == nullptr) return false;
  nccl_check(nccl().AllGather(send, recv, bytes, 0 /* ncclInt8 */, ctx->nccl_comm, stream), "ncclAllGather");
  return true;
}

std::pair<cudaEvent_t, cudaEvent_t> NextProfileEvents(lbk_context* ctx)
{
  constexpr size_t kMaxProfiledLaunches = 4096;
  if (ctx->prof_used < ctx->prof_events.size()) return ctx->prof_events[ctx->prof_used++];
  if (ctx->prof_events.size() >= kMaxProfiledLaunches) return ctx->prof_events.back();
  std::pair<cudaEvent_t, cudaEvent_t> ev{nullptr, nullptr};
  LBK_CUDA(cudaEventCreate(&ev.first));
  LBK_CUDA(cudaEventCreate(&ev.second));
  ctx->prof_events.push_back(ev);
  ctx->prof_used = ctx->prof_events.size();
  return ev;
}

void CheckDeviceStatus(lbk_context* ctx, cudaStream_t stream)
{
  int h = 0;
  LBK_CUDA(cudaMemcpyAsync(&h, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, stream));
  LBK_CUDA(cudaStreamSynchronize(stream));
  if (h != 0) {
    LBK_CUDA(cudaMemsetAsync(ctx->d_status, 0, sizeof(int), stream));
    throw Error(LBK_ERR_DEVICE, "a kernel reported fault code " + std::to_string(h));
  }
}

// ABI boundary: exceptions never cross it.
int Guard(lbk_context* ctx, const std::function<void()>& f)
{
  try {
    f();
    return LBK_OK;
  } catch (const Error& e) {
    (ctx ? ctx->err : tls_error) = e.what();
    return e.code;
  } catch (const std::exception& e) {
    (ctx ? ctx->err : tls_error) = e.what();
    return LBK_ERR_ARGUMENT;
  }
}
}  // namespace lbk

extern "C" {

int lbk_version(void) { return 1000; }

int lbk_context_create(int device, lbk_context** out)
{
  return lbk::Guard(nullptr, [&] {
    LBK_EXPECT(out != nullptr, "out is null");
    int n = 0;
    LBK_CUDA(cudaGetDeviceCount(&n));
    LBK_EXPECT(device >= 0 && device < n, "no such CUDA device");
    LBK_CUDA(cudaSetDevice(device));
    auto* c   = new lbk_context();
    c->device = device;
    try {
      LBK_CUDA(cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device));
      LBK_CUDA(cudaDeviceGetAttribute(&c->max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
      cudaMemPoolProps props = {};
      props.allocType        = cudaMemAllocationTypePinned;
      props.handleTypes      = cudaMemHandleTypeNone;
      props.location.type    = cudaMemLocationTypeDevice;
      props.location.id      = device;
      LBK_CUDA(cudaMemPoolCreate(&c->pool, &props));
      uint64_t keep = UINT64_MAX;  // keep freed scratch cached between calls
      LBK_CUDA(cudaMemPoolSetAttribute(c->pool, cudaMemPoolAttrReleaseThreshold, &keep));
      LBK_CUDA(cudaMalloc(&c->d_status, sizeof(int)));
      LBK_CUDA(cudaMemset(c->d_status, 0, sizeof(int)));
    } catch (...) {
      if (c->pool) cudaMemPoolDestroy(c->pool);
      if (c->d_status) cudaFree(c->d_status);
      delete c;
      throw;
    }
    *out = c;
  });
}

void lbk_context_destroy(lbk_context* ctx)
{
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  cudaDeviceSynchronize();
  lbk::DestroyExchange(ctx);
  if (ctx->owns_nccl && ctx->nccl_comm && nccl().CommDestroy) nccl().CommDestroy(ctx->nccl_comm);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->pool) cudaMemPoolDestroy(ctx->pool);
  for (auto& ev : ctx->prof_events) {
    cudaEventDestroy(ev.first);
    cudaEventDestroy(ev.second);
  }
  delete ctx;
}

const char* lbk_last_error(const lbk_context* ctx) { return ctx ? ctx->err.c_str() : tls_error.c_str(); }

int lbk_context_trim(lbk_context* ctx)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "context is null");
    LBK_CUDA(cudaSetDevice(ctx->device));
    LBK_CUDA(cudaDeviceSynchronize());
    LBK_CUDA(cudaMemPoolTrimTo(ctx->pool, 0));
  });
}

int lbk_context_set_allocator(lbk_context* ctx, lbk_alloc_fn alloc, lbk_release_fn release, void* user)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "context is null");
    LBK_EXPECT((alloc == nullptr) == (release == nullptr), "give both callbacks or neither");
    ctx->alloc_cb   = alloc;
    ctx->release_cb = release;
    ctx->alloc_user = user;
  });
}

int lbk_context_pool_bytes(lbk_context* ctx, size_t* reserved)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && reserved, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    uint64_t v = 0;
    LBK_CUDA(cudaMemPoolGetAttribute(ctx->pool, cudaMemPoolAttrReservedMemCurrent, &v));
    *reserved = static_cast<size_t>(v);
  });
}

int lbk_comm_unique_id(void* id_out)
{
  return lbk::Guard(nullptr, [&] {
    LBK_EXPECT(id_out != nullptr, "id_out is null");
    require_nccl();
    UniqueId id;
    std::memset(&id, 0, sizeof(id));
    nccl_check(nccl().GetUniqueId(&id), "ncclGetUniqueId");
    std::memcpy(id_out, &id, sizeof(id));
  });
}

int lbk_comm_init(lbk_context* ctx, const void* id, int rank, int n_ranks)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && id, "null argument");
    LBK_EXPECT(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "bad rank");
    require_nccl();
    LBK_CUDA(cudaSetDevice(ctx->device));
    UniqueId uid;
    std::memcpy(&uid, id, sizeof(uid));
    using InitFn = int (*)(void**, int, UniqueId, int);  // ncclCommInitRank(comm*, nranks, id, rank)
    auto init    = reinterpret_cast<InitFn>(nccl().CommInitRankRaw);
    void* comm   = nullptr;
    nccl_check(init(&comm, n_ranks, uid, rank), "ncclCommInitRank");
    ctx->nccl_comm = comm;
    ctx->owns_nccl = true;
    ctx->rank      = rank;
    ctx->n_ranks   = n_ranks;
    ctx->cb        = nullptr;
  });
}

int lbk_comm_attach_nccl(lbk_context* ctx, void* nccl_comm, int rank, int n_ranks)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && nccl_comm, "null argument");
    LBK_EXPECT(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "bad rank");
    require_nccl();
    ctx->nccl_comm = nccl_comm;
    ctx->owns_nccl = false;
    ctx->rank      = rank;
    ctx->n_ranks   = n_ranks;
    ctx->cb        = nullptr;
  });
}

int lbk_comm_set_callback(lbk_context* ctx, lbk_allreduce_fn fn, void* user, int rank, int n_ranks)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && fn, "null argument");
    LBK_EXPECT(n_ranks >= 1 && rank >= 0 && rank < n_ranks, "bad rank");
    ctx->cb      = fn;
    ctx->cb_user = user;
    ctx->rank    = rank;
    ctx->n_ranks = n_ranks;
  });
}

int lbk_comm_size(const lbk_context* ctx) { return ctx ? ctx->n_ranks : 0; }

int lbk_owned_features(int rank, int n_ranks, int n_features, int* begin, int* end)
{
  return lbk::Guard(nullptr, [&] {
    LBK_EXPECT(begin && end, "null argument");
    LBK_EXPECT(n_ranks >= 1 && rank >= 0 && rank < n_ranks && n_features >= 0, "bad rank or shape");
    *begin = lbk::OwnedBegin(rank, n_ranks, n_features);
    *end   = lbk::OwnedBegin(rank + 1, n_ranks, n_features);
  });
}

int lbk_profile_enable(lbk_context* ctx, int on)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "context is null");
    ctx->profile   = on != 0;
    ctx->prof_used = 0;
  });
}

int lbk_profile_histogram_ms(lbk_context* ctx, float* ms)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && ms, "null argument");
    LBK_EXPECT(ctx->profile && ctx->prof_used > 0, "no histogram launch has been timed");
    LBK_CUDA(cudaSetDevice(ctx->device));
    const auto& ev = ctx->prof_events[ctx->prof_used - 1];
    LBK_CUDA(cudaEventSynchronize(ev.second));
    LBK_CUDA(cudaEventElapsedTime(ms, ev.first, ev.second));
  });
}

int lbk_profile_histogram_total(lbk_context* ctx, float* ms, int* launches)
{
  return lbk::Guard(ctx, [&] {
    LBK_EXPECT(ctx && ms && launches, "null argument");
    LBK_EXPECT(ctx->profile, "the histogram timing is not enabled");
    LBK_CUDA(cudaSetDevice(ctx->device));
    float total = 0.f;
    for (size_t i = 0; i < ctx->prof_used; ++i) {
      float t = 0.f;
      LBK_CUDA(cudaEventSynchronize(ctx->prof_events[i].second));
      LBK_CUDA(cudaEventElapsedTime(&t, ctx->prof_events[i].first, ctx->prof_events[i].second));
      total += t;
    }
    *ms            = total;
    *launches      = static_cast<int>(ctx->prof_used);
    ctx->prof_used = 0;
  });
}

}  // extern "C"
