// Stand-in for the parts of the legate runtime API that the reference's tree task bodies
// (src/models/tree/build_tree.cc, build_tree.cu, predict.cc, predict.cu and the headers they
// include) use.
// TEST INFRASTRUCTURE: it exists so that those unmodified reference sources can be compiled
// into oracle/_ref/libref_cpu.so (host compiler) and oracle/_ref/libref_gpu.so (nvcc) and used to
// check the oracle's restatement.  Stores are thin views over caller-owned memory; there is one
// rank, no runtime, no task registration.  Under nvcc the views are usable in device code and
// scratch buffers are device memory.
#pragma once
#if defined(__CUDACC__)
#include <cuda_runtime.h>
#define LBSTUB_HD __host__ __device__
#else
#define LBSTUB_HD
#endif
#include <array>
#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <memory>
#include <optional>
#include <ostream>
#include <sstream>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <vector>

namespace Legion {
class Logger {
 public:
  explicit Logger(const char*) {}
};
}  // namespace Legion

namespace legate {

using coord_t = long long;

template <int N, typename T = coord_t>
struct Point {
  T x[N];
  LBSTUB_HD Point()
  {
    for (int i = 0; i < N; ++i) x[i] = 0;
  }
  template <typename... A, typename = std::enable_if_t<sizeof...(A) == N>>
  LBSTUB_HD Point(A... a) : x{static_cast<T>(a)...}
  {
  }
  LBSTUB_HD T& operator[](int i) { return x[i]; }
  LBSTUB_HD const T& operator[](int i) const { return x[i]; }
  LBSTUB_HD static Point ZEROES() { return Point(); }
  LBSTUB_HD Point operator+(const Point& o) const
  {
    Point r;
    for (int i = 0; i < N; ++i) r.x[i] = x[i] + o.x[i];
    return r;
  }
  LBSTUB_HD Point operator-(const Point& o) const
  {
    Point r;
    for (int i = 0; i < N; ++i) r.x[i] = x[i] - o.x[i];
    return r;
  }
};

template <int N, typename T = coord_t>
struct Rect {
  Point<N, T> lo, hi;
  LBSTUB_HD bool empty() const
  {
    for (int i = 0; i < N; ++i)
      if (hi[i] < lo[i]) return true;
    return false;
  }
  LBSTUB_HD std::size_t volume() const
  {
    if (empty()) return 0;
    std::size_t v = 1;
    for (int i = 0; i < N; ++i) v *= static_cast<std::size_t>(hi[i] - lo[i] + 1);
    return v;
  }
};
// Row-major walk over the points of a rectangle (the last dimension moves fastest).
template <int N, typename T = coord_t>
class PointInRectIterator {
 public:
  explicit PointInRectIterator(const Rect<N, T>& r) : rect_(r), p_(r.lo), valid_(!r.empty()) {}
  bool valid() const { return valid_; }
  const Point<N, T>& operator*() const { return p_; }
  PointInRectIterator& operator++()
  {
    for (int d = N - 1; d >= 0; --d) {
      if (p_[d] < rect_.hi[d]) {
        ++p_[d];
        return *this;
      }
      p_[d] = rect_.lo[d];
    }
    valid_ = false;
    return *this;
  }
  PointInRectIterator operator++(int)
  {
    PointInRectIterator t = *this;
    ++(*this);
    return t;
  }

 private:
  Rect<N, T> rect_;
  Point<N, T> p_;
  bool valid_;
};

template <int N, typename T>
std::ostream& operator<<(std::ostream& os, const Rect<N, T>& r)
{
  os << "<";
  for (int i = 0; i < N; ++i) os << r.lo[i] << (i + 1 < N ? "," : "");
  os << ">..<";
  for (int i = 0; i < N; ++i) os << r.hi[i] << (i + 1 < N ? "," : "");
  return os << ">";
}

struct Type {
  enum class Code : int { BOOL = 0, INT32 = 3, INT64 = 4, FLOAT32 = 10, FLOAT64 = 11 };
  Code c;
  Code code() const { return c; }
};
template <typename T>
struct type_code_of;
template <>
struct type_code_of<float> {
  static constexpr Type::Code value = Type::Code::FLOAT32;
};
template <>
struct type_code_of<double> {
  static constexpr Type::Code value = Type::Code::FLOAT64;
};
template <>
struct type_code_of<int32_t> {
  static constexpr Type::Code value = Type::Code::INT32;
};
template <>
struct type_code_of<int64_t> {
  static constexpr Type::Code value = Type::Code::INT64;
};
template <>
struct type_code_of<bool> {
  static constexpr Type::Code value = Type::Code::BOOL;
};
template <typename T>
inline constexpr Type::Code type_code_of_v = type_code_of<T>::value;

struct TaskException : public std::runtime_error {
  explicit TaskException(const std::string& s) : std::runtime_error(s) {}
};

// Strided view; strides are in elements, a promoted dimension has stride 0.  Trivially copyable,
// so that a device lambda can capture one by value.
template <typename T, int N>
struct AccessorBase {
  T* base = nullptr;
  long long stride[N]{};
  long long origin[N]{};  // coordinates of base[0]
  // what the reference reaches as `accessor.accessor` (Legion's affine accessor): its own copy of
  // the strides, set by the store that makes the view
  struct Inner {
    long long stride[N]{};
    template <typename R>
    bool is_dense_row_major(const R& r) const
    {
      long long expect = 1;
      for (int d = N - 1; d >= 0; --d) {
        long long extent = r.hi[d] - r.lo[d] + 1;
        if (extent > 1 && stride[d] != expect) return false;
        expect *= extent;
      }
      return true;
    }
  } accessor;
  LBSTUB_HD T& at(const Point<N>& p) const
  {
    long long off = 0;
    for (int d = 0; d < N; ++d) off += (p[d] - origin[d]) * stride[d];
    return base[off];
  }
  // address of one element, and of the first element of a rectangle together with the strides (in
  // elements) of its dimensions: what an adapter needs to hand a store to a C library
  T* ptr(const Point<N>& p) const { return &at(p); }
  T* ptr(const Rect<N>& r, std::size_t* strides) const
  {
    for (int d = 0; d < N; ++d) strides[d] = static_cast<std::size_t>(stride[d]);
    return &at(r.lo);
  }
};
template <typename T, int N>
struct AccessorRO : AccessorBase<const T, N> {
  LBSTUB_HD const T& operator[](const Point<N>& p) const { return this->at(p); }
};
template <typename T, int N>
struct AccessorWO : AccessorBase<T, N> {
  LBSTUB_HD T& operator[](const Point<N>& p) const { return this->at(p); }
};

class PhysicalStore {
 public:
  void* ptr = nullptr;
  Type::Code tcode{};
  int ndim = 0;
  std::array<long long, 4> lo{}, hi{}, stride{};
  Type::Code code() const { return tcode; }
  Type type() const { return Type{tcode}; }
  int dim() const { return ndim; }
  template <int N>
  Rect<N> shape() const
  {
    Rect<N> r;
    for (int i = 0; i < N; ++i) {
      r.lo[i] = lo[i];
      r.hi[i] = hi[i];
    }
    return r;
  }
  template <typename T, int N, bool = false>
  AccessorRO<T, N> read_accessor() const
  {
    AccessorRO<T, N> a;
    a.base = static_cast<const T*>(ptr);
    for (int i = 0; i < N; ++i) {
      a.stride[i]          = stride[i];
      a.accessor.stride[i] = stride[i];
      a.origin[i]          = lo[i];
    }
    return a;
  }
  template <typename T, int N, bool = false>
  AccessorWO<T, N> write_accessor() const
  {
    AccessorWO<T, N> a;
    a.base = static_cast<T*>(ptr);
    for (int i = 0; i < N; ++i) {
      a.stride[i]          = stride[i];
      a.accessor.stride[i] = stride[i];
      a.origin[i]          = lo[i];
    }
    return a;
  }
};

class PhysicalArray {
 public:
  PhysicalStore store;
  const PhysicalStore& data() const { return store; }
  int dim() const { return store.ndim; }
  Type type() const { return store.type(); }
  template <int N>
  Rect<N> shape() const
  {
    return store.shape<N>();
  }
};

class Scalar {
 public:
  unsigned char bytes[8]{};
  template <typename T>
  T value() const
  {
    T v;
    __builtin_memcpy(&v, bytes, sizeof(T));
    return v;
  }
  template <typename T>
  static Scalar make(T v)
  {
    Scalar s;
    __builtin_memcpy(s.bytes, &v, sizeof(T));
    return s;
  }
};

struct Domain {
  std::size_t get_volume() const { return 1; }
};
struct DomainPoint {
  long long operator[](int) const { return 0; }
};
struct Communicator {
  template <typename T>
  T get() const
  {
    return T{};
  }
};

class TaskContext {
 public:
  struct State {
    std::vector<PhysicalArray> inputs, outputs;
    std::vector<Scalar> scalars;
    void* stream = nullptr;
  };
  std::shared_ptr<State> st = std::make_shared<State>();
  const PhysicalArray& input(std::size_t i) const { return st->inputs.at(i); }
  const PhysicalArray& output(std::size_t i) const { return st->outputs.at(i); }
  const std::vector<PhysicalArray>& inputs() const { return st->inputs; }
  const std::vector<Scalar>& scalars() const { return st->scalars; }
  const Scalar& scalar(std::size_t i) const { return st->scalars.at(i); }
  Domain get_launch_domain() const { return {}; }
  DomainPoint get_task_index() const { return {}; }
  std::size_t num_communicators() const { return 0; }
  Communicator communicator(int) const { return {}; }
#if defined(__CUDACC__)
  cudaStream_t get_task_stream() const { return static_cast<cudaStream_t>(st->stream); }
#endif
};

// Scratch buffers live until the end of the task, as the runtime's do: a temporary Buffer
// object going out of scope must not release its memory.  The driver calls
// detail::release_task_buffers() after the task body returns.
namespace detail {
inline void* raw_alloc(std::size_t bytes)
{
#if defined(__CUDACC__)
  void* p = nullptr;
  if (cudaMalloc(&p, bytes > 0 ? bytes : 1) != cudaSuccess) throw std::runtime_error("stand-in: cudaMalloc failed");
  return p;
#else
  return std::malloc(bytes > 0 ? bytes : 1);
#endif
}
inline void raw_free(void* p)
{
#if defined(__CUDACC__)
  cudaFree(p);
#else
  std::free(p);
#endif
}
inline std::vector<void*>& task_buffers()
{
  static thread_local std::vector<void*> v;
  return v;
}
inline void release_task_buffers()
{
  for (void* p : task_buffers())
    if (p) raw_free(p);
  task_buffers().clear();
}
}  // namespace detail

template <typename T, int DIM = 1>
class Buffer {
 public:
  T* mem = nullptr;
  long long extent[DIM]{};
  LBSTUB_HD long long offset(const Point<DIM>& p) const
  {
    long long off = 0;
    for (int d = 0; d < DIM; ++d) off = off * extent[d] + p[d];
    return off;
  }
  LBSTUB_HD T& operator[](const Point<DIM>& p) const { return mem[offset(p)]; }
  LBSTUB_HD T* ptr(const Point<DIM>& p) const { return mem + offset(p); }
  void destroy()
  {
    auto& v = detail::task_buffers();
    for (auto& q : v)
      if (q == mem) {
        detail::raw_free(q);
        q = nullptr;
      }
    mem = nullptr;
  }
};
template <typename T, int DIM = 1>
Buffer<T, DIM> create_buffer(const Point<DIM>& extents)
{
  static_assert(std::is_trivially_destructible_v<T>, "buffers hold plain data");
  Buffer<T, DIM> b;
  std::size_t n = 1;
  for (int d = 0; d < DIM; ++d) {
    b.extent[d] = extents[d];
    n *= static_cast<std::size_t>(extents[d] > 0 ? extents[d] : 0);
  }
  b.mem = static_cast<T*>(detail::raw_alloc(sizeof(T) * (n > 0 ? n : 1)));
  detail::task_buffers().push_back(b.mem);
  return b;
}

template <typename T, typename I, typename = std::enable_if_t<std::is_integral_v<I>>>
Buffer<T, 1> create_buffer(I n)
{
  return create_buffer<T, 1>(Point<1>(n));
}

// Memory kinds and the allocator thrust's temporary storage goes through (nvcc build only uses it).
struct Memory {
  enum Kind { SYSTEM_MEM, GPU_FB_MEM, Z_COPY_MEM };
};
class ScopedAllocator {
 public:
  explicit ScopedAllocator(Memory::Kind) {}
  ~ScopedAllocator()
  {
    for (void* p : live_) detail::raw_free(p);
  }
  ScopedAllocator(const ScopedAllocator&)            = delete;
  ScopedAllocator& operator=(const ScopedAllocator&) = delete;
  ScopedAllocator(ScopedAllocator&& o) noexcept : live_(std::move(o.live_)) { o.live_.clear(); }
  void* allocate(std::size_t bytes)
  {
    void* p = detail::raw_alloc(bytes);
    live_.push_back(p);
    return p;
  }
  void deallocate(void* p)
  {
    for (auto& q : live_)
      if (q == p) {
        detail::raw_free(q);
        q = live_.back();
        live_.pop_back();
        return;
      }
  }

 private:
  std::vector<void*> live_;
};

struct VariantOptions {
  constexpr VariantOptions with_has_allocations(bool) const { return *this; }
};
struct LocalTaskID {
  int id;
};
struct TaskConfig {
  LocalTaskID id;
};
class TaskRegistrar {};
template <typename T>
struct LegateTask {
  static void register_variants() {}
};

template <typename Functor, typename... Args>
decltype(auto) dim_dispatch(int dim, Functor&& f, Args&&... args)
{
  throw std::runtime_error("dim_dispatch is not part of the stand-in");
}

}  // namespace legate
