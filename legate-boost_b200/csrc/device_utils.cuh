// Device-side arithmetic shared by the kernels: the reference's random-number and hash
// functions restated with plain integer arithmetic, and its gain / leaf-value formulas.
// Translation units that include this file are compiled with -fmad=false so that no product
// is fused into a following add (the results are compared bit-for-bit with a CPU restatement
// compiled with -ffp-contract=off).
#pragma once
#include <cstdint>

#include "internal.h"

namespace lbk {

// thrust::default_random_engine (minstd_rand): x <- 48271 x mod (2^31-1); a seed congruent to 0
// becomes 1; the seed argument is first converted to the engine's 32-bit unsigned state type.
struct MinStd {
  uint32_t x;
  __host__ __device__ explicit MinStd(uint32_t s)
  {
    uint32_t r = s % 2147483647u;
    x          = r == 0 ? 1u : r;
  }
  __host__ __device__ uint32_t next()
  {
    x = static_cast<uint32_t>((48271ull * x) % 2147483647ull);
    return x;
  }
  __host__ __device__ void discard(unsigned long long z)
  {
    unsigned long long mult = 48271ull, mult_z = 1ull;
    while (z > 0) {
      if (z & 1ull) mult_z = (mult_z * mult) % 2147483647ull;
      z >>= 1;
      mult = (mult * mult) % 2147483647ull;
    }
    x = static_cast<uint32_t>((mult_z * x) % 2147483647ull);
  }
  // thrust::uniform_real_distribution<double>(a,b)
  __host__ __device__ double uniform_real(double a, double b)
  {
    double r = static_cast<double>(next() - 1u);
    r /= 2147483646.0;
    return (r * (b - a)) + a;
  }
  // thrust::uniform_int_distribution<int64_t>(a,b): truncated real draw from [a, b+1)
  __host__ __device__ long long uniform_int(long long a, long long b)
  {
    return static_cast<long long>(uniform_real(static_cast<double>(a), static_cast<double>(b) + 1.0));
  }
};

// MurmurHash3 fmix64 on a signed value and boost-style hash_combine (reference:
// build_tree.cu:143-165).  Right shifts are arithmetic, multiplications and additions wrap.
__host__ __device__ inline long long Hash64(long long k)
{
  k ^= k >> 33;
  k = static_cast<long long>(static_cast<unsigned long long>(k) * 0xff51afd7ed558ccdULL);
  k ^= k >> 33;
  k = static_cast<long long>(static_cast<unsigned long long>(k) * 0xc4ceb9fe1a85ec53ULL);
  k ^= k >> 33;
  return k;
}
__host__ __device__ inline long long HashCombine1(long long seed, long long v)
{
  unsigned long long add = static_cast<unsigned long long>(Hash64(v)) + 0x9e3779b9ULL +
                           (static_cast<unsigned long long>(seed) << 6) +
                           static_cast<unsigned long long>(seed >> 2);
  return seed ^ static_cast<long long>(add);
}
__host__ __device__ inline long long HashCombine(long long seed, long long a, long long b)
{
  return HashCombine1(HashCombine1(seed, a), b);
}

// Stochastic rounding of one (g,h) pair (reference: QuantiseStochasticRounding,
// build_tree.cu:112-129): first uniform draw for the gradient, second for the hessian.
__device__ inline int2 QuantisePair(double g, double h, const QuantParams& qp, long long seed)
{
  MinStd eng(static_cast<uint32_t>(static_cast<unsigned long long>(seed)));
  const double sg = g * qp.scale_g;
  const double sh = h * qp.scale_h;
  const double fg = floor(sg);
  const double fh = floor(sh);
  const double rg = sg - fg;
  const double rh = sh - fh;
  const double ug = eng.uniform_real(0.0, 1.0);
  const double uh = eng.uniform_real(0.0, 1.0);
  const long long qg = static_cast<long long>(fg + static_cast<double>(ug < rg));
  const long long qh = static_cast<long long>(fh + static_cast<double>(uh < rh));
  return make_int2(static_cast<int>(qg), static_cast<int>(qh));
}

__device__ inline GPairF64 Dequantise(GPairI64 v, const QuantParams& qp)
{
  GPairF64 r;
  r.grad = static_cast<double>(v.grad) * qp.inv_g;
  r.hess = static_cast<double>(v.hess) * qp.inv_h;
  return r;
}

// reference: build_tree.h:106-152
__device__ inline double LeafGain(GPairF64 s, double l1, double reg)
{
  double z = 0.0;
  if (s.grad > l1) {
    z = s.grad - l1;
  } else if (s.grad < -l1) {
    z = s.grad + l1;
  }
  return (z * z) / (s.hess + reg);
}
__device__ inline double CalculateGain(GPairF64 l, GPairF64 r, GPairF64 p, double l1, double l2, double msg)
{
  const double reg = fmax(1e-5, l2);
  return (0.5 * (LeafGain(l, l1, reg) + LeafGain(r, l1, reg) - LeafGain(p, l1, reg))) - msg;
}
__device__ inline double CalculateLeafValue(double G, double H, double l1, double l2)
{
  double z = 0.0;
  if (G > l1) {
    z = G - l1;
  } else if (G < -l1) {
    z = G + l1;
  }
  return -z / (H + l2);
}

__device__ inline GPairI64 LoadPair(const GPairI64* p)
{
  const longlong2 v = *reinterpret_cast<const longlong2*>(p);
  return GPairI64{v.x, v.y};
}
__device__ inline void StorePair(GPairI64* p, GPairI64 v)
{
  *reinterpret_cast<longlong2*>(p) = make_longlong2(v.grad, v.hess);
}
__device__ inline void StorePair(GPairF64* p, GPairF64 v)
{
  *reinterpret_cast<double2*>(p) = make_double2(v.grad, v.hess);
}
// 16-byte loads that go to L2 / the owning GPU every time (no L1 copy): for memory that another
// GPU or an earlier level wrote
__device__ inline GPairI64 LoadPairStreaming(const GPairI64* p)
{
  const longlong2 v = __ldcg(reinterpret_cast<const longlong2*>(p));
  return GPairI64{v.x, v.y};
}
__device__ inline GPairF64 LoadPairStreaming(const GPairF64* p)
{
  const double2 v = __ldcg(reinterpret_cast<const double2*>(p));
  return GPairF64{v.x, v.y};
}

}  // namespace lbk
