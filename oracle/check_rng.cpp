// Cross-check of the oracle's restated random-number arithmetic against the CUDA toolkit's
// thrust headers compiled for the host (test infrastructure).  The reference draws its
// split-sample rows and its stochastic-rounding uniforms with thrust::default_random_engine
// (src/models/tree/build_tree.cu:112-129, 882-888).  Exit code 0 = identical.
#include <thrust/random.h>
#include <cstdint>
#include <cstdio>
#include <vector>

extern "C" {
void lbo_sample_rows(int seed, int S, int64_t n_rows, int64_t* out);
void lbo_uniform_pair(int64_t seed, double* out2);
}

int main()
{
  int bad = 0;
  const int seeds[]      = {0, 1, 2, 12345, 2147483646, 2147483647, 48271, 1790989824};
  const int64_t nrows[]  = {1, 2, 3, 1000, 200000, 100000000, 5000000000LL};
  for (int seed : seeds)
    for (int64_t n : nrows) {
      const int S = 300;
      std::vector<int64_t> got(S);
      lbo_sample_rows(seed, S, n, got.data());
      for (int i = 0; i < S; ++i) {
        thrust::default_random_engine eng(seed);
        thrust::uniform_int_distribution<int64_t> dist(0, n - 1);
        eng.discard(i);
        int64_t want = dist(eng);
        if (want != got[i]) {
          if (bad < 10) std::printf("rows mismatch seed=%d n=%lld i=%d want=%lld got=%lld\n", seed, (long long)n, i, (long long)want, (long long)got[i]);
          ++bad;
        }
      }
    }
  const int64_t seeds64[] = {0, 1, -1, 2147483647, 2147483648LL, 4294967295LL, 4294967296LL,
                             -8446744073709551615LL, 0x7fffffffffffffffLL, 123456789012345LL,
                             2147483647LL * 3, -2147483647LL};
  for (int64_t s : seeds64) {
    double got[2];
    lbo_uniform_pair(s, got);
    thrust::default_random_engine eng(s);
    thrust::uniform_real_distribution<double> dist(0.0, 1.0);
    double w0 = dist(eng), w1 = dist(eng);
    if (w0 != got[0] || w1 != got[1]) {
      std::printf("uniform mismatch seed=%lld\n", (long long)s);
      ++bad;
    }
  }
  std::printf(bad ? "FAIL %d\n" : "OK\n", bad);
  return bad ? 1 : 0;
}
