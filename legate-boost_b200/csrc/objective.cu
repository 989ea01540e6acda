// Weighted gradients of the boosting round: g = d loss / d raw prediction times the learning rate,
// h = second derivative floored at 1e-8, both float64 [n_rows, n_outputs].
//
// Reference behaviour restated here: LBBase._get_weighted_gradient, legateboost/legateboost.py:189-224
// (unit sample weights, no subsampling), over the objectives' transform + gradient:
// SquaredErrorObjective (objectives.py:131-135): g = pred - y, h = 1;
// LogLossObjective (objectives.py:489-512): binary p = 1 / (1 + exp(-raw)), g = p - y, h = p (1 - p);
// multi-class softmax with the row maximum taken out, g = p - onehot(label), h = p (1 - p).
// The reference runs them as a chain of array operations (about ten passes over N x K float64);
// here a row is read once and its pairs are written once.
#include "device_utils.cuh"
#include "internal.h"

namespace lbk {
namespace {

constexpr int kMaxClassesInRegisters = 32;

__global__ void __launch_bounds__(256)
  k_gradient_squared_error(const double* __restrict__ raw, const double* __restrict__ y, int64_t n, double lr,
                           double* __restrict__ g, double* __restrict__ h)
{
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  g[i] = (raw[i] - y[i]) * lr;
  h[i] = 1.0;
}

__global__ void __launch_bounds__(256)
  k_gradient_logloss_binary(const double* __restrict__ raw, const double* __restrict__ y, int64_t n, double lr,
                            double* __restrict__ g, double* __restrict__ h)
{
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= n) return;
  const double p = 1.0 / (1.0 + exp(-raw[i]));
  g[i]           = (p - y[i]) * lr;
  h[i]           = fmax(p * (1.0 - p), 1e-8);
}

// one thread per row; the exponentials of up to 32 classes stay in registers, more are recomputed
__global__ void __launch_bounds__(256)
  k_gradient_softmax(const double* __restrict__ raw, const double* __restrict__ label, int64_t n_rows, int K, double lr,
                     double* __restrict__ g, double* __restrict__ h)
{
  const int64_t row = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (row >= n_rows) return;
  const double* r = raw + row * K;
  double s        = r[0];
  for (int k = 1; k < K; ++k) s = fmax(s, r[k]);
  double e[kMaxClassesInRegisters];
  double div = 0.0;
  for (int k = 0; k < K; ++k) {
    const double v = exp(r[k] - s);
    if (k < kMaxClassesInRegisters) e[k] = v;
    div += v;
  }
  const int cls = static_cast<int>(label[row]);
  for (int k = 0; k < K; ++k) {
    const double v = k < kMaxClassesInRegisters ? e[k] : exp(r[k] - s);
    const double p = v / div;
    g[row * K + k] = (k == cls ? p - 1.0 : p) * lr;
    h[row * K + k] = fmax(p * (1.0 - p), 1e-8);
  }
}

}  // namespace
}  // namespace lbk

extern "C" int lbk_gradient(lbk_context* ctx, int objective, const double* raw_pred, const double* y, int64_t n_rows,
                            int n_outputs, double learning_rate, double* g, double* h, void* stream_)
{
  using namespace lbk;
  return Guard(ctx, [&] {
    LBK_EXPECT(ctx != nullptr, "context is null");
    LBK_EXPECT(objective == LBK_SQUARED_ERROR || objective == LBK_LOG_LOSS, "unknown objective");
    LBK_EXPECT(n_rows >= 0 && n_outputs >= 1, "bad shape");
    if (n_rows == 0) return;
    LBK_EXPECT(raw_pred && y && g && h, "null argument");
    LBK_CUDA(cudaSetDevice(ctx->device));
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    const int64_t n     = n_rows * n_outputs;
    if (objective == LBK_SQUARED_ERROR) {
      k_gradient_squared_error<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(raw_pred, y, n, learning_rate,
                                                                                          g, h);
    } else if (n_outputs == 1) {
      k_gradient_logloss_binary<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(raw_pred, y, n, learning_rate,
                                                                                           g, h);
    } else {
      k_gradient_softmax<<<static_cast<unsigned>((n_rows + 255) / 256), 256, 0, stream>>>(raw_pred, y, n_rows, n_outputs,
                                                                                         learning_rate, g, h);
    }
    LBK_LAUNCH_CHECK();
  });
}
