// Measurement aid, built as its own small library (libb2sprobe.so) and used by bench.py only:
// n divergent 8-byte gathers x[idx[i]] and nothing else.  Timed over an L2-resident x it gives
// the ceiling the SpMV gather of x runs against (about one gather per clock per SM on B200).
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

// 128 threads x 8 gathers per pass, grid-stride over whole passes; the tail of fewer than 1024
// indices is taken by the first CTA one index per thread.
__global__ void __launch_bounds__(128, 12)
    probe_gather_kernel(const int32_t* __restrict__ idx, int64_t n, const double* __restrict__ x,
                        double* __restrict__ sink) {
  constexpr int U = 8;
  const int64_t pass = 128 * U;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * pass;
  double acc = 0.0;
  for (int64_t b = blockIdx.x * pass; b + pass <= n; b += stride) {
    int32_t c[U];
#pragma unroll
    for (int u = 0; u < U; ++u) c[u] = __ldcs(idx + b + u * 128 + threadIdx.x);
    double v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = __ldg(x + c[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) acc += v[u];
  }
  if (blockIdx.x == 0)
    for (int64_t i = n - n % pass + threadIdx.x; i < n; i += 128) acc += __ldg(x + idx[i]);
  if (acc == -1.2345678e300) *sink = acc;
}

}  // namespace

// idx values must lie in [0, n_x); *sink_dev (one double) is written only if a sum takes a value
// it cannot take.  Returns 0, or 2 for a bad argument, 4 for a failed launch.
extern "C" int b2s_probe_gather(const int32_t* idx_dev, int64_t n, const double* x_dev,
                                int64_t n_x, double* sink_dev, void* stream) {
  if (n < 0 || n_x <= 0) return 2;
  if (n == 0) return 0;
  if (!idx_dev || !x_dev || !sink_dev) return 2;
  const int64_t want = (n + 1023) / 1024;
  const unsigned grid = static_cast<unsigned>(want > 148 * 12 ? 148 * 12 : want);
  probe_gather_kernel<<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(idx_dev, n, x_dev,
                                                                           sink_dev);
  return cudaGetLastError() == cudaSuccess ? 0 : 4;
}
