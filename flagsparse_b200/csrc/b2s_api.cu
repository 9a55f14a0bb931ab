// Entry points that are not tied to one operator: version, status text, the input-contract scan
// and the merge-path tile plan.
#include <mutex>

#include "b2s_tile.cuh"

namespace b2s {

void ensure_dyn_smem(const void* kernel, size_t bytes) {
  struct Seen {
    const void* k;
    int dev;
  };
  static Seen seen[512];
  static int n_seen = 0;
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_seen; ++i)
    if (seen[i].k == kernel && seen[i].dev == dev) return;
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                       static_cast<int>(bytes));
  if (n_seen < 512) seen[n_seen++] = {kernel, dev};
}

// ---- input contract --------------------------------------------------------------------------
__global__ void inspect_init_kernel(int64_t* stats) {
  stats[0] = 0;
  stats[1] = 0;
  stats[2] = 0;
  stats[3] = INT64_MAX;
  stats[4] = INT64_MIN;
  stats[5] = 0;
  stats[6] = 0;
  stats[7] = 0;
}

__device__ inline int64_t warp_max(int64_t v) {
  for (int m = 16; m > 0; m >>= 1) {
    int64_t o = __shfl_xor_sync(0xffffffffu, v, m);
    v = o > v ? o : v;
  }
  return v;
}
__device__ inline int64_t warp_min(int64_t v) {
  for (int m = 16; m > 0; m >>= 1) {
    int64_t o = __shfl_xor_sync(0xffffffffu, v, m);
    v = o < v ? o : v;
  }
  return v;
}
__device__ inline int64_t warp_add(int64_t v) {
  for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
  return v;
}

// Integer atomics only: min / max / add commute, so the eight words do not depend on the order
// in which warps arrive.
template <class P>
__global__ void inspect_ptr_kernel(const P* __restrict__ ptr, int64_t n_rows, int64_t* stats) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t bad = 0, longest = 0, empty = 0;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_rows;
       i += stride) {
    const int64_t a = static_cast<int64_t>(ptr[i]), b = static_cast<int64_t>(ptr[i + 1]);
    const int64_t len = b - a;
    bad += len < 0;
    empty += len == 0;
    longest = len > longest ? len : longest;
  }
  bad = warp_add(bad);
  empty = warp_add(empty);
  longest = warp_max(longest);
  if ((threadIdx.x & 31) == 0) {
    if (bad) atomicAdd(reinterpret_cast<unsigned long long*>(stats + 2),
                       static_cast<unsigned long long>(bad));
    if (empty) atomicAdd(reinterpret_cast<unsigned long long*>(stats + 6),
                         static_cast<unsigned long long>(empty));
    atomicMax(reinterpret_cast<long long*>(stats + 5), static_cast<long long>(longest));
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    stats[0] = static_cast<int64_t>(ptr[0]);
    stats[1] = static_cast<int64_t>(ptr[n_rows]);
  }
}

template <class I>
__global__ void inspect_idx_kernel(const I* __restrict__ idx, int64_t nnz, int64_t* stats) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  int64_t lo = INT64_MAX, hi = INT64_MIN;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < nnz;
       i += stride) {
    const int64_t c = static_cast<int64_t>(idx[i]);
    lo = c < lo ? c : lo;
    hi = c > hi ? c : hi;
  }
  lo = warp_min(lo);
  hi = warp_max(hi);
  if ((threadIdx.x & 31) == 0) {
    atomicMin(reinterpret_cast<long long*>(stats + 3), static_cast<long long>(lo));
    atomicMax(reinterpret_cast<long long*>(stats + 4), static_cast<long long>(hi));
  }
}

// ---- tile plan -------------------------------------------------------------------------------
// Merge-path search: tile t starts where diagonal d = t*items crosses the merge of the row-end
// offsets ptr[1..R] with the non-zero indices 0..nnz-1.  A row-end marker is consumed once all
// non-zeros of its row have been.
template <class P>
__global__ void tile_plan_kernel(const P* __restrict__ ptr, int64_t n_rows, int64_t nnz,
                                 int items, int64_t n_tiles, int64_t* __restrict__ tile_row) {
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t > n_tiles) return;
  const int64_t total = n_rows + nnz;
  int64_t d = t * static_cast<int64_t>(items);
  if (d > total) d = total;
  int64_t lo = d > nnz ? d - nnz : 0;
  int64_t hi = d < n_rows ? d : n_rows;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(ptr[mid + 1]) <= d - mid - 1)
      lo = mid + 1;
    else
      hi = mid;
  }
  tile_row[t] = lo;
}

}  // namespace b2s

extern "C" int b2s_version(void) { return B2S_VERSION; }

extern "C" const char* b2s_status_string(int status) {
  switch (status) {
    case B2S_OK: return "ok";
    case B2S_ERR_DTYPE: return "unsupported value or index dtype code";
    case B2S_ERR_ARG: return "invalid argument (null pointer or inconsistent size)";
    case B2S_ERR_ALIGNMENT: return "pointer not aligned to its element size";
    case B2S_ERR_LAUNCH: return "CUDA kernel launch failed";
    case B2S_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case B2S_ERR_WORKSPACE: return "scratch buffer too small";
    case B2S_ERR_RANGE: return "size does not fit the index dtype";
    case B2S_ERR_TOO_LARGE: return "problem exceeds the fixed scratch of b2s_spmv_csr_fixed";
    case B2S_ERR_BOUNDS: return "an index read from the matrix points outside its array";
  }
  return "unknown status";
}

extern "C" int b2s_csr_inspect(const void* indptr_dev, int ptr_type, const void* indices_dev,
                               int idx_type, int64_t n_rows, int64_t nnz, int64_t* stats_dev,
                               b2s_stream stream) {
  if (!stats_dev || !indptr_dev || n_rows < 0 || nnz < 0) return B2S_ERR_ARG;
  if (nnz > 0 && !indices_dev) return B2S_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  b2s::inspect_init_kernel<<<1, 1, 0, s>>>(stats_dev);
  const int threads = 256;
  {
    const int64_t want = (n_rows + threads - 1) / threads;
    const unsigned grid = static_cast<unsigned>(want < 1 ? 1 : (want > 148 * 8 ? 148 * 8 : want));
    B2S_DISPATCH_I(ptr_type, P, {
      (b2s::inspect_ptr_kernel<P><<<grid, threads, 0, s>>>(static_cast<const P*>(indptr_dev),
                                                           n_rows, stats_dev));
    });
  }
  if (nnz > 0) {
    const int64_t want = (nnz + threads - 1) / threads;
    const unsigned grid = static_cast<unsigned>(want > 148 * 8 ? 148 * 8 : want);
    B2S_DISPATCH_I(idx_type, I, {
      (b2s::inspect_idx_kernel<I><<<grid, threads, 0, s>>>(static_cast<const I*>(indices_dev),
                                                           nnz, stats_dev));
    });
  }
  return b2s::launch_status();
}

extern "C" int64_t b2s_tile_count(int64_t n_rows, int64_t nnz, int tile_items) {
  if (n_rows <= 0 || nnz < 0 || tile_items <= 0) return 0;
  return (n_rows + nnz + tile_items - 1) / tile_items;
}

extern "C" int b2s_tile_plan(const void* indptr_dev, int ptr_type, int64_t n_rows, int64_t nnz,
                             int tile_items, int64_t* tile_row_dev, b2s_stream stream) {
  if (n_rows < 0 || nnz < 0 || tile_items <= 0) return B2S_ERR_ARG;
  const int64_t n_tiles = b2s_tile_count(n_rows, nnz, tile_items);
  if (n_tiles == 0) return B2S_OK;
  if (!indptr_dev || !tile_row_dev) return B2S_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 128;
  const unsigned grid = static_cast<unsigned>((n_tiles + 1 + threads - 1) / threads);
  B2S_DISPATCH_I(ptr_type, P, {
    (b2s::tile_plan_kernel<P><<<grid, threads, 0, s>>>(static_cast<const P*>(indptr_dev), n_rows,
                                                       nnz, tile_items, n_tiles, tile_row_dev));
  });
  return b2s::launch_status();
}
