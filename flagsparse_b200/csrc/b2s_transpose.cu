// CSR -> CSC for sm_100a: the transpose behind op = trans / conj, built once per matrix.
//
// A stable least-significant-digit radix sort (8-bit digits) of the non-zeros by column, with
// the source position as payload.  Stability keeps, inside one column, the order in which the
// non-zeros appear in the CSR arrays (ascending source row), which is what a stable argsort on
// the column ids gives.  Ranks are computed with warp match / ballot and integer counters, so
// the permutation -- and therefore the order in which SpMV / SpMM later add the entries of a
// transposed row -- is the same on every run.
#include "b2s_tile.cuh"

namespace b2s {

constexpr int kRxThreads = 256;
constexpr int kRxWarps = kRxThreads / 32;
constexpr int kRxRounds = 16;                        // keys per lane
constexpr int kRxWarpChunk = 32 * kRxRounds;         // keys per warp, contiguous
constexpr int kRxChunk = kRxWarpChunk * kRxWarps;    // keys per CTA
constexpr int kScanThreads = 256;
constexpr int kScanPer = 8;
constexpr int kScanChunk = kScanThreads * kScanPer;

// ---- per-CTA digit histogram ----------------------------------------------------------------
template <class W, class KeyIn>
__global__ void __launch_bounds__(kRxThreads)
radix_hist_kernel(const KeyIn* __restrict__ keys, int64_t n, int shift, W* __restrict__ hist,
                  int64_t n_blocks) {
  __shared__ unsigned int cnt[256];
  cnt[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = blockIdx.x * static_cast<int64_t>(kRxChunk);
  for (int q = 0; q < kRxChunk / kRxThreads; ++q) {
    const int64_t i = base + q * kRxThreads + threadIdx.x;
    if (i < n) {
      const unsigned d = static_cast<unsigned>((static_cast<uint64_t>(keys[i]) >> shift) & 255u);
      atomicAdd(&cnt[d], 1u);
    }
  }
  __syncthreads();
  hist[threadIdx.x * n_blocks + blockIdx.x] = static_cast<W>(cnt[threadIdx.x]);
}

// ---- exclusive scan (three small kernels, applied recursively from the host) ------------------
template <class W>
__global__ void __launch_bounds__(kScanThreads)
scan_block_kernel(W* __restrict__ data, int64_t n, W* __restrict__ sums) {
  __shared__ W warp_tot[kScanThreads / 32];
  const int64_t base = blockIdx.x * static_cast<int64_t>(kScanChunk) + threadIdx.x * kScanPer;
  W v[kScanPer];
  W run = 0;
#pragma unroll
  for (int i = 0; i < kScanPer; ++i) {
    v[i] = (base + i < n) ? data[base + i] : 0;
    run += v[i];
  }
  // inclusive scan of the thread totals across the warp, then across warps
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  W inc = run;
  for (int o = 1; o < 32; o <<= 1) {
    const W up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  if (lane == 31) warp_tot[warp] = inc;
  __syncthreads();
  W warp_off = 0;
  for (int w = 0; w < warp; ++w) warp_off += warp_tot[w];
  W excl = warp_off + inc - run;
#pragma unroll
  for (int i = 0; i < kScanPer; ++i) {
    if (base + i < n) data[base + i] = excl;
    excl += v[i];
  }
  if (threadIdx.x == kScanThreads - 1 && sums) sums[blockIdx.x] = warp_off + inc;
}

template <class W>
__global__ void scan_add_kernel(W* __restrict__ data, int64_t n, const W* __restrict__ sums) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < n) data[i] += sums[i / kScanChunk];
}

template <class W>
void exclusive_scan(W* data, int64_t n, W* scratch, cudaStream_t s) {
  if (n <= 0) return;
  const int64_t blocks = (n + kScanChunk - 1) / kScanChunk;
  if (blocks == 1) {
    scan_block_kernel<W><<<1, kScanThreads, 0, s>>>(data, n, nullptr);
    return;
  }
  scan_block_kernel<W><<<static_cast<unsigned>(blocks), kScanThreads, 0, s>>>(data, n, scratch);
  exclusive_scan<W>(scratch, blocks, scratch + blocks, s);
  scan_add_kernel<W><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(data, n, scratch);
}

inline int64_t scan_scratch_elems(int64_t n) {
  int64_t tot = 0;
  while (n > kScanChunk) {
    n = (n + kScanChunk - 1) / kScanChunk;
    tot += n;
  }
  return tot + 1;
}

// ---- stable scatter --------------------------------------------------------------------------
// Each warp owns a contiguous run of keys; lanes take consecutive keys round by round, so
// (warp, round, lane) is memory order.  rank = keys with the same digit that come earlier.
template <class W, class KeyIn>
__global__ void __launch_bounds__(kRxThreads)
radix_scatter_kernel(const KeyIn* __restrict__ keys_in, const W* __restrict__ vals_in,
                     W* __restrict__ keys_out, W* __restrict__ vals_out, int64_t n, int shift,
                     const W* __restrict__ offsets, int64_t n_blocks) {
  __shared__ unsigned int warp_cnt[kRxWarps][256];
  __shared__ W gbase[256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kRxWarps * 256; i += kRxThreads) (&warp_cnt[0][0])[i] = 0;
  __syncthreads();

  const int64_t wbase = blockIdx.x * static_cast<int64_t>(kRxChunk) + warp * kRxWarpChunk;
  unsigned int rank[kRxRounds];
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int q = 0; q < kRxRounds; ++q) {
    const int64_t i = wbase + q * 32 + lane;
    const bool live = i < n;
    unsigned d = 256u + lane;  // dead lanes match nobody
    if (live) d = static_cast<unsigned>((static_cast<uint64_t>(keys_in[i]) >> shift) & 255u);
    const unsigned peers = __match_any_sync(0xffffffffu, d);
    const unsigned before = __popc(peers & lt_mask);
    unsigned prev = 0;
    if (live) prev = warp_cnt[warp][d];
    __syncwarp();
    if (live && before == 0) warp_cnt[warp][d] = prev + __popc(peers);
    __syncwarp();
    rank[q] = prev + before;
  }
  __syncthreads();
  {
    const int d = threadIdx.x;  // one thread per digit
    unsigned run = 0;
#pragma unroll
    for (int w = 0; w < kRxWarps; ++w) {
      const unsigned c = warp_cnt[w][d];
      warp_cnt[w][d] = run;
      run += c;
    }
    gbase[d] = offsets[d * n_blocks + blockIdx.x];
  }
  __syncthreads();
#pragma unroll
  for (int q = 0; q < kRxRounds; ++q) {
    const int64_t i = wbase + q * 32 + lane;
    if (i < n) {
      const W key = static_cast<W>(keys_in[i]);
      const unsigned d = static_cast<unsigned>((static_cast<uint64_t>(key) >> shift) & 255u);
      const W dst = gbase[d] + warp_cnt[warp][d] + rank[q];
      keys_out[dst] = key;
      vals_out[dst] = vals_in ? vals_in[i] : static_cast<W>(i);
    }
  }
}

// ---- column pointers from the sorted column ids -----------------------------------------------
template <class W, class P>
__global__ void csc_ptr_kernel(const W* __restrict__ sorted_cols, int64_t nnz, int64_t n_cols,
                               P* __restrict__ t_ptr) {
  const int64_t k = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (k > nnz) return;
  const int64_t prev = k > 0 ? static_cast<int64_t>(sorted_cols[k - 1]) : -1;
  const int64_t cur = k < nnz ? static_cast<int64_t>(sorted_cols[k]) : n_cols;
  for (int64_t c = prev + 1; c <= cur; ++c) t_ptr[c] = static_cast<P>(k);
}

// ---- gather values (optionally conjugated) and source rows ------------------------------------
template <class V, class I, class P, class W>
__global__ void csc_gather_kernel(const V* __restrict__ data, const P* __restrict__ ptr,
                                  int64_t n_rows, const W* __restrict__ src_pos, int64_t nnz,
                                  int conj, V* __restrict__ t_data, I* __restrict__ t_idx) {
  const int64_t k = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (k >= nnz) return;
  const int64_t j = static_cast<int64_t>(src_pos[k]);
  // last row r with ptr[r] <= j  (empty rows share their offset with the next row)
  int64_t lo = 0, hi = n_rows;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(ptr[mid + 1]) <= j)
      lo = mid + 1;
    else
      hi = mid;
  }
  V v = data[j];
  if (conj) v = vt<V>::conj(v);
  t_data[k] = v;
  t_idx[k] = static_cast<I>(lo);
}

template <class P>
__global__ void fill_zero_kernel(P* p, int64_t n) {
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i < n) p[i] = 0;
}

inline int64_t align256(int64_t b) { return (b + 255) / 256 * 256; }

inline bool wide_needed(int64_t n_cols, int64_t nnz) {
  return n_cols > 0x7fffffffLL || nnz > 0x7fffffffLL;
}

template <class W>
int64_t csr2csc_scratch_bytes(int64_t nnz) {
  const int64_t n_blocks = (nnz + kRxChunk - 1) / kRxChunk;
  const int64_t hist = 256 * n_blocks;
  return 4 * align256(nnz * sizeof(W)) + align256(hist * sizeof(W)) +
         align256(scan_scratch_elems(hist) * sizeof(W));
}

template <class V, class I, class P, class W>
int csr2csc_run(const void* data, const void* indices, const void* indptr, int64_t n_rows,
                int64_t n_cols, int64_t nnz, int conj, void* t_data, void* t_idx, void* t_ptr,
                void* scratch, int64_t scratch_bytes, cudaStream_t s) {
  if (csr2csc_scratch_bytes<W>(nnz) > scratch_bytes) return B2S_ERR_WORKSPACE;
  unsigned char* p = static_cast<unsigned char*>(scratch);
  W* keys[2];
  W* vals[2];
  keys[0] = reinterpret_cast<W*>(p); p += align256(nnz * sizeof(W));
  keys[1] = reinterpret_cast<W*>(p); p += align256(nnz * sizeof(W));
  vals[0] = reinterpret_cast<W*>(p); p += align256(nnz * sizeof(W));
  vals[1] = reinterpret_cast<W*>(p); p += align256(nnz * sizeof(W));
  const int64_t n_blocks = (nnz + kRxChunk - 1) / kRxChunk;
  const int64_t hist_n = 256 * n_blocks;
  W* hist = reinterpret_cast<W*>(p); p += align256(hist_n * sizeof(W));
  W* scan_ws = reinterpret_cast<W*>(p);

  int bits = 0;
  while (bits < 64 && ((n_cols - 1) >> bits) > 0) ++bits;
  int passes = (bits + 7) / 8;
  if (passes < 1) passes = 1;
  const unsigned grid = static_cast<unsigned>(n_blocks);
  int cur = 0;
  for (int pass = 0; pass < passes; ++pass) {
    const int shift = 8 * pass;
    if (pass == 0) {
      radix_hist_kernel<W, I><<<grid, kRxThreads, 0, s>>>(static_cast<const I*>(indices), nnz,
                                                          shift, hist, n_blocks);
      exclusive_scan<W>(hist, hist_n, scan_ws, s);
      radix_scatter_kernel<W, I><<<grid, kRxThreads, 0, s>>>(
          static_cast<const I*>(indices), nullptr, keys[0], vals[0], nnz, shift, hist, n_blocks);
      cur = 0;
    } else {
      radix_hist_kernel<W, W><<<grid, kRxThreads, 0, s>>>(keys[cur], nnz, shift, hist, n_blocks);
      exclusive_scan<W>(hist, hist_n, scan_ws, s);
      radix_scatter_kernel<W, W><<<grid, kRxThreads, 0, s>>>(
          keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], nnz, shift, hist, n_blocks);
      cur ^= 1;
    }
  }
  csc_ptr_kernel<W, P><<<static_cast<unsigned>((nnz + 1 + 255) / 256), 256, 0, s>>>(
      keys[cur], nnz, n_cols, static_cast<P*>(t_ptr));
  csc_gather_kernel<V, I, P, W><<<static_cast<unsigned>((nnz + 255) / 256), 256, 0, s>>>(
      static_cast<const V*>(data), static_cast<const P*>(indptr), n_rows, vals[cur], nnz, conj,
      static_cast<V*>(t_data), static_cast<I*>(t_idx));
  return launch_status();
}

// ---- column-panel layout ------------------------------------------------------------------------
// The non-zeros are stably sorted by panel id = col >> panel_shift (one radix pass), so the result
// is a stack of n_panels CSR matrices over the same rows, each touching only its own slice of x.
// Columns become panel-local int32; stacked row p * n_rows + r holds the entries of row r that
// fall into panel p, in their original order.
template <class V, class P, class W>
__global__ void panel_gather_kernel(const V* __restrict__ data, const P* __restrict__ ptr,
                                    int64_t n_rows, const W* __restrict__ sorted_cols,
                                    const W* __restrict__ src_pos, int64_t nnz, int panel_shift,
                                    V* __restrict__ p_data, int32_t* __restrict__ p_cols,
                                    int64_t* __restrict__ stacked_row, int global_cols) {
  const int64_t k = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (k >= nnz) return;
  const int64_t j = static_cast<int64_t>(src_pos[k]);
  const int64_t c = static_cast<int64_t>(sorted_cols[k]);
  int64_t lo = 0, hi = n_rows;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (static_cast<int64_t>(ptr[mid + 1]) <= j)
      lo = mid + 1;
    else
      hi = mid;
  }
  p_data[k] = data[j];
  p_cols[k] = static_cast<int32_t>(global_cols ? c : (c & ((int64_t{1} << panel_shift) - 1)));
  stacked_row[k] = (c >> panel_shift) * n_rows + lo;
}

template <class PP>
__global__ void panel_start_kernel(const PP* __restrict__ p_ptr, int64_t n_rows, int n_panels,
                                   int64_t* __restrict__ panel_start) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p <= n_panels) panel_start[p] = static_cast<int64_t>(p_ptr[p * n_rows]);
}

// ---- dropping the empty rows of the stack ------------------------------------------------------
// Most rows have entries in only some panels (a row with one entry is empty in all panels but
// one).  pos[q] = 1 if stacked row q has entries; after an exclusive scan pos[q] is its index
// among the non-empty rows.
template <class PP>
__global__ void panel_flag_kernel(const PP* __restrict__ p_ptr, int64_t n_stacked,
                                  uint32_t* __restrict__ pos) {
  const int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (q < n_stacked) pos[q] = p_ptr[q + 1] > p_ptr[q] ? 1u : 0u;
}

// subpos[q] = index of stacked row q among the non-empty ones, or -1; the last thread also
// stores the number of non-empty rows
template <class PP>
__global__ void panel_subpos_kernel(const PP* __restrict__ p_ptr, int64_t n_stacked,
                                    const uint32_t* __restrict__ pos,
                                    int32_t* __restrict__ subpos, int64_t* __restrict__ count) {
  const int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (q >= n_stacked) return;
  const bool full = p_ptr[q + 1] > p_ptr[q];
  subpos[q] = full ? static_cast<int32_t>(pos[q]) : -1;
  if (q == n_stacked - 1) *count = static_cast<int64_t>(pos[q]) + (full ? 1 : 0);
}

// row pointers of the non-empty rows only
template <class PP>
__global__ void panel_compact_ptr_kernel(const PP* __restrict__ p_ptr, int64_t n_stacked,
                                         const int32_t* __restrict__ subpos, int64_t n_compact,
                                         PP* __restrict__ c_ptr) {
  const int64_t q = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (q >= n_stacked) return;
  const int32_t c = subpos[q];
  if (c >= 0) c_ptr[c] = p_ptr[q];
  if (q == n_stacked - 1) c_ptr[n_compact] = p_ptr[n_stacked];
}

template <class W>
int64_t panel_scratch_bytes(int64_t nnz) {
  const int64_t n_blocks = (nnz + kRxChunk - 1) / kRxChunk;
  const int64_t hist = 256 * n_blocks;
  return 2 * align256(nnz * sizeof(W)) + align256(hist * sizeof(W)) +
         align256(scan_scratch_elems(hist) * sizeof(W)) + align256(nnz * sizeof(int64_t));
}

template <class V, class I, class P, class PP, class W>
int panel_build_run(const void* data, const void* indices, const void* indptr, int64_t n_rows,
                    int64_t nnz, int n_panels, int panel_shift, void* p_data, int32_t* p_cols,
                    void* p_ptr, int64_t* panel_start, void* scratch, int64_t scratch_bytes,
                    cudaStream_t s, int global_cols) {
  if (panel_scratch_bytes<W>(nnz) > scratch_bytes) return B2S_ERR_WORKSPACE;
  unsigned char* p = static_cast<unsigned char*>(scratch);
  W* keys = reinterpret_cast<W*>(p); p += align256(nnz * sizeof(W));
  W* vals = reinterpret_cast<W*>(p); p += align256(nnz * sizeof(W));
  const int64_t n_blocks = (nnz + kRxChunk - 1) / kRxChunk;
  const int64_t hist_n = 256 * n_blocks;
  W* hist = reinterpret_cast<W*>(p); p += align256(hist_n * sizeof(W));
  W* scan_ws = reinterpret_cast<W*>(p); p += align256(scan_scratch_elems(hist_n) * sizeof(W));
  int64_t* stacked = reinterpret_cast<int64_t*>(p);
  const unsigned grid = static_cast<unsigned>(n_blocks);
  radix_hist_kernel<W, I><<<grid, kRxThreads, 0, s>>>(static_cast<const I*>(indices), nnz,
                                                      panel_shift, hist, n_blocks);
  exclusive_scan<W>(hist, hist_n, scan_ws, s);
  radix_scatter_kernel<W, I><<<grid, kRxThreads, 0, s>>>(static_cast<const I*>(indices), nullptr,
                                                         keys, vals, nnz, panel_shift, hist,
                                                         n_blocks);
  panel_gather_kernel<V, P, W><<<static_cast<unsigned>((nnz + 255) / 256), 256, 0, s>>>(
      static_cast<const V*>(data), static_cast<const P*>(indptr), n_rows, keys, vals, nnz,
      panel_shift, static_cast<V*>(p_data), p_cols, stacked, global_cols);
  csc_ptr_kernel<int64_t, PP><<<static_cast<unsigned>((nnz + 1 + 255) / 256), 256, 0, s>>>(
      stacked, nnz, n_rows * n_panels, static_cast<PP*>(p_ptr));
  panel_start_kernel<PP><<<(n_panels + 1 + 63) / 64, 64, 0, s>>>(static_cast<const PP*>(p_ptr),
                                                                 n_rows, n_panels, panel_start);
  return launch_status();
}

}  // namespace b2s

extern "C" int64_t b2s_panel_compact_bytes(int64_t n_stacked) {
  if (n_stacked <= 0) return 256;
  return b2s::align256(n_stacked * sizeof(uint32_t)) +
         b2s::align256(b2s::scan_scratch_elems(n_stacked) * sizeof(uint32_t));
}

extern "C" int b2s_panel_compact(const void* p_ptr_dev, int p_ptr_type, int64_t n_stacked,
                                 int32_t* subpos_dev, int64_t* count_dev, void* c_ptr_dev,
                                 int64_t n_compact, void* scratch_dev, int64_t scratch_bytes,
                                 b2s_stream stream) {
  if (!p_ptr_dev || !subpos_dev || n_stacked <= 0 || n_stacked > 0x7fffffffLL) return B2S_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>((n_stacked + 255) / 256);
  if (c_ptr_dev == nullptr) {
    // phase 1: positions of the non-empty rows and their number
    if (!count_dev || !scratch_dev) return B2S_ERR_ARG;
    if (b2s_panel_compact_bytes(n_stacked) > scratch_bytes) return B2S_ERR_WORKSPACE;
    uint32_t* pos = static_cast<uint32_t*>(scratch_dev);
    uint32_t* scan_ws = reinterpret_cast<uint32_t*>(static_cast<unsigned char*>(scratch_dev) +
                                                    b2s::align256(n_stacked * sizeof(uint32_t)));
    B2S_DISPATCH_I(p_ptr_type, PP, {
      (b2s::panel_flag_kernel<PP><<<grid, 256, 0, s>>>(static_cast<const PP*>(p_ptr_dev),
                                                       n_stacked, pos));
      b2s::exclusive_scan<uint32_t>(pos, n_stacked, scan_ws, s);
      (b2s::panel_subpos_kernel<PP><<<grid, 256, 0, s>>>(static_cast<const PP*>(p_ptr_dev),
                                                         n_stacked, pos, subpos_dev, count_dev));
    });
    return b2s::launch_status();
  }
  // phase 2: the compacted row pointers (n_compact + 1 entries)
  if (n_compact < 0) return B2S_ERR_ARG;
  B2S_DISPATCH_I(p_ptr_type, PP, {
    (b2s::panel_compact_ptr_kernel<PP><<<grid, 256, 0, s>>>(
        static_cast<const PP*>(p_ptr_dev), n_stacked, subpos_dev, n_compact,
        static_cast<PP*>(c_ptr_dev)));
  });
  return b2s::launch_status();
}

extern "C" int64_t b2s_panel_bytes(int64_t n_cols, int64_t nnz) {
  if (nnz <= 0) return 256;
  return b2s::wide_needed(n_cols, nnz) ? b2s::panel_scratch_bytes<uint64_t>(nnz)
                                       : b2s::panel_scratch_bytes<uint32_t>(nnz);
}

static int panel_build_any(int val_type, int idx_type, int ptr_type, const void* data_dev,
                           const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                           int64_t n_cols, int64_t nnz, int n_panels, int panel_shift,
                           void* p_data_dev, int32_t* p_cols_dev, void* p_ptr_dev,
                           int p_ptr_type, int64_t* panel_start_dev, void* scratch_dev,
                           int64_t scratch_bytes, b2s_stream stream, int global_cols) {
  if (n_rows <= 0 || n_cols <= 0 || nnz <= 0) return B2S_ERR_ARG;
  if (global_cols && n_cols > 0x7fffffffLL) return B2S_ERR_RANGE;
  if (n_panels < 1 || n_panels > 256 || panel_shift < 1 || panel_shift > 31) return B2S_ERR_ARG;
  if (((n_cols - 1) >> panel_shift) >= n_panels) return B2S_ERR_ARG;
  if (p_ptr_type == B2S_I32 && nnz > 0x7fffffffLL) return B2S_ERR_RANGE;
  if (!data_dev || !indices_dev || !indptr_dev || !p_data_dev || !p_cols_dev || !p_ptr_dev ||
      !panel_start_dev || !scratch_dev)
    return B2S_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool wide = b2s::wide_needed(n_cols, nnz);
  B2S_DISPATCH_MOVE(val_type, B2S_DISPATCH_I(idx_type, I, B2S_DISPATCH_I(ptr_type, P,
      B2S_DISPATCH_I(p_ptr_type, PP, {
    if (wide)
      return (b2s::panel_build_run<V, I, P, PP, uint64_t>(
          data_dev, indices_dev, indptr_dev, n_rows, nnz, n_panels, panel_shift, p_data_dev,
          p_cols_dev, p_ptr_dev, panel_start_dev, scratch_dev, scratch_bytes, s, global_cols));
    return (b2s::panel_build_run<V, I, P, PP, uint32_t>(
        data_dev, indices_dev, indptr_dev, n_rows, nnz, n_panels, panel_shift, p_data_dev,
        p_cols_dev, p_ptr_dev, panel_start_dev, scratch_dev, scratch_bytes, s, global_cols));
  }))));
  return B2S_ERR_DTYPE;
}

extern "C" int b2s_panel_build(int val_type, int idx_type, int ptr_type, const void* data_dev,
                               const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                               int64_t n_cols, int64_t nnz, int n_panels, int panel_shift,
                               void* p_data_dev, int32_t* p_cols_dev, void* p_ptr_dev,
                               int p_ptr_type, int64_t* panel_start_dev, void* scratch_dev,
                               int64_t scratch_bytes, b2s_stream stream) {
  return panel_build_any(val_type, idx_type, ptr_type, data_dev, indices_dev, indptr_dev, n_rows,
                         n_cols, nnz, n_panels, panel_shift, p_data_dev, p_cols_dev, p_ptr_dev,
                         p_ptr_type, panel_start_dev, scratch_dev, scratch_bytes, stream, 0);
}

extern "C" int b2s_panel_build_global(int val_type, int idx_type, int ptr_type,
                                      const void* data_dev, const void* indices_dev,
                                      const void* indptr_dev, int64_t n_rows, int64_t n_cols,
                                      int64_t nnz, int n_panels, int panel_shift,
                                      void* p_data_dev, int32_t* p_cols_dev, void* p_ptr_dev,
                                      int p_ptr_type, int64_t* panel_start_dev, void* scratch_dev,
                                      int64_t scratch_bytes, b2s_stream stream) {
  return panel_build_any(val_type, idx_type, ptr_type, data_dev, indices_dev, indptr_dev, n_rows,
                         n_cols, nnz, n_panels, panel_shift, p_data_dev, p_cols_dev, p_ptr_dev,
                         p_ptr_type, panel_start_dev, scratch_dev, scratch_bytes, stream, 1);
}

extern "C" int64_t b2s_csr2csc_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz) {
  (void)n_rows;
  if (nnz <= 0) return 256;
  return b2s::wide_needed(n_cols, nnz) ? b2s::csr2csc_scratch_bytes<uint64_t>(nnz)
                                       : b2s::csr2csc_scratch_bytes<uint32_t>(nnz);
}

extern "C" int b2s_csr2csc(int val_type, int idx_type, int ptr_type, const void* data_dev,
                           const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                           int64_t n_cols, int64_t nnz, int conj, void* t_data_dev,
                           void* t_indices_dev, void* t_indptr_dev, void* scratch_dev,
                           int64_t scratch_bytes, b2s_stream stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return B2S_ERR_ARG;
  if (!t_indptr_dev || !indptr_dev) return B2S_ERR_ARG;
  if (idx_type == B2S_I32 && n_rows > 0x7fffffffLL) return B2S_ERR_RANGE;
  if (ptr_type == B2S_I32 && nnz > 0x7fffffffLL) return B2S_ERR_RANGE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (nnz == 0) {
    B2S_DISPATCH_I(ptr_type, P, {
      (b2s::fill_zero_kernel<P><<<static_cast<unsigned>((n_cols + 1 + 255) / 256), 256, 0, s>>>(
          static_cast<P*>(t_indptr_dev), n_cols + 1));
    });
    return b2s::launch_status();
  }
  if (!data_dev || !indices_dev || !t_data_dev || !t_indices_dev || !scratch_dev)
    return B2S_ERR_ARG;
  const bool wide = b2s::wide_needed(n_cols, nnz);
  B2S_DISPATCH_MOVE(val_type, B2S_DISPATCH_I(idx_type, I, B2S_DISPATCH_I(ptr_type, P, {
    if (wide)
      return (b2s::csr2csc_run<V, I, P, uint64_t>(data_dev, indices_dev, indptr_dev, n_rows,
                                                  n_cols, nnz, conj, t_data_dev, t_indices_dev,
                                                  t_indptr_dev, scratch_dev, scratch_bytes, s));
    return (b2s::csr2csc_run<V, I, P, uint32_t>(data_dev, indices_dev, indptr_dev, n_rows,
                                                n_cols, nnz, conj, t_data_dev, t_indices_dev,
                                                t_indptr_dev, scratch_dev, scratch_bytes, s));
  })));
  return B2S_ERR_DTYPE;
}

// =================================================================================================
// Dense transpose (column-major B / C around the row-major SpMM kernel)
// =================================================================================================
namespace b2s {

// dst[c * ld_dst + r] = src[r * ld_src + c] for a rows x cols matrix.  32 x 32 tiles through
// padded shared memory: 32 consecutive elements of a source row are read by one warp and 32
// consecutive elements of a destination row are written by one warp.  One-dimensional grid over
// the tiles (tile rows can exceed the 65,535 limit of the other grid dimensions).
template <class T>
__global__ void __launch_bounds__(256)
    dense_transpose_kernel(const T* __restrict__ src, int64_t rows, int64_t cols, int64_t ld_src,
                           T* __restrict__ dst, int64_t ld_dst, int64_t tiles_x) {
  __shared__ T tile[32][33];
  const int64_t t = blockIdx.x;
  const int64_t r0 = (t / tiles_x) * 32;
  const int64_t c0 = (t % tiles_x) * 32;
  const int tx = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;  // 0..7
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    const int64_t r = r0 + ty + k, c = c0 + tx;
    if (r < rows && c < cols) tile[ty + k][tx] = src[r * ld_src + c];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < 32; k += 8) {
    const int64_t c = c0 + ty + k, r = r0 + tx;
    if (r < rows && c < cols) dst[c * ld_dst + r] = tile[tx][ty + k];
  }
}

template <class T>
int dense_transpose_launch(const void* src, int64_t rows, int64_t cols, int64_t ld_src, void* dst,
                           int64_t ld_dst, cudaStream_t s) {
  const int64_t tiles_x = (cols + 31) / 32, tiles_y = (rows + 31) / 32;
  const int64_t tiles = tiles_x * tiles_y;
  if (tiles > 0x7fffffffLL) return B2S_ERR_RANGE;
  dense_transpose_kernel<T><<<static_cast<unsigned>(tiles), 256, 0, s>>>(
      static_cast<const T*>(src), rows, cols, ld_src, static_cast<T*>(dst), ld_dst, tiles_x);
  return launch_status();
}

}  // namespace b2s

extern "C" int b2s_dense_transpose(int elem_bytes, const void* src_dev, int64_t rows, int64_t cols,
                                   int64_t ld_src, void* dst_dev, int64_t ld_dst,
                                   b2s_stream stream) {
  if (rows < 0 || cols < 0 || ld_src < cols || ld_dst < rows) return B2S_ERR_ARG;
  if (rows == 0 || cols == 0) return B2S_OK;
  if (!src_dev || !dst_dev) return B2S_ERR_ARG;
  if (elem_bytes != 2 && elem_bytes != 4 && elem_bytes != 8 && elem_bytes != 16)
    return B2S_ERR_DTYPE;
  const uintptr_t both =
      reinterpret_cast<uintptr_t>(src_dev) | reinterpret_cast<uintptr_t>(dst_dev);
  if (both % static_cast<uintptr_t>(elem_bytes)) return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (elem_bytes == 2)
    return b2s::dense_transpose_launch<uint16_t>(src_dev, rows, cols, ld_src, dst_dev, ld_dst, s);
  if (elem_bytes == 4)
    return b2s::dense_transpose_launch<uint32_t>(src_dev, rows, cols, ld_src, dst_dev, ld_dst, s);
  if (elem_bytes == 8)
    return b2s::dense_transpose_launch<uint64_t>(src_dev, rows, cols, ld_src, dst_dev, ld_dst, s);
  return b2s::dense_transpose_launch<uint4>(src_dev, rows, cols, ld_src, dst_dev, ld_dst, s);
}
