// CSR SpMV for sm_100a: y = alpha * A x + beta * y_in.
//
// One CTA per merge-path tile.  A tile's col / val range is brought into shared memory by two
// bulk asynchronous copies (TMA engine) that complete on an mbarrier; the products val * x[col]
// overwrite the staged values; rows are then reduced out of shared memory with a strategy chosen
// from the row lengths inside the tile:
//   1. vector-per-row : a group of T = 1..32 lanes per row, T the power of two that covers the
//                       tile's mean row length, butterfly (__shfl_xor) reduction;
//   2. warp-per-row   : rows longer than 8*T (up to 1024 entries) are queued and taken by whole
//                       warps;
//   3. CTA-per-row    : longer pieces are reduced by the whole CTA; a row that crosses tile
//                       borders leaves one partial sum per tile in `carry`, and a second kernel
//                       adds those partials to the row in ascending tile order.
// No floating-point atomics: every sum has a fixed shape, so results repeat bit for bit.
#include "b2s_tile.cuh"

namespace b2s {

template <class V, class I>
struct SpmvCfg {
  static constexpr int THREADS = 256;
  static constexpr int ITEMS = 2048;
};

constexpr int kWarpRowMax = 1024;   // longest in-tile row piece a single warp takes
constexpr int kQueue2Cap = 512;     // queue of warp-per-row pieces (each longer than 8)
constexpr int kQueue3Cap = 8;       // queue of CTA-per-row pieces (each longer than 1024)

template <int THREADS, int ITEMS, class V, class I>
constexpr size_t spmv_smem_bytes() {
  return 16                                   // mbarrier
         + sizeof(int) * (ITEMS + 4)          // row_end (+ padding to keep 16-byte alignment)
         + sizeof(I) * ITEMS + 16             // staged columns
         + sizeof(V) * ITEMS + 16             // staged values -> products
         + sizeof(int) * (kQueue2Cap + kQueue3Cap + 4)  // queues + counters
         + sizeof(V) * (THREADS / 32);        // per-warp partials
}

template <class V, class I, class P, int THREADS, int ITEMS>
__global__ void __launch_bounds__(THREADS)
spmv_tile_kernel(const V* __restrict__ val, const I* __restrict__ col, const P* __restrict__ ptr,
                 const V* __restrict__ x, const V* y_in, V* y, V* __restrict__ carry,
                 const int64_t* __restrict__ tile_row, int64_t n_rows, int64_t nnz, V alpha,
                 V beta, int has_beta, int32_t* status) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  int* row_end = reinterpret_cast<int*>(smem + 16);
  unsigned char* col_buf = smem + 16 + sizeof(int) * (ITEMS + 4);
  unsigned char* val_buf = col_buf + sizeof(I) * ITEMS + 16;
  int* queue2 = reinterpret_cast<int*>(val_buf + sizeof(V) * ITEMS + 16);
  int* queue3 = queue2 + kQueue2Cap;
  int* qcount = queue3 + kQueue3Cap;  // [0] = n2, [1] = n3
  V* wpart = reinterpret_cast<V*>(qcount + 4);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  // an earlier CTA already gave up on a copy: do not queue more waits behind it
  if (status && *reinterpret_cast<volatile int32_t*>(status) != 0) return;
  const int64_t t = blockIdx.x;
  const TileCoord tc = tile_coord(tile_row, t, ITEMS, n_rows + nnz);
  const int n_nz = static_cast<int>(tc.j1 - tc.j0);
  const int n_end = static_cast<int>(tc.r1 - tc.r0);  // rows that end in this tile

  const I* gcol = col + tc.j0;
  const V* gval = val + tc.j0;
  const Staged<I> sc = stage_layout<I>(col_buf, gcol, n_nz);
  const Staged<V> sv = stage_layout<V>(val_buf, gval, n_nz);
  const uint32_t tx = stage_bytes(sc) + stage_bytes(sv);

  if (tid == 0) {
    qcount[0] = 0;
    qcount[1] = 0;
    if (tx) mbar_init(bar, 1);
  }
  __syncthreads();
  if (tid == 0 && tx) {
    const uint64_t pol = policy_evict_first();  // col / val are read once
    mbar_expect_tx(bar, tx);
    stage_issue(sc, gcol, bar, pol);
    stage_issue(sv, gval, bar, pol);
  }
  // while the copies fly: ragged edges and the row ends of this tile
  stage_edges(sc, gcol, n_nz, tid, THREADS);
  stage_edges(sv, gval, n_nz, tid, THREADS);
  for (int k = tid; k < n_end; k += THREADS)
    row_end[k] = static_cast<int>(static_cast<int64_t>(ptr[tc.r0 + 1 + k]) - tc.j0);
  if (tid == 0) row_end[n_end] = n_nz;  // the open row runs to the end of the tile
  if (tx) {
    if (!mbar_wait(bar, 0)) {
      if (status) atomicOr(status, 1 << B2S_ERR_TIMEOUT);
      mbar_wait(bar, 0);  // second bounded wait: do not leave with a copy in flight
    }
  }
  __syncthreads();

  // products, in place
  {
    const I* scol = sc.s;
    V* sval = sv.s;
#pragma unroll 4
    for (int i = tid; i < n_nz; i += THREADS) {
      const int64_t c = static_cast<int64_t>(scol[i]);
      sval[i] = sval[i] * ldg_val(x + c);
    }
  }
  __syncthreads();

  const V* prod = sv.s;
  const bool open_row = tc.r1 < n_rows;
  const int n_seg = n_end + 1;  // row pieces in the tile; the last one is the open row
  // lanes per row: power of two covering the mean piece length
  int T = 1;
  {
    const int mean = (n_nz + n_seg - 1) / n_seg;
    while (T < mean && T < 32) T <<= 1;
  }
  const int p1max = (T == 32) ? kWarpRowMax : 8 * T;

  // ---- strategy 1: vector-per-row ---------------------------------------------------------
  {
    const int sub = tid & (T - 1);
    const int grp = tid / T;
    const int n_grp = THREADS / T;
    for (int kb = 0; kb < n_seg; kb += n_grp) {  // uniform trip count: shuffles stay converged
      const int k = kb + grp;
      const bool live = k < n_seg;
      int s = 0, e = 0;
      if (live) {
        s = k ? row_end[k - 1] : 0;
        e = row_end[k];
      }
      const int len = e - s;
      V acc = vt<V>::zero();
      if (len <= p1max) {
        for (int i = s + sub; i < e; i += T) acc = acc + prod[i];
      } else if (sub == 0) {
        if (len <= kWarpRowMax) {
          const int q = atomicAdd(&qcount[0], 1);
          if (q < kQueue2Cap) queue2[q] = k;
        } else {
          const int q = atomicAdd(&qcount[1], 1);
          if (q < kQueue3Cap) queue3[q] = k;
        }
      }
      acc = group_sum(acc, T);
      if (live && sub == 0 && len <= p1max) {
        if (k < n_end) {
          const int64_t r = tc.r0 + k;
          y[r] = axpby(alpha, acc, has_beta != 0, beta, y_in + r);
        } else if (open_row) {
          carry[t] = acc;
        }
      }
    }
  }
  __syncthreads();

  // ---- strategy 2: warp-per-row -----------------------------------------------------------
  const int n2 = min(qcount[0], kQueue2Cap);
  for (int q = warp; q < n2; q += THREADS / 32) {
    const int k = queue2[q];
    const int s = k ? row_end[k - 1] : 0;
    const int e = row_end[k];
    V acc = vt<V>::zero();
    for (int i = s + lane; i < e; i += 32) acc = acc + prod[i];
    acc = group_sum(acc, 32);
    if (lane == 0) {
      if (k < n_end) {
        const int64_t r = tc.r0 + k;
        y[r] = axpby(alpha, acc, has_beta != 0, beta, y_in + r);
      } else if (open_row) {
        carry[t] = acc;
      }
    }
  }

  // ---- strategy 3: CTA-per-row ------------------------------------------------------------
  const int n3 = min(qcount[1], kQueue3Cap);
  for (int q = 0; q < n3; ++q) {
    const int k = queue3[q];
    const int s = k ? row_end[k - 1] : 0;
    const int e = row_end[k];
    V acc = vt<V>::zero();
    for (int i = s + tid; i < e; i += THREADS) acc = acc + prod[i];
    acc = group_sum(acc, 32);
    if (lane == 0) wpart[warp] = acc;
    __syncthreads();
    if (tid == 0) {
      V tot = wpart[0];
#pragma unroll
      for (int w = 1; w < THREADS / 32; ++w) tot = tot + wpart[w];
      if (k < n_end) {
        const int64_t r = tc.r0 + k;
        y[r] = axpby(alpha, tot, has_beta != 0, beta, y_in + r);
      } else if (open_row) {
        carry[t] = tot;
      }
    }
    __syncthreads();
  }
}

// Adds to each row that began in an earlier tile the partial sums those tiles left behind,
// oldest tile first.  Only the first row of a tile can have such partials.
template <class V>
__global__ void spmv_fixup_kernel(V* y, const V* __restrict__ carry,
                                  const int64_t* __restrict__ tile_row, int64_t n_tiles,
                                  V alpha) {
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t < 1 || t >= n_tiles) return;
  const int64_t r = tile_row[t];
  if (tile_row[t + 1] <= r) return;  // row r does not end in tile t
  int64_t u0 = t - 1;
  while (u0 >= 1 && tile_row[u0] == r) --u0;  // tile u0-1 also ended with row r open
  V s = carry[u0];
  for (int64_t u = u0 + 1; u < t; ++u) s = s + carry[u];
  y[r] = y[r] + alpha * s;
}

template <class V, class I, class P>
int spmv_launch(const void* data, const void* indices, const void* indptr, int64_t n_rows,
                int64_t nnz, const void* x, const void* y_in, void* y, const void* alpha,
                const void* beta, const int64_t* tile_row, void* carry, int32_t* status,
                cudaStream_t stream) {
  using Cfg = SpmvCfg<V, I>;
  constexpr int THREADS = Cfg::THREADS, ITEMS = Cfg::ITEMS;
  const int64_t n_tiles = b2s_tile_count(n_rows, nnz, ITEMS);
  if (n_tiles == 0) return B2S_OK;
  if (n_tiles > 0x7fffffffLL) return B2S_ERR_RANGE;
  const V a = *static_cast<const V*>(alpha);
  const V b = *static_cast<const V*>(beta);
  const int has_beta = vt<V>::is_zero(b) ? 0 : 1;
  if (has_beta && y_in == nullptr) return B2S_ERR_ARG;
  auto kern = spmv_tile_kernel<V, I, P, THREADS, ITEMS>;
  constexpr size_t smem = spmv_smem_bytes<THREADS, ITEMS, V, I>();
  ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem);
  kern<<<static_cast<unsigned>(n_tiles), THREADS, smem, stream>>>(
      static_cast<const V*>(data), static_cast<const I*>(indices),
      static_cast<const P*>(indptr), static_cast<const V*>(x), static_cast<const V*>(y_in),
      static_cast<V*>(y), static_cast<V*>(carry), tile_row, n_rows, nnz, a, b, has_beta, status);
  if (n_tiles > 1) {
    const int fb = 256;
    spmv_fixup_kernel<V><<<static_cast<unsigned>((n_tiles + fb - 1) / fb), fb, 0, stream>>>(
        static_cast<V*>(y), static_cast<const V*>(carry), tile_row, n_tiles, a);
  }
  return launch_status();
}

}  // namespace b2s

extern "C" int b2s_spmv_tile_items(int val_type, int idx_type) {
  (void)val_type;
  (void)idx_type;
  return b2s::SpmvCfg<float, int32_t>::ITEMS;
}

extern "C" int b2s_spmv_csr(int val_type, int idx_type, int ptr_type, const void* data_dev,
                            const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                            int64_t n_cols, int64_t nnz, const void* x_dev, const void* y_in_dev,
                            void* y_dev, const void* alpha, const void* beta,
                            const int64_t* tile_row_dev, void* carry_dev, int32_t* status_dev,
                            b2s_stream stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0 || !alpha || !beta) return B2S_ERR_ARG;
  if (n_rows == 0) return B2S_OK;
  if (!indptr_dev || !y_dev || !tile_row_dev || !carry_dev) return B2S_ERR_ARG;
  if (nnz > 0 && (!data_dev || !indices_dev || !x_dev)) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(data_dev) & m) || (reinterpret_cast<uintptr_t>(x_dev) & m) ||
      (reinterpret_cast<uintptr_t>(y_dev) & m) || (reinterpret_cast<uintptr_t>(y_in_dev) & m) ||
      (reinterpret_cast<uintptr_t>(carry_dev) & m))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_V(val_type, B2S_DISPATCH_I(idx_type, I, B2S_DISPATCH_I(ptr_type, P, {
    return (b2s::spmv_launch<V, I, P>(data_dev, indices_dev, indptr_dev, n_rows, nnz, x_dev,
                                      y_in_dev, y_dev, alpha, beta, tile_row_dev, carry_dev,
                                      status_dev, s));
  })));
  return B2S_ERR_DTYPE;
}
