// CSR SpMV for sm_100a: y = alpha * A x + beta * y_in.
//
// One CTA per merge-path tile (b2s_tile_plan).  The tile's col / val range is read straight from
// global memory, coalesced, a batch of independent loads per thread, followed by the gathers of x;
// the products go to shared memory.  The row pieces of the tile are then binned by length and
// reduced out of shared memory:
//   <= 8 entries   one thread per row, serial sum;
//   9 .. 64        vector-per-row: 8 lanes per row, butterfly (__shfl_xor) reduction;
//   65 .. 1024     warp-per-row, 32-lane butterfly;
//   longer         the whole CTA; a row that crosses tile borders leaves one partial sum per
//                  tile in `carry`, and a second kernel adds those partials to the row in
//                  ascending tile order.
// Row sums are staged in shared memory and written with a coalesced alpha / beta epilogue.
// No floating-point atomics: every sum has a fixed shape, so results repeat bit for bit.
//
// Column-panel layout (b2s_spmv_panels): the same kernel runs over a stack of CSR matrices, one
// per panel of columns, with panel-local int32 columns; partial results per (panel, row) are
// added in ascending panel order by panel_combine_kernel.
//
// B2S_SPMV_DIRECT=0 selects the earlier variant that stages col / val with cp.async.bulk and an
// mbarrier; it is kept for comparison (measured slower: the bulk-copy fills and the re-reads of
// shared memory load the same L1 data pipe the gathers need).
#include <mutex>

#include "b2s_tile.cuh"

namespace b2s {

#ifndef B2S_SPMV_PERSISTENT
#define B2S_SPMV_PERSISTENT 0  // 1: one CTA per resident slot walks the tiles (see the kernel)
#endif
#ifndef B2S_SPMV_THREADS
#define B2S_SPMV_THREADS 128
#endif
#ifndef B2S_SPMV_ITEMS
#define B2S_SPMV_ITEMS 1024
#endif
#ifndef B2S_SPMV_DIRECT
#define B2S_SPMV_DIRECT 1  // 1: col / val straight from global memory; 0: staged by bulk copies
#endif
#ifndef B2S_SPMV_PREFETCH_AHEAD
#define B2S_SPMV_PREFETCH_AHEAD 0  // tiles ahead whose col / val are prefetched into L2 (0 = off)
#endif
#ifndef B2S_SPMV_UNROLL
#define B2S_SPMV_UNROLL 8
#endif

template <class V, class I>
struct SpmvCfg {
  static constexpr int THREADS = B2S_SPMV_THREADS;
  static constexpr int ITEMS = B2S_SPMV_ITEMS;
};

#ifdef B2S_PHASES
__device__ unsigned long long g_phase_cycles[8];
__device__ unsigned long long g_s1_by_T[16];
#define B2S_TICK(n)                                                             \
  do {                                                                          \
    if (threadIdx.x == 0) {                                                     \
      const long long now_ = clock64();                                         \
      atomicAdd(&g_phase_cycles[n], static_cast<unsigned long long>(now_ - tick_)); \
      tick_ = now_;                                                             \
    }                                                                           \
  } while (0)
#else
#define B2S_TICK(n)
#endif

static_assert(B2S_SPMV_ITEMS <= 4096, "queue capacities below assume at most 4096 items per tile");
constexpr int kSpmvUnroll = B2S_SPMV_UNROLL;  // gathers in flight per thread
constexpr int kThreadRowMax = 8;    // longest in-tile row piece one thread sums serially
constexpr int kGroupRowMax = 64;    // longest piece a group of 8 lanes takes
constexpr int kWarpRowMax = 1024;   // longest piece a single warp takes
constexpr int kQueueACap = 512;     // pieces of 9..64 entries (at most ITEMS / 9)
constexpr int kQueueBCap = 64;      // pieces of 65..1024 entries (at most ITEMS / 65)
constexpr int kQueueCCap = 8;       // longer pieces (at most ITEMS / 1025 + 1)

template <int THREADS, int ITEMS, class V, class I>
constexpr size_t spmv_smem_bytes() {
  return 16                                   // mbarrier
         + sizeof(int) * (ITEMS + 4)          // row_end (+ padding to keep 16-byte alignment)
         + (B2S_SPMV_DIRECT ? 0 : sizeof(I) * ITEMS + 16)  // staged columns
         + sizeof(V) * ITEMS + 32             // staged values -> products, then row sums
         + sizeof(int) * (kQueueACap + kQueueBCap + kQueueCCap + 4)  // queues + counters
         + sizeof(V) * (THREADS / 32);        // per-warp partials
}

// CTAs per SM the register allocation aims at.  12 x 128 threads (<= 42 registers) measured 13 %
// faster than the 10 the compiler settles on by itself (more gathers in flight); 16-byte values
// and 8-byte column indices need more registers and would spill at that limit.
template <class V, class I, int THREADS>
constexpr int spmv_min_blocks() {
#ifdef B2S_SPMV_MINBLOCKS
  return B2S_SPMV_MINBLOCKS;
#else
  constexpr int want = (sizeof(V) <= 8 && sizeof(I) == 4) ? 12 : (sizeof(V) <= 8 ? 10 : 8);
  constexpr int fit = 2048 / THREADS;  // resident threads per SM
  return want < fit ? want : fit;
#endif
}

template <class V, class I, class P, int THREADS, int ITEMS>
__global__ void __launch_bounds__(THREADS, spmv_min_blocks<V, I, THREADS>())
spmv_tile_kernel(const V* __restrict__ val, const I* __restrict__ col, const P* __restrict__ ptr,
                 const V* __restrict__ x, const V* y_in, V* y, V* __restrict__ carry,
                 const int64_t* __restrict__ tile_row, int64_t n_rows, int64_t nnz, V alpha,
                 V beta, int has_beta, int gather_policy, int32_t* status,
                 const int64_t* __restrict__ panel_start, int n_panels, int panel_shift) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  int* row_end = reinterpret_cast<int*>(smem + 16);
  unsigned char* col_buf = smem + 16 + sizeof(int) * (ITEMS + 4);
  unsigned char* val_buf = col_buf + (B2S_SPMV_DIRECT ? 0 : sizeof(I) * ITEMS + 16);
  int* queueA = reinterpret_cast<int*>(val_buf + sizeof(V) * ITEMS + 32);
  int* queueB = queueA + kQueueACap;
  int* queueC = queueB + kQueueBCap;
  int* qcount = queueC + kQueueCCap;  // number of entries in queues A, B, C
  V* wpart = reinterpret_cast<V*>(qcount + 4);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
#ifdef B2S_PHASES
  long long tick_ = clock64();
#endif
  // an earlier CTA already gave up on a copy: do not queue more waits behind it
  if (status && *reinterpret_cast<volatile int32_t*>(status) != 0) return;
#if B2S_SPMV_PERSISTENT
  // one CTA per slot of the GPU walks the tiles blockIdx.x, blockIdx.x + gridDim.x, ...: the
  // CTAs resident at any time still cover a contiguous window of tiles (the x slice of a panel
  // stays the one in L2), no CTA is launched or retired between tiles, and the plan entries of
  // the next tile are requested while the current one is multiplied
  const int64_t n_tiles_all = (n_rows + nnz + ITEMS - 1) / ITEMS;
  int64_t next_r0 = tile_row[blockIdx.x], next_r1 = tile_row[blockIdx.x + 1];
  for (int64_t t = blockIdx.x; t < n_tiles_all; t += gridDim.x) {
  const TileCoord tc = tile_coord_from(next_r0, next_r1, t, ITEMS, n_rows + nnz);
  if (t + gridDim.x < n_tiles_all) {
    next_r0 = tile_row[t + gridDim.x];
    next_r1 = tile_row[t + gridDim.x + 1];
  }
#else
  const int64_t t = blockIdx.x;
  const TileCoord tc = tile_coord(tile_row, t, ITEMS, n_rows + nnz);
  {
#endif
  const int n_nz = static_cast<int>(tc.j1 - tc.j0);
  const int n_end = static_cast<int>(tc.r1 - tc.r0);  // rows that end in this tile

  const I* gcol = col + tc.j0;
  const V* gval = val + tc.j0;
  V* prod_w;  // products of the tile, in shared memory
  if (tid == 0) {
    qcount[0] = 0;
    qcount[1] = 0;
    qcount[2] = 0;
  }
  if constexpr (B2S_SPMV_DIRECT) {
    // col / val are read straight from global memory, coalesced, with all loads of a batch in
    // flight before the gathers; measured cheaper for the load/store pipe than staging them
    // (bulk-copy fills of shared memory and the re-reads count against the same data pipe)
    prod_w = reinterpret_cast<V*>(val_buf);
#if B2S_SPMV_PREFETCH_AHEAD > 0
    // pull the col / val range of the tile that will run in this CTA's slot one wave from now
    // into L2, so that its loads find them there instead of waiting on DRAM
    {
      const int64_t ta = t + B2S_SPMV_PREFETCH_AHEAD;
      if (ta < static_cast<int64_t>(gridDim.x)) {
        const int64_t total = n_rows + nnz;
        int64_t da = ta * static_cast<int64_t>(ITEMS);
        if (da > total) da = total;
        const int64_t ja = da - tile_row[ta];
        int64_t na = nnz - ja;
        if (na > ITEMS) na = ITEMS;
        const char* pc = reinterpret_cast<const char*>(col + ja);
        const char* pv = reinterpret_cast<const char*>(val + ja);
        const int64_t bc = na * static_cast<int64_t>(sizeof(I));
        const int64_t bv = na * static_cast<int64_t>(sizeof(V));
        for (int64_t o = tid * 128LL; o < bc; o += THREADS * 128LL)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(pc + o));
        for (int64_t o = tid * 128LL; o < bv; o += THREADS * 128LL)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(pv + o));
      }
    }
#endif
    const uint64_t once = policy_evict_first();
    const uint64_t keep = policy_evict_last();
    for (int k = tid; k < n_end; k += THREADS)
      row_end[k] = static_cast<int>(static_cast<int64_t>(ptr[tc.r0 + 1 + k]) - tc.j0);
    if (tid == 0) row_end[n_end] = n_nz;  // the open row runs to the end of the tile
    // column-panel layout: the matrix is a stack of panels, columns are panel-local and the
    // non-zeros of panel p start at panel_start[p]; find the panel of the tile's first entry
    int p_lo = 0;
    int64_t p_next = INT64_MAX;  // first non-zero (global index) of the panel after p_lo
    if (panel_start != nullptr && n_nz > 0) {
      int lo = 0, hi = n_panels - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (panel_start[mid] <= tc.j0) lo = mid; else hi = mid - 1;
      }
      p_lo = lo;
      p_next = panel_start[p_lo + 1];
    }
    for (int base = tid; base < n_nz; base += kSpmvUnroll * THREADS) {
      I c[kSpmvUnroll];
      V a[kSpmvUnroll];
#pragma unroll
      for (int u = 0; u < kSpmvUnroll; ++u) {
        const int i = base + u * THREADS;
        if (i < n_nz) {
          c[u] = stream_val(gcol + i, once);
          a[u] = stream_val(gval + i, once);
        }
      }
#pragma unroll
      for (int u = 0; u < kSpmvUnroll; ++u) {
        const int i = base + u * THREADS;
        if (i < n_nz) {
          int64_t xc = static_cast<int64_t>(c[u]);
          if (panel_start != nullptr) {
            int pp = p_lo;
            if (tc.j0 + i >= p_next) {  // rare: the tile straddles a panel border
              ++pp;
              while (pp + 1 < n_panels && tc.j0 + i >= panel_start[pp + 1]) ++pp;
            }
            xc += static_cast<int64_t>(pp) << panel_shift;
          }
          a[u] = a[u] * gather_val(x + xc, gather_policy, keep);
        }
      }
#pragma unroll
      for (int u = 0; u < kSpmvUnroll; ++u) {
        const int i = base + u * THREADS;
        if (i < n_nz) prod_w[i] = a[u];
      }
    }
    __syncthreads();
    B2S_TICK(1);
  } else {
    const Staged<I> sc = stage_layout<I>(col_buf, gcol, n_nz);
    const Staged<V> sv = stage_layout<V>(val_buf, gval, n_nz);
    const uint32_t tx = stage_bytes(sc) + stage_bytes(sv);
    if (tid == 0 && tx) mbar_init(bar, 1);
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
    // one warp waits for the copies; the CTA barrier that follows releases everybody else
    if (tx && warp == 0) {
      if (!mbar_wait(bar, 0)) {
        if (status && lane == 0) atomicOr(status, 1 << B2S_ERR_TIMEOUT);
        mbar_wait(bar, 0);  // second bounded wait: do not leave with a copy in flight
      }
    }
    __syncthreads();
    B2S_TICK(0);
    const I* scol = sc.s;
    V* sval = sv.s;
    prod_w = sv.s;
    const uint64_t keep = policy_evict_last();
    for (int base = tid; base < n_nz; base += kSpmvUnroll * THREADS) {
      V xv[kSpmvUnroll];
#pragma unroll
      for (int u = 0; u < kSpmvUnroll; ++u) {
        const int i = base + u * THREADS;
        if (i < n_nz)
          xv[u] = gather_val(x + static_cast<int64_t>(scol[i]), gather_policy, keep);
      }
#pragma unroll
      for (int u = 0; u < kSpmvUnroll; ++u) {
        const int i = base + u * THREADS;
        if (i < n_nz) sval[i] = sval[i] * xv[u];
      }
    }
    __syncthreads();
    B2S_TICK(1);
  }

  const V* prod = prod_w;
  V* rsum = prod_w + n_nz;  // row sums live behind the products (n_nz + n_end + 1 <= ITEMS + 1)
  const bool open_row = tc.r1 < n_rows;
  const int n_seg = n_end + 1;  // row pieces in the tile; the last one is the open row

  // ---- bin the row pieces of the tile by length; the shortest are summed on the spot ----------
  //   <= kThreadRowMax : one thread per piece, serial sum
  //   <= kGroupRowMax  : queue A, a group of 8 lanes per piece (vector-per-row)
  //   <= kWarpRowMax   : queue B, a warp per piece
  //   longer           : queue C, the whole CTA per piece
  for (int k = tid; k < n_seg; k += THREADS) {
    const int s = k ? row_end[k - 1] : 0;
    const int e = row_end[k];
    const int len = e - s;
    if (len <= kThreadRowMax) {
      V acc = vt<V>::zero();
      for (int i = s; i < e; ++i) acc = acc + prod[i];
      rsum[k] = acc;
    } else if (len <= kGroupRowMax) {
      const int q = atomicAdd(&qcount[0], 1);
      if (q < kQueueACap) queueA[q] = k;
    } else if (len <= kWarpRowMax) {
      const int q = atomicAdd(&qcount[1], 1);
      if (q < kQueueBCap) queueB[q] = k;
    } else {
      const int q = atomicAdd(&qcount[2], 1);
      if (q < kQueueCCap) queueC[q] = k;
    }
  }
  __syncthreads();
  B2S_TICK(2);

  // ---- queue A: vector-per-row, 8 lanes per piece, butterfly reduction ------------------------
  {
    const int nA = min(qcount[0], kQueueACap);
    const int sub = tid & 7;
    const int grp = tid >> 3;
    for (int qb = 0; qb < nA; qb += THREADS / 8) {  // uniform trip count: shuffles stay converged
      const int q = qb + grp;
      const bool live = q < nA;
      int k = 0, s = 0, e = 0;
      if (live) {
        k = queueA[q];
        s = k ? row_end[k - 1] : 0;
        e = row_end[k];
      }
      V acc = vt<V>::zero();
      for (int i = s + sub; i < e; i += 8) acc = acc + prod[i];
      acc = group_sum(acc, 8);
      if (live && sub == 0) rsum[k] = acc;
    }
  }

  // ---- queue B: warp-per-row -------------------------------------------------------------------
  {
    const int nB = min(qcount[1], kQueueBCap);
    for (int q = warp; q < nB; q += THREADS / 32) {
      const int k = queueB[q];
      const int s = k ? row_end[k - 1] : 0;
      const int e = row_end[k];
      V acc = vt<V>::zero();
      for (int i = s + lane; i < e; i += 32) acc = acc + prod[i];
      acc = group_sum(acc, 32);
      if (lane == 0) rsum[k] = acc;
    }
  }

  // ---- queue C: CTA-per-row --------------------------------------------------------------------
  {
    const int nC = min(qcount[2], kQueueCCap);
    for (int q = 0; q < nC; ++q) {
      const int k = queueC[q];
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
        rsum[k] = tot;
      }
      __syncthreads();
    }
  }
  __syncthreads();
  B2S_TICK(3);

  // ---- epilogue: the rows that end in this tile are consecutive, so y is read and written
  // coalesced, with every load of a batch issued before the first store
  for (int kb = 0; kb < n_end; kb += 4 * THREADS) {
    V old[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = kb + u * THREADS + tid;
      old[u] = (has_beta && k < n_end) ? y_in[tc.r0 + k] : vt<V>::zero();
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = kb + u * THREADS + tid;
      if (k < n_end) {
        V r = alpha * rsum[k];
        if (has_beta) r = r + beta * old[u];
        y[tc.r0 + k] = r;
      }
    }
  }
  if (tid == 0 && open_row) carry[t] = rsum[n_end];
  B2S_TICK(4);
#if B2S_SPMV_PERSISTENT
  __syncthreads();  // the next tile reuses the shared-memory buffers
#endif
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
                int64_t n_cols, int64_t nnz, const void* x, const void* y_in, void* y, const void* alpha,
                const void* beta, const int64_t* tile_row, void* carry, int32_t* status,
                cudaStream_t stream, const int64_t* panel_start = nullptr, int n_panels = 0,
                int panel_shift = 0) {
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
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(n_tiles));
#if B2S_SPMV_PERSISTENT
  {
    // as many CTAs as the device keeps resident at once
    static int slots = 0;
    if (slots == 0) {
      int dev = 0, sms = 0, per_sm = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, THREADS, smem);
      slots = sms * (per_sm > 0 ? per_sm : 1);
    }
    if (n_tiles > slots) cfg.gridDim = dim3(static_cast<unsigned>(slots));
  }
#endif
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (g_knobs[KNOB_PERSIST_BYTES] > 0 && n_cols > 0) {
    // keep as much of x as the persisting carve-out holds; the rest is treated as streaming
    const double x_bytes = static_cast<double>(n_cols) * sizeof(V);
    attr[0].id = cudaLaunchAttributeAccessPolicyWindow;
    attr[0].val.accessPolicyWindow.base_ptr = const_cast<void*>(x);
    attr[0].val.accessPolicyWindow.num_bytes = static_cast<size_t>(x_bytes);
    double ratio = static_cast<double>(g_knobs[KNOB_PERSIST_BYTES]) / x_bytes;
    attr[0].val.accessPolicyWindow.hitRatio = static_cast<float>(ratio > 1.0 ? 1.0 : ratio);
    attr[0].val.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
    attr[0].val.accessPolicyWindow.missProp = cudaAccessPropertyStreaming;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaLaunchKernelEx(&cfg, kern, static_cast<const V*>(data), static_cast<const I*>(indices),
                     static_cast<const P*>(indptr), static_cast<const V*>(x),
                     static_cast<const V*>(y_in), static_cast<V*>(y), static_cast<V*>(carry),
                     tile_row, n_rows, nnz, a, b, has_beta,
                     static_cast<int>(g_knobs[KNOB_GATHER_POLICY]), status, panel_start, n_panels,
                     panel_shift);
  if (n_tiles > 1) {
    const int fb = 256;
    spmv_fixup_kernel<V><<<static_cast<unsigned>((n_tiles + fb - 1) / fb), fb, 0, stream>>>(
        static_cast<V*>(y), static_cast<const V*>(carry), tile_row, n_tiles, a);
  }
  return launch_status();
}

// y[r] = alpha * (ypart[0][r] + ypart[1][r] + ...) + beta * y_in[r]; panels are added in
// ascending order, so the result does not depend on scheduling.
template <class V>
__global__ void panel_combine_kernel(const V* __restrict__ ypart, int64_t n_rows, int n_panels,
                                     const V* y_in, V* y, V alpha, V beta, int has_beta) {
  const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (r >= n_rows) return;
  V s = ypart[r];
  for (int p = 1; p < n_panels; ++p) s = s + ypart[p * n_rows + r];
  V out = alpha * s;
  if (has_beta) out = out + beta * y_in[r];
  y[r] = out;
}

// The same with the empty rows of the stack dropped: subpos[p * n_rows + r] is the position of
// (panel p, row r) among the non-empty stacked rows, or -1.
template <class V>
__global__ void panel_combine_sparse_kernel(const V* __restrict__ ypart,
                                            const int32_t* __restrict__ subpos, int64_t n_rows,
                                            int n_panels, const V* y_in, V* y, V alpha, V beta,
                                            int has_beta) {
  const int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (r >= n_rows) return;
  V s = vt<V>::zero();
  for (int p = 0; p < n_panels; ++p) {
    const int32_t c = subpos[p * n_rows + r];
    if (c >= 0) s = s + ypart[c];
  }
  V out = alpha * s;
  if (has_beta) out = out + beta * y_in[r];
  y[r] = out;
}

// ---- the same combine with the all-gather fused in ---------------------------------------------
// Every rank of a row-partitioned product owns rows [row_offset, row_offset + n_rows) of the
// assembled y.  Instead of writing its block locally and handing it to a collective, the combine
// stores each finished value straight into the y buffer of every rank (its own included) through
// peer-mapped pointers: ordinary coalesced stores that travel over NVLink.
struct PeerList {
  void* p[16];
};

template <class V>
__global__ void panel_combine_peers_kernel(const V* __restrict__ ypart,
                                           const int32_t* __restrict__ subpos, int64_t n_rows,
                                           int n_panels, const V* y_in, PeerList peers,
                                           int n_peers, int64_t row_offset, V alpha, V beta,
                                           int has_beta) {
  // grid-stride: with one thread per row the loop runs once; a small grid (grid_limit of the
  // entry point) keeps the kernel to a few CTAs per SM so that it can drain over NVLink beside
  // the tile kernel of the next row block instead of filling the GPU with stalled stores
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t r = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; r < n_rows;
       r += stride) {
    V s = vt<V>::zero();
    for (int p = 0; p < n_panels; ++p) {
      if (subpos != nullptr) {
        const int32_t c = subpos[p * n_rows + r];
        if (c >= 0) s = s + ypart[c];
      } else {
        s = s + ypart[p * n_rows + r];
      }
    }
    V out = alpha * s;
    if (has_beta) out = out + beta * y_in[r];
    for (int q = 0; q < n_peers; ++q) static_cast<V*>(peers.p[q])[row_offset + r] = out;
  }
}

// Plain block of bytes to the same offset of every peer buffer (16-byte vectors, grid-stride).
__global__ void peer_scatter_kernel(const uint4* __restrict__ src, int64_t n16, PeerList peers,
                                    int n_peers, int64_t dst_off16) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n16;
       i += stride) {
    const uint4 v = src[i];
    for (int q = 0; q < n_peers; ++q) static_cast<uint4*>(peers.p[q])[dst_off16 + i] = v;
  }
}

template <class V, class P>
int spmv_panels_launch(const void* p_data, const int32_t* p_cols, const void* p_ptr,
                       int64_t n_rows, int64_t n_cols, int64_t nnz, int n_panels, int panel_shift,
                       const int64_t* panel_start, const void* x, const void* y_in, void* y,
                       const void* alpha, const void* beta, const int64_t* tile_row, void* carry,
                       void* ypart, int32_t* status, cudaStream_t stream,
                       int64_t n_stacked, const int32_t* subpos,
                       const PeerList* peers = nullptr, int n_peers = 0,
                       int64_t row_offset = 0) {
  // 1) the stacked matrix (n_panels * n_rows rows, panel-local int32 columns) times x with
  //    alpha = 1, beta = 0 -> one partial result per (panel, row)
  const V one = vt<V>::one(), zero = vt<V>::zero();
  int st = spmv_launch<V, int32_t, P>(p_data, p_cols, p_ptr, n_stacked, n_cols, nnz, x,
                                      nullptr, ypart, &one, &zero, tile_row, carry, status,
                                      stream, panel_start, n_panels, panel_shift);
  if (st != B2S_OK) return st;
  if (y == nullptr && peers == nullptr) return launch_status();  // caller combines separately
  // 2) add the panels of each row and apply alpha / beta
  const V a = *static_cast<const V*>(alpha);
  const V b = *static_cast<const V*>(beta);
  const int has_beta = vt<V>::is_zero(b) ? 0 : 1;
  if (has_beta && y_in == nullptr) return B2S_ERR_ARG;
  const int threads = 256;
  const unsigned grid = static_cast<unsigned>((n_rows + threads - 1) / threads);
  if (peers != nullptr)
    panel_combine_peers_kernel<V><<<grid, threads, 0, stream>>>(
        static_cast<const V*>(ypart), subpos, n_rows, n_panels, static_cast<const V*>(y_in),
        *peers, n_peers, row_offset, a, b, has_beta);
  else if (subpos != nullptr)
    panel_combine_sparse_kernel<V><<<grid, threads, 0, stream>>>(
        static_cast<const V*>(ypart), subpos, n_rows, n_panels, static_cast<const V*>(y_in),
        static_cast<V*>(y), a, b, has_beta);
  else
    panel_combine_kernel<V><<<grid, threads, 0, stream>>>(
        static_cast<const V*>(ypart), n_rows, n_panels, static_cast<const V*>(y_in),
        static_cast<V*>(y), a, b, has_beta);
  return launch_status();
}

}  // namespace b2s

#ifdef B2S_PHASES
extern "C" int b2s_debug_phases(unsigned long long* out8, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out8, b2s::g_phase_cycles, sizeof(unsigned long long) * 8);
  cudaMemcpyFromSymbol(out8 + 8, b2s::g_s1_by_T, sizeof(unsigned long long) * 16);
  if (reset) {
    unsigned long long z[8] = {0};
    cudaMemcpyToSymbol(b2s::g_phase_cycles, z, sizeof(z));
    unsigned long long z2[16] = {0};
    cudaMemcpyToSymbol(b2s::g_s1_by_T, z2, sizeof(z2));
  }
  return 0;
}
#endif

extern "C" int b2s_spmv_tile_items(int val_type, int idx_type) {
  (void)val_type;
  (void)idx_type;
  return b2s::SpmvCfg<float, int32_t>::ITEMS;
}

extern "C" int b2s_spmv_panels(int val_type, int ptr_type, const void* p_data_dev,
                               const int32_t* p_cols_dev, const void* p_ptr_dev, int64_t n_rows,
                               int64_t n_cols, int64_t nnz, int n_panels, int panel_shift,
                               const int64_t* panel_start_dev, const void* x_dev,
                               const void* y_in_dev, void* y_dev, const void* alpha,
                               const void* beta, const int64_t* tile_row_dev, void* carry_dev,
                               void* ypart_dev, int32_t* status_dev, b2s_stream stream,
                               int64_t n_stacked, const int32_t* subpos_dev) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0 || !alpha || !beta) return B2S_ERR_ARG;
  if (subpos_dev == nullptr) n_stacked = n_rows * n_panels;
  if (n_stacked < 0 || n_stacked > n_rows * n_panels) return B2S_ERR_ARG;
  if (n_panels < 1 || n_panels > 256 || panel_shift < 0 || panel_shift > 40) return B2S_ERR_ARG;
  if (n_rows == 0) return B2S_OK;
  if (!p_ptr_dev || !tile_row_dev || !carry_dev || !ypart_dev || !panel_start_dev)
    return B2S_ERR_ARG;  // y_dev == NULL: leave the per-panel partials in ypart_dev
  if (nnz > 0 && (!p_data_dev || !p_cols_dev || !x_dev)) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(p_data_dev) & m) || (reinterpret_cast<uintptr_t>(x_dev) & m) ||
      (reinterpret_cast<uintptr_t>(y_dev) & m) || (reinterpret_cast<uintptr_t>(y_in_dev) & m) ||
      (reinterpret_cast<uintptr_t>(carry_dev) & m) || (reinterpret_cast<uintptr_t>(ypart_dev) & m))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_V(val_type, B2S_DISPATCH_I(ptr_type, P, {
    return (b2s::spmv_panels_launch<V, P>(p_data_dev, p_cols_dev, p_ptr_dev, n_rows, n_cols, nnz,
                                          n_panels, panel_shift, panel_start_dev, x_dev, y_in_dev,
                                          y_dev, alpha, beta, tile_row_dev, carry_dev, ypart_dev,
                                          status_dev, s, n_stacked, subpos_dev));
  }));
  return B2S_ERR_DTYPE;
}

static int make_peer_list(void* const* peer_ptrs, int n_peers, size_t align,
                          b2s::PeerList* out) {
  if (!peer_ptrs || n_peers < 1 || n_peers > 16) return B2S_ERR_ARG;
  for (int q = 0; q < 16; ++q) out->p[q] = nullptr;
  for (int q = 0; q < n_peers; ++q) {
    if (!peer_ptrs[q]) return B2S_ERR_ARG;
    if (reinterpret_cast<uintptr_t>(peer_ptrs[q]) % align) return B2S_ERR_ALIGNMENT;
    out->p[q] = peer_ptrs[q];
  }
  return B2S_OK;
}

extern "C" int b2s_spmv_panels_peers(int val_type, int ptr_type, const void* p_data_dev,
                                     const int32_t* p_cols_dev, const void* p_ptr_dev,
                                     int64_t n_rows, int64_t n_cols, int64_t nnz, int n_panels,
                                     int panel_shift, const int64_t* panel_start_dev,
                                     const void* x_dev, const void* y_in_dev,
                                     void* const* peer_y, int n_peers, int64_t row_offset,
                                     int64_t peer_rows, const void* alpha, const void* beta,
                                     const int64_t* tile_row_dev, void* carry_dev,
                                     void* ypart_dev, int32_t* status_dev, b2s_stream stream,
                                     int64_t n_stacked, const int32_t* subpos_dev) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0 || row_offset < 0 || !alpha || !beta) return B2S_ERR_ARG;
  if (row_offset + n_rows > peer_rows) return B2S_ERR_ARG;  // block must fit the peers' buffers
  if (subpos_dev == nullptr) n_stacked = n_rows * n_panels;
  if (n_stacked < 0 || n_stacked > n_rows * n_panels) return B2S_ERR_ARG;
  if (n_panels < 1 || n_panels > 256 || panel_shift < 0 || panel_shift > 40) return B2S_ERR_ARG;
  if (n_rows == 0) return B2S_OK;
  if (!p_ptr_dev || !tile_row_dev || !carry_dev || !ypart_dev || !panel_start_dev)
    return B2S_ERR_ARG;
  if (nnz > 0 && (!p_data_dev || !p_cols_dev || !x_dev)) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  b2s::PeerList peers;
  const int pst = make_peer_list(peer_y, n_peers, vs, &peers);
  if (pst != B2S_OK) return pst;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_V(val_type, B2S_DISPATCH_I(ptr_type, P, {
    return (b2s::spmv_panels_launch<V, P>(p_data_dev, p_cols_dev, p_ptr_dev, n_rows, n_cols, nnz,
                                          n_panels, panel_shift, panel_start_dev, x_dev, y_in_dev,
                                          nullptr, alpha, beta, tile_row_dev, carry_dev,
                                          ypart_dev, status_dev, s, n_stacked, subpos_dev, &peers,
                                          n_peers, row_offset));
  }));
  return B2S_ERR_DTYPE;
}

extern "C" int b2s_panel_combine_peers(int val_type, const void* ypart_dev,
                                       const int32_t* subpos_dev, int64_t n_rows, int n_panels,
                                       const void* y_in_dev, void* const* peer_y, int n_peers,
                                       int64_t row_offset, int64_t peer_rows, const void* alpha,
                                       const void* beta, int grid_limit, b2s_stream stream) {
  if (n_rows < 0 || row_offset < 0 || n_panels < 1 || n_panels > 256 || !alpha || !beta ||
      grid_limit < 0)
    return B2S_ERR_ARG;
  if (row_offset + n_rows > peer_rows) return B2S_ERR_ARG;
  if (n_rows == 0) return B2S_OK;
  if (!ypart_dev) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  b2s::PeerList peers;
  const int pst = make_peer_list(peer_y, n_peers, vs, &peers);
  if (pst != B2S_OK) return pst;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  int64_t want = (n_rows + threads - 1) / threads;
  if (grid_limit > 0 && want > grid_limit) want = grid_limit;
  const unsigned grid = static_cast<unsigned>(want);
  B2S_DISPATCH_V(val_type, {
    const V a = *static_cast<const V*>(alpha);
    const V b = *static_cast<const V*>(beta);
    const int has_beta = b2s::vt<V>::is_zero(b) ? 0 : 1;
    if (has_beta && y_in_dev == nullptr) return B2S_ERR_ARG;
    (b2s::panel_combine_peers_kernel<V><<<grid, threads, 0, s>>>(
        static_cast<const V*>(ypart_dev), subpos_dev, n_rows, n_panels,
        static_cast<const V*>(y_in_dev), peers, n_peers, row_offset, a, b, has_beta));
  });
  return b2s::launch_status();
}

extern "C" int b2s_peer_scatter(const void* src_dev, int64_t bytes, void* const* peer_dst,
                                int n_peers, int64_t dst_offset_bytes, int64_t peer_bytes,
                                b2s_stream stream) {
  if (bytes < 0 || dst_offset_bytes < 0) return B2S_ERR_ARG;
  if (dst_offset_bytes + bytes > peer_bytes) return B2S_ERR_ARG;  // must fit the peers' buffers
  if (bytes == 0) return B2S_OK;
  if (!src_dev) return B2S_ERR_ARG;
  if ((bytes % 16) || (dst_offset_bytes % 16) || (reinterpret_cast<uintptr_t>(src_dev) % 16))
    return B2S_ERR_ALIGNMENT;
  b2s::PeerList peers;
  const int pst = make_peer_list(peer_dst, n_peers, 16, &peers);
  if (pst != B2S_OK) return pst;
  const int64_t n16 = bytes / 16;
  const int threads = 256;
  int64_t want = (n16 + threads - 1) / threads;
  const unsigned grid = static_cast<unsigned>(want > 148 * 8 ? 148 * 8 : want);
  b2s::peer_scatter_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src_dev), n16, peers, n_peers, dst_offset_bytes / 16);
  return b2s::launch_status();
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
    return (b2s::spmv_launch<V, I, P>(data_dev, indices_dev, indptr_dev, n_rows, n_cols, nnz, x_dev,
                                      y_in_dev, y_dev, alpha, beta, tile_row_dev, carry_dev,
                                      status_dev, s));
  })));
  return B2S_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// SpMV without any allocation: tile plan and carries live in a fixed device array
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int64_t kFixedMaxTiles = 1 << 16;  // 65,536 tiles = 67,108,864 rows + non-zeros

struct FixedScratch {
  int64_t tile_row[kFixedMaxTiles + 1];
  alignas(16) unsigned char carry[kFixedMaxTiles * 16];  // one value of the widest dtype per tile
};

// About 1.5 MB of device memory on every GPU that loads the library, held until exit.
static __device__ __align__(256) unsigned char g_fixed_scratch[sizeof(FixedScratch)];

// In host code the name g_fixed_scratch is only a stand-in for the device array, not its
// address; the address is looked up once per device and kept here.
FixedScratch* g_fixed_ptr[64] = {};
std::mutex g_fixed_mu;

int fixed_scratch_for_current_device(FixedScratch** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B2S_ERR_ARG;
  std::lock_guard<std::mutex> lock(g_fixed_mu);
  if (g_fixed_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fixed_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return B2S_ERR_LAUNCH;
    }
    g_fixed_ptr[dev] = static_cast<FixedScratch*>(p);
  }
  *out = g_fixed_ptr[dev];
  return B2S_OK;
}

}  // namespace

extern "C" int64_t b2s_spmv_csr_fixed_max_items(void) {
  return kFixedMaxTiles * static_cast<int64_t>(b2s::SpmvCfg<float, int32_t>::ITEMS);
}

extern "C" int b2s_spmv_csr_fixed(int val_type, int idx_type, int ptr_type, const void* data_dev,
                                  const void* indices_dev, const void* indptr_dev,
                                  int64_t n_rows, int64_t n_cols, int64_t nnz, const void* x_dev,
                                  const void* y_in_dev, void* y_dev, const void* alpha,
                                  const void* beta, b2s_stream stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return B2S_ERR_ARG;
  const int items = b2s_spmv_tile_items(val_type, idx_type);
  if (b2s_tile_count(n_rows, nnz, items) > kFixedMaxTiles) return B2S_ERR_TOO_LARGE;
  if (n_rows == 0) return B2S_OK;
  FixedScratch* fs = nullptr;
  int st = fixed_scratch_for_current_device(&fs);
  if (st != B2S_OK) return st;
  // Nothing in the array has to start at zero: the plan is rewritten in full here, and every
  // carry the fix-up reads was written by the tile kernel of this same call.
  st = b2s_tile_plan(indptr_dev, ptr_type, n_rows, nnz, items, fs->tile_row, stream);
  if (st != B2S_OK) return st;
  return b2s_spmv_csr(val_type, idx_type, ptr_type, data_dev, indices_dev, indptr_dev, n_rows,
                      n_cols, nnz, x_dev, y_in_dev, y_dev, alpha, beta, fs->tile_row, fs->carry,
                      nullptr, stream);
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait: one warp waits on an mbarrier that nothing ever completes, with
// a small iteration limit.  The wait gives up, the kernel ORs B2S_ERR_TIMEOUT into the status
// word and returns normally; the context stays usable.  Used by the failure-path test.
// ---------------------------------------------------------------------------------------------
namespace b2s {
__global__ void wait_timeout_selftest_kernel(int32_t* status, int limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) mbar_init(&bar, 1);
  __syncthreads();
  const uint32_t a = smem_addr(&bar);
  bool done = false;
  for (int it = 0; it < limit && !done; ++it) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; "
        "selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(a), "r"(0u), "r"(1000u)
        : "memory");
    done = ok != 0;
  }
  if (!done && threadIdx.x == 0) atomicOr(status, 1 << B2S_ERR_TIMEOUT);
}
}  // namespace b2s

extern "C" int b2s_selftest_wait_timeout(int32_t* status_dev, int spin_limit, b2s_stream stream) {
  if (!status_dev || spin_limit < 1 || spin_limit > 100000) return B2S_ERR_ARG;
  b2s::wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status_dev,
                                                                                   spin_limit);
  return b2s::launch_status();
}
