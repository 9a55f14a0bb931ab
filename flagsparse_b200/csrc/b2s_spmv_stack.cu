// SpMV over the "end-flag stack": the layout the column-panel path of SpMV keeps its matrix in.
//
// b2s_panel_build + b2s_panel_compact turn a CSR matrix into a stack of column panels whose
// stacked rows (one per (panel, row) pair that has entries) are all non-empty.  In that layout
// the row pointers can be folded into the column words: bit 31 of a column word marks the LAST
// entry of its stacked row, bit 30 marks a padding entry that must add nothing, the low bits
// are the panel-local column.  The kernel then needs no row pointers, no search and no
// shared-memory bit map:
//   * a tile is a fixed chunk of TILE consecutive entries (always vector aligned), tile_ord[t]
//     is the ordinal of the stacked row that is active at its first entry;
//   * every thread reads SPT consecutive entries with 32-byte vector loads, gathers x, and sums
//     its products serially, cutting after each end flag; the ordinal of the row a thread is
//     in comes from ballots of the flags (no memory traffic);
//   * sums that begin and end inside one thread are stored straight to ypart[ordinal]; the
//     others are completed by the same segmented warp scan and cross-warp carry as in
//     spmv_tile_kernel, and rows that cross tile borders by the same carry fix-up.
// Two ways to read x:
//   GLOBAL  panels as wide as L2 allows: x[panel offset + column] through the read-only path;
//   SHARED  narrow panels (an x slice of at most 64 KB) for the long rows of a matrix: a CTA copies the
//           x slice of its panel into shared memory once (one bulk copy) and then walks a run
//           of tiles of that panel; the gathers never leave the SM.  Panels are padded to
//           whole tiles so that no tile sees two slices.
// Sums have fixed shapes; nothing is atomic; results repeat bit for bit.
#include "b2s_tile.cuh"

namespace b2s {

constexpr uint32_t kStackEndBit = 0x80000000u;
constexpr uint32_t kStackPadBit = 0x40000000u;
constexpr uint32_t kStackColMask = 0x3fffffffu;
constexpr int kStackSharedBytes = 64 * 1024;  // largest x slice of the SHARED variant

// A tile is what one warp multiplies at a time: SPT consecutive entries per lane.
template <class V>
struct StackShape {
  static constexpr int SPT = sizeof(V) <= 8 ? 8 : 4;
  static constexpr int TILE = 32 * SPT;
  static constexpr int THREADS = 128;         // wide panels: four independent warps per CTA
  static constexpr int SHARED_THREADS = 256;  // shared x slice: eight warps per slice
};

// N consecutive elements from p (aligned to 32 bytes, or to 16 when the run is 16 bytes long):
// read-only path, no L1 allocation, L2 evict-first.  The arrays are padded to whole tiles, so
// every chunk may be read.
template <class T, int N>
__device__ inline void stack_load_run(const T* p, T (&out)[N], uint64_t pol) {
  constexpr int BYTES = N * static_cast<int>(sizeof(T));
  constexpr int CB = BYTES >= 32 ? 32 : 16;
  static_assert(BYTES % CB == 0, "a lane's run is a whole number of chunks");
  uint64_t w[BYTES / 8];
#pragma unroll
  for (int q = 0; q < BYTES / CB; ++q) {
    const char* src = reinterpret_cast<const char*>(p) + CB * q;
    if constexpr (CB == 32)
      asm volatile(
          "ld.global.nc.L1::no_allocate.L2::cache_hint.v4.b64 {%0,%1,%2,%3}, [%4], %5;"
          : "=l"(w[4 * q]), "=l"(w[4 * q + 1]), "=l"(w[4 * q + 2]), "=l"(w[4 * q + 3])
          : "l"(src), "l"(pol));
    else
      asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.b64 {%0,%1}, [%2], %3;"
                   : "=l"(w[2 * q]), "=l"(w[2 * q + 1])
                   : "l"(src), "l"(pol));
  }
  memcpy(out, w, BYTES);
}

// One value of V at a 32-bit shared-memory address.
__device__ inline float lds_val(uint32_t a, float*) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
  return v;
}
__device__ inline double lds_val(uint32_t a, double*) {
  double v;
  asm volatile("ld.shared.f64 %0, [%1];" : "=d"(v) : "r"(a));
  return v;
}
__device__ inline c64 lds_val(uint32_t a, c64*) {
  c64 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.re), "=f"(v.im) : "r"(a));
  return v;
}
__device__ inline c128 lds_val(uint32_t a, c128*) {
  c128 v;
  asm volatile("ld.shared.v2.f64 {%0,%1}, [%2];" : "=d"(v.re), "=d"(v.im) : "r"(a));
  return v;
}

// CTAs per SM the register allocation aims at.  Wide panels: 8 CTAs of four warps (64 registers,
// nothing spilled) measured 1.32 ms per product on the 2^24-row power-law matrix, the same as 6,
// 7 and 9; 10 and 12 (48 / 40 registers, spills) 1.42 and 1.65 ms.  Shared slice: two CTAs of
// eight warps, each warp with two tiles in flight.
template <class V, bool SHARED>
constexpr int stack_min_blocks() {
  return SHARED ? 2 : (sizeof(V) <= 8 ? 8 : 6);
}

// The entries of tile t that lane `lane` owns.
template <class V>
__device__ inline void stack_tile_load(const V* __restrict__ val,
                                       const uint32_t* __restrict__ col, int64_t t, int lane,
                                       uint32_t (&c)[StackShape<V>::SPT],
                                       V (&v)[StackShape<V>::SPT]) {
  const int64_t jt = t * StackShape<V>::TILE + static_cast<int64_t>(lane) * StackShape<V>::SPT;
  const uint64_t once = policy_evict_first();
  stack_load_run(col + jt, c, once);
  stack_load_run(val + jt, v, once);
}

// One warp multiplies one tile whose entries are already in registers.  SHARED: xs32 is the
// shared-memory address of the x slice and `cut` the mask that keeps a column inside it;
// otherwise x_base + x_off is the panel's slice of x in global memory.  The warp shares
// nothing with the other warps of its CTA.
template <class V, bool SHARED>
__device__ inline void stack_tile(uint32_t (&c)[StackShape<V>::SPT], V (&v)[StackShape<V>::SPT],
                                  uint32_t xs32, uint32_t cut, const V* __restrict__ x_base,
                                  int64_t x_off, int64_t t, int lane, int64_t ord0, int64_t ord1,
                                  V* __restrict__ ypart, int64_t n_stacked,
                                  V* __restrict__ carry, int64_t n_cols,
                                  const int64_t* __restrict__ panel_start, int p_lo,
                                  int n_panels, int panel_shift, int32_t* status) {
  using S = StackShape<V>;
  constexpr int SPT = S::SPT, TILE = S::TILE;
  uint32_t ends = 0;  // bit i: entry i is the last of its stacked row
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    ends |= (c[i] >> 31) << i;
    if (c[i] & kStackPadBit) v[i] = vt<V>::zero();
    c[i] &= kStackColMask;  // padding entries carry column 0
  }

  // ---- gathers ---------------------------------------------------------------------------------
  V xv[SPT];
  if constexpr (SHARED) {
    // the column is cut to the width of the slice, so that not even a corrupt entry can read
    // outside the shared-memory copy
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
#ifdef B2S_CHECKED
      if (c[i] > cut) {
        if (status) atomicOr(status, 1 << B2S_ERR_BOUNDS);
        v[i] = vt<V>::zero();
      }
#endif
      xv[i] = lds_val(xs32 + (c[i] & cut) * static_cast<uint32_t>(sizeof(V)),
                      static_cast<V*>(nullptr));
    }
  } else {
    bool straddles = false;
    if (panel_start != nullptr)
      straddles = panel_start[p_lo + 1] < (t + 1) * static_cast<int64_t>(TILE);
    if (!straddles) {
      const V* xp = x_base + x_off;
#pragma unroll
      for (int i = 0; i < SPT; ++i) {
#ifdef B2S_CHECKED
        if (static_cast<uint64_t>(x_off + static_cast<int64_t>(c[i])) >=
            static_cast<uint64_t>(n_cols)) {
          if (status) atomicOr(status, 1 << B2S_ERR_BOUNDS);
          c[i] = 0;
          v[i] = vt<V>::zero();
        }
#endif
        xv[i] = ldg_val(xp + c[i]);
      }
    } else {
      // the tile reaches into later panels (at most n_panels - 1 tiles of a matrix do)
      const int64_t jt = t * TILE + static_cast<int64_t>(lane) * SPT;
#pragma unroll
      for (int i = 0; i < SPT; ++i) {
        int pp = p_lo;
        while (pp + 1 < n_panels && jt + i >= panel_start[pp + 1]) ++pp;
        int64_t xc = (static_cast<int64_t>(pp) << panel_shift) + static_cast<int64_t>(c[i]);
        if (static_cast<uint64_t>(xc) >= static_cast<uint64_t>(n_cols)) {
          // only padding behind the last entry can point here; it adds nothing
#ifdef B2S_CHECKED
          if (!vt<V>::is_zero(v[i]) && status) atomicOr(status, 1 << B2S_ERR_BOUNDS);
#endif
          xc = 0;
          v[i] = vt<V>::zero();
        }
        xv[i] = ldg_val(x_base + xc);
      }
    }
  }

  if (ord1 == ord0) {
    // ---- no row ends in this tile: one long row, plain fixed-tree sum ---------------------------
    V acc = vt<V>::zero();
#pragma unroll
    for (int i = 0; i < SPT; ++i) acc = acc + v[i] * xv[i];
    acc = group_sum(acc, 32);
    if (lane == 0) carry[t] = acc;
    return;
  }

  // ---- ordinal of the stacked row each lane starts in: ballots of the end flags -----------------
  int before = 0;  // ends in lower lanes of the warp
  {
    const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
    for (int i = 0; i < SPT; ++i)
      before += __popc(__ballot_sync(0xffffffffu, (ends >> i) & 1u) & lt);
  }

  // ---- open sum after the lane's last end (all of its products if it has no end) ----------------
  const bool seen = ends != 0;
  V tail = vt<V>::zero();
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    tail = tail + v[i] * xv[i];
    if ((ends >> i) & 1u) tail = vt<V>::zero();
  }

  // ---- open sums across the lanes: a lane with an end starts afresh with its tail ----------------
  const uint32_t heads_w = __ballot_sync(0xffffffffu, seen);
  const uint32_t upto = heads_w & (0xffffffffu >> (31 - lane));  // lanes with an end, <= this one
  const int reach = upto ? lane - (31 - __clz(upto)) : lane;     // lanes below in the same run
  V incl = tail;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const V below = shfl_up(incl, d);
    if (d <= reach) incl = below + incl;
  }
  V inflow = shfl_up(incl, 1);  // open sum that enters this lane
  if (lane == 0) inflow = vt<V>::zero();

  // ---- rows that end in this lane: the first one takes the sum that flowed in --------------------
  if (seen) {
    int64_t ord = ord0 + before;
    V run = inflow;
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      run = run + v[i] * xv[i];
      if ((ends >> i) & 1u) {
#ifdef B2S_CHECKED
        if (ord < 0 || ord >= n_stacked) {  // flags and tile_ord disagree
          if (status) atomicOr(status, 1 << B2S_ERR_BOUNDS);
        } else
#endif
          ypart[ord] = run;
        ++ord;
        run = vt<V>::zero();
      }
    }
  }
  if (lane == 31) carry[t] = incl;  // the row still open at the end of the tile
}

template <class V>
__global__ void __launch_bounds__(StackShape<V>::THREADS, stack_min_blocks<V, false>())
spmv_stack_kernel(const V* __restrict__ val, const uint32_t* __restrict__ col,
                  const V* __restrict__ x, V* __restrict__ ypart, int64_t n_stacked,
                  V* __restrict__ carry, const int64_t* __restrict__ tile_ord, int64_t n_tiles,
                  int64_t n_cols, const int64_t* __restrict__ panel_start,
                  const int32_t* __restrict__ tile_panel, int n_panels, int panel_shift,
                  int32_t* status, int64_t tile_begin) {
  using S = StackShape<V>;
  const int lane = threadIdx.x & 31;
  // this launch covers tiles tile_begin .. n_tiles - 1 (n_tiles: end of the range)
  const int64_t t =
      tile_begin + static_cast<int64_t>(blockIdx.x) * (S::THREADS / 32) + (threadIdx.x >> 5);
  if (t >= n_tiles) return;  // warps share no barrier: leaving early is safe
  uint32_t c[S::SPT];
  V v[S::SPT];
  stack_tile_load(val, col, t, lane, c, v);
  const int p_lo = tile_panel != nullptr ? tile_panel[t] : 0;
  stack_tile<V, false>(c, v, 0u, 0u, x, static_cast<int64_t>(p_lo) << panel_shift, t, lane,
                       tile_ord[t], tile_ord[t + 1], ypart, n_stacked, carry, n_cols,
                       panel_start, p_lo, n_panels, panel_shift, status);
}

// SHARED: CTA u copies the x slice of panel unit[3u] into shared memory; its warps then walk
// tiles unit[3u + 1] .. unit[3u + 1] + unit[3u + 2] - 1 (all of that panel) round robin, each
// warp with the entries of its next tile already requested while it multiplies the current one.
template <class V>
__global__ void __launch_bounds__(StackShape<V>::SHARED_THREADS, stack_min_blocks<V, true>())
spmv_stack_shared_kernel(const V* __restrict__ val, const uint32_t* __restrict__ col,
                         const V* __restrict__ x, V* __restrict__ ypart, int64_t n_stacked,
                         V* __restrict__ carry, const int64_t* __restrict__ tile_ord,
                         int64_t n_tiles, int64_t n_cols, const int32_t* __restrict__ unit,
                         int panel_shift, int32_t* status) {
  using S = StackShape<V>;
  constexpr int THREADS = S::SHARED_THREADS, WARPS = THREADS / 32, SPT = S::SPT;
  extern __shared__ __align__(128) unsigned char smem[];  // the x slice (+ 16 bytes of phase)
  __shared__ __align__(8) uint64_t bar_slot;
  uint64_t* bar = &bar_slot;
  V* xs = reinterpret_cast<V*>(smem);
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int p = unit[3 * blockIdx.x];
  const int64_t t0 = unit[3 * blockIdx.x + 1];
  const int n_t = unit[3 * blockIdx.x + 2];
  const int64_t c0 = static_cast<int64_t>(p) << panel_shift;
#ifdef B2S_CHECKED
  if (p < 0 || c0 >= n_cols || t0 < 0 || n_t < 0 || t0 + n_t > n_tiles) {  // a bad unit table
    if (status && tid == 0) atomicOr(status, 1 << B2S_ERR_BOUNDS);
    return;
  }
#endif
  int64_t width = n_cols - c0;
  if (width > (int64_t{1} << panel_shift)) width = int64_t{1} << panel_shift;
  if (width < 0) width = 0;
  // the slice: one bulk copy for the part that is a multiple of 16 bytes from a 16-byte aligned
  // address, plain loads for what is left at either end
  const V* src = x + c0;
  const uintptr_t addr = reinterpret_cast<uintptr_t>(src);
  int head = static_cast<int>(((16 - (addr & 15)) & 15) / sizeof(V));
  if (head > width) head = static_cast<int>(width);
  const int per16 = sizeof(V) >= 16 ? 1 : 16 / static_cast<int>(sizeof(V));
  const int body = static_cast<int>((width - head) / per16) * per16;
  // shared copy keeps the 16-byte phase of the source
  V* xdst = xs + (sizeof(V) >= 16 ? 0 : (addr & 15) / sizeof(V));
  const uint32_t tx = static_cast<uint32_t>(body) * static_cast<uint32_t>(sizeof(V));
  if (tid == 0 && tx) mbar_init(bar, 1);
  __syncthreads();
  if (tid == 0 && tx) {
    mbar_expect_tx(bar, tx);
    bulk_g2s(xdst + head, src + head, tx, bar, policy_evict_last());
  }
  // the entries of each warp's first tile travel while the slice is copied
  const int64_t t_end = t0 + n_t;
  int64_t t = t0 + (tid >> 5);
  uint32_t c[SPT];
  V v[SPT];
  if (t < t_end) stack_tile_load(val, col, t, lane, c, v);
  for (int i = tid; i < head; i += THREADS) xdst[i] = src[i];
  for (int i = head + body + tid; i < width; i += THREADS) xdst[i] = src[i];
  // every thread observes the completion of the copy itself
  bool arrived = true;
  if (tx) {
    arrived = mbar_wait(bar, 0);
    if (!arrived) arrived = mbar_wait(bar, 0);  // second bounded wait
  }
  if (__syncthreads_or(!arrived)) {  // do not multiply from a slice that never came
    if (status && tid == 0) atomicOr(status, 1 << B2S_ERR_TIMEOUT);
    return;
  }
  const uint32_t xs32 = smem_addr(xdst);
  const uint32_t cut = (1u << panel_shift) - 1u;
  while (t < t_end) {
    const int64_t t_next = t + WARPS;
    uint32_t cn[SPT];
    V vn[SPT];
    if (t_next < t_end) stack_tile_load(val, col, t_next, lane, cn, vn);
    stack_tile<V, true>(c, v, xs32, cut, nullptr, 0, t, lane, tile_ord[t], tile_ord[t + 1], ypart,
                        n_stacked, carry, n_cols, nullptr, 0, 0, panel_shift, status);
    if (t_next < t_end) {
#pragma unroll
      for (int i = 0; i < SPT; ++i) {
        c[i] = cn[i];
        v[i] = vn[i];
      }
    }
    t = t_next;
  }
}

// ypart[r] += carries of the tiles row r crossed, oldest first (r = row active at a tile start).
template <class V>
__global__ void stack_fixup_kernel(V* ypart, const V* __restrict__ carry,
                                   const int64_t* __restrict__ tile_ord, int64_t n_tiles) {
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t < 1 || t >= n_tiles) return;
  const int64_t r = tile_ord[t];
  if (tile_ord[t + 1] <= r) return;  // row r does not end in tile t
  int64_t u0 = t - 1;                // tiles u0 .. t-1 ended with row r open
  if (u0 >= 1 && tile_ord[u0] == r) {
    int64_t lo = 0, hi = u0;  // first tile that starts in row r
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (tile_ord[mid] < r) lo = mid + 1; else hi = mid;
    }
    u0 = lo > 0 ? lo - 1 : 0;
  }
  V s = carry[u0];
  for (int64_t u = u0 + 1; u < t; ++u) s = s + carry[u];
  ypart[r] = ypart[r] + s;
}

// out[j] = sum of the partials of long row j, in ascending panel order.  One warp per long row:
// lane l adds partials l, l + 32, ... in order, then a fixed butterfly.
template <class V>
__global__ void stack_rows_combine_kernel(const V* __restrict__ part,
                                          const int64_t* __restrict__ seg_ptr,
                                          const int32_t* __restrict__ seg_ids, int64_t n_long,
                                          int64_t n_part, int32_t* status, V* __restrict__ out) {
  const int64_t j = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (j >= n_long) return;
  V s = vt<V>::zero();
  for (int64_t k = seg_ptr[j] + lane; k < seg_ptr[j + 1]; k += 32) {
#ifdef B2S_CHECKED
    if (seg_ids[k] < 0 || seg_ids[k] >= n_part) {
      if (status) atomicOr(status, 1 << B2S_ERR_BOUNDS);
      continue;
    }
#endif
    s = s + part[seg_ids[k]];
  }
  s = group_sum(s, 32);
  if (lane == 0) out[j] = s;
}

}  // namespace b2s

extern "C" int b2s_spmv_stack_tile_items(int val_type) {
  B2S_DISPATCH_V(val_type, { return b2s::StackShape<V>::TILE; });
  return 0;
}

extern "C" int b2s_spmv_stack_shared_cols(int val_type) {
  const size_t vs = b2s::vsize(val_type);
  return vs ? static_cast<int>(b2s::kStackSharedBytes / vs) : 0;
}

extern "C" int b2s_spmv_stack_tiles(int val_type, const void* s_data_dev,
                                    const uint32_t* s_cols_dev, int64_t n_entries,
                                    int64_t n_stacked, int64_t n_cols, int n_panels,
                                    int panel_shift, const int64_t* panel_start_dev,
                                    const int32_t* tile_panel_dev, const int64_t* tile_ord_dev,
                                    const void* x_dev, void* ypart_dev, void* carry_dev,
                                    int32_t* status_dev, int64_t tile_begin, int64_t tile_count,
                                    int run_fixup, b2s_stream stream) {
  if (n_entries < 0 || n_stacked < 0 || n_cols < 0 || tile_begin < 0 || tile_count < 0)
    return B2S_ERR_ARG;
  if (n_panels < 1 || panel_shift < 0 || panel_shift > 30) return B2S_ERR_ARG;
  if (n_entries == 0 || n_stacked == 0) return B2S_OK;
  if (!s_data_dev || !s_cols_dev || !tile_ord_dev || !x_dev || !ypart_dev || !carry_dev)
    return B2S_ERR_ARG;
  if (n_panels > 1 && (!panel_start_dev || !tile_panel_dev)) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(s_data_dev) % 32) || (reinterpret_cast<uintptr_t>(s_cols_dev) % 32))
    return B2S_ERR_ALIGNMENT;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(x_dev) & m) || (reinterpret_cast<uintptr_t>(ypart_dev) & m) ||
      (reinterpret_cast<uintptr_t>(carry_dev) & m))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_V(val_type, {
    constexpr int THREADS = b2s::StackShape<V>::THREADS;
    constexpr int TILE = b2s::StackShape<V>::TILE;
    if (n_entries % TILE) return B2S_ERR_ARG;  // the arrays are padded to whole tiles
    const int64_t n_tiles = n_entries / TILE;
    if (tile_begin + tile_count > n_tiles) return B2S_ERR_ARG;
    const int64_t n_ctas = (tile_count + THREADS / 32 - 1) / (THREADS / 32);
    if (n_ctas > 0x7fffffffLL) return B2S_ERR_RANGE;
    if (n_ctas > 0)
      (b2s::spmv_stack_kernel<V><<<static_cast<unsigned>(n_ctas), THREADS, 0, s>>>(
          static_cast<const V*>(s_data_dev), s_cols_dev, static_cast<const V*>(x_dev),
          static_cast<V*>(ypart_dev), n_stacked, static_cast<V*>(carry_dev), tile_ord_dev,
          tile_begin + tile_count, n_cols,
          n_panels > 1 ? panel_start_dev : nullptr, n_panels > 1 ? tile_panel_dev : nullptr,
          n_panels, panel_shift, status_dev, tile_begin));
    if (run_fixup && n_tiles > 1)
      (b2s::stack_fixup_kernel<V><<<static_cast<unsigned>((n_tiles + 255) / 256), 256, 0, s>>>(
          static_cast<V*>(ypart_dev), static_cast<const V*>(carry_dev), tile_ord_dev, n_tiles));
    return b2s::launch_status();
  });
  return B2S_ERR_DTYPE;
}

extern "C" int b2s_spmv_stack(int val_type, const void* s_data_dev, const uint32_t* s_cols_dev,
                              int64_t n_entries, int64_t n_stacked, int64_t n_cols,
                              int n_panels, int panel_shift, const int64_t* panel_start_dev,
                              const int32_t* tile_panel_dev, const int64_t* tile_ord_dev,
                              const void* x_dev, void* ypart_dev, void* carry_dev,
                              int32_t* status_dev, b2s_stream stream) {
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  if (n_entries < 0) return B2S_ERR_ARG;
  int tile = 0;
  B2S_DISPATCH_V(val_type, { tile = b2s::StackShape<V>::TILE; });
  return b2s_spmv_stack_tiles(val_type, s_data_dev, s_cols_dev, n_entries, n_stacked, n_cols,
                              n_panels, panel_shift, panel_start_dev, tile_panel_dev,
                              tile_ord_dev, x_dev, ypart_dev, carry_dev, status_dev, 0,
                              n_entries / tile, 1, stream);
}

extern "C" int b2s_spmv_stack_shared(int val_type, const void* s_data_dev,
                                     const uint32_t* s_cols_dev, int64_t n_entries,
                                     int64_t n_stacked, int64_t n_cols, int panel_shift,
                                     const int32_t* unit_dev, int64_t n_units,
                                     const int64_t* tile_ord_dev, const void* x_dev,
                                     void* ypart_dev, void* carry_dev, int32_t* status_dev,
                                     b2s_stream stream) {
  if (n_entries < 0 || n_stacked < 0 || n_cols < 0 || n_units < 0) return B2S_ERR_ARG;
  if (panel_shift < 0 || panel_shift > 20) return B2S_ERR_ARG;
  if (n_entries == 0 || n_stacked == 0 || n_units == 0) return B2S_OK;
  if (!s_data_dev || !s_cols_dev || !tile_ord_dev || !x_dev || !ypart_dev || !carry_dev ||
      !unit_dev)
    return B2S_ERR_ARG;
  if (n_units > 0x7fffffffLL) return B2S_ERR_RANGE;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  if ((reinterpret_cast<uintptr_t>(s_data_dev) % 32) || (reinterpret_cast<uintptr_t>(s_cols_dev) % 32))
    return B2S_ERR_ALIGNMENT;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(x_dev) & m) || (reinterpret_cast<uintptr_t>(ypart_dev) & m) ||
      (reinterpret_cast<uintptr_t>(carry_dev) & m))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_V(val_type, {
    constexpr int THREADS = b2s::StackShape<V>::SHARED_THREADS;
    constexpr int TILE = b2s::StackShape<V>::TILE;
    if (n_entries % TILE) return B2S_ERR_ARG;
    if ((static_cast<size_t>(1) << panel_shift) * sizeof(V) > b2s::kStackSharedBytes)
      return B2S_ERR_ARG;
    const int64_t n_tiles = n_entries / TILE;
    const size_t smem = (static_cast<size_t>(1) << panel_shift) * sizeof(V) + 16;
    auto kern = b2s::spmv_stack_shared_kernel<V>;
    b2s::ensure_dyn_smem(reinterpret_cast<const void*>(kern), b2s::kStackSharedBytes + 16);
    kern<<<static_cast<unsigned>(n_units), THREADS, smem, s>>>(
        static_cast<const V*>(s_data_dev), s_cols_dev, static_cast<const V*>(x_dev),
        static_cast<V*>(ypart_dev), n_stacked, static_cast<V*>(carry_dev), tile_ord_dev, n_tiles,
        n_cols, unit_dev, panel_shift, status_dev);
    if (n_tiles > 1)
      (b2s::stack_fixup_kernel<V><<<static_cast<unsigned>((n_tiles + 255) / 256), 256, 0, s>>>(
          static_cast<V*>(ypart_dev), static_cast<const V*>(carry_dev), tile_ord_dev, n_tiles));
    return b2s::launch_status();
  });
  return B2S_ERR_DTYPE;
}

extern "C" int b2s_spmv_stack_rows_combine(int val_type, const void* part_dev,
                                           const int64_t* seg_ptr_dev, const int32_t* seg_ids_dev,
                                           int64_t n_long, int64_t n_part, void* out_dev,
                                           int32_t* status_dev, b2s_stream stream) {
  if (n_long < 0 || n_part < 0) return B2S_ERR_ARG;
  if (n_long == 0) return B2S_OK;
  if (!part_dev || !seg_ptr_dev || !seg_ids_dev || !out_dev) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(part_dev) & m) || (reinterpret_cast<uintptr_t>(out_dev) & m))
    return B2S_ERR_ALIGNMENT;
  const int threads = 256;
  const int64_t grid = (n_long * 32 + threads - 1) / threads;
  if (grid > 0x7fffffffLL) return B2S_ERR_RANGE;
  B2S_DISPATCH_V(val_type, {
    (b2s::stack_rows_combine_kernel<V><<<static_cast<unsigned>(grid), threads, 0,
                                         static_cast<cudaStream_t>(stream)>>>(
        static_cast<const V*>(part_dev), seg_ptr_dev, seg_ids_dev, n_long, n_part, status_dev,
        static_cast<V*>(out_dev)));
    return b2s::launch_status();
  });
  return B2S_ERR_DTYPE;
}
