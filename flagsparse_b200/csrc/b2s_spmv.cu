// CSR SpMV for sm_100a: y = alpha * A x + beta * y_in.
//
// One CTA of 128 threads per merge-path tile (b2s_tile_plan).  The non-zeros of a tile occupy
// consecutive "slots"; slot 0 is moved back to a 32-byte boundary of the col / val arrays, so
// every thread owns SPT consecutive slots that it reads with 32-byte vector loads, coalesced
// across the warp, straight into registers.  The gathers of x follow (SPT per thread in
// flight) and the products never leave the register file:
//   1. the rows that end in the tile mark the slot after their last non-zero in a shared-memory
//      bit map ("heads": the slot starts a new row piece);
//   2. each thread sums its slots serially, cutting at its head bits; a piece that begins and
//      ends inside the thread is finished on the spot;
//   3. a warp-wide segmented scan (shuffles, keyed on the ballot of the head bits) carries the
//      open sums across lanes, four words of shared memory carry them across warps;
//   4. the sum of each piece is stored at the slot of the head that ends it, and the rows read
//      them back for a coalesced alpha / beta epilogue.
// A row that crosses tile borders leaves one partial sum per tile in `carry`; a second kernel
// adds those partials to the row in ascending tile order.  No floating-point atomics and only
// fixed trees: results repeat bit for bit for a given matrix and build.
//
// Matrices whose x does not fit L2 are multiplied from a column-panel layout by the kernels of
// b2s_spmv_stack.cu; the combine kernels at the end of this file add the per-panel partials.
#include <mutex>
#include <type_traits>

#include "b2s_tile.cuh"

namespace b2s {

// Tile geometry.  SPT slots per thread: 8 consecutive non-zeros for values up to 8 bytes, 4 for
// complex128.  A tile holds ITEMS merge items = SLOTS - SPT, which leaves room to begin the
// slots on the vector boundary below the tile's first non-zero.
template <class V>
struct SpmvShape {
  static constexpr int THREADS = 128;
  static constexpr int SPT = sizeof(V) <= 8 ? 8 : 4;
  static constexpr int SLOTS = THREADS * SPT;
  static constexpr int ITEMS = SLOTS - SPT;
};

// CTAs per SM the register allocation aims at.
template <class V, class I>
constexpr int spmv_min_blocks() {
#ifdef B2S_SPMV_MINBLOCKS
  return B2S_SPMV_MINBLOCKS;
#else
  return (sizeof(V) <= 8 && sizeof(I) == 4) ? 10 : 8;
#endif
}

// Bytes of one vector load of a thread's run of N elements of T: 32, or 16 when the whole run
// is only 16 bytes long (4 int32 columns beside 4 complex128 values).
template <class T, int N>
__host__ __device__ constexpr int run_chunk_bytes() {
  return N * static_cast<int>(sizeof(T)) >= 32 ? 32 : 16;
}

// N consecutive elements starting at p (p aligned to the chunk size) with 32-byte loads through
// the read-only path, no L1 allocation, L2 evict-first: col / val are read exactly once.  Only
// the chunks that hold a live element (index in [lo, hi)) are requested, so a load never leaves
// the aligned 32-byte sector of an element that belongs to the arrays.
template <class T, int N>
__device__ inline void load_run(const T* p, T (&out)[N], int lo, int hi, uint64_t pol) {
  constexpr int BYTES = N * static_cast<int>(sizeof(T));
  constexpr int CB = run_chunk_bytes<T, N>();
  static_assert(BYTES % CB == 0, "a thread's run is a whole number of chunks");
  constexpr int CHUNKS = BYTES / CB;
  constexpr int EPC = N / CHUNKS;  // elements per chunk
  constexpr int WPC = CB / 8;      // 8-byte words per chunk
  uint64_t w[BYTES / 8];
#pragma unroll
  for (int q = 0; q < CHUNKS; ++q) {
#pragma unroll
    for (int k = 0; k < WPC; ++k) w[WPC * q + k] = 0;
    if ((q + 1) * EPC > lo && q * EPC < hi) {
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
  }
  memcpy(out, w, BYTES);
}

// S: storage type of val, x and y (V itself, or a 16-bit float type with V = float).  With a
// 16-bit S the last piece of a row that began in an earlier tile is not written to y but left,
// unrounded, in first_part[t]; the fix-up adds it to the carries and rounds the row once.
template <class V, class I, class P, class S = V>
__global__ void __launch_bounds__(SpmvShape<V>::THREADS, spmv_min_blocks<V, I>())
spmv_tile_kernel(const S* __restrict__ val, const I* __restrict__ col, const P* __restrict__ ptr,
                 const S* __restrict__ x, const S* y_in, S* y, V* __restrict__ carry,
                 V* __restrict__ first_part, const int64_t* __restrict__ tile_row,
                 int64_t n_rows, int64_t n_cols, int64_t nnz, V alpha, V beta, int has_beta,
                 int phase, int32_t* status) {
  constexpr bool kNarrow = !std::is_same<S, V>::value;
  using Shape = SpmvShape<V>;
  constexpr int THREADS = Shape::THREADS, SPT = Shape::SPT, SLOTS = Shape::SLOTS;
  constexpr int ITEMS = Shape::ITEMS;
  constexpr int WARPS = THREADS / 32;
  __shared__ uint32_t head[SLOTS / 32];
  __shared__ __align__(16) unsigned char seg_raw[sizeof(V) * SLOTS];
  __shared__ __align__(16) unsigned char wtail_raw[sizeof(V) * WARPS];
  __shared__ int whead[WARPS];
  V* seg_at = reinterpret_cast<V*>(seg_raw);    // sum of the piece that ends before a head slot
  V* wtail = reinterpret_cast<V*>(wtail_raw);   // open sum at the end of each warp

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int64_t t = blockIdx.x;
  const TileCoord tc = tile_coord(tile_row, t, ITEMS, n_rows + nnz);
  const int n_nz = static_cast<int>(tc.j1 - tc.j0);
  const int n_end = static_cast<int>(tc.r1 - tc.r0);  // rows that end in this tile

  // slot 0 sits on a vector boundary at or below the first non-zero of the tile; `phase` is the
  // element offset of the arrays' base addresses from such a boundary (-1: no common one, the
  // arrays are then read element by element)
  const int a = static_cast<int>((tc.j0 + (phase > 0 ? phase : 0)) & (SPT - 1));
  const int64_t jb = tc.j0 - a;       // non-zero index of slot 0 (may lie below the tile)
  const int sb = tid * SPT;           // first slot of this thread
  const int64_t jt = jb + sb;
  const int lo = a - sb;              // this thread's live elements are lo <= i < hi
  const int hi = a + n_nz - sb;
  const bool live = hi > 0 && lo < SPT;

  // ---- col / val of this thread's slots, and the first row end, all in flight together --------
  I c[SPT];
  V v[SPT];
  {
    S vs[SPT];  // as stored
#pragma unroll
    for (int i = 0; i < SPT; ++i) {
      c[i] = 0;
      vs[i] = storage_of<S>::from_acc(vt<V>::zero());
    }
    if (live) {
      if (phase >= 0) {
        const uint64_t once = policy_evict_first();
        load_run(col + jt, c, lo, hi, once);
        load_run(val + jt, vs, lo, hi, once);
      } else {
#pragma unroll
        for (int i = 0; i < SPT; ++i)
          if (i >= lo && i < hi) {
            c[i] = col[jt + i];
            vs[i] = val[jt + i];
          }
      }
    }
#pragma unroll
    for (int i = 0; i < SPT; ++i) v[i] = to_acc(vs[i]);
  }
  int64_t e_first = 0;
  if (tid < n_end) e_first = static_cast<int64_t>(ptr[tc.r0 + 1 + tid]);
  if (tid < SLOTS / 32) head[tid] = 0;
  __syncthreads();

  // ---- gathers of x ---------------------------------------------------------------------------
  V xv[SPT];
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    xv[i] = vt<V>::zero();
    if (i >= lo && i < hi) {
#ifdef B2S_CHECKED
      if (static_cast<uint64_t>(c[i]) >= static_cast<uint64_t>(n_cols)) {
        if (status) atomicOr(status, 1 << B2S_ERR_BOUNDS);  // never follow a column outside x
        continue;
      }
#endif
      xv[i] = to_acc(ldg_val(x + static_cast<int64_t>(c[i])));
    }
  }

  // ---- heads: the slot after the last non-zero of every row that ends here ----------------------
  // (a row end at or below slot a closes an empty piece and needs no bit; rows that end on the
  // same slot share one)
  for (int k = tid; k < n_end; k += THREADS) {
    const int64_t e64 = (k == tid ? e_first : static_cast<int64_t>(ptr[tc.r0 + 1 + k])) - jb;
#ifdef B2S_CHECKED
    if (e64 < a || e64 > a + n_nz) {  // row pointers that disagree with the tile plan
      if (status) atomicOr(status, 1 << B2S_ERR_BOUNDS);
      continue;
    }
#endif
    const int e = static_cast<int>(e64);
    if (e > a) atomicOr(&head[e >> 5], 1u << (e & 31));
  }
  if (tid == 0) atomicOr(&head[(a + n_nz) >> 5], 1u << ((a + n_nz) & 31));  // end of the tile
  __syncthreads();

  uint32_t flags;
  if constexpr (SPT == 8)
    flags = reinterpret_cast<const unsigned char*>(head)[tid];
  else
    flags = (head[tid >> 3] >> ((tid & 7) * 4)) & 15u;

  // ---- serial pass over this thread's slots -----------------------------------------------------
  // first: sum before the thread's first head (continues a piece from the lanes below);
  // acc at the end: sum after its last head (continues into the lanes above)
  V acc = vt<V>::zero(), first = vt<V>::zero();
  bool seen = false;
#pragma unroll
  for (int i = 0; i < SPT; ++i) {
    if ((flags >> i) & 1u) {
      if (!seen) {
        first = acc;
        seen = true;
      } else {
        seg_at[sb + i] = acc;
      }
      acc = vt<V>::zero();
    }
    if (i >= lo && i < hi) acc = acc + v[i] * xv[i];
  }

  // ---- open sums across the lanes of the warp ---------------------------------------------------
  const uint32_t heads_w = __ballot_sync(0xffffffffu, seen);
  const uint32_t upto = heads_w & (0xffffffffu >> (31 - lane));  // head lanes <= this lane
  const int reach = upto ? lane - (31 - __clz(upto)) : lane;     // lanes below in the same piece
  V incl = acc;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const V below = shfl_up(incl, d);
    if (d <= reach) incl = below + incl;
  }
  V cin = shfl_up(incl, 1);  // open sum that enters this lane
  if (lane == 0) cin = vt<V>::zero();
  if (lane == 31) {
    wtail[warp] = incl;
    whead[warp] = heads_w != 0;
  }
  __syncthreads();
  if (seen) {
    V total = cin;
    if ((heads_w & ((1u << lane) - 1u)) == 0) {  // the piece began in an earlier warp
      V wc = vt<V>::zero();
      for (int w = 0; w < warp; ++w) wc = whead[w] ? wtail[w] : wc + wtail[w];
      total = wc + cin;
    }
    seg_at[sb + __ffs(flags) - 1] = total + first;
  }
  __syncthreads();

  // ---- epilogue: the rows that end in this tile are consecutive, y is read and written coalesced
  for (int k = tid; k < n_end; k += THREADS) {
    const int64_t s64 = static_cast<int64_t>(ptr[tc.r0 + k]) - jb;
    const int s = s64 < a ? a : static_cast<int>(s64);
    const int e = static_cast<int>(
        (k == tid ? e_first : static_cast<int64_t>(ptr[tc.r0 + 1 + k])) - jb);
#ifdef B2S_CHECKED
    if (e < a || e > a + n_nz) continue;
#endif
    const V sum = e > s ? seg_at[e] : vt<V>::zero();
    if (kNarrow && k == 0 && s64 < a) {  // began in an earlier tile: rounded by the fix-up
      first_part[t] = sum;
      continue;
    }
    V r = alpha * sum;
    if (has_beta) r = r + beta * to_acc(y_in[tc.r0 + k]);
    y[tc.r0 + k] = storage_of<S>::from_acc(r);
  }
  if (tid == 0 && tc.r1 < n_rows) {  // the row still open at the end of the tile
    const int64_t s64 = static_cast<int64_t>(ptr[tc.r1]) - jb;
    const int s = s64 < a ? a : static_cast<int>(s64);
    const int e = a + n_nz;
    carry[t] = e > s ? seg_at[e] : vt<V>::zero();
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

// The same for 16-bit storage: the row's pieces (carries of the earlier tiles, then the piece
// the tile it ends in has left in first_part) are added in float32 and the row is rounded once.
template <class V, class S, class P>
__global__ void spmv_fixup_narrow_kernel(S* y, const S* y_in, const V* __restrict__ carry,
                                         const V* __restrict__ first_part,
                                         const int64_t* __restrict__ tile_row,
                                         const P* __restrict__ ptr, int64_t n_tiles, int items,
                                         int64_t total, V alpha, V beta, int has_beta) {
  const int64_t t = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (t < 1 || t >= n_tiles) return;
  const int64_t r = tile_row[t];
  if (tile_row[t + 1] <= r) return;  // row r does not end in tile t
  int64_t d0 = t * static_cast<int64_t>(items);
  if (d0 > total) d0 = total;
  if (static_cast<int64_t>(ptr[r]) >= d0 - r) return;  // row r starts in tile t: written there
  int64_t u0 = t - 1;
  while (u0 >= 1 && tile_row[u0] == r) --u0;
  V s = carry[u0];
  for (int64_t u = u0 + 1; u < t; ++u) s = s + carry[u];
  s = s + first_part[t];
  V out = alpha * s;
  if (has_beta) out = out + beta * to_acc(y_in[r]);
  y[r] = storage_of<S>::from_acc(out);
}

// Element offset of the two arrays from a common vector boundary, or -1 when they have
// none (then the kernel reads element by element).  Slices taken at the same element offset of
// two aligned allocations, as a row block of a larger matrix is, do have one.
template <class V, class I, class S>
int spmv_vector_phase(const void* data, const void* indices) {
  constexpr int SPT = SpmvShape<V>::SPT;
  const uintptr_t d = reinterpret_cast<uintptr_t>(data), c = reinterpret_cast<uintptr_t>(indices);
  if (d % sizeof(S) || c % sizeof(I)) return -1;
  constexpr uintptr_t vb = run_chunk_bytes<S, SPT>(), cb = run_chunk_bytes<I, SPT>();
  for (int o = 0; o < SPT; ++o)
    if ((d - o * sizeof(S)) % vb == 0 && (c - o * sizeof(I)) % cb == 0) return o;
  return -1;
}

template <class V, class I, class P, class S = V>
int spmv_launch(const void* data, const void* indices, const void* indptr, int64_t n_rows,
                int64_t n_cols, int64_t nnz, const void* x, const void* y_in, void* y, const void* alpha,
                const void* beta, const int64_t* tile_row, void* carry, int32_t* status,
                cudaStream_t stream) {
  using Shape = SpmvShape<V>;
  const int64_t n_tiles = b2s_tile_count(n_rows, nnz, Shape::ITEMS);
  if (n_tiles == 0) return B2S_OK;
  if (n_tiles > 0x7fffffffLL) return B2S_ERR_RANGE;
  const V a = *static_cast<const V*>(alpha);
  const V b = *static_cast<const V*>(beta);
  const int has_beta = vt<V>::is_zero(b) ? 0 : 1;
  if (has_beta && y_in == nullptr) return B2S_ERR_ARG;
  const int phase = nnz > 0 ? spmv_vector_phase<V, I, S>(data, indices) : 0;
  V* first_part = static_cast<V*>(carry) + n_tiles;  // used by the 16-bit dtypes only
  spmv_tile_kernel<V, I, P, S><<<static_cast<unsigned>(n_tiles), Shape::THREADS, 0, stream>>>(
      static_cast<const S*>(data), static_cast<const I*>(indices), static_cast<const P*>(indptr),
      static_cast<const S*>(x), static_cast<const S*>(y_in), static_cast<S*>(y),
      static_cast<V*>(carry), first_part, tile_row, n_rows, n_cols, nnz, a, b, has_beta, phase,
      status);
  if (n_tiles > 1) {
    const int fb = 256;
    const unsigned grid = static_cast<unsigned>((n_tiles + fb - 1) / fb);
    if constexpr (std::is_same<S, V>::value)
      spmv_fixup_kernel<V><<<grid, fb, 0, stream>>>(static_cast<V*>(y),
                                                    static_cast<const V*>(carry), tile_row,
                                                    n_tiles, a);
    else
      spmv_fixup_narrow_kernel<V, S, P><<<grid, fb, 0, stream>>>(
          static_cast<S*>(y), static_cast<const S*>(y_in), static_cast<const V*>(carry),
          first_part, tile_row, static_cast<const P*>(indptr), n_tiles, Shape::ITEMS,
          n_rows + nnz, a, b, has_beta);
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

// A thread finishes the 16 / sizeof(V) consecutive rows that make up 16 bytes of y and stores
// them to every peer with one 16-byte store (vec_ok: the peers' buffers are 16-byte aligned and
// row_offset is a multiple of that row count); ragged ends and unaligned blocks store by value.
// NVSwitch multicast: one store to an address of the multicast mapping of the ranks' buffers is
// replicated by the switch into every rank's copy (multimem.st), so a block leaves this GPU once
// instead of once per peer.  The payload travels as 32-bit lanes; a store changes no bits.
__device__ inline void multimem_store4(void* mc, uint32_t a) {
  asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(mc), "f"(__uint_as_float(a))
               : "memory");
}
__device__ inline void multimem_store8(void* mc, uint2 v) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1,%2};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y))
               : "memory");
}
__device__ inline void multimem_store16(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc),
               "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
               "f"(__uint_as_float(v.w))
               : "memory");
}
template <class V>
__device__ inline void multimem_store_value(V* mc, const V& v) {
  if constexpr (sizeof(V) == 4)
    multimem_store4(mc, *reinterpret_cast<const uint32_t*>(&v));
  else if constexpr (sizeof(V) == 8)
    multimem_store8(mc, *reinterpret_cast<const uint2*>(&v));
  else
    multimem_store16(mc, *reinterpret_cast<const uint4*>(&v));
}

// MC: peers.p[0] is the multicast address of the assembled result (n_peers is 1)
template <class V, bool MC = false>
__global__ void panel_combine_peers_kernel(const V* __restrict__ ypart,
                                           const int32_t* __restrict__ subpos, int64_t n_rows,
                                           int n_panels, const V* y_in, PeerList peers,
                                           int n_peers, int64_t row_offset, V alpha, V beta,
                                           int has_beta, int vec_ok) {
  constexpr int RP = sizeof(V) >= 16 ? 1 : 16 / static_cast<int>(sizeof(V));
  // grid-stride: with one thread per row group the loop runs once; a small grid (grid_limit of
  // the entry point) keeps the kernel to a few CTAs per SM so that it can drain over NVLink
  // beside the tile kernel of the next row block instead of filling the GPU with stalled stores
  const int64_t n_groups = (n_rows + RP - 1) / RP;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; g < n_groups;
       g += stride) {
    const int64_t r0 = g * RP;
    alignas(16) V out[RP];
#pragma unroll
    for (int j = 0; j < RP; ++j) {
      const int64_t r = r0 + j;
      V s = vt<V>::zero();
      if (r < n_rows) {
        for (int p = 0; p < n_panels; ++p) {
          if (subpos != nullptr) {
            const int32_t c = subpos[p * n_rows + r];
            if (c >= 0) s = s + ypart[c];
          } else {
            s = s + ypart[p * n_rows + r];
          }
        }
        s = alpha * s;
        if (has_beta) s = s + beta * y_in[r];
      }
      out[j] = s;
    }
    if (vec_ok && r0 + RP <= n_rows) {
      const uint4 raw = *reinterpret_cast<const uint4*>(out);
      if constexpr (MC) {
        multimem_store16(static_cast<V*>(peers.p[0]) + row_offset + r0, raw);
      } else {
        for (int q = 0; q < n_peers; ++q)
          *reinterpret_cast<uint4*>(static_cast<V*>(peers.p[q]) + row_offset + r0) = raw;
      }
    } else {
#pragma unroll
      for (int j = 0; j < RP; ++j)
        if (r0 + j < n_rows) {
          if constexpr (MC) {
            multimem_store_value(static_cast<V*>(peers.p[0]) + row_offset + r0 + j, out[j]);
          } else {
            for (int q = 0; q < n_peers; ++q)
              static_cast<V*>(peers.p[q])[row_offset + r0 + j] = out[j];
          }
        }
    }
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

}  // namespace b2s

extern "C" int b2s_spmv_tile_items(int val_type, int idx_type) {
  (void)idx_type;
  B2S_DISPATCH_VS(val_type, {
    (void)sizeof(S);
    return b2s::SpmvShape<V>::ITEMS;
  });
  return 0;
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

extern "C" int b2s_panel_combine(int val_type, const void* ypart_dev, const int32_t* subpos_dev,
                                 int64_t n_rows, int n_panels, const void* y_in_dev, void* y_dev,
                                 const void* alpha, const void* beta, b2s_stream stream) {
  if (n_rows < 0 || n_panels < 1 || n_panels > 256 || !alpha || !beta) return B2S_ERR_ARG;
  if (n_rows == 0) return B2S_OK;
  if (!ypart_dev || !y_dev) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(ypart_dev) & m) || (reinterpret_cast<uintptr_t>(y_dev) & m) ||
      (reinterpret_cast<uintptr_t>(y_in_dev) & m))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const unsigned grid = static_cast<unsigned>((n_rows + threads - 1) / threads);
  B2S_DISPATCH_V(val_type, {
    const V a = *static_cast<const V*>(alpha);
    const V b = *static_cast<const V*>(beta);
    const int has_beta = b2s::vt<V>::is_zero(b) ? 0 : 1;
    if (has_beta && y_in_dev == nullptr) return B2S_ERR_ARG;
    if (subpos_dev != nullptr)
      (b2s::panel_combine_sparse_kernel<V><<<grid, threads, 0, s>>>(
          static_cast<const V*>(ypart_dev), subpos_dev, n_rows, n_panels,
          static_cast<const V*>(y_in_dev), static_cast<V*>(y_dev), a, b, has_beta));
    else
      (b2s::panel_combine_kernel<V><<<grid, threads, 0, s>>>(
          static_cast<const V*>(ypart_dev), n_rows, n_panels, static_cast<const V*>(y_in_dev),
          static_cast<V*>(y_dev), a, b, has_beta));
  });
  return b2s::launch_status();
}

static int panel_combine_to_ranks(int val_type, const void* ypart_dev,
                                  const int32_t* subpos_dev, int64_t n_rows, int n_panels,
                                  const void* y_in_dev, void* const* peer_y, int n_peers,
                                  int64_t row_offset, int64_t peer_rows, const void* alpha,
                                  const void* beta, int grid_limit, b2s_stream stream,
                                  bool multicast) {
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
  const int64_t rows_per_thread = vs >= 16 ? 1 : 16 / static_cast<int64_t>(vs);
  int vec_ok = row_offset % rows_per_thread == 0;
  for (int q = 0; q < n_peers; ++q)
    if (reinterpret_cast<uintptr_t>(peer_y[q]) % 16) vec_ok = 0;
  const int64_t n_groups = (n_rows + rows_per_thread - 1) / rows_per_thread;
  int64_t want = (n_groups + threads - 1) / threads;
  if (grid_limit > 0 && want > grid_limit) want = grid_limit;
  const unsigned grid = static_cast<unsigned>(want);
  B2S_DISPATCH_V(val_type, {
    const V a = *static_cast<const V*>(alpha);
    const V b = *static_cast<const V*>(beta);
    const int has_beta = b2s::vt<V>::is_zero(b) ? 0 : 1;
    if (has_beta && y_in_dev == nullptr) return B2S_ERR_ARG;
    if (multicast)
      (b2s::panel_combine_peers_kernel<V, true><<<grid, threads, 0, s>>>(
          static_cast<const V*>(ypart_dev), subpos_dev, n_rows, n_panels,
          static_cast<const V*>(y_in_dev), peers, 1, row_offset, a, b, has_beta, vec_ok));
    else
      (b2s::panel_combine_peers_kernel<V, false><<<grid, threads, 0, s>>>(
          static_cast<const V*>(ypart_dev), subpos_dev, n_rows, n_panels,
          static_cast<const V*>(y_in_dev), peers, n_peers, row_offset, a, b, has_beta, vec_ok));
  });
  return b2s::launch_status();
}

extern "C" int b2s_panel_combine_peers(int val_type, const void* ypart_dev,
                                       const int32_t* subpos_dev, int64_t n_rows, int n_panels,
                                       const void* y_in_dev, void* const* peer_y, int n_peers,
                                       int64_t row_offset, int64_t peer_rows, const void* alpha,
                                       const void* beta, int grid_limit, b2s_stream stream) {
  return panel_combine_to_ranks(val_type, ypart_dev, subpos_dev, n_rows, n_panels, y_in_dev,
                                peer_y, n_peers, row_offset, peer_rows, alpha, beta, grid_limit,
                                stream, false);
}

extern "C" int b2s_panel_combine_multicast(int val_type, const void* ypart_dev,
                                           const int32_t* subpos_dev, int64_t n_rows,
                                           int n_panels, const void* y_in_dev, void* multicast_y,
                                           int64_t row_offset, int64_t peer_rows,
                                           const void* alpha, const void* beta, int grid_limit,
                                           b2s_stream stream) {
  void* one[1] = {multicast_y};
  return panel_combine_to_ranks(val_type, ypart_dev, subpos_dev, n_rows, n_panels, y_in_dev, one,
                                1, row_offset, peer_rows, alpha, beta, grid_limit, stream, true);
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
      (reinterpret_cast<uintptr_t>(carry_dev) & (b2s::acc_size(val_type) - 1)))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_VS(val_type, B2S_DISPATCH_I(idx_type, I, B2S_DISPATCH_I(ptr_type, P, {
    return (b2s::spmv_launch<V, I, P, S>(data_dev, indices_dev, indptr_dev, n_rows, n_cols, nnz, x_dev,
                                      y_in_dev, y_dev, alpha, beta, tile_row_dev, carry_dev,
                                      status_dev, s));
  })));
  return B2S_ERR_DTYPE;
}

// ---------------------------------------------------------------------------------------------
// SpMV without any allocation: tile plan and carries live in a fixed device array
// ---------------------------------------------------------------------------------------------
namespace {

constexpr int64_t kFixedMaxItems = 1 << 26;  // rows + non-zeros one call may bring
// tiles of the narrowest tile shape (complex128) that many items make
constexpr int64_t kFixedMaxTiles =
    (kFixedMaxItems + b2s::SpmvShape<b2s::c128>::ITEMS - 1) / b2s::SpmvShape<b2s::c128>::ITEMS;

struct FixedScratch {
  int64_t tile_row[kFixedMaxTiles + 1];
  alignas(16) unsigned char carry[kFixedMaxTiles * 16];  // one value of the widest dtype per tile
};

// About 3.2 MB of device memory on every GPU that loads the library, held until exit.
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
  return kFixedMaxItems;
}

extern "C" int b2s_spmv_csr_fixed(int val_type, int idx_type, int ptr_type, const void* data_dev,
                                  const void* indices_dev, const void* indptr_dev,
                                  int64_t n_rows, int64_t n_cols, int64_t nnz, const void* x_dev,
                                  const void* y_in_dev, void* y_dev, const void* alpha,
                                  const void* beta, b2s_stream stream) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0) return B2S_ERR_ARG;
  const int items = b2s_spmv_tile_items(val_type, idx_type);
  if (items <= 0) return B2S_ERR_DTYPE;
  if (n_rows + nnz > kFixedMaxItems || b2s_tile_count(n_rows, nnz, items) > kFixedMaxTiles)
    return B2S_ERR_TOO_LARGE;
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
