// CSR SpMM for sm_100a: C = alpha * A B + beta * C_in, B and C row-major.
//
// Same merge-path tiles as SpMV.  A tile's col / val range is streamed into shared memory by
// bulk asynchronous copies; rows of B are read with 16-byte loads, G lanes per B row
// (G * 16 bytes covers one dense-column tile; G is picked from N).  Each lane owns 16 bytes of
// the output row, so there is no reduction across lanes of one group; groups that share a row
// combine with a fixed butterfly (inside a warp) or a fixed-order pass over shared memory
// (whole CTA).  Rows that cross tile borders leave N-wide partials in `carry`; a second kernel
// adds them in ascending tile order.  No floating-point atomics.
#include <type_traits>

#include "b2s_tile.cuh"

namespace b2s {

#ifndef B2S_SPMM_CHUNKED
#define B2S_SPMM_CHUNKED 2  // 0: team-per-row kernel; 1: chunk kernel; 2: chunk kernel for narrow B rows
#endif
#ifndef B2S_SPMM_GROUP_NNZ
#define B2S_SPMM_GROUP_NNZ 32  // entries one group of lanes takes before a row is split over more groups
#endif
#ifndef B2S_SPMM_CHUNK_WIDE
#define B2S_SPMM_CHUNK_WIDE 16  // chunk length of the chunk kernel when B rows take more than 4 lanes
#endif
#ifndef B2S_SPMM_RUN_MEAN
#define B2S_SPMM_RUN_MEAN 12  // mean entries per row piece of a tile up to which groups walk runs of rows
#endif
#ifndef B2S_SPMM_WIN_MINBLOCKS
#define B2S_SPMM_WIN_MINBLOCKS 6  // CTAs per SM the float32 / int32 windowed kernel is compiled for
#endif
#ifndef B2S_SPMM_WIN_ITEMS
#define B2S_SPMM_WIN_ITEMS 1536  // merge items per tile of that kernel
#endif
#ifndef B2S_SPMM_THREADS
#define B2S_SPMM_THREADS 128
#endif
#ifndef B2S_SPMM_ITEMS
#define B2S_SPMM_ITEMS 1024
#endif

template <class V, class I>
struct SpmmCfg {
  static constexpr int THREADS = B2S_SPMM_THREADS;
  static constexpr int ITEMS = B2S_SPMM_ITEMS;
};

constexpr size_t kSpmmWindowMaxBytes = 32 * 1024;  // largest shared-memory window of B rows
constexpr int kSpmmWarpRowMax = 512;
constexpr int kSpmmQueue2Cap = 256;
constexpr int kSpmmQueue3Cap = 8;

// What one lane owns of a B / C row: the values held in 16 bytes of storage (S), kept as
// accumulation type V (S itself, or float for the 16-bit storage types: 8 values per lane).
template <class V, class S = V>
struct alignas(16) Pack {
  static constexpr int N = sizeof(S) >= 16 ? 1 : 16 / static_cast<int>(sizeof(S));
  V e[N];
};

template <class V, class S = V>
__device__ inline Pack<V, S> pack_zero() {
  Pack<V, S> p;
#pragma unroll
  for (int i = 0; i < Pack<V, S>::N; ++i) p.e[i] = vt<V>::zero();
  return p;
}

// 16 bytes of storage -> the lane's values in accumulation type, and back (rounding once)
template <class V, class S>
__device__ inline Pack<V, S> unpack16(const uint4& raw) {
  Pack<V, S> p;
  if constexpr (std::is_same<S, V>::value) {
    *reinterpret_cast<uint4*>(&p) = raw;
  } else {
    S s[Pack<V, S>::N];
    *reinterpret_cast<uint4*>(s) = raw;
#pragma unroll
    for (int i = 0; i < Pack<V, S>::N; ++i) p.e[i] = to_acc(s[i]);
  }
  return p;
}
template <class V, class S>
__device__ inline uint4 pack16(const Pack<V, S>& p) {
  uint4 raw;
  if constexpr (std::is_same<S, V>::value) {
    raw = *reinterpret_cast<const uint4*>(&p);
  } else {
    alignas(16) S s[Pack<V, S>::N];
#pragma unroll
    for (int i = 0; i < Pack<V, S>::N; ++i) s[i] = storage_of<S>::from_acc(p.e[i]);
    raw = *reinterpret_cast<const uint4*>(s);
  }
  return raw;
}

// load the lane's slice of B row `brow` (elements e0 .. e0+N-1 of n_dense)
template <class V, class S>
__device__ inline Pack<V, S> load_pack(const S* __restrict__ brow, int64_t e0, int64_t n_dense,
                                       bool vec_ok) {
  if (vec_ok && e0 + Pack<V, S>::N <= n_dense)
    return unpack16<V, S>(__ldg(reinterpret_cast<const uint4*>(brow + e0)));
  Pack<V, S> p;
#pragma unroll
  for (int i = 0; i < Pack<V, S>::N; ++i)
    p.e[i] = (e0 + i < n_dense) ? to_acc(ldg_val(brow + e0 + i)) : vt<V>::zero();
  return p;
}

template <class V, class S>
__device__ inline void fma_pack(Pack<V, S>& acc, V a, const Pack<V, S>& b) {
#pragma unroll
  for (int i = 0; i < Pack<V, S>::N; ++i) fma_acc(acc.e[i], a, b.e[i]);
}

template <class V, class S>
__device__ inline Pack<V, S> add_pack(const Pack<V, S>& a, const Pack<V, S>& b) {
  Pack<V, S> r;
#pragma unroll
  for (int i = 0; i < Pack<V, S>::N; ++i) r.e[i] = a.e[i] + b.e[i];
  return r;
}

template <class V, class S>
__device__ inline Pack<V, S> shfl_xor_pack(const Pack<V, S>& a, int m) {
  Pack<V, S> r;
#pragma unroll
  for (int i = 0; i < Pack<V, S>::N; ++i) r.e[i] = shfl_xor(a.e[i], m);
  return r;
}

// out[e0..] = alpha * acc + beta * in[e0..], rounded to the storage type; `cs` is the distance
// between two columns of the row (1: row-major C, one 16-byte store; n_rows: column-major C,
// one store per value, consecutive rows of a column being neighbours in memory)
template <class V, class S>
__device__ inline void store_pack(S* out, const S* in, int64_t e0, int64_t n_dense,
                                  const Pack<V, S>& acc, V alpha, V beta, bool has_beta,
                                  bool vec_ok, int64_t cs = 1) {
  if (e0 >= n_dense) return;
  constexpr int N = Pack<V, S>::N;
  Pack<V, S> r;
  if (cs != 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if (e0 + i < n_dense) {
        V v = alpha * acc.e[i];
        if (has_beta) v = v + beta * to_acc(in[(e0 + i) * cs]);
        out[(e0 + i) * cs] = storage_of<S>::from_acc(v);
      }
    }
    return;
  }
  if (vec_ok && e0 + N <= n_dense) {
    if (has_beta) {
      const Pack<V, S> old = unpack16<V, S>(*reinterpret_cast<const uint4*>(in + e0));
#pragma unroll
      for (int i = 0; i < N; ++i) r.e[i] = alpha * acc.e[i] + beta * old.e[i];
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) r.e[i] = alpha * acc.e[i];
    }
    *reinterpret_cast<uint4*>(out + e0) = pack16<V, S>(r);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      if (e0 + i < n_dense) {
        V v = alpha * acc.e[i];
        if (has_beta) v = v + beta * to_acc(in[e0 + i]);
        out[e0 + i] = storage_of<S>::from_acc(v);
      }
    }
  }
}

// unrounded partial sums (carries) in accumulation type
template <class V, class S>
__device__ inline void store_raw(V* out, int64_t e0, int64_t n_dense, const Pack<V, S>& acc) {
#pragma unroll
  for (int i = 0; i < Pack<V, S>::N; ++i)
    if (e0 + i < n_dense) out[e0 + i] = acc.e[i];
}

template <int THREADS, int ITEMS, class V, class I, class S = V>
__host__ __device__ constexpr size_t spmm_smem_bytes() {
  return 16 + sizeof(int) * (ITEMS + 4) + sizeof(I) * ITEMS + 16 + sizeof(V) * ITEMS + 16 +
         sizeof(int) * (kSpmmQueue2Cap + kSpmmQueue3Cap + 4) + sizeof(Pack<V, S>) * THREADS;
}

// Accumulate A[piece] * B over non-zeros s + first, s + first + step, ... < e of the staged tile.
// Four gathers of B are in flight per lane before the first multiply.
// VEC: every lane that owns columns owns a full, 16-byte aligned pack, so a B row slice is one
// 128-bit read-only load at Bv + col * stride16 (Bv already points at the lane's columns).
// WIN: the rows of B the tile touches have been copied to shared memory and Bv points into that
// window, shifted so that Bv + col * stride still is the row of column col (see the kernel);
// loads are then ordinary shared-memory reads and `mask_col` (the first column of the window)
// replaces column 0 as the harmless address of a masked entry.
template <bool WIN>
__device__ inline uint4 load_b16(const uint4* p) {
  if constexpr (WIN)
    return *p;
  else
    return __ldg(p);
}

template <class V, class I, bool VEC, bool WIN = false, class S = V>
__device__ inline void accumulate(Pack<V, S>& acc, const I* __restrict__ scol,
                                  const S* __restrict__ sval, int s, int e, int first, int step,
                                  const S* __restrict__ B, int64_t ldb, int64_t e0,
                                  int64_t n_dense, const uint4* Bv, int64_t stride16,
                                  uint32_t mask_col = 0) {
  int i = s + first;
  if constexpr (VEC) {
    if (e0 >= n_dense) return;  // lane beyond the last column: nothing to add
    if (stride16 < 0) {
      // all of B lies within 2^32 sixteen-byte units: 32-bit row offsets (one multiply, one
      // widening add per gather instead of a 64-bit multiply)
      const uint32_t s32 = static_cast<uint32_t>(-stride16);
      if constexpr (sizeof(I) == 4 && sizeof(V) == 4 && std::is_same<S, V>::value) {
        // consecutive entries, 4-byte col and val staged with the same 16-byte phase: four
        // columns and four values per 128-bit shared-memory read
        const unsigned phase_c = (static_cast<unsigned>(smem_addr(scol)) >> 2) & 3u;
        const unsigned phase_v = (static_cast<unsigned>(smem_addr(sval)) >> 2) & 3u;
        if (step == 1 && phase_c == phase_v) {
          // whole aligned quads from the quad that contains the first entry to the one that
          // contains the last; entries of a quad outside [i, e) are masked (column 0, not
          // added), so there are no ragged head / tail loops to diverge on (reads stay inside
          // the staging buffers: the quad below index 0 and the one above the last entry fall
          // into their 16-byte slack or the neighbouring buffer)
          if (i >= e) return;
          const int first = i;
          for (int a = i - static_cast<int>((static_cast<unsigned>(i) + phase_c) & 3u); a < e;
               a += 4) {
            uint4 c4 = *reinterpret_cast<const uint4*>(scol + a);
            Pack<V, S> a4;
            *reinterpret_cast<uint4*>(&a4) = *reinterpret_cast<const uint4*>(sval + a);
            const bool k0 = a >= first, k1 = a + 1 >= first && a + 1 < e,
                       k2 = a + 2 >= first && a + 2 < e, k3 = a + 3 < e;
            // masked entries read a row that certainly is there (row 0 of B, or the first row
            // of the window) and are not added
            if (!k0) c4.x = mask_col;
            if (!k1) c4.y = mask_col;
            if (!k2) c4.z = mask_col;
            if (!k3) c4.w = mask_col;
            Pack<V, S> b0, b1, b2, b3;
            b0 = unpack16<V, S>(load_b16<WIN>(Bv + c4.x * s32));
            b1 = unpack16<V, S>(load_b16<WIN>(Bv + c4.y * s32));
            b2 = unpack16<V, S>(load_b16<WIN>(Bv + c4.z * s32));
            b3 = unpack16<V, S>(load_b16<WIN>(Bv + c4.w * s32));
            if (k0) fma_pack(acc, a4.e[0], b0);
            if (k1) fma_pack(acc, a4.e[1], b1);
            if (k2) fma_pack(acc, a4.e[2], b2);
            if (k3) fma_pack(acc, a4.e[3], b3);
          }
          return;
        }
      }
      for (; i + 3 * step < e; i += 4 * step) {
        const uint32_t o0 = static_cast<uint32_t>(scol[i]) * s32;
        const uint32_t o1 = static_cast<uint32_t>(scol[i + step]) * s32;
        const uint32_t o2 = static_cast<uint32_t>(scol[i + 2 * step]) * s32;
        const uint32_t o3 = static_cast<uint32_t>(scol[i + 3 * step]) * s32;
        Pack<V, S> b0, b1, b2, b3;
        b0 = unpack16<V, S>(load_b16<WIN>(Bv + o0));
        b1 = unpack16<V, S>(load_b16<WIN>(Bv + o1));
        b2 = unpack16<V, S>(load_b16<WIN>(Bv + o2));
        b3 = unpack16<V, S>(load_b16<WIN>(Bv + o3));
        fma_pack(acc, to_acc(sval[i]), b0);
        fma_pack(acc, to_acc(sval[i + step]), b1);
        fma_pack(acc, to_acc(sval[i + 2 * step]), b2);
        fma_pack(acc, to_acc(sval[i + 3 * step]), b3);
      }
      for (; i < e; i += step) {
        Pack<V, S> b;
        b = unpack16<V, S>(load_b16<WIN>(Bv + static_cast<uint32_t>(scol[i]) * s32));
        fma_pack(acc, to_acc(sval[i]), b);
      }
      return;
    }
    for (; i + 3 * step < e; i += 4 * step) {
      const I c0 = scol[i], c1 = scol[i + step], c2 = scol[i + 2 * step], c3 = scol[i + 3 * step];
      Pack<V, S> b0, b1, b2, b3;
      b0 = unpack16<V, S>(__ldg(Bv + static_cast<int64_t>(c0) * stride16));
      b1 = unpack16<V, S>(__ldg(Bv + static_cast<int64_t>(c1) * stride16));
      b2 = unpack16<V, S>(__ldg(Bv + static_cast<int64_t>(c2) * stride16));
      b3 = unpack16<V, S>(__ldg(Bv + static_cast<int64_t>(c3) * stride16));
      fma_pack(acc, to_acc(sval[i]), b0);
      fma_pack(acc, to_acc(sval[i + step]), b1);
      fma_pack(acc, to_acc(sval[i + 2 * step]), b2);
      fma_pack(acc, to_acc(sval[i + 3 * step]), b3);
    }
    for (; i < e; i += step) {
      Pack<V, S> b;
      b = unpack16<V, S>(__ldg(Bv + static_cast<int64_t>(scol[i]) * stride16));
      fma_pack(acc, to_acc(sval[i]), b);
    }
  } else {
    for (; i + 3 * step < e; i += 4 * step) {
      const int64_t c0 = scol[i], c1 = scol[i + step], c2 = scol[i + 2 * step],
                    c3 = scol[i + 3 * step];
      const Pack<V, S> b0 = load_pack<V, S>(B + c0 * ldb, e0, n_dense, false);
      const Pack<V, S> b1 = load_pack<V, S>(B + c1 * ldb, e0, n_dense, false);
      const Pack<V, S> b2 = load_pack<V, S>(B + c2 * ldb, e0, n_dense, false);
      const Pack<V, S> b3 = load_pack<V, S>(B + c3 * ldb, e0, n_dense, false);
      fma_pack(acc, to_acc(sval[i]), b0);
      fma_pack(acc, to_acc(sval[i + step]), b1);
      fma_pack(acc, to_acc(sval[i + 2 * step]), b2);
      fma_pack(acc, to_acc(sval[i + 3 * step]), b3);
    }
    for (; i < e; i += step) {
      const int64_t c = scol[i];
      const Pack<V, S> b = load_pack<V, S>(B + c * ldb, e0, n_dense, false);
      fma_pack(acc, to_acc(sval[i]), b);
    }
  }
}

// Bounds-checked build: every staged column must name a row of B (and, with a window, a row of
// the window), every staged row end must lie inside the tile and not before the previous one.
// A tile that fails sets B2S_ERR_BOUNDS and is skipped by the whole CTA.
#ifdef B2S_CHECKED
template <class I>
__device__ inline bool spmm_tile_is_sound(const I* scol, const int* row_end, int n_nz, int n_end,
                                          int64_t n_cols, int64_t lo, int64_t hi, int tid,
                                          int threads, int32_t* status) {
  int bad = 0;
  for (int j = tid; j < n_nz; j += threads) {
    const int64_t c = static_cast<int64_t>(scol[j]);
    if (c < 0 || c >= n_cols || c < lo || c >= hi) bad = 1;
  }
  for (int k = tid; k <= n_end; k += threads) {
    const int e = row_end[k], s = k ? row_end[k - 1] : 0;
    if (e < s || e > n_nz || s < 0) bad = 1;
  }
  if (__syncthreads_or(bad)) {
    if (status && tid == 0) atomicOr(status, 1 << B2S_ERR_BOUNDS);
    return false;
  }
  return true;
}
#endif

// ---- float32 / int32 window path ---------------------------------------------------------------
// The staged columns and values of the tile and its window of B rows are all in shared memory;
// everything is addressed with 32-bit shared addresses (one multiply-add per gather, no generic
// loads).  A row piece [i, e) is walked in aligned quads of the staging buffers: one masked
// quad at the head, unmasked quads in the middle, one masked quad at the tail, so that the mask
// arithmetic is paid twice per row instead of once per quad.  Same order of additions as
// accumulate().
__device__ inline uint4 lds_u4(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a));
  return v;
}

template <bool MASKED>
__device__ inline void window_quad(Pack<float>& acc, uint32_t col32, uint32_t val32, int a,
                                   int first, int e, uint32_t win32, uint32_t pitch,
                                   uint32_t mask_col) {
  uint4 c4 = lds_u4(col32 + 4u * static_cast<uint32_t>(a));
  const uint4 v4 = lds_u4(val32 + 4u * static_cast<uint32_t>(a));
  bool k0 = true, k1 = true, k2 = true, k3 = true;
  if constexpr (MASKED) {
    k0 = a >= first;
    k1 = a + 1 >= first && a + 1 < e;
    k2 = a + 2 >= first && a + 2 < e;
    k3 = a + 3 < e;
    // masked entries read the first row of the window and are not added
    if (!k0) c4.x = mask_col;
    if (!k1) c4.y = mask_col;
    if (!k2) c4.z = mask_col;
    if (!k3) c4.w = mask_col;
  }
  Pack<float> b0, b1, b2, b3;
  if constexpr (MASKED) {
    // a masked entry is not loaded at all: its lanes add no wavefront to the shared-memory pipe
    b0 = b1 = b2 = b3 = pack_zero<float, float>();
    if (k0) b0 = unpack16<float, float>(lds_u4(win32 + c4.x * pitch));
    if (k1) b1 = unpack16<float, float>(lds_u4(win32 + c4.y * pitch));
    if (k2) b2 = unpack16<float, float>(lds_u4(win32 + c4.z * pitch));
    if (k3) b3 = unpack16<float, float>(lds_u4(win32 + c4.w * pitch));
  } else {
    b0 = unpack16<float, float>(lds_u4(win32 + c4.x * pitch));
    b1 = unpack16<float, float>(lds_u4(win32 + c4.y * pitch));
    b2 = unpack16<float, float>(lds_u4(win32 + c4.z * pitch));
    b3 = unpack16<float, float>(lds_u4(win32 + c4.w * pitch));
  }
  if (k0) fma_pack(acc, __uint_as_float(v4.x), b0);
  if (k1) fma_pack(acc, __uint_as_float(v4.y), b1);
  if (k2) fma_pack(acc, __uint_as_float(v4.z), b2);
  if (k3) fma_pack(acc, __uint_as_float(v4.w), b3);
}

// col32 / val32: shared addresses of the staged columns / values (same 16-byte phase);
// win32 + col * pitch: shared address of the lane's 16 bytes of B row `col`
__device__ inline void accumulate_window_quads(Pack<float>& acc, uint32_t col32, uint32_t val32,
                                               int i, int e, uint32_t win32, uint32_t pitch,
                                               uint32_t mask_col) {
  if (i >= e) return;
  int a = i - static_cast<int>((static_cast<unsigned>(i) + ((col32 >> 2) & 3u)) & 3u);
  window_quad<true>(acc, col32, val32, a, i, e, win32, pitch, mask_col);
  a += 4;
  for (; a + 4 <= e; a += 4)
    window_quad<false>(acc, col32, val32, a, i, e, win32, pitch, mask_col);
  if (a < e) window_quad<true>(acc, col32, val32, a, i, e, win32, pitch, mask_col);
}

// CTAs per SM the register allocation of the tile kernel aims at.  With 4-byte column indices and
// values of up to 8 bytes, 12 CTAs (40 registers, a few bytes of spills) measured faster than
// the 10 the compiler settles on by itself: banded float32 N = 32 1.27 -> 1.15 ms, transposed
// Poisson matrix N = 64 0.95 -> 0.81 ms, both pieces of the long-row split of the power-law
// matrix 3-6 % (same box).  With 8-byte indices the same limit made the one-launch product of
// that matrix slower (13.6 -> 15.4 ms), so those instantiations stay unconstrained.
// The windowed variants hold a window of B rows per CTA and are not squeezed into 40 registers:
// the float32 / int32 one is compiled for the 6 CTAs its 37 KB of shared memory allow (80
// registers), the others keep the compiler's choice.
template <class V, class I, bool WIN = false>
constexpr int spmm_min_blocks() {
#ifdef B2S_SPMM_MINBLOCKS
  return B2S_SPMM_MINBLOCKS;
#else
  if (WIN) return (sizeof(I) == 4 && sizeof(V) == 4) ? B2S_SPMM_WIN_MINBLOCKS : 1;
  return (sizeof(I) == 4 && sizeof(V) <= 8) ? 12 : 1;
#endif
}

// G = lanes per B row (power of two, 1..32); blockIdx.y selects the dense-column tile of
// G * Pack::N columns when N is wider than one tile.
// WIN (needs VEC, one dense-column tile, 32-bit row offsets): the rows of B between the smallest
// and the largest column of the tile are copied into shared memory by one bulk copy and every
// gather of the tile is a shared-memory read; `win_rows_cap` rows fit the buffer behind the
// other arrays (the host has checked that no tile of the matrix spans more).
// ST: storage type of val, B and C (V itself, or a 16-bit float type with V = float: eight
// columns per lane, float32 sums, one rounding).  With a 16-bit ST the last piece of a row that
// began in an earlier tile is left unrounded in first_part (one row of n_dense values per tile)
// and the fix-up rounds the row once.
template <class V, class I, class P, int THREADS, int ITEMS, bool VEC, bool WIN = false,
          class ST = V>
__global__ void __launch_bounds__(THREADS, spmm_min_blocks<V, I, WIN>())
spmm_tile_kernel(const ST* __restrict__ val, const I* __restrict__ col, const P* __restrict__ ptr,
                 const ST* __restrict__ B, int64_t ldb, int64_t n_dense, const ST* C_in, ST* C,
                 int64_t ldc, int64_t cs, V* __restrict__ carry, V* __restrict__ first_part,
                 const int64_t* __restrict__ tile_row,
                 int64_t n_rows, int64_t n_cols, int64_t nnz, V alpha, V beta, int has_beta_i,
                 int G, int small_b,
                 int vec_c, int32_t* status, int win_rows_cap = 0,
                 const int32_t* __restrict__ tile_win = nullptr) {
  static_assert(!WIN || VEC, "the shared-memory window is read with 16-byte loads");
  extern __shared__ __align__(16) unsigned char smem[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  int* row_end = reinterpret_cast<int*>(smem + 16);
  unsigned char* col_buf = smem + 16 + sizeof(int) * (ITEMS + 4);
  unsigned char* val_buf = col_buf + sizeof(I) * ITEMS + 16;
  int* queue2 = reinterpret_cast<int*>(val_buf + sizeof(V) * ITEMS + 16);
  int* queue3 = queue2 + kSpmmQueue2Cap;
  int* qcount = queue3 + kSpmmQueue3Cap;
  Pack<V, ST>* part = reinterpret_cast<Pack<V, ST>*>(qcount + 4);  // one slot per thread

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  // an earlier CTA already gave up on a copy: do not queue more waits behind it (one thread
  // reads the word and the whole CTA leaves or stays together)
  {
    const int gave_up =
        (tid == 0 && status) ? (*reinterpret_cast<volatile int32_t*>(status) != 0) : 0;
    if (__syncthreads_or(gave_up)) return;
  }
  const bool has_beta = has_beta_i != 0;
  const int64_t t = blockIdx.x;
  const TileCoord tc = tile_coord(tile_row, t, ITEMS, n_rows + nnz);
  const int n_nz = static_cast<int>(tc.j1 - tc.j0);
  const int n_end = static_cast<int>(tc.r1 - tc.r0);

  const I* gcol = col + tc.j0;
  const ST* gval = val + tc.j0;
  const Staged<I> sc = stage_layout<I>(col_buf, gcol, n_nz);
  const Staged<ST> sv = stage_layout<ST>(val_buf, gval, n_nz);
  const uint32_t tx = stage_bytes(sc) + stage_bytes(sv);
  if (tid == 0) {
    qcount[0] = 0;
    qcount[1] = 0;
    if (tx || WIN) mbar_init(bar, 1);
  }
  // WIN: first column and number of B rows of this tile's window, from the plan; the window is
  // requested together with col / val, on the same barrier
  int win_lo = 0, win_rows = 0;
  uint32_t win_bytes = 0;
  constexpr size_t win_off =
      (spmm_smem_bytes<THREADS, ITEMS, V, I, ST>() + 15) & ~static_cast<size_t>(15);
  if constexpr (WIN) {
    win_lo = tile_win[2 * t];
    win_rows = tile_win[2 * t + 1];
    if (win_rows > win_rows_cap || win_rows < 0) {  // the host sized the buffer: never expected
      if (status && tid == 0) atomicOr(status, 1 << B2S_ERR_WORKSPACE);
      return;
    }
    // whole rows but for the last one, of which only the n_dense values are read (B may be a
    // view whose last row has nothing behind it)
    if (win_rows > 0)
      win_bytes = static_cast<uint32_t>(win_rows - 1) *
                      static_cast<uint32_t>(ldb * static_cast<int64_t>(sizeof(ST))) +
                  static_cast<uint32_t>(n_dense * static_cast<int64_t>(sizeof(ST)));
  }
  __syncthreads();
  if (tid == 0 && (tx || win_bytes)) {
    const uint64_t pol = policy_evict_first();
    mbar_expect_tx(bar, tx + win_bytes);
    stage_issue(sc, gcol, bar, pol);
    stage_issue(sv, gval, bar, pol);
    if constexpr (WIN) {
      if (win_bytes)
        bulk_g2s(smem + win_off, B + static_cast<int64_t>(win_lo) * ldb, win_bytes, bar,
                 policy_evict_last());
    }
  }
  stage_edges(sc, gcol, n_nz, tid, THREADS);
  stage_edges(sv, gval, n_nz, tid, THREADS);
  for (int k = tid; k < n_end; k += THREADS)
    row_end[k] = static_cast<int>(static_cast<int64_t>(ptr[tc.r0 + 1 + k]) - tc.j0);
  if (tid == 0) row_end[n_end] = n_nz;
  // one warp waits for the copies; the CTA barrier that follows releases everybody else
  if ((tx || win_bytes) && warp == 0) {
    if (!mbar_wait(bar, 0)) {
      if (status && lane == 0) atomicOr(status, 1 << B2S_ERR_TIMEOUT);
      mbar_wait(bar, 0);  // second bounded wait: do not leave with a copy in flight
    }
  }
  __syncthreads();

  const I* scol = sc.s;
  const ST* sval = sv.s;
#ifdef B2S_CHECKED
  if (!spmm_tile_is_sound(scol, row_end, n_nz, n_end, n_cols,
                          WIN ? static_cast<int64_t>(win_lo) : 0,
                          WIN ? static_cast<int64_t>(win_lo) + win_rows : n_cols, tid, THREADS,
                          status))
    return;
#endif
  const bool open_row = tc.r1 < n_rows;
  const int n_seg = n_end + 1;
  const int64_t e0 =
      (static_cast<int64_t>(blockIdx.y) * G + (tid & (G - 1))) * Pack<V, ST>::N;  // lane's columns
  const bool vc = VEC || vec_c != 0;
  const uint4* Bv = reinterpret_cast<const uint4*>(B + (VEC && e0 < n_dense ? e0 : 0));
  int64_t stride16 = VEC ? ldb * static_cast<int64_t>(sizeof(ST)) / 16 : 0;
  if (VEC && small_b) stride16 = -stride16;  // flag for 32-bit row offsets (see accumulate)
  V* carry_row = carry + t * n_dense;
  // 16-bit storage: the tile's first row, when it began in an earlier tile, is finished (and
  // rounded once) by the fix-up; its piece here goes to first_part instead of C
  V* first_row = nullptr;
  if constexpr (!std::is_same<ST, V>::value) {
    if (tc.r0 < n_rows && static_cast<int64_t>(ptr[tc.r0]) < tc.j0)
      first_row = first_part + t * n_dense;
  }
  uint32_t mask_col = 0;
  if constexpr (WIN) {
    const uint32_t pitch = static_cast<uint32_t>(ldb * static_cast<int64_t>(sizeof(ST)));
    // base such that base + col * (pitch / 16) sixteen-byte units is the lane's slice of row col
    const uintptr_t lane_bytes = static_cast<uintptr_t>(e0 < n_dense ? e0 : 0) * sizeof(ST);
    const uintptr_t base = reinterpret_cast<uintptr_t>(smem + win_off) + lane_bytes -
                           static_cast<uintptr_t>(win_lo) * pitch;
    Bv = reinterpret_cast<const uint4*>(base);
    stride16 = -(static_cast<int64_t>(pitch) / 16);
    mask_col = static_cast<uint32_t>(win_lo);
  }

  // groups per row piece: power of two so that each group sees at most about 16 non-zeros
  const int groups_per_warp = 32 / G;
  int S = 1;
  {
    const int mean = (n_nz + n_seg - 1) / n_seg;
    while (S * B2S_SPMM_GROUP_NNZ < mean && S < groups_per_warp) S <<= 1;
  }
  // float32 / int32 window, one group per row piece: the quad walk on shared addresses
  bool quads = false;
  uint32_t col32 = 0, val32 = 0, win32 = 0, pitch32 = 0;
  if constexpr (WIN && sizeof(I) == 4 && std::is_same<V, float>::value &&
                std::is_same<ST, float>::value) {
    col32 = smem_addr(scol);
    val32 = smem_addr(sval);
    pitch32 = static_cast<uint32_t>(ldb * static_cast<int64_t>(sizeof(ST)));
    win32 = smem_addr(smem + win_off) +
            static_cast<uint32_t>((e0 < n_dense ? e0 : 0) * sizeof(ST)) -
            static_cast<uint32_t>(win_lo) * pitch32;
    quads = S == 1 && (((col32 ^ val32) >> 2) & 3u) == 0;
  }
  const int team = S * G;  // lanes per row piece
  const int p1max = (S == groups_per_warp) ? kSpmmWarpRowMax : 64 * S;

  // ---- strategy 1 for short rows: one group per run of consecutive row pieces ------------------
  // With a handful of entries per row a group that takes one row at a time has one or two
  // gathers in flight.  Here the row pieces and entries of the tile are dealt out in equal
  // shares of their merged sequence, whole pieces only; a group walks the entries of its pieces
  // as one run, four gathers in flight across row borders, and stores a row whenever the run
  // passes its end.  Sums are taken in entry order, as in the loop below.  Pieces longer than
  // p1max are left to the warp / CTA strategies as before.
  bool run_walk = false;
  if constexpr (VEC && !WIN && std::is_same<ST, V>::value) {
    // measured on the short-row part of the 2^24-row power-law matrix, N = 32 float64 (16
    // lanes per row): 11.7 -> 11.0 ms for the whole product; with 4 lanes per row (N = 16
    // float32, 2^26-row matrix) the walk was 4 % slower, so narrow rows keep the loop below
    run_walk = S == 1 && stride16 < 0 && G >= 8 &&
               (n_nz + n_seg - 1) / n_seg <= B2S_SPMM_RUN_MEAN;
  }
  if (run_walk) {
    if constexpr (VEC && !WIN && std::is_same<ST, V>::value) {
      const int team_id = tid / G;
      const int n_team = THREADS / G;
      const int total = n_seg + n_nz;
      auto first_piece = [&](int m) {   // first piece k with k + (its first entry) >= m
        int a = 0, b = n_seg;
        while (a < b) {
          const int mid = (a + b) >> 1;
          if (mid + (mid ? row_end[mid - 1] : 0) < m) a = mid + 1; else b = mid;
        }
        return a;
      };
      int k = first_piece(static_cast<int>(static_cast<int64_t>(total) * team_id / n_team));
      const int kend =
          first_piece(static_cast<int>(static_cast<int64_t>(total) * (team_id + 1) / n_team));
      const uint32_t s32 = static_cast<uint32_t>(-stride16);
      const bool owner = e0 < n_dense;            // lanes beyond the last column only follow
      auto flush = [&](int kk, const Pack<V, ST>& sum) {
        if (!owner) return;
        if (kk < n_end) {
          const int64_t r = tc.r0 + kk;
          store_pack(C + r * ldc, C_in + r * ldc, e0, n_dense, sum, alpha, beta, has_beta, vc, cs);
        } else if (open_row) {
          store_raw(carry_row, e0, n_dense, sum);
        }
      };
      int i = k ? row_end[k - 1] : 0;
      int stretch_end = i;                        // entries before it belong to short pieces
      int e_k = k < kend ? row_end[k] : 0;
      bool at_start = true;
      Pack<V, ST> acc = pack_zero<V, ST>();
      while (k < kend) {
        if (at_start) {
          if (i >= stretch_end) {
            if (e_k - i > p1max) {                // a long piece: queued, skipped here
              if ((tid & (G - 1)) == 0) {
                if (e_k - i <= kSpmmWarpRowMax) {
                  const int q = atomicAdd(&qcount[0], 1);
                  if (q < kSpmmQueue2Cap) queue2[q] = k;
                } else {
                  const int q = atomicAdd(&qcount[1], 1);
                  if (q < kSpmmQueue3Cap) queue3[q] = k;
                }
              }
              i = e_k;
              ++k;
              e_k = k < kend ? row_end[k] : 0;
              stretch_end = i;
              continue;
            }
            int j = k, pos = i;
            while (j < kend) {
              const int ej = row_end[j];
              if (ej - pos > p1max) break;
              pos = ej;
              ++j;
            }
            stretch_end = pos;
          }
          if (e_k == i) {                         // an empty piece
            flush(k, acc);
            ++k;
            e_k = k < kend ? row_end[k] : 0;
            continue;
          }
        }
        const int n = min(4, stretch_end - i);    // >= 1: piece k has an entry at i
        const int last = stretch_end - 1;
        const int i1 = min(i + 1, last), i2 = min(i + 2, last), i3 = min(i + 3, last);
        Pack<V, ST> b[4];
        b[0] = unpack16<V, ST>(__ldg(Bv + static_cast<uint32_t>(scol[i]) * s32));
        b[1] = unpack16<V, ST>(__ldg(Bv + static_cast<uint32_t>(scol[i1]) * s32));
        b[2] = unpack16<V, ST>(__ldg(Bv + static_cast<uint32_t>(scol[i2]) * s32));
        b[3] = unpack16<V, ST>(__ldg(Bv + static_cast<uint32_t>(scol[i3]) * s32));
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (j < n) {
            fma_pack(acc, to_acc(sval[i + j]), b[j]);
            at_start = false;
            while (k < kend && e_k == i + j + 1) {   // the piece ends here (and empty ones follow)
              flush(k, acc);
              acc = pack_zero<V, ST>();
              ++k;
              e_k = k < kend ? row_end[k] : 0;
              at_start = true;
            }
          }
        }
        i += n;
      }
    }
  } else {
    const int team_id = tid / team;
    const int n_team = THREADS / team;
    const int grp_in_team = (tid % team) / G;
    for (int kb = 0; kb < n_seg; kb += n_team) {
      const int k = kb + team_id;
      const bool live = k < n_seg;
      int s = 0, e = 0;
      if (live) {
        s = k ? row_end[k - 1] : 0;
        e = row_end[k];
      }
      const int len = e - s;
      Pack<V, ST> acc = pack_zero<V, ST>();
      if (len <= p1max) {
        bool done = false;
        if constexpr (WIN && sizeof(I) == 4 && std::is_same<V, float>::value &&
                      std::is_same<ST, float>::value) {
          if (quads) {
            if (e0 < n_dense)
              accumulate_window_quads(acc, col32, val32, s, e, win32, pitch32, mask_col);
            done = true;
          }
        }
        if (!done)
          accumulate<V, I, VEC, WIN, ST>(acc, scol, sval, s, e, grp_in_team, S, B, ldb, e0,
                                         n_dense, Bv, stride16, mask_col);
      } else if ((tid % team) == 0) {
        if (len <= kSpmmWarpRowMax) {
          const int q = atomicAdd(&qcount[0], 1);
          if (q < kSpmmQueue2Cap) queue2[q] = k;
        } else {
          const int q = atomicAdd(&qcount[1], 1);
          if (q < kSpmmQueue3Cap) queue3[q] = k;
        }
      }
      for (int m = team >> 1; m >= G; m >>= 1) acc = add_pack(acc, shfl_xor_pack(acc, m));
      if (live && grp_in_team == 0 && len <= p1max) {
        if (k < n_end) {
          const int64_t r = tc.r0 + k;
          if (k == 0 && first_row != nullptr)
            store_raw(first_row, e0, n_dense, acc);
          else
            store_pack(C + r * ldc, C_in + r * ldc, e0, n_dense, acc, alpha, beta, has_beta, vc, cs);
        } else if (open_row) {
          store_raw(carry_row, e0, n_dense, acc);
        }
      }
    }
  }
  __syncthreads();

  // ---- strategy 2: one warp per row piece -----------------------------------------------------
  const int n2 = min(qcount[0], kSpmmQueue2Cap);
  for (int q = warp; q < n2; q += THREADS / 32) {
    const int k = queue2[q];
    const int s = k ? row_end[k - 1] : 0;
    const int e = row_end[k];
    Pack<V, ST> acc = pack_zero<V, ST>();
    accumulate<V, I, VEC, WIN, ST>(acc, scol, sval, s, e, lane / G, groups_per_warp, B, ldb, e0,
                               n_dense, Bv, stride16, mask_col);
    for (int m = 16; m >= G; m >>= 1) acc = add_pack(acc, shfl_xor_pack(acc, m));
    if (lane < G) {
      if (k < n_end) {
        const int64_t r = tc.r0 + k;
        if (k == 0 && first_row != nullptr)
          store_raw(first_row, e0, n_dense, acc);
        else
          store_pack(C + r * ldc, C_in + r * ldc, e0, n_dense, acc, alpha, beta, has_beta, vc, cs);
      } else if (open_row) {
        store_raw(carry_row, e0, n_dense, acc);
      }
    }
  }

  // ---- strategy 3: the whole CTA on one row piece ---------------------------------------------
  const int n3 = min(qcount[1], kSpmmQueue3Cap);
  const int n_grp = THREADS / G;
  for (int q = 0; q < n3; ++q) {
    const int k = queue3[q];
    const int s = k ? row_end[k - 1] : 0;
    const int e = row_end[k];
    Pack<V, ST> acc = pack_zero<V, ST>();
    accumulate<V, I, VEC, WIN, ST>(acc, scol, sval, s, e, tid / G, n_grp, B, ldb, e0, n_dense, Bv,
                               stride16, mask_col);
    part[tid] = acc;
    __syncthreads();
    if (tid < G) {
      Pack<V, ST> tot = part[tid];
      for (int g = 1; g < n_grp; ++g) tot = add_pack(tot, part[g * G + tid]);
      if (k < n_end) {
        const int64_t r = tc.r0 + k;
        if (k == 0 && first_row != nullptr)
          store_raw(first_row, e0, n_dense, tot);
        else
          store_pack(C + r * ldc, C_in + r * ldc, e0, n_dense, tot, alpha, beta, has_beta, vc, cs);
      } else if (open_row) {
        store_raw(carry_row, e0, n_dense, tot);
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// Chunked SpMM tile kernel.  The staged non-zeros of a tile are cut into chunks of CH consecutive
// entries; a team of G lanes takes a chunk, issues the B-row gathers of the chunk in batches of 8
// (every lane has up to 8 independent 16-byte loads in flight whatever the row lengths are), and
// walks the chunk in order, flushing a row whenever its end is passed.  A row that lies inside
// one chunk is stored at once.  The first row that ends in a chunk may have begun in earlier
// chunks: its partial goes to shared memory (`first`), as does the partial of the row still
// open at the chunk's end (`carry`); a second pass adds, for every such first row, the carries
// of the preceding chunks in ascending order.  Work per team is uniform (CH entries), sums have
// a fixed order, nothing is atomic.
// ---------------------------------------------------------------------------------------------
constexpr int kSpmmMaxChunks = B2S_SPMM_ITEMS / 4;
static_assert(B2S_SPMM_ITEMS <= 4 * kSpmmMaxChunks, "the shortest chunk has 4 entries");

template <int ITEMS, class V, class I>
constexpr size_t spmm_chunk_smem_base() {
  return 16 + sizeof(int) * (ITEMS + 4) + sizeof(I) * ITEMS + 16 + sizeof(V) * ITEMS + 16 +
         sizeof(int) * 2 * kSpmmMaxChunks;
}

template <class V, class I, class P, int THREADS, int ITEMS, bool VEC>
__global__ void __launch_bounds__(THREADS)
spmm_chunk_kernel(const V* __restrict__ val, const I* __restrict__ col,
                  const P* __restrict__ ptr, const V* __restrict__ B, int64_t ldb,
                  int64_t n_dense, const V* C_in, V* C, int64_t ldc, int64_t cs,
                  V* __restrict__ carry, const int64_t* __restrict__ tile_row, int64_t n_rows,
                  int64_t n_cols, int64_t nnz, V alpha, V beta, int has_beta_i, int G, int CH,
                  int vec_c,
                  int32_t* status) {
  extern __shared__ __align__(16) unsigned char smem[];
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  int* row_end = reinterpret_cast<int*>(smem + 16);
  unsigned char* col_buf = smem + 16 + sizeof(int) * (ITEMS + 4);
  unsigned char* val_buf = col_buf + sizeof(I) * ITEMS + 16;
  int* first_k = reinterpret_cast<int*>(val_buf + sizeof(V) * ITEMS + 16);
  int* open_k = first_k + kSpmmMaxChunks;
  Pack<V>* slots = reinterpret_cast<Pack<V>*>(open_k + kSpmmMaxChunks);  // [chunk][2][G]

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  {
    const int gave_up =
        (tid == 0 && status) ? (*reinterpret_cast<volatile int32_t*>(status) != 0) : 0;
    if (__syncthreads_or(gave_up)) return;
  }
  const bool has_beta = has_beta_i != 0;
  const int64_t t = blockIdx.x;
  const TileCoord tc = tile_coord(tile_row, t, ITEMS, n_rows + nnz);
  const int n_nz = static_cast<int>(tc.j1 - tc.j0);
  const int n_end = static_cast<int>(tc.r1 - tc.r0);

  const I* gcol = col + tc.j0;
  const V* gval = val + tc.j0;
  const Staged<I> sc = stage_layout<I>(col_buf, gcol, n_nz);
  const Staged<V> sv = stage_layout<V>(val_buf, gval, n_nz);
  const uint32_t tx = stage_bytes(sc) + stage_bytes(sv);
  if (tid == 0 && tx) mbar_init(bar, 1);
  __syncthreads();
  if (tid == 0 && tx) {
    const uint64_t pol = policy_evict_first();
    mbar_expect_tx(bar, tx);
    stage_issue(sc, gcol, bar, pol);
    stage_issue(sv, gval, bar, pol);
  }
  stage_edges(sc, gcol, n_nz, tid, THREADS);
  stage_edges(sv, gval, n_nz, tid, THREADS);
  for (int k = tid; k < n_end; k += THREADS)
    row_end[k] = static_cast<int>(static_cast<int64_t>(ptr[tc.r0 + 1 + k]) - tc.j0);
  if (tid == 0) row_end[n_end] = n_nz;
  if (tx && warp == 0) {
    if (!mbar_wait(bar, 0)) {
      if (status && lane == 0) atomicOr(status, 1 << B2S_ERR_TIMEOUT);
      mbar_wait(bar, 0);
    }
  }
  __syncthreads();
#ifdef B2S_CHECKED
  if (!spmm_tile_is_sound(sc.s, row_end, n_nz, n_end, n_cols, 0, n_cols, tid, THREADS, status))
    return;
#endif

  const I* scol = sc.s;
  const V* sval = sv.s;
  const bool open_row = tc.r1 < n_rows;
  const int sub = tid & (G - 1);
  const int team = tid / G;
  const int n_teams = THREADS / G;
  const int64_t e0 = (static_cast<int64_t>(blockIdx.y) * G + sub) * Pack<V>::N;  // lane's columns
  const bool lane_on = e0 < n_dense;
  const bool vc = VEC || vec_c != 0;
  const uint4* Bv = reinterpret_cast<const uint4*>(B + (VEC && lane_on ? e0 : 0));
  const int64_t stride16 = VEC ? ldb * static_cast<int64_t>(sizeof(V)) / 16 : 0;
  V* carry_row = carry + t * n_dense;
  const int n_chunks = n_nz > 0 ? (n_nz + CH - 1) / CH : 1;

  auto load_b = [&](I c) -> Pack<V> {
    Pack<V> b;
    if constexpr (VEC) {
      if (lane_on)
        *reinterpret_cast<uint4*>(&b) = __ldg(Bv + static_cast<int64_t>(c) * stride16);
      else
        b = pack_zero<V>();
    } else {
      b = load_pack<V, V>(B + static_cast<int64_t>(c) * ldb, e0, n_dense, false);
    }
    return b;
  };
  auto store_row = [&](int k, const Pack<V>& acc) {
    const int64_t r = tc.r0 + k;
    store_pack(C + r * ldc, C_in + r * ldc, e0, n_dense, acc, alpha, beta, has_beta, vc, cs);
  };

  // rows without entries in this tile: alpha * 0 + beta * C_in, all teams in parallel
  for (int k = team; k < n_end; k += n_teams) {
    const int s = k ? row_end[k - 1] : 0;
    if (row_end[k] == s) store_row(k, pack_zero<V>());
  }

  // ---- pass 1: one team per chunk ---------------------------------------------------------------
  for (int c = team; c < n_chunks; c += n_teams) {
    const int i0 = c * CH;
    const int i1 = min(i0 + CH, n_nz);
    int k = 0;
    if (c > 0) {  // first piece whose end lies beyond i0
      int lo = 0, hi = n_end;
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (row_end[mid] <= i0) lo = mid + 1; else hi = mid;
      }
      k = lo;
    }
    int start = k ? row_end[k - 1] : 0;
    int next_end = k < n_end ? row_end[k] : 0x7fffffff;
    int fk = -1;
    Pack<V> acc = pack_zero<V>();
    Pack<V>* my_first = slots + (static_cast<size_t>(c) * 2 + 0) * G + sub;
    Pack<V>* my_carry = slots + (static_cast<size_t>(c) * 2 + 1) * G + sub;

    auto pass_ends = [&](int upto) {  // flush every piece that ends at or before `upto`
      while (next_end <= upto) {
        if (next_end > start) {  // pieces without entries were written above
          if (fk < 0) {
            fk = k;
            *my_first = acc;
          } else {
            store_row(k, acc);
          }
          acc = pack_zero<V>();
        }
        start = next_end;
        ++k;
        next_end = k < n_end ? row_end[k] : 0x7fffffff;
      }
    };

    for (int b0 = i0; b0 < i1; b0 += 8) {
      Pack<V> bb[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (b0 + u < i1) bb[u] = load_b(scol[b0 + u]);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = b0 + u;
        if (i < i1) {
          pass_ends(i);
          fma_pack(acc, sval[i], bb[u]);
        }
      }
    }
    pass_ends(i1);
    *my_carry = acc;  // partial of the piece still open at the end of the chunk
    if (sub == 0) {
      first_k[c] = fk;
      open_k[c] = k;
    }
  }
  __syncthreads();

  // ---- pass 2: complete the first row of every chunk with the carries before it ----------------
  for (int c = team; c < n_chunks; c += n_teams) {
    const int fk = first_k[c];
    if (fk < 0) continue;
    int c_lo = c;
    while (c_lo > 0 && open_k[c_lo - 1] == fk) --c_lo;
    Pack<V> tot = slots[(static_cast<size_t>(c) * 2 + 0) * G + sub];
    if (c_lo < c) {
      Pack<V> run = slots[(static_cast<size_t>(c_lo) * 2 + 1) * G + sub];
      for (int cc = c_lo + 1; cc < c; ++cc)
        run = add_pack(run, slots[(static_cast<size_t>(cc) * 2 + 1) * G + sub]);
      tot = add_pack(run, tot);
    }
    store_row(fk, tot);
  }
  if (team == 0 && open_row) {  // what this tile contributes to the row that continues after it
    int c_lo = n_chunks;
    while (c_lo > 0 && open_k[c_lo - 1] == n_end) --c_lo;
    Pack<V> run = pack_zero<V>();
    if (c_lo < n_chunks) {
      run = slots[(static_cast<size_t>(c_lo) * 2 + 1) * G + sub];
      for (int cc = c_lo + 1; cc < n_chunks; ++cc)
        run = add_pack(run, slots[(static_cast<size_t>(cc) * 2 + 1) * G + sub]);
    }
    store_raw(carry_row, e0, n_dense, run);
  }
}

template <class V>
__global__ void spmm_fixup_kernel(V* C, int64_t ldc, int64_t cs, int64_t n_dense,
                                  const V* __restrict__ carry,
                                  const int64_t* __restrict__ tile_row, int64_t n_tiles,
                                  V alpha) {
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t t = idx / n_dense;
  const int64_t n = idx - t * n_dense;
  if (t < 1 || t >= n_tiles) return;
  const int64_t r = tile_row[t];
  if (tile_row[t + 1] <= r) return;
  int64_t u0 = t - 1;
  while (u0 >= 1 && tile_row[u0] == r) --u0;
  V s = carry[u0 * n_dense + n];
  for (int64_t u = u0 + 1; u < t; ++u) s = s + carry[u * n_dense + n];
  C[r * ldc + n * cs] = C[r * ldc + n * cs] + alpha * s;
}

// 16-bit storage: the pieces of the row (carries of the earlier tiles, then the piece the tile
// it ends in left in first_part) are added in float32 and the row is rounded once.
template <class V, class S, class P>
__global__ void spmm_fixup_narrow_kernel(S* C, const S* C_in, int64_t ldc, int64_t cs,
                                         int64_t n_dense,
                                         const V* __restrict__ carry,
                                         const V* __restrict__ first_part,
                                         const int64_t* __restrict__ tile_row,
                                         const P* __restrict__ ptr, int64_t n_tiles, int items,
                                         int64_t total, V alpha, V beta, int has_beta) {
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t t = idx / n_dense;
  const int64_t n = idx - t * n_dense;
  if (t < 1 || t >= n_tiles) return;
  const int64_t r = tile_row[t];
  if (tile_row[t + 1] <= r) return;
  int64_t d0 = t * static_cast<int64_t>(items);
  if (d0 > total) d0 = total;
  if (static_cast<int64_t>(ptr[r]) >= d0 - r) return;  // row r starts in tile t: written there
  int64_t u0 = t - 1;
  while (u0 >= 1 && tile_row[u0] == r) --u0;
  V s = carry[u0 * n_dense + n];
  for (int64_t u = u0 + 1; u < t; ++u) s = s + carry[u * n_dense + n];
  s = s + first_part[t * n_dense + n];
  V out = alpha * s;
  if (has_beta) out = out + beta * to_acc(C_in[r * ldc + n * cs]);
  C[r * ldc + n * cs] = storage_of<S>::from_acc(out);
}

// Tile length of the windowed kernel.  float32 values with int32 columns (the quad walk) run
// 1536-item tiles, 6 CTAs per SM: on the banded benchmark matrix 0.79 ms against 1.03 ms with
// 1024-item tiles at 5 CTAs (more rows per tile for the 16 teams, a smaller share of halo rows
// in the window).
template <class V, class I>
constexpr int spmm_window_items() {
  return (std::is_same<V, float>::value && sizeof(I) == 4) ? B2S_SPMM_WIN_ITEMS
                                                             : SpmmCfg<V, I>::ITEMS;
}

// Whether the windowed kernel can run this product: whole, 16-byte aligned packs in B, C and
// C_in, one dense-column tile, 32-bit row offsets into B, the window within its buffer.
template <class V>
bool spmm_window_usable(const void* B, int64_t ldb, int64_t n_dense, const void* C_in,
                        const void* C, int64_t ldc, int64_t n_cols, int64_t window_rows) {
  constexpr int PN = Pack<V>::N;
  if (window_rows <= 0 || n_dense <= 0 || n_dense % PN != 0) return false;
  if ((n_dense + PN - 1) / PN > 32) return false;
  const bool aligned = reinterpret_cast<uintptr_t>(B) % 16 == 0 && (ldb * sizeof(V)) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(C) % 16 == 0 && (ldc * sizeof(V)) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(C_in) % 16 == 0;
  if (!aligned) return false;
  if (static_cast<double>(n_cols) * static_cast<double>(ldb) * sizeof(V) / 16.0 >= 4.0e9)
    return false;
  return static_cast<uint64_t>(window_rows) * static_cast<uint64_t>(ldb) * sizeof(V) <=
         kSpmmWindowMaxBytes;
}

template <class V, class I, class P, class S = V>
int spmm_launch(const void* data, const void* indices, const void* indptr, int64_t n_rows,
                int64_t n_cols, int64_t nnz, const void* B, int64_t ldb, int64_t n_dense, const void* C_in,
                void* C, int64_t ldc, const void* alpha, const void* beta,
                const int64_t* tile_row, void* carry, int32_t* status, cudaStream_t stream,
                int64_t window_rows = 0, const int32_t* tile_win = nullptr, int64_t cs = 1) {
  using Cfg = SpmmCfg<V, I>;
  constexpr int THREADS = Cfg::THREADS, ITEMS = Cfg::ITEMS;
  constexpr int WITEMS = spmm_window_items<V, I>();
  // with a window the caller's tile plan, window table and carries are those of WITEMS-item tiles
  const bool windowed = window_rows > 0;
  if (windowed) {
    if (!std::is_same<S, V>::value || tile_win == nullptr || cs != 1 ||
        !spmm_window_usable<V>(B, ldb, n_dense, C_in, C, ldc, n_cols, window_rows))
      return B2S_ERR_ARG;
  }
  const int64_t n_tiles = b2s_tile_count(n_rows, nnz, windowed ? WITEMS : ITEMS);
  if (n_tiles == 0 || n_dense == 0) return B2S_OK;
  if (n_tiles > 0x7fffffffLL) return B2S_ERR_RANGE;
  const V a = *static_cast<const V*>(alpha);
  const V b = *static_cast<const V*>(beta);
  const int has_beta = vt<V>::is_zero(b) ? 0 : 1;
  if (has_beta && C_in == nullptr) return B2S_ERR_ARG;
  constexpr int PN = Pack<V, S>::N;
  constexpr bool kNarrow = !std::is_same<S, V>::value;
  V* first_part = static_cast<V*>(carry) + n_tiles * n_dense;  // 16-bit dtypes only
  // lanes per B row: enough 16-byte slices to cover N, at most a warp
  const int64_t slices = (n_dense + PN - 1) / PN;
  int G = 1;
  while (G < slices && G < 32) G <<= 1;
  const int64_t col_tiles = (slices + G - 1) / G;
  if (col_tiles > 65535) return B2S_ERR_RANGE;
  const int vec_b = (reinterpret_cast<uintptr_t>(B) % 16 == 0) && ((ldb * sizeof(S)) % 16 == 0);
  const int vec_c = cs == 1 && (reinterpret_cast<uintptr_t>(C) % 16 == 0) &&
                    ((ldc * sizeof(S)) % 16 == 0) &&
                    (!has_beta || reinterpret_cast<uintptr_t>(C_in) % 16 == 0);
  dim3 grid(static_cast<unsigned>(n_tiles), static_cast<unsigned>(col_tiles));
  // fast path: every pack is whole and 16-byte aligned in B, C and C_in
  const bool vec = vec_b && vec_c && (n_dense % PN == 0);
  // B spans fewer than 2^32 sixteen-byte units (64 GB): row offsets fit 32 bits
  const int small_b = (static_cast<double>(n_cols) * static_cast<double>(ldb) * sizeof(S) / 16.0) < 4.0e9;
  // Two tile kernels.  Narrow rows of B (G <= 4 lanes, e.g. N = 16 float32): the chunk kernel,
  // where every team has 8 gathers in flight whatever the row lengths (measured on the 2^26-row
  // power-law matrix, N = 16: 30 ms against 40 ms).  Wider rows: the team-per-row kernel, whose
  // smaller footprint keeps more CTAs resident (N = 32 float64 on the 2^24-row matrix: 18.5 ms
  // against 35 ms; banded N = 32 float32: 1.4 ms against 3.1 ms).
  // With 4-byte column indices the team-per-row kernel (12 CTAs per SM) is the faster one for
  // narrow rows too: the two pieces of the long-row split of that matrix, N = 16, take
  // 18.7 + 4.8 ms against 21.1 + 9.8 ms with the chunk kernel.
  const bool chunked = !kNarrow && !windowed && (B2S_SPMM_CHUNKED == 1 ||
                                    (B2S_SPMM_CHUNKED == 2 && G <= 4 && sizeof(I) == 8));
  if constexpr (kNarrow) {
    // 16-bit storage: the team-per-row kernel only (no chunk kernel, no shared-memory window)
    constexpr size_t smem = spmm_smem_bytes<THREADS, ITEMS, V, I, S>();
    auto launch = [&](auto kern) {
      ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem);
      kern<<<grid, THREADS, smem, stream>>>(
          static_cast<const S*>(data), static_cast<const I*>(indices),
          static_cast<const P*>(indptr), static_cast<const S*>(B), ldb, n_dense,
          static_cast<const S*>(C_in), static_cast<S*>(C), ldc, cs, static_cast<V*>(carry),
          first_part, tile_row, n_rows, n_cols, nnz, a, b, has_beta, G, small_b, vec_c, status, 0,
          nullptr);
    };
    if (vec)
      launch(spmm_tile_kernel<V, I, P, THREADS, ITEMS, true, false, S>);
    else
      launch(spmm_tile_kernel<V, I, P, THREADS, ITEMS, false, false, S>);
    if (n_tiles > 1) {
      const int fb = 256;
      const int64_t work = n_tiles * n_dense;
      spmm_fixup_narrow_kernel<V, S, P><<<static_cast<unsigned>((work + fb - 1) / fb), fb, 0,
                                          stream>>>(
          static_cast<S*>(C), static_cast<const S*>(C_in), ldc, cs, n_dense,
          static_cast<const V*>(carry), first_part, tile_row, static_cast<const P*>(indptr),
          n_tiles, ITEMS, n_rows + nnz, a, b, has_beta);
    }
    return launch_status();
  } else if (chunked) {
    // shorter chunks for very narrow rows: all teams busy
    const int CH = G > 4 ? B2S_SPMM_CHUNK_WIDE : (G == 4 ? 16 : 4 * G);
    const size_t smem = spmm_chunk_smem_base<ITEMS, V, I>() +
                        static_cast<size_t>(ITEMS / CH) * 2 * G * sizeof(Pack<V>);
    constexpr size_t smem_max = spmm_chunk_smem_base<ITEMS, V, I>() +
                                static_cast<size_t>(ITEMS / 16) * 2 * 32 * sizeof(Pack<V>);
    auto launch = [&](auto kern) {
      ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem_max);
      kern<<<grid, THREADS, smem, stream>>>(
          static_cast<const V*>(data), static_cast<const I*>(indices),
          static_cast<const P*>(indptr), static_cast<const V*>(B), ldb, n_dense,
          static_cast<const V*>(C_in), static_cast<V*>(C), ldc, cs, static_cast<V*>(carry),
          tile_row, n_rows, n_cols, nnz, a, b, has_beta, G, CH, vec_c, status);
    };
    if (vec)
      launch(spmm_chunk_kernel<V, I, P, THREADS, ITEMS, true>);
    else
      launch(spmm_chunk_kernel<V, I, P, THREADS, ITEMS, false>);
  } else if (windowed) {
    // the B rows of every tile fit a shared-memory window: gather from there
    constexpr size_t base =
        (spmm_smem_bytes<THREADS, WITEMS, V, I>() + 15) & ~static_cast<size_t>(15);
    const size_t smem = base + static_cast<size_t>(window_rows) * static_cast<size_t>(ldb) * sizeof(V);
    auto kern = spmm_tile_kernel<V, I, P, THREADS, WITEMS, true, true>;
    ensure_dyn_smem(reinterpret_cast<const void*>(kern), base + kSpmmWindowMaxBytes);
    kern<<<grid, THREADS, smem, stream>>>(
        static_cast<const V*>(data), static_cast<const I*>(indices),
        static_cast<const P*>(indptr), static_cast<const V*>(B), ldb, n_dense,
        static_cast<const V*>(C_in), static_cast<V*>(C), ldc, cs, static_cast<V*>(carry),
        first_part, tile_row, n_rows, n_cols, nnz, a, b, has_beta, G, small_b, vec_c, status,
        static_cast<int>(window_rows), tile_win);
  } else {
    constexpr size_t smem = spmm_smem_bytes<THREADS, ITEMS, V, I>();
    auto launch = [&](auto kern) {
      ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem);
      kern<<<grid, THREADS, smem, stream>>>(
          static_cast<const V*>(data), static_cast<const I*>(indices),
          static_cast<const P*>(indptr), static_cast<const V*>(B), ldb, n_dense,
          static_cast<const V*>(C_in), static_cast<V*>(C), ldc, cs, static_cast<V*>(carry),
          first_part, tile_row, n_rows, n_cols, nnz, a, b, has_beta, G, small_b, vec_c, status, 0,
          nullptr);
    };
    if (vec)
      launch(spmm_tile_kernel<V, I, P, THREADS, ITEMS, true>);
    else
      launch(spmm_tile_kernel<V, I, P, THREADS, ITEMS, false>);
  }
  if (n_tiles > 1) {
    const int fb = 256;
    const int64_t work = n_tiles * n_dense;
    spmm_fixup_kernel<V><<<static_cast<unsigned>((work + fb - 1) / fb), fb, 0, stream>>>(
        static_cast<V*>(C), ldc, cs, n_dense, static_cast<const V*>(carry), tile_row, n_tiles, a);
  }
  return launch_status();
}

}  // namespace b2s

extern "C" int b2s_spmm_tile_items(int val_type, int idx_type) {
  (void)val_type;
  (void)idx_type;
  return b2s::SpmmCfg<float, int32_t>::ITEMS;
}

extern "C" int b2s_spmm_window_tile_items(int val_type, int idx_type) {
  return (val_type == B2S_F32 && idx_type == B2S_I32) ? b2s::spmm_window_items<float, int32_t>()
                                                      : b2s::SpmmCfg<float, int32_t>::ITEMS;
}

extern "C" int b2s_spmm_window_usable(int val_type, const void* B_dev, int64_t ldb,
                                      int64_t n_dense, const void* C_in_dev, const void* C_dev,
                                      int64_t ldc, int64_t n_cols, int64_t window_rows) {
  switch (val_type) {
    case B2S_F32: return b2s::spmm_window_usable<float>(B_dev, ldb, n_dense, C_in_dev, C_dev, ldc, n_cols, window_rows);
    case B2S_F64: return b2s::spmm_window_usable<double>(B_dev, ldb, n_dense, C_in_dev, C_dev, ldc, n_cols, window_rows);
    case B2S_C64: return b2s::spmm_window_usable<b2s::c64>(B_dev, ldb, n_dense, C_in_dev, C_dev, ldc, n_cols, window_rows);
    case B2S_C128: return b2s::spmm_window_usable<b2s::c128>(B_dev, ldb, n_dense, C_in_dev, C_dev, ldc, n_cols, window_rows);
    default: return 0;
  }
}

namespace b2s {

// Widest column span (largest - smallest column + 1) over the tiles of a matrix: one CTA per
// tile, a block-wide min / max of the tile's column indices, one atomicMax per tile.
template <class I>
__global__ void __launch_bounds__(256)
    spmm_window_stat_kernel(const I* __restrict__ col, const int64_t* __restrict__ tile_row,
                            int64_t n_rows, int64_t nnz, int items,
                            unsigned long long* __restrict__ widest,
                            int32_t* __restrict__ tile_win) {
  __shared__ long long s_lo[8], s_hi[8];
  const TileCoord tc = tile_coord(tile_row, blockIdx.x, items, n_rows + nnz);
  long long lo = INT64_MAX, hi = -1;
  for (int64_t j = tc.j0 + threadIdx.x; j < tc.j1; j += blockDim.x) {
    const long long c = static_cast<long long>(col[j]);
    lo = c < lo ? c : lo;
    hi = c > hi ? c : hi;
  }
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) {
    const long long ol = __shfl_xor_sync(0xffffffffu, lo, m);
    const long long oh = __shfl_xor_sync(0xffffffffu, hi, m);
    lo = ol < lo ? ol : lo;
    hi = oh > hi ? oh : hi;
  }
  if ((threadIdx.x & 31) == 0) {
    s_lo[threadIdx.x >> 5] = lo;
    s_hi[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < static_cast<int>(blockDim.x >> 5); ++w) {
      lo = s_lo[w] < lo ? s_lo[w] : lo;
      hi = s_hi[w] > hi ? s_hi[w] : hi;
    }
    const long long span = hi >= lo ? hi - lo + 1 : 0;
    if (span > 0) atomicMax(widest, static_cast<unsigned long long>(span));
    if (tile_win != nullptr) {  // first column and rows of the tile's window (0 rows: no entries)
      const bool fits = span > 0 && hi <= 0x7fffffffLL;
      tile_win[2 * static_cast<int64_t>(blockIdx.x)] = fits ? static_cast<int32_t>(lo) : 0;
      tile_win[2 * static_cast<int64_t>(blockIdx.x) + 1] =
          fits ? static_cast<int32_t>(span) : (span > 0 ? 0x7fffffff : 0);
    }
  }
}

__global__ void spmm_window_zero_kernel(unsigned long long* widest) { *widest = 0ull; }

}  // namespace b2s

extern "C" int b2s_spmm_window_stat(int idx_type, const void* indices_dev, int64_t n_rows,
                                    int64_t nnz, const int64_t* tile_row_dev, int tile_items,
                                    int64_t* widest_dev, int32_t* tile_win_dev,
                                    b2s_stream stream) {
  if (n_rows < 0 || nnz < 0 || tile_items <= 0 || !widest_dev) return B2S_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  unsigned long long* out = reinterpret_cast<unsigned long long*>(widest_dev);
  b2s::spmm_window_zero_kernel<<<1, 1, 0, s>>>(out);
  const int64_t n_tiles = b2s_tile_count(n_rows, nnz, tile_items);
  if (n_tiles == 0 || nnz == 0) return b2s::launch_status();
  if (!indices_dev || !tile_row_dev) return B2S_ERR_ARG;
  if (n_tiles > 0x7fffffffLL) return B2S_ERR_RANGE;
  B2S_DISPATCH_I(idx_type, I, {
    (b2s::spmm_window_stat_kernel<I><<<static_cast<unsigned>(n_tiles), 256, 0, s>>>(
        static_cast<const I*>(indices_dev), tile_row_dev, n_rows, nnz, tile_items, out,
        tile_win_dev));
  });
  return b2s::launch_status();
}

static int spmm_csr_any(int val_type, int idx_type, int ptr_type, const void* data_dev,
                        const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                        int64_t n_cols, int64_t nnz, const void* B_dev, int64_t ldb,
                        int64_t n_dense, const void* C_in_dev, void* C_dev, int64_t ldc,
                        const void* alpha, const void* beta, const int64_t* tile_row_dev,
                        void* carry_dev, int32_t* status_dev, b2s_stream stream,
                        int64_t window_rows, const int32_t* tile_win_dev, int64_t c_col_stride);

extern "C" int b2s_spmm_csr(int val_type, int idx_type, int ptr_type, const void* data_dev,
                            const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                            int64_t n_cols, int64_t nnz, const void* B_dev, int64_t ldb,
                            int64_t n_dense, const void* C_in_dev, void* C_dev, int64_t ldc,
                            const void* alpha, const void* beta, const int64_t* tile_row_dev,
                            void* carry_dev, int32_t* status_dev, b2s_stream stream) {
  return spmm_csr_any(val_type, idx_type, ptr_type, data_dev, indices_dev, indptr_dev, n_rows,
                      n_cols, nnz, B_dev, ldb, n_dense, C_in_dev, C_dev, ldc, alpha, beta,
                      tile_row_dev, carry_dev, status_dev, stream, 0, nullptr, 1);
}

extern "C" int b2s_spmm_csr_windowed(int val_type, int idx_type, int ptr_type,
                                     const void* data_dev, const void* indices_dev,
                                     const void* indptr_dev, int64_t n_rows, int64_t n_cols,
                                     int64_t nnz, const void* B_dev, int64_t ldb, int64_t n_dense,
                                     const void* C_in_dev, void* C_dev, int64_t ldc,
                                     const void* alpha, const void* beta,
                                     const int64_t* tile_row_dev, void* carry_dev,
                                     int32_t* status_dev, int64_t window_rows,
                                     const int32_t* tile_win_dev, b2s_stream stream) {
  if (window_rows < 0 || window_rows > 0x7fffffffLL) return B2S_ERR_ARG;
  if (window_rows > 0 && !tile_win_dev) return B2S_ERR_ARG;
  return spmm_csr_any(val_type, idx_type, ptr_type, data_dev, indices_dev, indptr_dev, n_rows,
                      n_cols, nnz, B_dev, ldb, n_dense, C_in_dev, C_dev, ldc, alpha, beta,
                      tile_row_dev, carry_dev, status_dev, stream, window_rows, tile_win_dev, 1);
}

extern "C" int b2s_spmm_csr_colmajor_c(int val_type, int idx_type, int ptr_type,
                                       const void* data_dev, const void* indices_dev,
                                       const void* indptr_dev, int64_t n_rows, int64_t n_cols,
                                       int64_t nnz, const void* B_dev, int64_t ldb,
                                       int64_t n_dense, const void* C_in_dev, void* C_dev,
                                       int64_t ldc_col, const void* alpha, const void* beta,
                                       const int64_t* tile_row_dev, void* carry_dev,
                                       int32_t* status_dev, b2s_stream stream) {
  if (ldc_col < n_rows) return B2S_ERR_ARG;
  // element (r, n) of C at r + n * ldc_col: row stride 1, column stride ldc_col
  return spmm_csr_any(val_type, idx_type, ptr_type, data_dev, indices_dev, indptr_dev, n_rows,
                      n_cols, nnz, B_dev, ldb, n_dense, C_in_dev, C_dev, 1, alpha, beta,
                      tile_row_dev, carry_dev, status_dev, stream, 0, nullptr, ldc_col);
}

static int spmm_csr_any(int val_type, int idx_type, int ptr_type, const void* data_dev,
                        const void* indices_dev, const void* indptr_dev, int64_t n_rows,
                        int64_t n_cols, int64_t nnz, const void* B_dev, int64_t ldb,
                        int64_t n_dense, const void* C_in_dev, void* C_dev, int64_t ldc,
                        const void* alpha, const void* beta, const int64_t* tile_row_dev,
                        void* carry_dev, int32_t* status_dev, b2s_stream stream,
                        int64_t window_rows, const int32_t* tile_win_dev, int64_t c_col_stride) {
  if (n_rows < 0 || n_cols < 0 || nnz < 0 || n_dense < 0 || !alpha || !beta) return B2S_ERR_ARG;
  if (n_rows == 0 || n_dense == 0) return B2S_OK;
  if (ldb < n_dense || (c_col_stride == 1 && ldc < n_dense)) return B2S_ERR_ARG;
  if (!indptr_dev || !C_dev || !tile_row_dev || !carry_dev) return B2S_ERR_ARG;
  if (nnz > 0 && (!data_dev || !indices_dev || !B_dev)) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(data_dev) & m) || (reinterpret_cast<uintptr_t>(B_dev) & m) ||
      (reinterpret_cast<uintptr_t>(C_dev) & m) || (reinterpret_cast<uintptr_t>(C_in_dev) & m) ||
      (reinterpret_cast<uintptr_t>(carry_dev) & (b2s::acc_size(val_type) - 1)))
    return B2S_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B2S_DISPATCH_VS(val_type, B2S_DISPATCH_I(idx_type, I, B2S_DISPATCH_I(ptr_type, P, {
    return (b2s::spmm_launch<V, I, P, S>(data_dev, indices_dev, indptr_dev, n_rows, n_cols, nnz, B_dev, ldb,
                                      n_dense, C_in_dev, C_dev, ldc, alpha, beta, tile_row_dev,
                                      carry_dev, status_dev, s, window_rows, tile_win_dev,
                                      c_col_stride));
  })));
  return B2S_ERR_DTYPE;
}

// ---- long rows by column panel ---------------------------------------------------------------
// The long rows of a matrix, taken out and re-laid as a stack of column panels (one stacked row
// per (panel, long row) that has entries), are multiplied by the same tile kernel into one
// partial row of C per stacked row.  This kernel adds the partials of each long row in ascending
// panel order and accumulates alpha times the sum into the row of C the long row belongs to
// (which the product over the remaining rows has already set to beta * C_in).
namespace b2s {

template <class V>
__global__ void spmm_rows_combine_kernel(const V* __restrict__ part,
                                         const int32_t* __restrict__ subpos,
                                         const int64_t* __restrict__ rows, int64_t n_long,
                                         int n_panels, int64_t n_dense, V* C, int64_t ldc,
                                         V alpha) {
  const int64_t idx = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (idx >= n_long * n_dense) return;
  const int64_t j = idx / n_dense;
  const int64_t n = idx - j * n_dense;
  V s = vt<V>::zero();
  for (int p = 0; p < n_panels; ++p) {
    const int32_t c = subpos[p * n_long + j];
    if (c >= 0) s = s + part[c * n_dense + n];
  }
  V* out = C + rows[j] * ldc + n;
  *out = *out + alpha * s;
}

}  // namespace b2s

extern "C" int b2s_spmm_rows_combine(int val_type, const void* part_dev,
                                     const int32_t* subpos_dev, const int64_t* rows_dev,
                                     int64_t n_long, int n_panels, int64_t n_dense, void* C_dev,
                                     int64_t ldc, const void* alpha, b2s_stream stream) {
  if (n_long < 0 || n_dense < 0 || n_panels < 1 || n_panels > 256 || !alpha) return B2S_ERR_ARG;
  if (n_long == 0 || n_dense == 0) return B2S_OK;
  if (ldc < n_dense || !part_dev || !subpos_dev || !rows_dev || !C_dev) return B2S_ERR_ARG;
  const size_t vs = b2s::vsize(val_type);
  if (vs == 0) return B2S_ERR_DTYPE;
  const uintptr_t m = vs - 1;
  if ((reinterpret_cast<uintptr_t>(part_dev) & m) || (reinterpret_cast<uintptr_t>(C_dev) & m))
    return B2S_ERR_ALIGNMENT;
  const int64_t work = n_long * n_dense;
  const int threads = 256;
  const int64_t grid = (work + threads - 1) / threads;
  if (grid > 0x7fffffffLL) return B2S_ERR_RANGE;
  B2S_DISPATCH_V(val_type, {
    (b2s::spmm_rows_combine_kernel<V><<<static_cast<unsigned>(grid), threads, 0,
                                        static_cast<cudaStream_t>(stream)>>>(
        static_cast<const V*>(part_dev), subpos_dev, rows_dev, n_long, n_panels, n_dense,
        static_cast<V*>(C_dev), ldc, *static_cast<const V*>(alpha)));
    return b2s::launch_status();
  });
  return B2S_ERR_DTYPE;
}
