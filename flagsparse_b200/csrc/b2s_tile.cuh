// Merge-path tiles: coordinates of a tile and staging of its col / val range in shared memory.
#pragma once
#include "b2s_common.cuh"

namespace b2s {

// A tile is `ITEMS` consecutive entries of the merged sequence "row-end markers + non-zeros".
// Tile t starts at merge coordinate (row r0, non-zero j0) with r0 + j0 = min(t*ITEMS, R + nnz).
struct TileCoord {
  int64_t r0, r1;  // rows r0 .. r1-1 END inside the tile; row r1 (if < R) is still open at its end
  int64_t j0, j1;  // the tile holds non-zeros j0 .. j1-1
};

// from the two plan entries of tile t (r0 = tile_row[t], r1 = tile_row[t + 1])
__device__ inline TileCoord tile_coord_from(int64_t r0, int64_t r1, int64_t t, int items,
                                            int64_t total) {
  TileCoord c;
  c.r0 = r0;
  c.r1 = r1;
  int64_t d0 = t * (int64_t)items;
  if (d0 > total) d0 = total;
  int64_t d1 = d0 + items;
  if (d1 > total) d1 = total;
  c.j0 = d0 - c.r0;
  c.j1 = d1 - c.r1;
  return c;
}

__device__ inline TileCoord tile_coord(const int64_t* __restrict__ tile_row, int64_t t,
                                       int items, int64_t total) {
  TileCoord c;
  c.r0 = tile_row[t];
  c.r1 = tile_row[t + 1];
  int64_t d0 = t * (int64_t)items;
  if (d0 > total) d0 = total;
  int64_t d1 = d0 + items;
  if (d1 > total) d1 = total;
  c.j0 = d0 - c.r0;
  c.j1 = d1 - c.r1;
  return c;
}

// Where a global range g[0..n) sits in a 16-byte aligned shared buffer so that the part of the
// range that starts on a 16-byte boundary in global memory also starts on one in shared memory.
// That part (body) is fetched by one bulk copy; the ragged head and tail (< 16 bytes each) are
// fetched with ordinary loads.  The buffer needs n*sizeof(E) + 16 bytes.
template <class E>
struct Staged {
  E* s;      // shared address of element 0
  int head;  // elements before the body
  int body;  // elements in the body (body*sizeof(E) is a multiple of 16)
};

template <class E>
__device__ inline Staged<E> stage_layout(unsigned char* buf16, const E* g, int n) {
  const uintptr_t ga = reinterpret_cast<uintptr_t>(g);
  const int hb = static_cast<int>((16 - (ga & 15)) & 15);  // bytes up to the next boundary
  Staged<E> st;
  st.s = reinterpret_cast<E*>(buf16 + ((16 - hb) & 15));
  int head = hb / static_cast<int>(sizeof(E));
  if (head > n) head = n;
  st.head = head;
  const int per16 = sizeof(E) >= 16 ? 1 : 16 / static_cast<int>(sizeof(E));
  st.body = ((n - head) / per16) * per16;
  return st;
}

template <class E>
__device__ inline uint32_t stage_bytes(const Staged<E>& st) {
  return static_cast<uint32_t>(st.body) * static_cast<uint32_t>(sizeof(E));
}

// one thread
template <class E>
__device__ inline void stage_issue(const Staged<E>& st, const E* g, uint64_t* bar,
                                   uint64_t policy) {
  if (st.body > 0) bulk_g2s(st.s + st.head, g + st.head, stage_bytes(st), bar, policy);
}

// all threads
template <class E>
__device__ inline void stage_edges(const Staged<E>& st, const E* __restrict__ g, int n, int tid,
                                   int nthreads) {
  for (int i = tid; i < st.head; i += nthreads) st.s[i] = g[i];
  for (int i = st.head + st.body + tid; i < n; i += nthreads) st.s[i] = g[i];
}

// per-device, per-kernel opt-in to more than 48 KB of dynamic shared memory
void ensure_dyn_smem(const void* kernel, size_t bytes);  // b2s_api.cu

}  // namespace b2s
