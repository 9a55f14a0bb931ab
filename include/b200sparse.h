/*
 * b200sparse.h -- C ABI of libb200sparse.so: CSR SpMV / SpMM for NVIDIA B200 (sm_100a).
 *
 * The library is the device side of the Python functions flagsparse_spmv_csr and
 * flagsparse_spmm_csr.  FlagSparse itself has no native interface (its kernels are Triton
 * functions launched from Python), so every entry point below cites the Python function or
 * Triton kernel of FlagSparse whose work it takes over
 * (paths are relative to the FlagSparse source tree).
 *
 * Conventions
 *   - every pointer argument named *_dev is a CUDA device pointer on the current device;
 *     alpha / beta are HOST pointers to one scalar of the value dtype;
 *   - nothing here allocates, frees or synchronises: scratch memory is passed in by the caller,
 *     kernels are enqueued on `stream` and the call returns at once;
 *   - every function returns a b2s_status (0 = ok); none throws, aborts or traps;
 *   - value pointers must be aligned to the value size (16 bytes for complex128).
 */
#ifndef B200SPARSE_H_
#define B200SPARSE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2S_VERSION 100

typedef enum {
  B2S_OK = 0,
  B2S_ERR_DTYPE = 1,      /* unknown value / index dtype code                     */
  B2S_ERR_ARG = 2,        /* null pointer, negative size, inconsistent sizes      */
  B2S_ERR_ALIGNMENT = 3,  /* a pointer is not aligned to its element size         */
  B2S_ERR_LAUNCH = 4,     /* cudaGetLastError() reported a launch failure         */
  B2S_ERR_TIMEOUT = 5,    /* (device status word) a bounded wait in a kernel ran out */
  B2S_ERR_WORKSPACE = 6,  /* scratch buffer smaller than *_bytes() asked for      */
  B2S_ERR_RANGE = 7,      /* a size does not fit the requested index dtype        */
  B2S_ERR_TOO_LARGE = 8,  /* problem exceeds the fixed scratch of b2s_spmv_csr_fixed */
  B2S_ERR_BOUNDS = 9      /* (device status word, bounds-checked build only) a column index or
                             row pointer read from the matrix points outside its array; the
                             access was skipped                                       */
} b2s_status;

/* value dtypes (FlagSparse's SUPPORTED_VALUE_DTYPES, _common.py:21-29).  B2S_F16 / B2S_BF16:
 * the matrix values AND the dense operand AND the result are 16-bit arrays; every sum is a
 * float32 sum and the result is rounded once, the arithmetic FlagSparse's launchers do for these
 * dtypes (spmv_csr.py:124-129, spmm_csr.py:2716-2719) without its float32 copies; alpha / beta
 * then point at float32 scalars.  Accepted by b2s_spmv_csr, b2s_spmm_csr and b2s_csr2csc. */
typedef enum {
  B2S_F32 = 0, B2S_F64 = 1, B2S_C64 = 2, B2S_C128 = 3, B2S_F16 = 4, B2S_BF16 = 5
} b2s_vtype;
/* index dtypes (SUPPORTED_INDEX_DTYPES, _common.py:30) */
typedef enum { B2S_I32 = 0, B2S_I64 = 1 } b2s_itype;

/* Opaque CUDA stream handle (cudaStream_t); 0 is the legacy default stream. */
typedef void* b2s_stream;

int b2s_version(void);
const char* b2s_status_string(int status);

/* Failure-path self-test (no counterpart in the reference): launches one warp that waits, with
 * `spin_limit` (1..100000) bounded tries of about a microsecond each, on a barrier nothing
 * completes.  The wait runs out, bit B2S_ERR_TIMEOUT is ORed into *status_dev and the kernel
 * returns normally -- the behaviour every bounded wait in the library has when a copy is lost. */
int b2s_selftest_wait_timeout(int32_t* status_dev, int spin_limit, b2s_stream stream);

/* ---- input contract ------------------------------------------------------------------------
 * Replaces the device reductions behind the `.item()` checks of _prepare_spmv_csr_matrix
 * (spmv_csr.py:546-563) and _prepare_spmm_csr_matrix (spmm_csr.py:268-296).  One pass over
 * indptr and indices fills eight int64 words at stats_dev:
 *   [0] indptr[0]   [1] indptr[n_rows]   [2] number of i with indptr[i+1] < indptr[i]
 *   [3] min column  [4] max column       [5] max row length   [6] number of empty rows
 *   [7] reserved (0)
 * The caller zero-initialises nothing: the first kernel does.  min/max are INT64_MAX/INT64_MIN
 * when nnz == 0.
 */
int b2s_csr_inspect(const void* indptr_dev, int ptr_type, const void* indices_dev, int idx_type,
                    int64_t n_rows, int64_t nnz, int64_t* stats_dev, b2s_stream stream);

/* ---- tile plan -----------------------------------------------------------------------------
 * A plan cuts the merged sequence "row ends + non-zeros" of a CSR matrix into tiles of
 * `tile_items` entries (merge-path).  It replaces the per-call bucket construction of
 * _build_spmv_opt_buckets (spmv_csr.py:353-399) and the split-row bookkeeping of
 * _spmm_csr_split_part / _split_reduce (spmm_csr.py:2368-2402, 2969-3109).
 * b2s_tile_count gives the number of tiles T; the plan is (T+1) int64 words (first row of
 * each tile) written to tile_row_dev.
 */
int64_t b2s_tile_count(int64_t n_rows, int64_t nnz, int tile_items);
int b2s_tile_plan(const void* indptr_dev, int ptr_type, int64_t n_rows, int64_t nnz,
                  int tile_items, int64_t* tile_row_dev, b2s_stream stream);

/* Tile size (merge items per CTA) the SpMV / SpMM kernels of this build were compiled for. */
int b2s_spmv_tile_items(int val_type, int idx_type);
int b2s_spmm_tile_items(int val_type, int idx_type);

/* ---- SpMV ----------------------------------------------------------------------------------
 * y = alpha * A x + beta * y_in.  Replaces _spmv_csr_real_kernel (spmv_csr.py:167-192),
 * _spmv_csr_complex_kernel (:196-227) and the bucketed kernels (:234-351) with their launchers
 * (:412-461, :679-723).  One launch of the tile kernel plus one launch of the carry fix-up.
 *   y_in_dev  may be NULL when *beta == 0, and may equal y_dev;
 *   carry_dev scratch of T values (T = b2s_tile_count(..., b2s_spmv_tile_items(...))); for the
 *             16-bit dtypes 2 T float32 values (the second half holds the last piece of every
 *             row that crosses a tile border, so that such a row is rounded once, after all
 *             of its pieces have been added in float32);
 *   status_dev one int32 the kernels OR error bits into (B2S_ERR_TIMEOUT); may be NULL.
 * The result is bit-identical from run to run: no floating-point atomics, fixed reduction trees.
 */
int b2s_spmv_csr(int val_type, int idx_type, int ptr_type,
                 const void* data_dev, const void* indices_dev, const void* indptr_dev,
                 int64_t n_rows, int64_t n_cols, int64_t nnz,
                 const void* x_dev, const void* y_in_dev, void* y_dev,
                 const void* alpha, const void* beta,
                 const int64_t* tile_row_dev, void* carry_dev, int32_t* status_dev,
                 b2s_stream stream);

/* ---- SpMV for callers that may not allocate ----------------------------------------------------
 * No counterpart in the reference.  b2s_spmv_csr needs a tile plan and a carry buffer that the
 * caller allocates.  Some callers cannot: a service that handed all device memory to its own
 * arena at start-up, a solver loop under a no-allocation-after-initialisation rule, a plug-in
 * whose host owns the allocator.  b2s_spmv_csr_fixed computes the same y = alpha * A x +
 * beta * y_in with the same kernels and takes both scratch areas from one fixed array inside the
 * library (about 3.2 MB per GPU, held from library load to process exit).  It calls no
 * cudaMalloc / cudaFree and no allocating library routine.
 *   - Limit: n_rows + nnz <= b2s_spmv_csr_fixed_max_items() (67,108,864); larger problems return
 *     B2S_ERR_TOO_LARGE and launch nothing.
 *   - The tile plan is rebuilt on every call (one extra small kernel), so the call costs a few
 *     microseconds more than b2s_spmv_csr with a cached plan.
 *   - The first call on each device looks up the array's device address (current device must be
 *     the one the pointers live on); make that first call before any stream capture begins.
 *   - All calls on a device share the array, which keeps the last call's contents.  Nothing in
 *     it needs clearing between calls, but two calls whose kernels overlap on the GPU (different
 *     streams, no ordering) race on it: order them.
 */
int64_t b2s_spmv_csr_fixed_max_items(void);
int b2s_spmv_csr_fixed(int val_type, int idx_type, int ptr_type,
                       const void* data_dev, const void* indices_dev, const void* indptr_dev,
                       int64_t n_rows, int64_t n_cols, int64_t nnz,
                       const void* x_dev, const void* y_in_dev, void* y_dev,
                       const void* alpha, const void* beta, b2s_stream stream);

/* ---- column-panel layout for SpMV -------------------------------------------------------------
 * No counterpart in the reference.  When x is larger than the L2 cache, gathers of x miss and
 * each miss moves a 64-byte DRAM burst for 8 useful bytes.  b2s_panel_build re-lays the matrix
 * out once as a stack of n_panels (<= 256) CSR matrices over the same rows, panel p holding the
 * entries with col >> panel_shift == p (stable, so the order inside a row is kept), columns
 * stored panel-local as int32.  p_ptr has n_panels * n_rows + 1 entries of p_ptr_type;
 * panel_start_dev has n_panels + 1 int64 entries.
 * b2s_panel_compact drops the empty rows of the stack (a row with few entries is empty in most
 * panels): called with c_ptr_dev == NULL it fills subpos_dev (n_panels * n_rows int32: position
 * of each stacked row among the non-empty ones, or -1) and *count_dev; called again with
 * c_ptr_dev it writes the count + 1 row pointers of the non-empty rows.
 */
int64_t b2s_panel_compact_bytes(int64_t n_stacked);
int b2s_panel_compact(const void* p_ptr_dev, int p_ptr_type, int64_t n_stacked,
                      int32_t* subpos_dev, int64_t* count_dev, void* c_ptr_dev,
                      int64_t n_compact, void* scratch_dev, int64_t scratch_bytes,
                      b2s_stream stream);
int64_t b2s_panel_bytes(int64_t n_cols, int64_t nnz);
int b2s_panel_build(int val_type, int idx_type, int ptr_type,
                    const void* data_dev, const void* indices_dev, const void* indptr_dev,
                    int64_t n_rows, int64_t n_cols, int64_t nnz, int n_panels, int panel_shift,
                    void* p_data_dev, int32_t* p_cols_dev, void* p_ptr_dev, int p_ptr_type,
                    int64_t* panel_start_dev, void* scratch_dev, int64_t scratch_bytes,
                    b2s_stream stream);
/* The same re-layout with the caller's (global) column numbers kept, as int32 (n_cols must not
 * exceed 2^31): the stack then is an ordinary CSR matrix whose rows are sorted by panel, which
 * the SpMM kernel can multiply as it is (see b2s_spmm_rows_combine). */
int b2s_panel_build_global(int val_type, int idx_type, int ptr_type,
                           const void* data_dev, const void* indices_dev, const void* indptr_dev,
                           int64_t n_rows, int64_t n_cols, int64_t nnz, int n_panels,
                           int panel_shift, void* p_data_dev, int32_t* p_cols_dev,
                           void* p_ptr_dev, int p_ptr_type, int64_t* panel_start_dev,
                           void* scratch_dev, int64_t scratch_bytes, b2s_stream stream);

/* ---- SpMV over the end-flag stack ---------------------------------------------------------------
 * No counterpart in the reference (its kernels walk row pointers, spmv_csr.py:167-192).  Once the
 * stack of panels holds non-empty rows only, the row pointers are folded into the column words:
 *   bit 31  the entry is the LAST of its stacked row,
 *   bit 30  padding entry (adds nothing; its column bits are 0),
 *   low bits the panel-local column.
 * s_data_dev / s_cols_dev hold n_entries such entries, n_entries a multiple of the tile size
 * b2s_spmv_stack_tile_items(val_type) (pad behind the last real entry), both arrays
 * 32-byte aligned.  tile_ord_dev[t] (n_entries / tile + 1 int64 entries) is the number of end
 * flags before entry t * tile, i.e. the ordinal of the stacked row active at the start of tile
 * t.  The kernels write ypart_dev[r] = (sum of the products of stacked row r) for all
 * n_stacked rows; carry_dev is scratch of n_entries / tile values.  The per-panel partials are
 * then added per matrix row by b2s_panel_combine (or b2s_panel_combine_peers).
 *
 * b2s_spmv_stack: wide panels (n_panels <= 256 of 2^panel_shift columns, the x slice of a panel
 * sized for L2); panel_start_dev[p] = first entry of panel p (n_panels + 1 entries),
 * tile_panel_dev[t] = panel of the first entry of tile t; both may be NULL when n_panels == 1.
 * b2s_spmv_stack_tiles is the same kernel over tiles [tile_begin, tile_begin + tile_count)
 * only, with the carry fix-up (which needs every tile done) run when run_fixup != 0: a caller
 * whose x arrives slice by slice launches the tiles of a panel as soon as that panel's slice of
 * x is in place and asks for the fix-up with the last range.
 *
 * b2s_spmv_stack_shared: narrow panels of 2^panel_shift <= b2s_spmv_stack_shared_cols(val_type)
 * columns for the long rows of a matrix.  Every panel is padded to whole tiles; CTA u copies
 * the x slice of panel unit_dev[3u] into shared memory (one bulk copy) and multiplies tiles
 * unit_dev[3u + 1] .. + unit_dev[3u + 2] - 1 of that panel from there, so the gathers of x never
 * leave the SM.  status_dev: bit B2S_ERR_TIMEOUT if the bulk copy did not arrive.
 *
 * b2s_spmv_stack_rows_combine: the stacked rows here are (panel, long row) pairs; seg_ids_dev
 * [seg_ptr_dev[j] .. seg_ptr_dev[j + 1]) lists the stacked rows of long row j in ascending panel
 * order and the call writes their sum (fixed order) to out_dev[j].  The host side points the
 * position table of the wide-panel stack at these sums (one more "stacked row" per long row
 * behind the n_stacked real ones), so that b2s_panel_combine / b2s_panel_combine_peers add them
 * like any other partial.  n_part is the number of stacked rows (the bounds-checked build
 * verifies seg_ids against it).
 */
int b2s_spmv_stack_tile_items(int val_type);
int b2s_spmv_stack_shared_cols(int val_type);
int b2s_spmv_stack(int val_type, const void* s_data_dev, const uint32_t* s_cols_dev,
                   int64_t n_entries, int64_t n_stacked, int64_t n_cols, int n_panels,
                   int panel_shift, const int64_t* panel_start_dev,
                   const int32_t* tile_panel_dev, const int64_t* tile_ord_dev,
                   const void* x_dev, void* ypart_dev, void* carry_dev, int32_t* status_dev,
                   b2s_stream stream);
int b2s_spmv_stack_tiles(int val_type, const void* s_data_dev, const uint32_t* s_cols_dev,
                         int64_t n_entries, int64_t n_stacked, int64_t n_cols, int n_panels,
                         int panel_shift, const int64_t* panel_start_dev,
                         const int32_t* tile_panel_dev, const int64_t* tile_ord_dev,
                         const void* x_dev, void* ypart_dev, void* carry_dev,
                         int32_t* status_dev, int64_t tile_begin, int64_t tile_count,
                         int run_fixup, b2s_stream stream);
int b2s_spmv_stack_shared(int val_type, const void* s_data_dev, const uint32_t* s_cols_dev,
                          int64_t n_entries, int64_t n_stacked, int64_t n_cols, int panel_shift,
                          const int32_t* unit_dev, int64_t n_units,
                          const int64_t* tile_ord_dev, const void* x_dev, void* ypart_dev,
                          void* carry_dev, int32_t* status_dev, b2s_stream stream);
int b2s_spmv_stack_rows_combine(int val_type, const void* part_dev, const int64_t* seg_ptr_dev,
                                const int32_t* seg_ids_dev, int64_t n_long, int64_t n_part,
                                void* out_dev, int32_t* status_dev, b2s_stream stream);
/* y = alpha * (sum over panels p of ypart[subpos[p * n_rows + r]], ascending p) + beta * y_in,
 * for every matrix row r (subpos_dev == NULL: ypart holds n_panels * n_rows values, none
 * dropped).  y_in_dev may be NULL when *beta == 0 and may equal y_dev. */
int b2s_panel_combine(int val_type, const void* ypart_dev, const int32_t* subpos_dev,
                      int64_t n_rows, int n_panels, const void* y_in_dev, void* y_dev,
                      const void* alpha, const void* beta, b2s_stream stream);

/* ---- all-gather fused into the last kernel (several GPUs, no counterpart in the reference) ----
 * In a row-partitioned product every rank owns rows [row_offset, row_offset + n_rows) of the
 * assembled y and every rank wants all of y.  peer_y is a HOST array of n_peers (<= 16) device
 * pointers: the y buffer (peer_rows rows) of each rank, this rank's own included, as addresses
 * that kernels of the current device may write (symmetric / peer-mapped memory).
 * b2s_panel_combine_peers is b2s_panel_combine storing each value into all of them (plain
 * coalesced stores over NVLink) instead of into a local y; b2s_peer_scatter does the same for
 * an already computed block of bytes (16-byte multiples; peer_bytes = size of each
 * destination buffer), e.g. the C block of an SpMM.  Blocks that would not fit the destination
 * are refused.  The caller orders the ranks afterwards (any barrier across the ranks after these
 * kernels have finished); neither call waits for a peer.
 */
int b2s_peer_scatter(const void* src_dev, int64_t bytes, void* const* peer_dst, int n_peers,
                     int64_t dst_offset_bytes, int64_t peer_bytes, b2s_stream stream);
/* The combine + store step: adds the per-panel partials b2s_spmv_stack left in ypart_dev,
 * applies alpha / beta and stores into the peers.  A call of its own so that it can run on a
 * second stream while the tile kernel of the next row block is already running.  grid_limit > 0 caps the number of CTAs
 * (256 threads each, grid-stride over the rows): on a high-priority stream a few CTAs per SM
 * drain over NVLink beside the other kernel instead of occupying every free slot with stores
 * that wait for the link; 0 = one thread per row. */
int b2s_panel_combine_peers(int val_type, const void* ypart_dev, const int32_t* subpos_dev,
                            int64_t n_rows, int n_panels, const void* y_in_dev,
                            void* const* peer_y, int n_peers, int64_t row_offset,
                            int64_t peer_rows, const void* alpha, const void* beta,
                            int grid_limit, b2s_stream stream);
/* The same step with ONE store per value: multicast_y is the address of the assembled result in
 * a multicast mapping of the ranks' buffers (NVSwitch replicates a multimem.st into every
 * rank's copy, this rank's included), so a block leaves the GPU once instead of once per peer.
 * The caller provides the mapping (e.g. the multicast pointer of a symmetric-memory
 * allocation) and orders the ranks afterwards as above. */
int b2s_panel_combine_multicast(int val_type, const void* ypart_dev, const int32_t* subpos_dev,
                                int64_t n_rows, int n_panels, const void* y_in_dev,
                                void* multicast_y, int64_t row_offset, int64_t peer_rows,
                                const void* alpha, const void* beta, int grid_limit,
                                b2s_stream stream);

/* ---- dense transpose ---------------------------------------------------------------------------
 * dst[c * ld_dst + r] = src[r * ld_src + c] for a rows x cols matrix of 2-, 4-, 8- or 16-byte
 * elements.  Serves dense_layout="col" of the prepared SpMM route (_run_spmm_csr_base_route,
 * spmm_csr.py:713-788, with _materialize_dense_layout :617-627): a column-major B is turned
 * into the row-major operand the SpMM kernel gathers whole rows from, and the row-major result
 * into the column-major C the caller gets.  (The reference instead hands its kernel the two
 * strides of B and C and gathers single elements.) */
int b2s_dense_transpose(int elem_bytes, const void* src_dev, int64_t rows, int64_t cols,
                        int64_t ld_src, void* dst_dev, int64_t ld_dst, b2s_stream stream);

/* ---- SpMM ----------------------------------------------------------------------------------
 * C = alpha * A B + beta * C_in, B (n_cols x n_dense, leading dimension ldb) and
 * C (n_rows x n_dense, leading dimension ldc) row-major.  Replaces _spmm_csr_real_kernel
 * (spmm_csr.py:135-176), _spmm_csr_complex_kernel (:181-237) and _triton_spmm_csr_impl
 * (:2684-2789).  carry_dev: scratch of T * n_dense values with
 * T = b2s_tile_count(..., b2s_spmm_tile_items(...)); for B2S_F16 / B2S_BF16 2 * T * n_dense
 * float32 values (see b2s_spmv_csr) -- with those dtypes a lane owns eight columns of a row.
 */
int b2s_spmm_csr(int val_type, int idx_type, int ptr_type,
                 const void* data_dev, const void* indices_dev, const void* indptr_dev,
                 int64_t n_rows, int64_t n_cols, int64_t nnz,
                 const void* B_dev, int64_t ldb, int64_t n_dense,
                 const void* C_in_dev, void* C_dev, int64_t ldc,
                 const void* alpha, const void* beta,
                 const int64_t* tile_row_dev, void* carry_dev, int32_t* status_dev,
                 b2s_stream stream);

/* The same product with C (and C_in) column-major: element (r, n) at r + n * ldc_col
 * (ldc_col >= n_rows).  Serves dense_layout="col" of the prepared route
 * (_run_spmm_csr_base_route, spmm_csr.py:713-788, which hands its kernel the strides of C): the
 * kernel stores each value of a row by itself (the 16-byte store of the row-major case does
 * not apply), rows handled by neighbouring lane groups being neighbours in memory.  B is read
 * row-major as always. */
int b2s_spmm_csr_colmajor_c(int val_type, int idx_type, int ptr_type,
                            const void* data_dev, const void* indices_dev,
                            const void* indptr_dev, int64_t n_rows, int64_t n_cols, int64_t nnz,
                            const void* B_dev, int64_t ldb, int64_t n_dense,
                            const void* C_in_dev, void* C_dev, int64_t ldc_col,
                            const void* alpha, const void* beta,
                            const int64_t* tile_row_dev, void* carry_dev, int32_t* status_dev,
                            b2s_stream stream);

/* Banded / local matrices (no counterpart in the reference).  When the columns of every tile of
 * tile_items merge items lie within a narrow span, the rows of B a tile needs are one contiguous
 * block; b2s_spmm_csr_windowed copies that block into shared memory with one bulk copy per tile
 * and gathers from there instead of from L1 / L2.  b2s_spmm_window_stat writes to *widest_dev
 * the widest column span (largest - smallest column + 1) over the tiles of the matrix and, when
 * tile_win_dev is not NULL, to tile_win_dev[2t], [2t + 1] the first column and the span of
 * tile t (b2s_tile_count tiles).
 * b2s_spmm_csr_windowed with window_rows > 0 runs the windowed kernel; its tiles are
 * b2s_spmm_window_tile_items(...) merge items long (1536 for B2S_F32 with B2S_I32, else the
 * length b2s_spmm_tile_items gives), and tile_row_dev, tile_win_dev and the T * n_dense carries
 * must describe tiles of that length.  The kernel needs the window to fit (window_rows * ldb *
 * value size <= 32 KB), B, C and C_in 16-byte aligned with whole 16-byte packs per row, N within
 * one dense-column tile and B below 64 GB: b2s_spmm_window_usable answers 1 when all of that
 * holds (ask before building the plan); when it does not, the call returns B2S_ERR_ARG.
 * window_rows = 0: the call is b2s_spmm_csr. */
int b2s_spmm_window_tile_items(int val_type, int idx_type);
int b2s_spmm_window_usable(int val_type, const void* B_dev, int64_t ldb, int64_t n_dense,
                           const void* C_in_dev, const void* C_dev, int64_t ldc, int64_t n_cols,
                           int64_t window_rows);
int b2s_spmm_window_stat(int idx_type, const void* indices_dev, int64_t n_rows, int64_t nnz,
                         const int64_t* tile_row_dev, int tile_items, int64_t* widest_dev,
                         int32_t* tile_win_dev, b2s_stream stream);
int b2s_spmm_csr_windowed(int val_type, int idx_type, int ptr_type,
                          const void* data_dev, const void* indices_dev, const void* indptr_dev,
                          int64_t n_rows, int64_t n_cols, int64_t nnz,
                          const void* B_dev, int64_t ldb, int64_t n_dense,
                          const void* C_in_dev, void* C_dev, int64_t ldc,
                          const void* alpha, const void* beta,
                          const int64_t* tile_row_dev, void* carry_dev, int32_t* status_dev,
                          int64_t window_rows, const int32_t* tile_win_dev, b2s_stream stream);

/* Long rows of a power-law matrix by column panel (no counterpart in the reference).  On random
 * columns SpMM gathers one row of B per non-zero from DRAM.  The host side splits the matrix:
 * rows up to a length threshold stay as they are; the long rows are laid out by
 * b2s_panel_build_global + b2s_panel_compact as a stack of column panels whose slice of B fits
 * L2, and b2s_spmm_csr multiplies that stack into part_dev (one row of n_dense values per
 * non-empty (panel, long row), leading dimension n_dense).  This call adds, for each long row j,
 * the partials subpos_dev[p * n_long + j] >= 0 in ascending panel order and accumulates
 * alpha * sum into row rows_dev[j] of C, which the product over the short rows has set to
 * beta * C_in before. */
int b2s_spmm_rows_combine(int val_type, const void* part_dev, const int32_t* subpos_dev,
                          const int64_t* rows_dev, int64_t n_long, int n_panels, int64_t n_dense,
                          void* C_dev, int64_t ldc, const void* alpha, b2s_stream stream);

/* ---- CSR -> CSC (the transpose behind op = trans / conj) -----------------------------------
 * Replaces _transpose_csr_for_spmv (spmv_csr.py:477-515) and _transpose_csr_for_spmm
 * (spmm_csr.py:300-338): a stable sort of the non-zeros by column, so that inside one output
 * row the entries keep ascending source-row order, exactly like the stable argsort there.
 * conj != 0 conjugates complex values on the way (spmv_csr.py:615-618, spmm_csr.py:345-348).
 * Output arrays use the input dtypes: t_indices (idx_type, source row ids), t_indptr (ptr_type,
 * n_cols + 1 entries).  scratch_dev needs b2s_csr2csc_bytes() bytes.
 */
int64_t b2s_csr2csc_bytes(int64_t n_rows, int64_t n_cols, int64_t nnz);
int b2s_csr2csc(int val_type, int idx_type, int ptr_type,
                const void* data_dev, const void* indices_dev, const void* indptr_dev,
                int64_t n_rows, int64_t n_cols, int64_t nnz, int conj,
                void* t_data_dev, void* t_indices_dev, void* t_indptr_dev,
                void* scratch_dev, int64_t scratch_bytes, b2s_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* B200SPARSE_H_ */
