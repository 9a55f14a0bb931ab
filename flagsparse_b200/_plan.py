"""Per-matrix device state: the checked CSR arrays, merge-path tile plans, scratch and the
cached transpose.  Everything here is built by kernels of libb200sparse.so; torch only owns the
memory.

A plan is found again through a small LRU cache keyed on the identity of the three CSR tensors
(address, length, dtype, torch version counter), so that the steady-state call of
``flagsparse_spmv_csr`` / ``flagsparse_spmm_csr`` does no validation, no host synchronisation
and no allocation -- the role ``PreparedCsrSpmv`` plays in FlagSparse (spmv_csr.py:55-130),
extended to SpMM, which there re-validates and re-transposes on every call
(spmm_csr.py:3330-3390).
"""

from __future__ import annotations

from collections import OrderedDict

import torch

from . import _lib

INDEX_LIMIT_INT32 = 2**31 - 1

# stats words written by b2s_csr_inspect
ST_PTR0, ST_PTRN, ST_DECREASING, ST_MINCOL, ST_MAXCOL, ST_MAXLEN, ST_EMPTY = range(7)


def inspect_csr(indices, indptr, n_rows, nnz):
    """One pass over indptr / indices on the device; returns the eight statistics as ints.

    This is the only host synchronisation a new matrix costs.
    """
    lib = _lib.load()
    stats = torch.empty(8, dtype=torch.int64, device=indptr.device)
    with torch.cuda.device(indptr.device):
        st = lib.b2s_csr_inspect(
            _lib.ptr(indptr), _lib.INDEX_CODE[indptr.dtype],
            _lib.ptr(indices) if nnz > 0 else None, _lib.INDEX_CODE[indices.dtype],
            n_rows, nnz, _lib.ptr(stats), _lib.stream_handle(indptr.device))
    _lib.check(st, "b2s_csr_inspect")
    return [int(v) for v in stats.tolist()]


# Column-panel layout for SpMV (b2s_panel_build).  "auto": used when x does not fit the part of L2
# that survives the col / val stream; "off": never.
PANEL_POLICY = "auto"
PANEL_TRIGGER_BYTES = 48 << 20   # x larger than this is split into panels
PANEL_TARGET_BYTES = 40 << 20    # largest x slice of one panel
PANEL_MIN_NNZ = 1 << 22          # below this the conversion is not worth its memory


# Long rows of SpMV from shared memory (b2s_spmv_stack_shared): rows with at least
# LONG_SPMV_MIN_PER_PANEL entries per narrow panel on average are taken out of the wide-panel
# stack and multiplied with their x slices held in shared memory.  Used only together with the
# panel layout, and only when those rows hold at least LONG_SPMV_MIN_SHARE of the non-zeros.
LONG_SPMV_POLICY = "auto"
LONG_SPMV_MIN_PER_PANEL = 4
LONG_SPMV_MIN_SHARE = 0.1
LONG_SPMV_TILES_PER_UNIT = 128
LONG_SPMV_SLICE_COLS = None   # None: the widest slice the kernel holds (64 KB of x)


def set_long_spmv_policy(policy="auto", min_per_panel=None, min_share=None, tiles_per_unit=None,
                         slice_cols=None):
    """'auto' (default) or 'off': whether SpMV may multiply the long rows of a panel-layout
    matrix from shared-memory slices of x.  The other arguments override the thresholds
    (slice_cols: a narrower slice than the kernel could hold, a power of two; tests use it to
    get many narrow panels on small matrices)."""
    global LONG_SPMV_POLICY, LONG_SPMV_MIN_PER_PANEL, LONG_SPMV_MIN_SHARE
    global LONG_SPMV_TILES_PER_UNIT, LONG_SPMV_SLICE_COLS
    if slice_cols is not None:
        LONG_SPMV_SLICE_COLS = int(slice_cols) if slice_cols else None
    if policy not in ("auto", "off"):
        raise ValueError("long-row policy must be 'auto' or 'off'")
    LONG_SPMV_POLICY = policy
    if min_per_panel is not None:
        LONG_SPMV_MIN_PER_PANEL = float(min_per_panel)
    if min_share is not None:
        LONG_SPMV_MIN_SHARE = float(min_share)
    if tiles_per_unit is not None:
        LONG_SPMV_TILES_PER_UNIT = max(1, int(tiles_per_unit))


def panel_shift(value_dtype):
    """log2 of the column-panel width the panel layout uses for this value type (a function of
    the value size alone, so every rank of a partitioned matrix arrives at the same one)."""
    vbytes = torch.empty(0, dtype=value_dtype).element_size()
    shift = 1
    while (2 << shift) * vbytes <= PANEL_TARGET_BYTES:
        shift += 1
    return shift


def set_panel_policy(policy):
    """'auto' (default) or 'off': whether SpMV may keep a column-panel copy of large matrices."""
    global PANEL_POLICY
    if policy not in ("auto", "off"):
        raise ValueError("panel policy must be 'auto' or 'off'")
    PANEL_POLICY = policy


# Long rows by column panel for SpMM (b2s_panel_build_global + b2s_spmm_rows_combine).  On random
# columns every non-zero gathers a row of B from DRAM; the rows longer than LONG_ROW_MIN of a
# power-law matrix hold half of the non-zeros and revisit every slice of B many times, so they
# are multiplied panel by panel out of L2.  "auto": used when B does not fit L2 and the long rows
# hold at least LONG_ROW_MIN_SHARE of the non-zeros; "off": never.
LONG_ROW_POLICY = "auto"
LONG_ROW_MIN = 1024                  # rows longer than this are taken out of the main product
LONG_ROW_TRIGGER_BYTES = 96 << 20    # B larger than this is a candidate
LONG_ROW_TARGET_BYTES = 40 << 20     # largest slice of B one panel touches
LONG_ROW_MIN_SHARE = 0.2
LONG_ROW_MIN_NNZ = 1 << 22


def set_long_row_policy(policy="auto", min_len=None, trigger_bytes=None, target_bytes=None,
                        min_share=None, min_nnz=None):
    """'auto' (default) or 'off': whether SpMM may split the long rows of a matrix off and
    multiply them by column panel.  The other arguments override the thresholds (tests use them
    to exercise the split on small matrices); None leaves a threshold as it is."""
    global LONG_ROW_POLICY, LONG_ROW_MIN, LONG_ROW_TRIGGER_BYTES, LONG_ROW_TARGET_BYTES
    global LONG_ROW_MIN_SHARE, LONG_ROW_MIN_NNZ
    if policy not in ("auto", "off"):
        raise ValueError("long-row policy must be 'auto' or 'off'")
    LONG_ROW_POLICY = policy
    if min_len is not None:
        LONG_ROW_MIN = int(min_len)
    if trigger_bytes is not None:
        LONG_ROW_TRIGGER_BYTES = int(trigger_bytes)
    if target_bytes is not None:
        LONG_ROW_TARGET_BYTES = int(target_bytes)
    if min_share is not None:
        LONG_ROW_MIN_SHARE = float(min_share)
    if min_nnz is not None:
        LONG_ROW_MIN_NNZ = int(min_nnz)


def long_row_shift(n_cols, row_bytes):
    """Panel width (as a shift) for rows of B of `row_bytes` bytes, or None when the split does
    not apply: the widest power of two whose slice of B stays within LONG_ROW_TARGET_BYTES, made
    wider if that would need more than 256 panels."""
    if LONG_ROW_POLICY != "auto" or row_bytes <= 0 or n_cols * row_bytes <= LONG_ROW_TRIGGER_BYTES:
        return None
    shift = 1
    while (2 << shift) * row_bytes <= LONG_ROW_TARGET_BYTES:
        shift += 1
    while ((n_cols - 1) >> shift) + 1 > 256:
        shift += 1
    if shift > 31 or ((n_cols - 1) >> shift) + 1 < 2:
        return None
    return shift


def build_panel_stack(data, indices, indptr, n_rows, n_cols, n_panels, shift, global_cols):
    """Re-lay a CSR matrix as a stack of column panels with the empty rows of the stack dropped
    where the stack is small enough to index with int32.  Returns (p_data, p_cols, p_ptr,
    panel_start, n_stacked, subpos); subpos is None when nothing was dropped."""
    lib = _lib.load()
    device = data.device
    nnz = int(data.numel())
    vcode = _lib.VALUE_CODE[data.dtype]
    icode, pcode_in = _lib.INDEX_CODE[indices.dtype], _lib.INDEX_CODE[indptr.dtype]
    ptr_dtype = torch.int32 if nnz <= INDEX_LIMIT_INT32 else torch.int64
    p_data = torch.empty_like(data)
    p_cols = torch.empty(nnz, dtype=torch.int32, device=device)
    p_ptr = torch.empty(n_panels * n_rows + 1, dtype=ptr_dtype, device=device)
    panel_start = torch.empty(n_panels + 1, dtype=torch.int64, device=device)
    nbytes = int(lib.b2s_panel_bytes(n_cols, nnz))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
    build = lib.b2s_panel_build_global if global_cols else lib.b2s_panel_build
    with torch.cuda.device(device):
        st = build(vcode, icode, pcode_in, _lib.ptr(data), _lib.ptr(indices), _lib.ptr(indptr),
                   n_rows, n_cols, nnz, n_panels, shift, _lib.ptr(p_data), _lib.ptr(p_cols),
                   _lib.ptr(p_ptr), _lib.INDEX_CODE[ptr_dtype], _lib.ptr(panel_start),
                   _lib.ptr(ws), nbytes, _lib.stream_handle(device))
    _lib.check(st, "b2s_panel_build")
    del ws
    # drop the rows of the stack that have no entries (most short rows live in one panel)
    n_stacked = n_panels * n_rows
    subpos = None
    if n_stacked <= INDEX_LIMIT_INT32:
        subpos = torch.empty(n_stacked, dtype=torch.int32, device=device)
        count = torch.zeros(1, dtype=torch.int64, device=device)
        cbytes = int(lib.b2s_panel_compact_bytes(n_stacked))
        ws = torch.empty(cbytes, dtype=torch.uint8, device=device)
        pcode = _lib.INDEX_CODE[ptr_dtype]
        with torch.cuda.device(device):
            st = lib.b2s_panel_compact(_lib.ptr(p_ptr), pcode, n_stacked, _lib.ptr(subpos),
                                       _lib.ptr(count), None, 0, _lib.ptr(ws), cbytes,
                                       _lib.stream_handle(device))
        _lib.check(st, "b2s_panel_compact")
        n_compact = int(count.item())
        c_ptr = torch.empty(n_compact + 1, dtype=ptr_dtype, device=device)
        with torch.cuda.device(device):
            st = lib.b2s_panel_compact(_lib.ptr(p_ptr), pcode, n_stacked, _lib.ptr(subpos),
                                       None, _lib.ptr(c_ptr), n_compact, None, 0,
                                       _lib.stream_handle(device))
        _lib.check(st, "b2s_panel_compact")
        del ws
        p_ptr, n_stacked = c_ptr, n_compact
    return p_data, p_cols, p_ptr, panel_start, n_stacked, subpos


STACK_END = -(1 << 31)   # bit 31 of a column word: last entry of its stacked row
STACK_PAD = 1 << 30      # bit 30: padding entry


class StackLayout:
    """The matrix as a stack of wide column panels in end-flag form (include/b200sparse.h,
    b2s_spmv_stack): values and flagged panel-local columns padded to whole tiles, the ordinal
    of the stacked row active at each tile start, the panel of each tile, and the position
    table the combine uses."""

    def __init__(self, vals, cols, n_stacked, tile_ord, tile_panel, panel_start, n_panels, shift,
                 subpos, tile):
        self.vals, self.cols = vals, cols
        self.n_entries = int(vals.numel())
        self.n_stacked = int(n_stacked)
        self.tile_ord, self.tile_panel, self.panel_start = tile_ord, tile_panel, panel_start
        self.n_panels, self.shift = int(n_panels), int(shift)
        self.subpos = subpos                # int32[n_panels * n_rows]
        self.tile = int(tile)
        self.n_tiles = self.n_entries // int(tile)
        self.long_rows = None               # LongRowStack when the long rows were taken out
        self._tile_bounds = None

    def panel_tile_bounds(self):
        """Host list b of n_panels tile indices: the tiles that need no x beyond panel p are
        tiles [0, b[p]) (a tile that straddles two panels counts for the later one); b[-1] is
        the number of tiles.  One read-back, kept."""
        if self._tile_bounds is None:
            b = torch.div(self.panel_start[1:], self.tile, rounding_mode="floor").tolist()
            b = [min(int(v), self.n_tiles) for v in b]
            b[-1] = self.n_tiles
            self._tile_bounds = b
        return self._tile_bounds


class LongRowStack:
    """The long rows of a matrix as a stack of narrow column panels in end-flag form
    (b2s_spmv_stack_shared): every panel padded to whole tiles, `units` = (panel, first tile,
    tiles) triples, one per CTA; `rows` the matrix rows they came from and, per long row, the
    list of its stacked rows in ascending panel order (seg_ptr / seg_ids)."""

    def __init__(self, vals, cols, n_stacked, tile_ord, units, rows, seg_ptr, seg_ids, shift,
                 tile):
        self.vals, self.cols = vals, cols
        self.n_entries = int(vals.numel())
        self.n_stacked = int(n_stacked)
        self.tile_ord, self.units = tile_ord, units
        self.n_units = int(units.numel()) // 3
        self.rows, self.seg_ptr, self.seg_ids = rows, seg_ptr, seg_ids
        self.n_long = int(rows.numel())
        self.shift = int(shift)
        self.n_tiles = self.n_entries // int(tile)


def _exclusive_cumsum(counts):
    out = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    torch.cumsum(counts, 0, out=out[1:])
    return out


def row_entry_positions(ptr64, rows):
    """Positions (int64) of the entries of rows `rows` in the CSR arrays, row after row."""
    lens = ptr64[rows + 1] - ptr64[rows]
    ptr_l = _exclusive_cumsum(lens)
    total = int(ptr_l[-1].item())
    gidx = torch.repeat_interleave(ptr64[rows] - ptr_l[:-1], lens)
    gidx += torch.arange(total, dtype=torch.int64, device=ptr64.device)
    return gidx, lens


def build_stack_layout(data, indices, indptr, n_rows, n_cols, n_panels, shift):
    """End-flag stack of wide panels from a CSR matrix, or None when the stack cannot be
    compacted (more than 2^31 stacked rows)."""
    lib = _lib.load()
    p_data, p_cols, p_ptr, panel_start, n_stacked, subpos = build_panel_stack(
        data, indices, indptr, n_rows, n_cols, n_panels, shift, global_cols=False)
    if subpos is None:
        return None
    device = data.device
    nnz = int(p_data.numel())
    tile = int(lib.b2s_spmv_stack_tile_items(_lib.VALUE_CODE[data.dtype]))
    n_tiles = (nnz + tile - 1) // tile
    n_entries = n_tiles * tile
    vals = torch.zeros(n_entries, dtype=data.dtype, device=device)
    vals[:nnz] = p_data
    del p_data
    cols = torch.full((n_entries,), STACK_PAD, dtype=torch.int32, device=device)
    cols[:nnz] = p_cols
    del p_cols
    ptr64 = p_ptr.to(torch.int64)
    del p_ptr
    if n_stacked > 0:
        cols[ptr64[1:] - 1] |= STACK_END          # every stacked row is non-empty
    starts = torch.arange(n_tiles + 1, dtype=torch.int64, device=device) * tile
    # rows whose last entry lies before the tile start = ordinal of the row active there
    tile_ord = torch.searchsorted(ptr64[1:].contiguous(), starts, right=True)
    tile_panel = (torch.searchsorted(panel_start, starts[:n_tiles].contiguous(), right=True)
                  - 1).clamp_(0, n_panels - 1).to(torch.int32)
    return StackLayout(vals, cols, n_stacked, tile_ord, tile_panel, panel_start, n_panels, shift,
                       subpos, tile)


def build_long_row_stack(data, indices, indptr, rows, n_cols, shift, tiles_per_unit):
    """End-flag stack of narrow panels (2^shift columns) from rows `rows` (int64, ascending) of a
    CSR matrix; the one-off sort runs in torch."""
    lib = _lib.load()
    device = data.device
    tile = int(lib.b2s_spmv_stack_tile_items(_lib.VALUE_CODE[data.dtype]))
    n_long = int(rows.numel())
    gidx, lens = row_entry_positions(indptr.to(torch.int64), rows)
    nnz_l = int(gidx.numel())
    rid = torch.repeat_interleave(torch.arange(n_long, dtype=torch.int64, device=device), lens)
    col = indices[gidx].to(torch.int64)
    key = (col >> shift) * n_long + rid            # (panel, long row); stable: row order kept
    key, order = torch.sort(key, stable=True)
    del rid
    vals_sorted = data[gidx[order]]
    lcol = (col[order] & ((1 << shift) - 1)).to(torch.int32)
    del col, gidx, order
    end = torch.ones(nnz_l, dtype=torch.bool, device=device)
    end[:-1] = key[1:] != key[:-1]
    lcol[end] |= STACK_END
    panel = key // n_long
    n_panels = ((n_cols - 1) >> shift) + 1
    cnt = torch.bincount(panel, minlength=n_panels)
    padded = (cnt + tile - 1) // tile * tile
    pstart, qstart = _exclusive_cumsum(cnt), _exclusive_cumsum(padded)
    pos = qstart[panel] + (torch.arange(nnz_l, dtype=torch.int64, device=device) - pstart[panel])
    n_entries = int(qstart[-1].item())
    cols = torch.full((n_entries,), STACK_PAD, dtype=torch.int32, device=device)
    cols[pos] = lcol
    vals = torch.zeros(n_entries, dtype=data.dtype, device=device)
    vals[pos] = vals_sorted
    del lcol, vals_sorted
    end_pos = pos[end]                             # ascending
    seg_key = key[end]                             # (panel, long row) of each stacked row
    del key, pos, end, panel
    n_seg = int(seg_key.numel())
    n_tiles = n_entries // tile
    starts = torch.arange(n_tiles + 1, dtype=torch.int64, device=device) * tile
    tile_ord = torch.searchsorted(end_pos, starts, right=False)
    # one CTA per run of at most tiles_per_unit tiles of one panel
    tiles_p = (padded // tile).tolist()
    tile0_p = (qstart[:-1] // tile).tolist()
    units = []
    for p, (t0, nt) in enumerate(zip(tile0_p, tiles_p)):
        for k in range(0, nt, tiles_per_unit):
            units += [p, t0 + k, min(tiles_per_unit, nt - k)]
    units = torch.tensor(units, dtype=torch.int32, device=device)
    # stacked rows of each long row, ascending panel
    seg_rid = seg_key % n_long
    order2 = torch.argsort(seg_rid * n_panels + seg_key // n_long)
    seg_ids = order2.to(torch.int32)
    seg_ptr = _exclusive_cumsum(torch.bincount(seg_rid, minlength=n_long))
    return LongRowStack(vals, cols, n_seg, tile_ord, units, rows, seg_ptr, seg_ids, shift, tile)


# Shared-memory window of B rows for SpMM on banded / local matrices (b2s_spmm_csr_windowed).
# "auto": used when the widest column span of a tile, times the bytes of a B row, fits the
# window the kernel can hold; "off": never.
WINDOW_POLICY = "auto"
WINDOW_MAX_BYTES = 32 << 10


def set_window_policy(policy="auto"):
    """'auto' (default) or 'off': whether SpMM may gather B from a shared-memory window."""
    global WINDOW_POLICY
    if policy not in ("auto", "off"):
        raise ValueError("window policy must be 'auto' or 'off'")
    WINDOW_POLICY = policy


class LongRowSplit:
    """A matrix cut in two for SpMM: `short` (all rows, the long ones emptied) and `stack` (the
    long rows as a stack of column panels with global int32 columns; stacked row
    subpos[p * n_long + j] holds the entries of long row j = rows[j] that fall into panel p)."""

    def __init__(self, short, stack, rows, subpos, n_panels, shift):
        self.short, self.stack = short, stack
        self.rows, self.subpos = rows, subpos
        self.n_long = int(rows.numel())
        self.n_panels, self.shift = int(n_panels), int(shift)


class CsrPlan:
    """Device arrays of one CSR matrix plus everything derived from them."""

    def __init__(self, data, indices, indptr, shape, max_row_nnz, keepalive=()):
        self.data = data
        self.indices = indices
        self.indptr = indptr
        self.n_rows = int(shape[0])
        self.n_cols = int(shape[1])
        self.shape = (self.n_rows, self.n_cols)
        self.nnz = int(data.numel())
        self.max_row_nnz = int(max_row_nnz)
        self.device = data.device
        self.vcode = _lib.VALUE_CODE[data.dtype]
        self.icode = _lib.INDEX_CODE[indices.dtype]
        self.pcode = _lib.INDEX_CODE[indptr.dtype]
        self._keepalive = keepalive          # caller tensors this plan was derived from
        self._tiles = {}                     # tile_items -> (T, int64[T+1])
        self._scratch = {}                   # (tag, width, stream) -> tensor
        self._transposed = {}                # conj flag -> CsrPlan of the transpose
        self._panels = False                 # False: not decided yet; None: not used
        self._long_rows = {}                 # panel shift -> LongRowSplit or None (SpMM)
        self._window = {}                    # tile_items -> widest column span of a tile (SpMM)
        self._spmv_record = None             # prebuilt launch arguments (spmv.py)
        self._prepared = {}                  # memo of PreparedCsrSpmv handles (spmv.py)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status_checked = False
        self._launches = 0                   # launches since the status word was last read
        self._status_probe = None            # (pinned host copy, event) of a read in flight

    # -- tile plans ---------------------------------------------------------------------------
    def tiles(self, items):
        hit = self._tiles.get(items)
        if hit is not None:
            return hit
        lib = _lib.load()
        n_tiles = int(lib.b2s_tile_count(self.n_rows, self.nnz, items))
        tile_row = torch.empty(n_tiles + 1, dtype=torch.int64, device=self.device)
        if n_tiles > 0:
            with torch.cuda.device(self.device):
                st = lib.b2s_tile_plan(_lib.ptr(self.indptr), self.pcode, self.n_rows, self.nnz,
                                       items, _lib.ptr(tile_row),
                                       _lib.stream_handle(self.device))
            _lib.check(st, "b2s_tile_plan")
        self._tiles[items] = (n_tiles, tile_row)
        return self._tiles[items]

    def scratch(self, tag, n_values, dtype=None):
        """Scratch of n_values elements, one buffer per (purpose, size, stream)."""
        return self.scratch_on(tag, n_values, torch.cuda.current_stream(self.device).cuda_stream,
                               dtype)

    def carry_on(self, tag, n_tile_values, stream):
        """Scratch for the carries of n_tile_values (tiles, or tiles x dense columns): the
        accumulation dtype, and twice as many for the 16-bit dtypes, whose rows that cross tile
        borders are finished by the fix-up (include/b200sparse.h, b2s_spmv_csr)."""
        if self.data.element_size() < 4:
            return self.scratch_on(tag, 2 * int(n_tile_values), stream, torch.float32)
        return self.scratch_on(tag, n_tile_values, stream)

    def scratch_on(self, tag, n_values, stream, dtype=None):
        key = (tag, int(n_values), stream)
        buf = self._scratch.get(key)
        if buf is None:
            buf = torch.empty(max(int(n_values), 1), dtype=dtype or self.data.dtype,
                              device=self.device)
            self._scratch[key] = buf
        return buf

    # -- column panels ------------------------------------------------------------------------
    def panels(self):
        """StackLayout when the policy asks for a column-panel layout of this matrix, else None
        (built once).  Its `long_rows` holds the LongRowStack when the long rows were taken out
        for the shared-memory kernel."""
        if self._panels is not False:
            return self._panels
        self._panels = None
        vbytes = self.data.element_size()
        if (PANEL_POLICY != "auto" or vbytes < 4 or self.n_cols * vbytes <= PANEL_TRIGGER_BYTES
                or self.nnz < PANEL_MIN_NNZ or self.n_rows == 0):
            return None
        shift = panel_shift(self.data.dtype)
        n_panels = ((self.n_cols - 1) >> shift) + 1
        if n_panels < 2 or n_panels > 256 or shift > 29:
            return None
        data, indices, indptr = self.data, self.indices, self.indptr
        long_stack = self._long_rows_for_spmv()
        if long_stack is not None:
            # the wide-panel stack keeps every row but the long ones, which become empty
            ptr64 = indptr.to(torch.int64)
            lens = ptr64[1:] - ptr64[:-1]
            keep = torch.ones(self.nnz, dtype=torch.bool, device=self.device)
            rows = long_stack.rows
            keep[row_entry_positions(ptr64, rows)[0]] = False
            data, indices = data[keep], indices[keep]
            del keep
            lens[rows] = 0
            indptr = _exclusive_cumsum(lens)
            del lens, ptr64
        lay = build_stack_layout(data, indices, indptr, self.n_rows, self.n_cols, n_panels, shift)
        if lay is None:
            return None
        if long_stack is not None:
            # the sum of long row j sits behind the stacked rows of the wide panels; the combine
            # finds it through the position table like the partial of panel 0
            lay.subpos[long_stack.rows] = (lay.n_stacked + torch.arange(
                long_stack.n_long, dtype=torch.int64, device=self.device)).to(torch.int32)
        lay.long_rows = long_stack
        self._panels = lay
        return lay

    def _long_rows_for_spmv(self):
        """LongRowStack of the rows long enough for the shared-memory kernel, or None."""
        if LONG_SPMV_POLICY != "auto":
            return None
        lib = _lib.load()
        width = int(lib.b2s_spmv_stack_shared_cols(self.vcode))
        if LONG_SPMV_SLICE_COLS:
            width = max(2, min(width, LONG_SPMV_SLICE_COLS))
        shift = width.bit_length() - 1
        n_panels = ((self.n_cols - 1) >> shift) + 1
        min_len = max(int(LONG_SPMV_MIN_PER_PANEL * n_panels), 2)
        if 0 <= self.max_row_nnz < min_len:
            return None
        ptr64 = self.indptr.to(torch.int64)
        lens = ptr64[1:] - ptr64[:-1]
        rows = torch.nonzero(lens >= min_len).flatten()
        if rows.numel() == 0 or rows.numel() > 65536:
            return None
        if int(lens[rows].sum().item()) < LONG_SPMV_MIN_SHARE * self.nnz:
            return None
        del lens, ptr64
        return build_long_row_stack(self.data, self.indices, self.indptr, rows, self.n_cols,
                                    shift, LONG_SPMV_TILES_PER_UNIT)

    # -- long rows by column panel (SpMM) --------------------------------------------------------
    def long_row_split(self, row_bytes):
        """LongRowSplit for rows of B of `row_bytes` bytes when the policy asks for one for this
        matrix, else None (decided and built once per panel width)."""
        shift = long_row_shift(self.n_cols, row_bytes)
        if shift is None or self.nnz < LONG_ROW_MIN_NNZ or self.n_cols > INDEX_LIMIT_INT32:
            return None
        if self.data.element_size() < 4:      # 16-bit values: the one-launch product only
            return None
        if shift in self._long_rows:
            return self._long_rows[shift]
        self._long_rows[shift] = None
        if 0 <= self.max_row_nnz <= LONG_ROW_MIN:
            return None
        ptr64 = self.indptr.to(torch.int64)
        lens = ptr64[1:] - ptr64[:-1]
        long_mask = lens > LONG_ROW_MIN
        rows = torch.nonzero(long_mask).flatten()
        n_long = int(rows.numel())
        if n_long == 0:
            return None
        long_lens = lens[rows]
        nnz_long = int(long_lens.sum().item())
        n_panels = ((self.n_cols - 1) >> shift) + 1
        if nnz_long < LONG_ROW_MIN_SHARE * self.nnz or n_panels * n_long > INDEX_LIMIT_INT32:
            return None
        # the long rows as a CSR matrix of their own, and the matrix without them
        ptr_long = torch.zeros(n_long + 1, dtype=torch.int64, device=self.device)
        torch.cumsum(long_lens, 0, out=ptr_long[1:])
        gidx = torch.repeat_interleave(ptr64[rows] - ptr_long[:-1], long_lens)
        gidx += torch.arange(nnz_long, dtype=torch.int64, device=self.device)
        data_long, idx_long = self.data[gidx], self.indices[gidx]
        keep = torch.ones(self.nnz, dtype=torch.bool, device=self.device)
        keep[gidx] = False
        del gidx
        # (columns fit int32 here; the narrower index halves that stream and the staging buffer)
        data_short, idx_short = self.data[keep], self.indices[keep].to(torch.int32)
        del keep
        ptr_short = torch.zeros(self.n_rows + 1, dtype=torch.int64, device=self.device)
        torch.cumsum(lens.masked_fill(long_mask, 0), 0, out=ptr_short[1:])
        ptr_short = ptr_short.to(self.indptr.dtype)
        del lens, long_mask, ptr64
        p_data, p_cols, p_ptr, _, n_stacked, subpos = build_panel_stack(
            data_long, idx_long, ptr_long, n_long, self.n_cols, n_panels, shift, global_cols=True)
        del data_long, idx_long
        if subpos is None:
            return None
        short = CsrPlan(data_short, idx_short, ptr_short, self.shape, LONG_ROW_MIN)
        stack = CsrPlan(p_data, p_cols, p_ptr, (n_stacked, self.n_cols), -1)
        self._long_rows[shift] = LongRowSplit(short, stack, rows, subpos, n_panels, shift)
        return self._long_rows[shift]

    # -- widest column span of a tile (SpMM window) ----------------------------------------------
    def window_rows(self, items):
        """Largest (max column - min column + 1) over the tiles of `items` merge items, measured
        once per matrix (one pass over the column indices, one scalar read back)."""
        return self.window(items)[0]

    def window(self, items):
        """(widest span, int32[2 * tiles] table of first column and span per tile or None)."""
        hit = self._window.get(items)
        if hit is not None:
            return hit
        rows, table = 0, None
        if self.nnz > 0 and self.n_rows > 0:
            n_tiles, tile_row = self.tiles(items)
            out = torch.zeros(1, dtype=torch.int64, device=self.device)
            table = torch.zeros(2 * n_tiles, dtype=torch.int32, device=self.device)
            with torch.cuda.device(self.device):
                st = _lib.load().b2s_spmm_window_stat(
                    self.icode, _lib.ptr(self.indices), self.n_rows, self.nnz,
                    _lib.ptr(tile_row), items, _lib.ptr(out), _lib.ptr(table),
                    _lib.stream_handle(self.device))
            _lib.check(st, "b2s_spmm_window_stat")
            rows = int(out.item())
            if rows * 16 > WINDOW_MAX_BYTES:   # no B row is narrower than 16 bytes: never used
                table = None
        self._window[items] = (rows, table)
        return self._window[items]

    # -- transpose ----------------------------------------------------------------------------
    def transposed(self, conj):
        """CsrPlan of A^T (conj=False) or A^H (conj=True), built once by b2s_csr2csc."""
        conj = bool(conj) and self.data.dtype.is_complex
        hit = self._transposed.get(conj)
        if hit is not None:
            return hit
        lib = _lib.load()
        if self.indices.dtype == torch.int32 and self.n_rows > INDEX_LIMIT_INT32:
            raise ValueError("row ids of the transpose do not fit int32 indices")
        t_data = torch.empty_like(self.data)
        t_idx = torch.empty_like(self.indices)
        t_ptr = torch.empty(self.n_cols + 1, dtype=self.indptr.dtype, device=self.device)
        nbytes = int(lib.b2s_csr2csc_bytes(self.n_rows, self.n_cols, self.nnz))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            st = lib.b2s_csr2csc(self.vcode, self.icode, self.pcode, _lib.ptr(self.data),
                                 _lib.ptr(self.indices), _lib.ptr(self.indptr), self.n_rows,
                                 self.n_cols, self.nnz, 1 if conj else 0, _lib.ptr(t_data),
                                 _lib.ptr(t_idx), _lib.ptr(t_ptr), _lib.ptr(ws), nbytes,
                                 _lib.stream_handle(self.device))
        _lib.check(st, "b2s_csr2csc")
        ws.record_stream(torch.cuda.current_stream(self.device))
        del ws
        plan = CsrPlan(t_data, t_idx, t_ptr, (self.n_cols, self.n_rows), max_row_nnz=-1)
        self._transposed[conj] = plan
        return plan

    def derived_bytes(self):
        """Device bytes this plan keeps alive beyond the caller's three arrays: tile plans,
        scratch, the column-panel stack, the long-row layouts, cached transposes."""
        seen, total = set(), 0

        def add(obj):
            nonlocal total
            if torch.is_tensor(obj):
                key = obj.untyped_storage().data_ptr() if obj.numel() else 0
                if key and key not in seen:
                    seen.add(key)
                    total += obj.untyped_storage().nbytes()
            elif isinstance(obj, CsrPlan):
                if id(obj) not in seen:
                    seen.add(id(obj))
                    for t in (obj.data, obj.indices, obj.indptr):
                        add(t)
                    total += obj.derived_bytes()
            elif isinstance(obj, (list, tuple)):
                for o in obj:
                    add(o)
            elif isinstance(obj, dict):
                for o in obj.values():
                    add(o)
            elif hasattr(obj, "__dict__") and not callable(obj):
                add(vars(obj))

        for t in (self.data, self.indices, self.indptr):   # the caller's: not counted
            if torch.is_tensor(t) and t.numel():
                seen.add(t.untyped_storage().data_ptr())
        for name in ("_tiles", "_scratch", "_transposed", "_long_rows", "_window"):
            add(getattr(self, name))
        if self._panels not in (False, None):
            add(self._panels)
        return total

    STATUS_EVERY = 64   # launches between two non-blocking reads of the status word

    def note_launch(self):
        """Called after every launch that passed the status word.  The first launch of a plan
        reads the word at once (synchronises, like the reference's validation does for a new
        matrix); afterwards a non-blocking copy is started every STATUS_EVERY launches and
        examined at the next call, so that an error bit set later (a bounded wait that ran
        out, a bounds violation in the checked build) still raises, without a host
        synchronisation on the steady-state path."""
        if torch.cuda.is_current_stream_capturing():
            # inside a CUDA graph capture neither a copy to the host nor an event query is
            # allowed; the word is read again by the first launch outside the capture
            return
        if not self.status_checked:
            self.check_status()
            return
        probe = self._status_probe
        if probe is not None and probe[1].query():
            self._status_probe = None
            self._raise_for(int(probe[0].item()))
        self._launches += 1
        if self._launches >= self.STATUS_EVERY and self._status_probe is None:
            self._launches = 0
            host = torch.empty(1, dtype=torch.int32).pin_memory()
            host.copy_(self.status, non_blocking=True)
            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(self.device))
            self._status_probe = (host, event)

    def check_status(self):
        """Read the device status word (synchronises); raise if a kernel reported an error."""
        self.status_checked = True
        self._raise_for(int(self.status.item()))

    def _raise_for(self, bits):
        if bits:
            self.status.zero_()
            if bits & (1 << _lib.B2S_ERR_TIMEOUT):
                raise RuntimeError("a bounded wait inside a b200sparse kernel ran out "
                                   "(bulk copy did not complete)")
            if bits & (1 << _lib.B2S_ERR_BOUNDS):
                raise IndexError("a b200sparse kernel (bounds-checked build) met a column index "
                                 "or row pointer outside its array")
            raise RuntimeError(f"b200sparse kernels reported error bits {bits:#x}")


# -------------------------------------------------------------------------------------------------
# plan cache
# -------------------------------------------------------------------------------------------------
_CACHE = OrderedDict()
_CACHE_CAPACITY = 16
_CACHE_MAX_BYTES = None   # None: a quarter of the device's memory, decided at the first put


def set_plan_cache_capacity(n):
    """Number of matrices whose plans are kept (least recently used is dropped first)."""
    global _CACHE_CAPACITY
    _CACHE_CAPACITY = max(0, int(n))
    _trim_cache()


def set_plan_cache_bytes(n):
    """Upper bound, in bytes of device memory, on what the cached plans keep alive beyond the
    caller's own tensors: re-laid-out copies of the matrix, transposes, scratch (None = a
    quarter of the device's memory).  Least recently used plans are dropped first."""
    global _CACHE_MAX_BYTES
    _CACHE_MAX_BYTES = None if n is None else max(0, int(n))
    _trim_cache()


def clear_plan_cache():
    _CACHE.clear()


def tensor_version(t):
    """torch's in-place modification counter of a tensor; tensors made under
    torch.inference_mode() have none (and cannot be modified in place outside it): 0."""
    try:
        return t._version
    except RuntimeError:
        return 0


def _trim_cache():
    while len(_CACHE) > _CACHE_CAPACITY:
        _CACHE.popitem(last=False)
    if not _CACHE:
        return
    limit = _CACHE_MAX_BYTES
    if limit is None:
        any_plan = next(iter(_CACHE.values()))
        try:
            limit = torch.cuda.get_device_properties(any_plan.device).total_memory // 4
        except Exception:  # noqa: BLE001 - no device information: count-bound only
            return
    sizes = [(k, v.derived_bytes()) for k, v in _CACHE.items()]
    total = sum(b for _, b in sizes)
    for key, nbytes in sizes[:-1]:          # oldest first; the newest plan always stays
        if total <= limit:
            break
        _CACHE.pop(key, None)
        total -= nbytes


def plan_key(kind, data, indices, indptr, shape):
    return (
        kind,
        data.data_ptr(), indices.data_ptr(), indptr.data_ptr(),
        data.numel(), indptr.numel(),
        data.dtype, indices.dtype, indptr.dtype,
        tensor_version(data), tensor_version(indices), tensor_version(indptr),
        data.stride(0) if data.ndim == 1 and data.numel() > 1 else 1,
        indices.stride(0) if indices.ndim == 1 and indices.numel() > 1 else 1,
        indptr.stride(0) if indptr.ndim == 1 and indptr.numel() > 1 else 1,
        int(shape[0]), int(shape[1]),
        data.device.index,
    )


def cache_get(key):
    plan = _CACHE.get(key)
    if plan is not None:
        _CACHE.move_to_end(key)
    return plan


def cache_put(key, plan):
    if _CACHE_CAPACITY == 0:
        return
    _CACHE[key] = plan
    _CACHE.move_to_end(key)
    _trim_cache()
