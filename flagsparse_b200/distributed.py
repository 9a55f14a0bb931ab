"""Row-partitioned CSR SpMV / SpMM over several GPUs of one node (one process per GPU).

FlagSparse has no distributed code (no NCCL, no torch.distributed anywhere in its tree); its only
multi-GPU feature is the test runner spreading operators over devices.  This module is therefore
new: output rows are independent, so the matrix is cut into contiguous row blocks holding equal
shares of the non-zeros, x / B is replicated (broadcast from one rank), every rank multiplies its
block with the single-GPU kernels, and the row blocks of y / C are all-gathered.

The collectives go through ``torch.distributed`` (NCCL over NVLink on GPUs; gloo on CPU for the
tests of the host logic, where ``local_spmv`` / ``local_spmm`` are injected because the product
kernels have no CPU path).
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def partition_rows_by_nnz(indptr, parts):
    """Row boundaries r_0=0 <= r_1 <= ... <= r_parts=n_rows such that block p holds about
    nnz/parts non-zeros: r_p is the first row whose start offset reaches p*nnz/parts."""
    n_rows = int(indptr.numel()) - 1
    nnz = int(indptr[-1].item()) if n_rows >= 0 else 0
    targets = torch.tensor([(p * nnz) // parts for p in range(1, parts)], dtype=indptr.dtype,
                           device=indptr.device)
    inner = torch.searchsorted(indptr[:-1].contiguous(), targets, right=False)
    bounds = [0] + [min(int(v), n_rows) for v in inner.tolist()] + [n_rows]
    for i in range(1, len(bounds)):  # monotone even for degenerate inputs
        bounds[i] = max(bounds[i], bounds[i - 1])
    return bounds


def slice_rows(data, indices, indptr, r0, r1):
    """CSR arrays of rows r0..r1-1 with indptr re-based to zero."""
    j0, j1 = int(indptr[r0].item()), int(indptr[r1].item())
    return data[j0:j1], indices[j0:j1], (indptr[r0:r1 + 1] - indptr[r0])


def _default_local_spmv(data, indices, indptr, x, shape, **kw):
    from .spmv import flagsparse_spmv_csr
    return flagsparse_spmv_csr(data, indices, indptr, x, shape, **kw)


def _default_local_spmm(data, indices, indptr, B, shape, **kw):
    from .spmm import flagsparse_spmm_csr
    return flagsparse_spmm_csr(data, indices, indptr, B, shape, **kw)


class RowPartitionedCsr:
    """This rank's row block of a CSR matrix whose rows are spread over the process group."""

    def __init__(self, data, indices, indptr, n_cols, group=None, local_spmv=None,
                 local_spmm=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.data, self.indices, self.indptr = data, indices, indptr
        self.n_local = int(indptr.numel()) - 1
        self.n_cols = int(n_cols)
        self.local_spmv = local_spmv or _default_local_spmv
        self.local_spmm = local_spmm or _default_local_spmm
        counts = [None] * self.world
        dist.all_gather_object(counts, self.n_local, group=group)
        self.rows_per_rank = [int(c) for c in counts]
        self.max_rows = max(self.rows_per_rank) if self.rows_per_rank else 0
        self.n_rows = sum(self.rows_per_rank)
        self.row_offset = sum(self.rows_per_rank[: self.rank])
        self._pads = {}
        self._stages = None
        self._peer = None
        # CTAs (of 256 threads) of a combine + store kernel that drains beside the tile kernel
        # of the next stage; 0 = one thread per row
        self.peer_store_ctas = 2 * 148
        # how a finished block reaches the other ranks' copies of the result: 'stores' (the
        # last kernel stores into every copy itself), 'multicast' (it stores once into the
        # multicast mapping and the switch replicates; needs enable_peer_gather(multicast=True))
        # or 'dma' (it writes this rank's copy and the copy engines move the block)
        self.peer_transfer = "stores"
        # SpMV with the peer gather: broadcast x one column panel at a time and start the kernel
        # of a panel when its slice has landed.  Off by default: on 2 GPUs the four small
        # broadcasts and their waits cost more than the 0.2 ms of broadcast they hide
        # (1.75 ms against 1.69 ms per step).
        self.pipeline_broadcast = False

    @classmethod
    def from_global(cls, data, indices, indptr, shape, group=None, **kw):
        """Every rank passes the same full matrix (or a view of it) and keeps its own block."""
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        bounds = partition_rows_by_nnz(indptr, world)
        d, i, p = slice_rows(data, indices, indptr, bounds[rank], bounds[rank + 1])
        return cls(d.contiguous(), i.contiguous(), p.contiguous(), shape[1], group=group, **kw)

    # -- collectives ---------------------------------------------------------------------------
    def broadcast_dense(self, dense, src=0):
        """Replicate x / B: `dense` holds the data on `src` and is overwritten elsewhere."""
        dist.broadcast(dense, src=src, group=self.group)
        return dense

    def broadcast_by_panel(self, x, src=0):
        """Replicate x as one asynchronous broadcast per column panel of the SpMV panel layout
        (the panel width follows from the value type alone, so all ranks cut x alike).  Returns
        x_ready: x_ready(p) makes the current stream wait for the slices of panels 0..p,
        x_ready(None) for all of x -- the kernel of panel 0 starts when 1 / P of x has landed
        instead of all of it.  None when x is one panel wide (use broadcast_dense)."""
        from ._plan import panel_shift
        width = 1 << panel_shift(x.dtype)
        n = int(x.shape[0])
        if x.ndim != 1 or n <= width:
            return None
        works = [dist.broadcast(x[c0:min(c0 + width, n)], src=src, group=self.group,
                                async_op=True) for c0 in range(0, n, width)]
        waited = [0]

        def x_ready(p):
            upto = len(works) if p is None else min(int(p) + 1, len(works))
            while waited[0] < upto:
                works[waited[0]].wait()
                waited[0] += 1
        return x_ready

    def _padded(self, trailing, dtype, device):
        key = (tuple(trailing), dtype, device)
        bufs = self._pads.get(key)
        if bufs is None:
            mine = torch.zeros((self.max_rows, *trailing), dtype=dtype, device=device)
            everyone = torch.empty((self.world * self.max_rows, *trailing), dtype=dtype,
                                   device=device)
            bufs = self._pads[key] = (mine, everyone)
        return bufs

    def gather_rows(self, local, out=None):
        """All-gather the row blocks (unequal heights are padded to the tallest block for the
        collective and cut back afterwards).  Returns the full y / C on every rank."""
        trailing = tuple(local.shape[1:])
        if out is None:
            out = torch.empty((self.n_rows, *trailing), dtype=local.dtype, device=local.device)
        if all(r == self.max_rows for r in self.rows_per_rank) and local.is_contiguous() \
                and out.is_contiguous():
            # equal blocks: gather straight into the result, no padding or repacking
            dist.all_gather_into_tensor(out, local, group=self.group)
            return out
        mine, everyone = self._padded(trailing, local.dtype, local.device)
        mine[: self.n_local].copy_(local)
        dist.all_gather_into_tensor(everyone, mine, group=self.group)
        off = 0
        for p, rows in enumerate(self.rows_per_rank):
            out[off:off + rows].copy_(everyone[p * self.max_rows: p * self.max_rows + rows])
            off += rows
        return out

    # -- all-gather fused into the kernels: stores into every rank's buffer ------------------------
    def enable_peer_gather(self, dtype, trailing=(), multicast=False):
        """Allocate the assembled y / C in symmetric memory (one buffer per rank, each mapped
        into every process so that kernels can store into it over NVLink).  Afterwards spmv() /
        spmm() have their last kernel store this rank's block straight into all copies instead
        of calling an all-gather.  Collective: every rank calls it with the same arguments.
        multicast=False (default): plain peer stores only, NVLink multicast is switched off for
        these buffers.  multicast=True: the allocation is also bound to an NVSwitch multicast
        object where the platform offers one, and `peer_transfer = "multicast"` then stores every
        value once for all ranks; every process must make this choice before its first
        symmetric-memory allocation.

        The caller owns the ordering between steps: a rank may start storing the next result as
        soon as it has passed the end-of-step fence, so a consumer that reads the assembled
        result asynchronously must finish (or call ``fence()``) before the next product."""
        import ctypes
        import os
        if not multicast:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        dev = self.data.device
        group = self.group if self.group is not None else dist.group.WORLD
        # every rank issues the same collectives whether or not its own set-up succeeds; the
        # ranks then agree on the outcome, so that none is left waiting in a barrier
        failure, full, hdl, ptrs = None, None, None, []
        try:
            full = symm.empty((self.n_rows, *trailing), dtype=dtype, device=dev)
            hdl = symm.rendezvous(full, group)
            offset = int(getattr(hdl, "offset", 0) or 0)
            ptrs = [int(p) + offset for p in hdl.buffer_ptrs]
            if len(ptrs) != self.world or ptrs[self.rank] != full.data_ptr():
                raise RuntimeError("symmetric memory handle does not describe the buffer "
                                   "just made")
        except Exception as exc:  # noqa: BLE001 - reported after the ranks have agreed
            failure = exc
        ok = torch.tensor([0 if failure is not None else 1], dtype=torch.int32, device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
        if int(ok.item()) == 0:
            raise RuntimeError(f"peer gather could not be set up on every rank: {failure}")
        row_items = 1
        for t in trailing:
            row_items *= int(t)
        self._peer = {
            "full": full, "handle": hdl, "n": self.world,
            "array": (ctypes.c_void_p * self.world)(*ptrs),
            "array_self": (ctypes.c_void_p * 1)(ptrs[self.rank]),
            "multicast_ptr": self._multicast_address(hdl) if multicast else 0,
            "views": self._peer_views(hdl, full, trailing, dtype),
            "flag": torch.zeros(1, dtype=torch.int32, device=dev),
            "trailing": tuple(int(t) for t in trailing), "dtype": dtype,
            "row_bytes": row_items * full.element_size(),
        }
        dist.barrier(group=self.group)
        return full

    @staticmethod
    def _multicast_address(hdl):
        """Address of the buffer in the multicast mapping, 0 when there is none."""
        try:
            base = int(hdl.multicast_ptr or 0)
        except Exception:  # noqa: BLE001 - no multicast on this platform / build
            return 0
        return base + int(getattr(hdl, "offset", 0) or 0) if base else 0

    def _peer_views(self, hdl, full, trailing, dtype):
        """Tensors over every rank's copy of the assembled result (for copies by the copy
        engines, peer_transfer = 'dma'), or None when the handle does not hand them out or its
        view of this rank's copy is not the buffer itself."""
        try:
            start = int(getattr(hdl, "offset", 0) or 0) // full.element_size()
            views = [hdl.get_buffer(q, tuple(full.shape), dtype, start)
                     for q in range(self.world)]
            if views[self.rank].data_ptr() != full.data_ptr():
                return None
            return views
        except Exception:  # noqa: BLE001 - the store route does not need them
            return None

    def _dma_block(self, row_offset, rows):
        """Copy rows [row_offset, row_offset + rows) of this rank's assembled result to the same
        rows of every other rank's copy: one asynchronous device-to-device copy per peer, each
        on a stream of its own behind the kernels enqueued so far, so that the copy engines move
        the block over NVLink while the SMs go on with the next block."""
        peer = self._peer
        dev = peer["full"].device
        streams = peer.get("dma_streams")
        if streams is None:
            streams = peer["dma_streams"] = [torch.cuda.Stream(device=dev)
                                             for _ in range(self.world)]
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(dev))
        src = peer["full"][row_offset:row_offset + rows]
        for k in range(1, self.world):
            q = (self.rank + k) % self.world           # every rank starts with another peer
            streams[q].wait_event(done)
            with torch.cuda.stream(streams[q]):
                peer["views"][q][row_offset:row_offset + rows].copy_(src, non_blocking=True)

    def _dma_join(self):
        cur = torch.cuda.current_stream(self._peer["full"].device)
        for q, st in enumerate(self._peer.get("dma_streams") or []):
            if q != self.rank:
                cur.wait_stream(st)

    @staticmethod
    def _into(out, full):
        """The assembled result in the caller's `out` when one was given and is not already the
        buffer the kernels stored into."""
        if out is None or out.data_ptr() == full.data_ptr():
            return full
        out.copy_(full)
        return out

    def fence(self):
        """Stream-ordered barrier across the ranks (a one-element all-reduce): when it has
        completed here, every rank has finished the kernels it had enqueued before its own
        fence, so all their stores into this rank's buffer have landed."""
        dist.all_reduce(self._peer["flag"], group=self.group)

    def _peer_spmv(self, x, out_local, alpha, beta, x_ready=None):
        from .spmv import prepare_spmv_csr, spmv_block_to_peers
        peer = self._peer
        blocks = self._stages or [(self.data, self.indices, self.indptr)]
        if self._stages:
            starts, heights = self._stage_starts, self._stage_heights
        else:
            starts, heights = [0], [self.n_local]
        side = None
        dma = self.peer_transfer == "dma" and peer.get("views") is not None
        mc_ptr = peer.get("multicast_ptr", 0) if self.peer_transfer == "multicast" else 0
        if len(blocks) > 1 and not dma:
            # the stores of block s drain on a second stream while block s+1 is multiplied
            # (high priority: its few CTAs take the next free slots of the SMs instead of
            # queueing behind every CTA of the tile kernel launched after them)
            side = peer.get("side")
            if side is None:
                side = peer["side"] = torch.cuda.Stream(device=x.device, priority=-1)
        for s, (d, i, p) in enumerate(blocks):
            t, h = starts[s], heights[s]
            prepared = prepare_spmv_csr(d, i, p, (h, self.n_cols))
            y_in = None if out_local is None else out_local[t:t + h]
            if len(blocks) == 1:
                row_offset = self.row_offset
            else:
                row_offset = self.world * t + self.rank * h
            last = s + 1 == len(blocks)
            if dma:
                # the last kernel writes the block into this rank's copy only; the copy engines
                # take it to the other ranks while the next block is multiplied
                ok = spmv_block_to_peers(prepared, x, y_in, alpha, beta, peer["array_self"], 1,
                                         row_offset, self.n_rows,
                                         x_ready=x_ready if s == 0 else None)
                if ok:
                    self._dma_block(row_offset, h)
            else:
                ok = spmv_block_to_peers(prepared, x, y_in, alpha, beta, peer["array"],
                                         peer["n"], row_offset, self.n_rows, store_stream=side,
                                         store_ctas=0 if last else self.peer_store_ctas,
                                         x_ready=x_ready if s == 0 else None,
                                         multicast_ptr=mc_ptr)
            if not ok:
                if s == 0:
                    if x_ready is not None:
                        x_ready(None)
                    return None
                raise RuntimeError("row block cannot be stored to the peers")
        if side is not None:
            torch.cuda.current_stream(x.device).wait_stream(side)
        if dma:
            self._dma_join()
        self.fence()
        return peer["full"]

    # -- pipelined variant: several row blocks per rank ------------------------------------------
    def split_stages(self, stages, first_fraction=None):
        """Cut this rank's block into `stages` consecutive sub-blocks so that the gather of one
        sub-block can run while the next one is multiplied.  The global row order becomes
        stage-major: with sub-block s of every rank h_s rows tall and starting at local row
        t_s, sub-block s of rank p holds global rows [world * t_s + p * h_s, + h_s) -- i.e. the
        gather of stage s fills one contiguous slice of y / C and no repacking is needed.
        Heights are equal, or, with first_fraction (0 < f < 1 / stages), the first sub-block
        holds about that share of the rows and the others split the rest equally: the exchange
        can start no earlier than the first sub-block is done, so a short first one leaves
        more of the step for the exchange to hide in (measured on 8 GPUs with 4 sub-blocks:
        2.31 / 2.20 ms with a first share of 1/16 / 1/8 against 2.19 ms with equal heights, so
        equal heights stay the default).  Needs equal n_local on all ranks and
        heights that come out as multiples of 32 rows; otherwise returns False and the
        single-stage path stays in use."""
        stages = int(stages)
        self._stages = None
        if stages <= 1 or len(set(self.rows_per_rank)) != 1:
            return False
        heights = None
        if first_fraction and stages >= 2 and 0.0 < first_fraction < 1.0 / stages:
            h0 = int(self.n_local * first_fraction) // 32 * 32
            rest = self.n_local - h0
            if h0 > 0 and rest % (stages - 1) == 0 and (rest // (stages - 1)) % 32 == 0:
                heights = [h0] + [rest // (stages - 1)] * (stages - 1)
        if heights is None:
            if self.n_local % stages:
                return False
            heights = [self.n_local // stages] * stages
        starts = [0]
        for h in heights:
            starts.append(starts[-1] + h)
        self._stages = []
        for s in range(stages):
            d, i, p = slice_rows(self.data, self.indices, self.indptr, starts[s], starts[s + 1])
            self._stages.append((d.contiguous(), i.contiguous(), p.contiguous()))
        self._stage_heights, self._stage_starts = heights, starts[:-1]
        self._stage_rows = heights[0] if len(set(heights)) == 1 else None
        return True

    def stage_slices(self, rank):
        """[(global first row, rows)] of the sub-blocks of `rank` in the assembled result, in
        stage order (one entry, the rank's whole block, without stages)."""
        if not self._stages:
            return [(sum(self.rows_per_rank[:rank]), self.rows_per_rank[rank])]
        return [(self.world * t + rank * h, h)
                for t, h in zip(self._stage_starts, self._stage_heights)]

    def _pipelined(self, local_op, dense, out_local, out, alpha, beta):
        W = self.world
        trailing = tuple(dense.shape[1:])
        if out is None:
            out = torch.empty((self.n_rows, *trailing), dtype=dense.dtype, device=dense.device)
        if out_local is None:
            out_local = torch.empty((self.n_local, *trailing), dtype=dense.dtype,
                                    device=dense.device)
        works = []
        for (d, i, p), t, h in zip(self._stages, self._stage_starts, self._stage_heights):
            blk = out_local[t:t + h]
            local_op(d, i, p, dense, (h, self.n_cols), out=blk, alpha=alpha, beta=beta)
            # asynchronous: the collective waits for the kernels enqueued so far and runs on
            # NCCL's stream while the next stage is being multiplied
            works.append(dist.all_gather_into_tensor(out[W * t:W * (t + h)], blk,
                                                     group=self.group, async_op=True))
        for w in works:
            w.wait()
        return out

    # -- products ------------------------------------------------------------------------------
    def spmv_local(self, x, out=None, alpha=1.0, beta=0.0):
        return self.local_spmv(self.data, self.indices, self.indptr, x,
                               (self.n_local, self.n_cols), out=out, alpha=alpha, beta=beta)

    def spmm_local(self, B, out=None, alpha=1.0, beta=0.0):
        return self.local_spmm(self.data, self.indices, self.indptr, B,
                               (self.n_local, self.n_cols), out=out, alpha=alpha, beta=beta)

    def spmv(self, x, src=0, out_local=None, out=None, alpha=1.0, beta=0.0):
        """y = alpha * A x + beta * y0 with x taken from rank `src`; y0 is this rank's block in
        out_local.  Returns the assembled y on every rank.  After enable_peer_gather the result
        is the symmetric-memory buffer that call returned (the next product overwrites it); an
        `out` that is another tensor receives a copy."""
        peer = self._peer
        if peer is not None and peer["trailing"] == () and peer["dtype"] == x.dtype \
                and self.local_spmv is _default_local_spmv:
            x_ready = self.broadcast_by_panel(x, src) if self.pipeline_broadcast else None
            if x_ready is None:
                self.broadcast_dense(x, src)
            done = self._peer_spmv(x, out_local, alpha, beta, x_ready)
            if done is not None:
                return self._into(out, done)
        else:
            self.broadcast_dense(x, src)
        if getattr(self, "_stages", None):
            return self._pipelined(self.local_spmv, x, out_local, out, alpha, beta)
        y_local = self.spmv_local(x, out=out_local, alpha=alpha, beta=beta)
        return self.gather_rows(y_local, out=out)

    def spmm(self, B, src=0, out_local=None, out=None, alpha=1.0, beta=0.0):
        self.broadcast_dense(B, src)
        peer = self._peer
        if peer is not None and peer["trailing"] == tuple(B.shape[1:]) \
                and peer["dtype"] == B.dtype and not self._stages:
            from . import _lib
            C_local = self.spmm_local(B, out=out_local, alpha=alpha, beta=beta)
            row_bytes = peer["row_bytes"]
            nbytes, offset = self.n_local * row_bytes, self.row_offset * row_bytes
            if C_local.is_contiguous() and nbytes % 16 == 0 and offset % 16 == 0 \
                    and C_local.data_ptr() % 16 == 0:
                with torch.cuda.device(C_local.device):
                    st = _lib.load().b2s_peer_scatter(
                        _lib.ptr(C_local), nbytes, peer["array"], peer["n"], offset,
                        self.n_rows * row_bytes, _lib.stream_handle(C_local.device))
                _lib.check(st, "b2s_peer_scatter")
                self.fence()
                return self._into(out, peer["full"])
            return self.gather_rows(C_local, out=out)
        if getattr(self, "_stages", None):
            return self._pipelined(self.local_spmm, B, out_local, out, alpha, beta)
        C_local = self.spmm_local(B, out=out_local, alpha=alpha, beta=beta)
        return self.gather_rows(C_local, out=out)
