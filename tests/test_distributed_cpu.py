"""Host logic of the row-partitioned multi-GPU path on CPU: two gloo ranks, the local products
supplied by the CPU oracle (the CUDA kernels have no CPU path, so the local operator is
injected).  Covers the nnz-balanced partition, padding of unequal blocks, reassembly, and a rank
that fails before a step."""

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def _matrix(seed=0, n_rows=301, n_cols=97):
    rng = np.random.default_rng(seed)
    lengths = rng.integers(0, 9, n_rows)
    lengths[5] = 400          # one heavy row: nnz-balanced blocks differ in height
    ptr = np.zeros(n_rows + 1, dtype=np.int64)
    np.cumsum(lengths, out=ptr[1:])
    idx = rng.integers(0, n_cols, int(ptr[-1]))
    data = rng.standard_normal(int(ptr[-1]))
    return data, idx, ptr, (n_rows, n_cols)


def _oracle_spmv(data, indices, indptr, x, shape, out=None, alpha=1.0, beta=0.0):
    import oracle
    y0 = None if out is None else out.numpy()
    y = oracle.spmv(data.numpy(), indices.numpy(), indptr.numpy(), x.numpy(), shape, alpha=alpha,
                    beta=beta, y0=y0)
    y = torch.from_numpy(y)
    if out is not None:
        out.copy_(y)
        return out
    return y


def _oracle_spmm(data, indices, indptr, B, shape, out=None, alpha=1.0, beta=0.0):
    import oracle
    C0 = None if out is None else out.numpy()
    C = torch.from_numpy(oracle.spmm(data.numpy(), indices.numpy(), indptr.numpy(), B.numpy(),
                                     shape, alpha=alpha, beta=beta, C0=C0))
    if out is not None:
        out.copy_(C)
        return out
    return C


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from flagsparse_b200.distributed import RowPartitionedCsr, partition_rows_by_nnz
        data, idx, ptr, shape = _matrix()
        td, ti, tp = torch.from_numpy(data), torch.from_numpy(idx), torch.from_numpy(ptr)
        bounds = partition_rows_by_nnz(tp, world)
        part = RowPartitionedCsr.from_global(td, ti, tp, shape, local_spmv=_oracle_spmv,
                                             local_spmm=_oracle_spmm)
        assert part.n_rows == shape[0] and part.rows_per_rank[rank] == bounds[rank + 1] - bounds[rank]
        # x lives on rank 0 only
        x = torch.from_numpy(np.random.default_rng(1).standard_normal(shape[1]))
        x_in = x.clone() if rank == 0 else torch.zeros_like(x)
        y = part.spmv(x_in, src=0)
        expect = oracle.spmv(data, idx, ptr, x.numpy(), shape)
        ok_spmv = np.array_equal(y.numpy(), expect)      # same oracle arithmetic per row: exact
        B = torch.from_numpy(np.random.default_rng(2).standard_normal((shape[1], 5)))
        B_in = B.clone() if rank == 0 else torch.zeros_like(B)
        C = part.spmm(B_in, src=0)
        ok_spmm = np.array_equal(C.numpy(), oracle.spmm(data, idx, ptr, B.numpy(), shape))
        # alpha / beta with per-rank y0 blocks
        y0 = torch.from_numpy(np.random.default_rng(3).standard_normal(shape[0]))
        blk = y0[part.row_offset: part.row_offset + part.n_local].clone()
        y2 = part.spmv(x_in, src=0, out_local=blk, alpha=1.5, beta=0.5)
        ok_ab = np.allclose(y2.numpy(), oracle.spmv(data, idx, ptr, x.numpy(), shape, alpha=1.5,
                                                    beta=0.5, y0=y0.numpy()), rtol=1e-14)
        results[rank] = (ok_spmv, ok_spmm, ok_ab, part.rows_per_rank)
    finally:
        dist.destroy_process_group()


def _staged_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from flagsparse_b200.distributed import RowPartitionedCsr
        stages, h, n_cols = 3, 20, 64
        # every rank owns `stages` blocks of h rows; block (s, p) holds global rows
        # [(s*world + p)*h, ...): build all blocks, keep those of this rank
        rng = np.random.default_rng(11)
        blocks = {}
        for s in range(stages):
            for p in range(world):
                lengths = rng.integers(0, 7, h)
                ptr = np.zeros(h + 1, dtype=np.int64)
                np.cumsum(lengths, out=ptr[1:])
                blocks[(s, p)] = (rng.standard_normal(int(ptr[-1])),
                                  rng.integers(0, n_cols, int(ptr[-1])), ptr)
        mine = [blocks[(s, rank)] for s in range(stages)]
        data = np.concatenate([b[0] for b in mine])
        idx = np.concatenate([b[1] for b in mine])
        ptr = np.zeros(stages * h + 1, dtype=np.int64)
        off = 0
        for s, b in enumerate(mine):
            ptr[s * h + 1:(s + 1) * h + 1] = b[2][1:] + off
            off += b[2][-1]
        part = RowPartitionedCsr(torch.from_numpy(data), torch.from_numpy(idx),
                                 torch.from_numpy(ptr), n_cols, local_spmv=_oracle_spmv)
        assert part.split_stages(stages)
        x = torch.from_numpy(np.random.default_rng(5).standard_normal(n_cols))
        y = part.spmv(x.clone() if rank == 0 else torch.zeros_like(x), src=0)
        expect = np.concatenate([oracle.spmv(*blocks[(s, p)], x.numpy(), (h, n_cols))
                                 for s in range(stages) for p in range(world)])
        results[rank] = bool(np.array_equal(y.numpy(), expect))
        assert not part.split_stages(7)          # 60 rows do not split into 7 equal stages
    finally:
        dist.destroy_process_group()


def test_staged_block_cyclic_gather_on_two_gloo_ranks():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_staged_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert results[0] and results[1]


def _short_first_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from flagsparse_b200.distributed import RowPartitionedCsr
        n_local, n_cols = 2048, 50
        rng = np.random.default_rng(100 + rank)
        lengths = rng.integers(0, 5, n_local)
        ptr = np.zeros(n_local + 1, dtype=np.int64)
        np.cumsum(lengths, out=ptr[1:])
        idx = rng.integers(0, n_cols, int(ptr[-1]))
        data = rng.standard_normal(int(ptr[-1]))
        part = RowPartitionedCsr(torch.from_numpy(data), torch.from_numpy(idx),
                                 torch.from_numpy(ptr), n_cols, local_spmv=_oracle_spmv)
        # a first share that is not below 1 / stages is ignored: equal heights
        ok = part.split_stages(4, first_fraction=0.3) and part._stage_heights == [512] * 4
        ok = ok and part.split_stages(4, first_fraction=1.0 / 16)
        ok = ok and part._stage_heights == [128, 640, 640, 640]
        ok = ok and part.stage_slices(1) == [(128, 128), (2 * 128 + 640, 640),
                                             (2 * 768 + 640, 640), (2 * 1408 + 640, 640)]
        x = torch.from_numpy(np.random.default_rng(7).standard_normal(n_cols))
        y = part.spmv(x.clone() if rank == 0 else torch.zeros_like(x), src=0)
        mine = oracle.spmv(data, idx, ptr, x.numpy(), (n_local, n_cols))
        got = np.concatenate([y.numpy()[a:a + h] for a, h in part.stage_slices(rank)])
        results[rank] = bool(ok and np.array_equal(got, mine) and y.numel() == 2 * n_local)
    finally:
        dist.destroy_process_group()


def test_stages_with_a_short_first_sub_block_on_two_gloo_ranks():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_short_first_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert results[0] and results[1]


def _panel_broadcast_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flagsparse_b200._plan import panel_shift
        from flagsparse_b200.distributed import RowPartitionedCsr
        data, idx, ptr, shape = _matrix()
        part = RowPartitionedCsr(torch.from_numpy(data), torch.from_numpy(idx),
                                 torch.from_numpy(ptr), shape[1], local_spmv=_oracle_spmv)
        width = 1 << panel_shift(torch.float64)
        n = 2 * width + 1000                      # three slices, the last one ragged
        ref = torch.arange(n, dtype=torch.float64)
        x = ref.clone() if rank == 0 else torch.zeros(n, dtype=torch.float64)
        ready = part.broadcast_by_panel(x, src=0)
        ok = ready is not None
        ready(0)
        ok = ok and bool(torch.equal(x[:width], ref[:width]))
        ready(0)                                  # asking again is harmless
        ready(None)
        ok = ok and bool(torch.equal(x, ref))
        # x no wider than one panel: one ordinary broadcast is the better call
        ok = ok and part.broadcast_by_panel(torch.zeros(100, dtype=torch.float64)) is None
        results[rank] = ok
    finally:
        dist.destroy_process_group()


def test_broadcast_by_panel_delivers_x_slice_by_slice_on_two_gloo_ranks():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_panel_broadcast_worker, args=(world, _free_port(), results), nprocs=world,
                 join=True)
        assert results[0] and results[1]


def _free_port():
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_is_balanced_by_nnz():
    from flagsparse_b200.distributed import partition_rows_by_nnz, slice_rows
    data, idx, ptr, shape = _matrix()
    tp = torch.from_numpy(ptr)
    for parts in (1, 2, 3, 8):
        b = partition_rows_by_nnz(tp, parts)
        assert b[0] == 0 and b[-1] == shape[0] and all(b[i] <= b[i + 1] for i in range(parts))
        share = [int(ptr[b[i + 1]] - ptr[b[i]]) for i in range(parts)]
        assert sum(share) == int(ptr[-1])
        # no block exceeds its fair share by more than the longest row
        assert max(share) <= int(ptr[-1]) / parts + 400 + 9
    d, i, p = slice_rows(torch.from_numpy(data), torch.from_numpy(idx), tp, 3, 10)
    assert int(p[0]) == 0 and int(p[-1]) == d.numel() == int(ptr[10] - ptr[3])
    # degenerate inputs: empty matrix, more parts than rows
    assert partition_rows_by_nnz(torch.zeros(1, dtype=torch.int64), 4) == [0, 0, 0, 0, 0]
    assert partition_rows_by_nnz(torch.tensor([0, 2, 4]), 4)[-1] == 2


def test_two_gloo_ranks_reassemble_the_single_process_result():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            ok_spmv, ok_spmm, ok_ab, rows = results[rank]
            assert ok_spmv and ok_spmm and ok_ab
            assert rows[0] != rows[1], "blocks should differ in height (padding path)"


def _failing_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=5))
    from flagsparse_b200.distributed import RowPartitionedCsr
    data, idx, ptr, shape = _matrix()
    part = RowPartitionedCsr.from_global(torch.from_numpy(data), torch.from_numpy(idx),
                                         torch.from_numpy(ptr), shape, local_spmv=_oracle_spmv)
    if rank == 1:
        results[rank] = "left"
        os._exit(0)                       # leaves between steps, nothing in flight
    try:
        part.spmv(torch.zeros(shape[1], dtype=torch.float64), src=0)
        results[rank] = "no error"
    except Exception as exc:  # the collective ends with an error instead of hanging
        results[rank] = type(exc).__name__
    os._exit(0)


def test_rank_leaving_between_steps_surfaces_as_an_error():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_failing_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert results[1] == "left"
        assert results[0] != "no error"
