"""Two NCCL ranks on two GPUs: the row-partitioned SpMV / SpMM reassemble the single-GPU result.
Skipped on a machine with fewer than two GPUs (the host logic is covered on CPU with gloo in
test_distributed_cpu.py)."""

import os
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr, workloads
        from flagsparse_b200.distributed import RowPartitionedCsr
        p = workloads.cfg5_scaling(device="cuda", scale=512, seed=3)   # same matrix on every rank
        part = RowPartitionedCsr.from_global(p.data, p.indices, p.indptr, p.shape)
        x = p.x.clone() if rank == 0 else torch.zeros_like(p.x)
        y = part.spmv(x, src=0)
        single = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape)
        err = float(torch.linalg.vector_norm(y - single) / torch.linalg.vector_norm(single))
        # the documented limit of bit-identity across partitions, on a matrix with many short
        # rows: the shape of a longer row's sum follows the row's
        # position in its tile, but a row of one entry is one product and a row of two entries
        # one more addition, the same bits wherever the row block starts
        q = workloads.cfg2_powerlaw_spmv(device="cuda", scale=256, seed=3)
        part_q = RowPartitionedCsr.from_global(q.data, q.indices, q.indptr, q.shape)
        xq = q.x.clone() if rank == 0 else torch.zeros_like(q.x)
        yq = part_q.spmv(xq, src=0)
        single_q = flagsparse_spmv_csr(q.data, q.indices, q.indptr, q.x, q.shape)
        lens = (q.indptr[1:] - q.indptr[:-1])
        one, two = lens == 1, lens == 2
        same_short = (bool(torch.equal(yq[one], single_q[one])) and int(one.sum()) > 1000
                      and float(torch.linalg.vector_norm(yq - single_q)
                                / torch.linalg.vector_norm(single_q)) <= 1e-12)
        two_differ = int((yq[two] != single_q[two]).sum())
        del part_q
        B = p.B.clone() if rank == 0 else torch.zeros_like(p.B)
        C = part.spmm(B, src=0)
        single_C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
        err_mm = float(torch.linalg.matrix_norm(C - single_C) / torch.linalg.matrix_norm(single_C))
        # the same products with the all-gather fused into the last kernel (stores into every
        # rank's symmetric-memory buffer over NVLink)
        import flagsparse_b200._plan as plan_mod
        from flagsparse_b200 import clear_plan_cache
        y_full = part.enable_peer_gather(p.x.dtype)
        y2 = part.spmv(x, src=0)                       # scratch route (x fits L2: no panels)
        torch.cuda.synchronize()
        dist.barrier()
        same = bool(torch.equal(y2, y))
        plan_mod.PANEL_TRIGGER_BYTES, plan_mod.PANEL_MIN_NNZ = 0, 0
        plan_mod.PANEL_TARGET_BYTES = 4096 * 4
        clear_plan_cache()
        y3 = part.spmv(x, src=0).clone()               # panel route: the combine kernel stores
        torch.cuda.synchronize()
        dist.barrier()
        used_peer = y3 is not None and part._peer is not None
        part.peer_transfer = "dma"                     # same kernels, block moved by copy engines
        y4 = part.spmv(x, src=0).clone()
        torch.cuda.synchronize()
        dist.barrier()
        dma_same = bool(torch.equal(y4, y3)) and part._peer.get("views") is not None
        part.peer_transfer = "stores"
        err_panel = float(torch.linalg.vector_norm(y3 - single) / torch.linalg.vector_norm(single))
        plan_mod.PANEL_POLICY = "off"
        clear_plan_cache()
        part_mm = RowPartitionedCsr.from_global(p.data, p.indices, p.indptr, p.shape)
        C_full = part_mm.enable_peer_gather(p.B.dtype, trailing=(int(p.B.shape[1]),))
        C2 = part_mm.spmm(B, src=0)
        torch.cuda.synchronize()
        dist.barrier()
        same_mm = bool(torch.equal(C2, C))
        results[rank] = (err, err_mm, part.rows_per_rank, same, err_panel, same_mm,
                         y2.data_ptr() == y_full.data_ptr(), C2.data_ptr() == C_full.data_ptr(),
                         same_short, two_differ, dma_same)
    finally:
        dist.barrier()
        dist.destroy_process_group()


def _staged_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        import flagsparse_b200._plan as plan_mod
        from flagsparse_b200 import flagsparse_spmv_csr, workloads
        from flagsparse_b200.distributed import RowPartitionedCsr, slice_rows
        plan_mod.PANEL_TRIGGER_BYTES, plan_mod.PANEL_MIN_NNZ = 0, 0
        plan_mod.PANEL_TARGET_BYTES = 8192 * 8
        p = workloads.cfg2_powerlaw_spmv(device="cuda", scale=128, seed=9)   # float64, 131072 rows
        single = flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, alpha=1.5,
                                     beta=0.5, out=p.y0.clone())
        half = p.shape[0] // world
        d, i, ptr = slice_rows(p.data, p.indices, p.indptr, rank * half, (rank + 1) * half)
        y0_block = p.y0[rank * half:(rank + 1) * half].clone()
        stages, h = 4, half // 4
        expect = torch.cat([single[q * half + s * h: q * half + (s + 1) * h]
                            for s in range(stages) for q in range(world)])
        out = {}
        for gather in ("nccl", "peer", "peer_short_first", "nccl_short_first"):
            part = RowPartitionedCsr(d.contiguous(), i.contiguous(), ptr.contiguous(), p.shape[1])
            if gather.endswith("short_first"):
                # a first sub-block of 1/16 of the rows, the other three share the rest
                assert part.split_stages(stages, first_fraction=1.0 / 16)
                assert part._stage_heights == [half // 16, 5 * half // 16, 5 * half // 16,
                                               5 * half // 16]
                expect = torch.cat([single[q * half + t: q * half + t + hs]
                                    for t, hs in zip(part._stage_starts, part._stage_heights)
                                    for q in range(world)])
                assert part.stage_slices(1)[1] == (world * (half // 16) + 5 * half // 16,
                                                   5 * half // 16)
            else:
                assert part.split_stages(stages)
            if gather.startswith("peer"):
                part.enable_peer_gather(p.x.dtype)
            x = p.x.clone() if rank == 0 else torch.zeros_like(p.x)
            y = part.spmv(x, src=0, out_local=y0_block.clone(), alpha=1.5, beta=0.5)
            torch.cuda.synchronize()
            dist.barrier()
            out[gather] = float(torch.linalg.vector_norm(y - expect)
                                / torch.linalg.vector_norm(expect))
        results[rank] = out
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_block_cyclic_stages_with_nccl_and_with_peer_stores():
    """Four row sub-blocks per rank (block-cyclic global order): the NCCL all-gather of one
    stage overlapping the next kernel, and the combine kernel of one stage storing into the
    peers' buffers on a second stream while the next stage is multiplied."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_staged_worker, args=(2, port, results), nprocs=2, join=True)
        for rank in range(2):
            assert all(results[rank][k] <= 1e-12 for k in
                       ("nccl", "peer", "peer_short_first", "nccl_short_first")), results[rank]


def test_two_nccl_ranks_match_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
        for rank in range(2):
            (err, err_mm, rows, same, err_panel, same_mm, y_in_place, c_in_place,
             same_short, two_differ, dma_same) = results[rank]
            assert dma_same, "the copy-engine transfer gives another result than the peer stores"
            assert same_short, "rows of one entry differ between 1 and 2 GPUs"
            assert two_differ == 0, f"{two_differ} rows of two entries differ between 1 and 2 GPUs"
            assert err <= 1e-5 and err_mm <= 1e-5, (err, err_mm)   # float32 tolerance
            assert same and same_mm, "peer-store gather differs from the NCCL all-gather"
            assert err_panel <= 1e-5, err_panel
            assert c_in_place, "SpMM result did not come back in the symmetric buffer"
            assert sum(rows) == (1 << 26) // 512


def _multicast_worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        import flagsparse_b200._plan as plan_mod
        from flagsparse_b200 import flagsparse_spmv_csr, workloads
        from flagsparse_b200.distributed import RowPartitionedCsr
        plan_mod.PANEL_TRIGGER_BYTES, plan_mod.PANEL_MIN_NNZ = 0, 0
        plan_mod.PANEL_TARGET_BYTES = 4096 * 8
        q = workloads.cfg2_powerlaw_spmv(device="cuda", scale=256, seed=5)
        part = RowPartitionedCsr.from_global(q.data, q.indices, q.indptr, q.shape)
        part.enable_peer_gather(q.x.dtype, multicast=True)
        x = q.x.clone() if rank == 0 else torch.zeros_like(q.x)
        have = bool(part._peer.get("multicast_ptr"))
        y_stores = part.spmv(x, src=0).clone()          # peer stores (panel route)
        torch.cuda.synchronize()
        dist.barrier()
        part.peer_transfer = "multicast"
        y_mc = part.spmv(x, src=0).clone()              # one multimem store per value
        torch.cuda.synchronize()
        dist.barrier()
        single = flagsparse_spmv_csr(q.data, q.indices, q.indptr, q.x, q.shape)
        err = float(torch.linalg.vector_norm(y_mc - single) / torch.linalg.vector_norm(single))
        results[rank] = (have, bool(torch.equal(y_mc, y_stores)), err)
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_multicast_stores_give_the_same_assembled_result_as_peer_stores():
    """The combine kernel storing once into the NVSwitch multicast mapping of the ranks' result
    buffers (b2s_panel_combine_multicast) against the same kernel storing into every buffer.
    Skipped where the platform hands out no multicast mapping."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_multicast_worker, args=(2, port, results), nprocs=2, join=True)
        if not all(results[r][0] for r in range(2)):
            pytest.skip("no multicast mapping on this platform")
        for rank in range(2):
            have, same, err = results[rank]
            assert same and err <= 1e-12, (same, err)
