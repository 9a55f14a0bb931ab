"""Two NCCL ranks on two GPUs: the row-partitioned SpMV / SpMM reassemble the single-GPU result.
Skipped on a machine with fewer than two GPUs (the host logic is covered on CPU with gloo in
test_distributed_cpu.py)."""

import os
import sys
from pathlib import Path

import numpy as np
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
        B = p.B.clone() if rank == 0 else torch.zeros_like(p.B)
        C = part.spmm(B, src=0)
        single_C = flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape)
        err_mm = float(torch.linalg.matrix_norm(C - single_C) / torch.linalg.matrix_norm(single_C))
        torch.cuda.synchronize()
        results[rank] = (err, err_mm, part.rows_per_rank)
    finally:
        dist.barrier()
        dist.destroy_process_group()


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
            err, err_mm, rows = results[rank]
            assert err <= 1e-5 and err_mm <= 1e-5, (err, err_mm)   # float32 tolerance
            assert sum(rows) == (1 << 26) // 512
