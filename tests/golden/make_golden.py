"""Generate tests/golden/*.npz from FlagSparse's own kernels.

Run once, on a machine that has the FlagSparse source tree (no GPU needed):

    python tests/golden/make_golden.py /path/to/FlagSparse

FlagSparse's public functions reject CPU tensors, but its @triton.jit kernels run on CPU tensors
under Triton's interpreter (TRITON_INTERPRET=1) when launched directly.  This script launches
them the way the reference launchers do -- same dtype promotion, same tile sizes:

    SpMV   _triton_spmv_csr_impl_prepared   spmv_csr.py:679-723
    SpMM   _triton_spmm_csr_impl            spmm_csr.py:2684-2789
           launch config                    spmm_csr.py:384-419
    op     _transpose_csr_for_spmv + conj   spmv_csr.py:477-515, :615-618

and stores inputs and outputs.  Matrices follow the recipes of the reference's accuracy tests
(shapes: tests/pytest/param_shapes.py:23-31; Bernoulli mask with p = clamp(32/(M*N), .06, .25):
tests/pytest/test_spmv_csr_accuracy.py:53-69; SpMM value scale 0.125:
tests/pytest/test_spmm_csr_accuracy.py:22-36; the 1536-entry long row: tests/test_spmm.py:62-64,
:433-445), with a fixed seed here because the reference draws them unseeded.
"""

import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np  # noqa: E402
import torch  # noqa: E402

OUT_DIR = Path(__file__).resolve().parent
SPMV_SHAPES = [(1, 32), (160, 1024), (128, 256)]
SPMM_SHAPES = [(8, 4, 16), (64, 16, 96)]  # (M, N, K)
DTYPES = [torch.float32, torch.float64, torch.complex64, torch.complex128]
OPS = ["non", "trans", "conj"]


def rand_values(shape, dtype, gen, scale=1.0):
    if dtype in (torch.float32, torch.float64):
        return torch.randn(shape, dtype=dtype, generator=gen) * scale
    comp = torch.float32 if dtype == torch.complex64 else torch.float64
    return torch.complex(torch.randn(shape, dtype=comp, generator=gen) * scale,
                         torch.randn(shape, dtype=comp, generator=gen) * scale)


def random_csr(M, N, dtype, gen, scale=1.0):
    p = min(0.25, max(0.06, 32.0 / max(M * N, 1)))
    mask = torch.rand(M, N, generator=gen) < p
    if int(mask.sum()) == 0:
        mask[0, 0] = True
    dense = torch.where(mask, rand_values((M, N), dtype, gen, scale), torch.zeros((), dtype=dtype))
    rows, cols = torch.nonzero(mask, as_tuple=True)
    data = dense[rows, cols].contiguous()
    indptr = torch.zeros(M + 1, dtype=torch.int64)
    indptr[1:] = torch.cumsum(torch.bincount(rows, minlength=M), 0)
    return data, cols.to(torch.int64).contiguous(), indptr


def main(ref_root):
    sys.path.insert(0, str(Path(ref_root) / "src"))
    import triton.language as tl
    import flagsparse.sparse_operations.spmm_csr as mm
    import flagsparse.sparse_operations.spmv_csr as mv

    def materialize(data, indices, indptr, shape, op):
        if op == "non":
            return data, indices, indptr, shape
        if op == "conj" and data.is_complex():
            data = data.conj().resolve_conj()
        return mv._transpose_csr_for_spmv(data, indices, indptr, shape)

    def ref_spmv(data, indices, indptr, x, shape, op, block_nnz=256):
        data, indices, indptr, shape = materialize(data, indices, indptr, shape, op)
        M = shape[0]
        lens = indptr[1:] - indptr[:-1]
        max_len = int(lens.max()) if M > 0 else 0
        segs = max((max_len + block_nnz - 1) // block_nnz, 1)
        dtype = data.dtype
        if not dtype.is_complex:
            cd = torch.float64 if dtype == torch.float32 else dtype  # spmv_csr.py:124-129
            y = torch.empty(M, dtype=cd)
            mv._spmv_csr_real_kernel[(M,)](data.to(cd), indices, indptr, x.to(cd), y, n_rows=M,
                                           BLOCK_NNZ=block_nnz, MAX_SEGMENTS=segs)
            return y.to(dtype), (data, indices, indptr)
        d_ri = torch.view_as_real(data).reshape(-1)
        x_ri = torch.view_as_real(x.contiguous()).reshape(-1)
        y_ri = torch.empty(M * 2, dtype=d_ri.dtype)
        mv._spmv_csr_complex_kernel[(M,)](d_ri, indices, indptr, x_ri, y_ri, n_rows=M,
                                          BLOCK_NNZ=block_nnz, MAX_SEGMENTS=segs)
        return torch.view_as_complex(y_ri.reshape(M, 2)).clone(), (data, indices, indptr)

    def ref_spmm(data, indices, indptr, B, shape, op):
        data, indices, indptr, shape = materialize(data, indices, indptr, shape, op)
        M = shape[0]
        N = B.shape[1]
        lens = indptr[1:] - indptr[:-1]
        max_len = int(lens.max()) if M > 0 else 0
        cfg = mm._resolve_spmm_alg1_launch_config(N, max_len)
        bn, bnnz = cfg["block_n"], cfg["block_nnz"]
        grid = (M, -(-N // bn))
        ind32 = indices.to(torch.int32)
        ptr64 = indptr.to(torch.int64)
        dtype = data.dtype
        if not dtype.is_complex:
            cd = torch.float64 if dtype == torch.float32 else dtype  # spmm_csr.py:2720-2723
            Bc = B.to(cd).contiguous()
            C = torch.empty((M, N), dtype=cd)
            mm._spmm_csr_real_kernel[grid](data.to(cd), ind32, ptr64, Bc, C, M, N, Bc.stride(0),
                                           Bc.stride(1), C.stride(0), C.stride(1), BLOCK_N=bn,
                                           BLOCK_NNZ=bnnz, ACC_DTYPE=tl.float64)
            return C.to(dtype)
        d_ri = torch.view_as_real(data).contiguous().reshape(-1)
        B_ri = torch.view_as_real(B.contiguous()).contiguous()
        C_ri = torch.empty((M, N, 2), dtype=B_ri.dtype)
        acc = tl.float64 if B_ri.dtype == torch.float64 else tl.float32
        mm._spmm_csr_complex_kernel[grid](d_ri, ind32, ptr64, B_ri, C_ri, M, N, B_ri.stride(0),
                                          B_ri.stride(1), B_ri.stride(2), C_ri.stride(0),
                                          C_ri.stride(1), C_ri.stride(2), BLOCK_N=bn,
                                          BLOCK_NNZ=bnnz, ACC_DTYPE=acc)
        return torch.view_as_complex(C_ri.contiguous()).clone()

    def name(dt):
        return str(dt).replace("torch.", "")

    # ---- SpMV ------------------------------------------------------------------------------
    cases = {}
    gen = torch.Generator().manual_seed(20240607)
    for (M, N) in SPMV_SHAPES:
        for dt in DTYPES:
            data, idx, ptr = random_csr(M, N, dt, gen)
            for op in OPS:
                x = rand_values((M if op != "non" else N,), dt, gen)
                y, (t_data, t_idx, t_ptr) = ref_spmv(data, idx, ptr, x, (M, N), op)
                key = f"spmv_{M}x{N}_{name(dt)}_{op}"
                cases[key + "/data"] = data.numpy()
                cases[key + "/indices"] = idx.numpy()
                cases[key + "/indptr"] = ptr.numpy()
                cases[key + "/x"] = x.numpy()
                cases[key + "/y"] = y.numpy()
                if op != "non":  # the transposed triple pins the CSR -> CSC step bit for bit
                    cases[key + "/t_data"] = t_data.numpy()
                    cases[key + "/t_indices"] = t_idx.numpy()
                    cases[key + "/t_indptr"] = t_ptr.numpy()
                print(key, flush=True)
    # rows longer than one 256-entry segment (exercises the serial add of block sums)
    for dt in DTYPES:
        M, N = 6, 3000
        lens = torch.tensor([0, 700, 1, 257, 0, 2048])
        ptr = torch.zeros(M + 1, dtype=torch.int64)
        ptr[1:] = torch.cumsum(lens, 0)
        idx = torch.cat([torch.randperm(N, generator=gen)[: int(n)].sort().values for n in lens])
        data = rand_values((int(ptr[-1]),), dt, gen)
        x = rand_values((N,), dt, gen)
        y, _ = ref_spmv(data, idx, ptr, x, (M, N), "non")
        key = f"spmv_longrows_{name(dt)}_non"
        cases[key + "/data"] = data.numpy()
        cases[key + "/indices"] = idx.numpy()
        cases[key + "/indptr"] = ptr.numpy()
        cases[key + "/x"] = x.numpy()
        cases[key + "/y"] = y.numpy()
        print(key, flush=True)
    np.savez_compressed(OUT_DIR / "spmv_reference.npz", **cases)

    # ---- SpMM ------------------------------------------------------------------------------
    cases = {}
    gen = torch.Generator().manual_seed(20240608)
    for (M, N, K) in SPMM_SHAPES:
        for dt in DTYPES:
            data, idx, ptr = random_csr(M, K, dt, gen, scale=0.125)
            for op in OPS:
                B = rand_values((M if op != "non" else K, N), dt, gen, scale=0.125)
                C = ref_spmm(data, idx, ptr, B, (M, K), op)
                key = f"spmm_{M}x{K}x{N}_{name(dt)}_{op}"
                cases[key + "/data"] = data.numpy()
                cases[key + "/indices"] = idx.numpy()
                cases[key + "/indptr"] = ptr.numpy()
                cases[key + "/B"] = B.numpy()
                cases[key + "/C"] = C.numpy()
                print(key, flush=True)
    # the long-row case of the reference's CLI checks: row 0 holds columns 0..1535
    for dt in (torch.float32, torch.complex64):
        n_rows, n_cols, nnz0, N = 2, 2048, 1536, 48
        idx = torch.cat([torch.arange(nnz0), torch.tensor([7, 129, 511, 1024])]).to(torch.int64)
        ptr = torch.tensor([0, nnz0, nnz0 + 4], dtype=torch.int64)
        data = rand_values((idx.numel(),), dt, gen)
        B = rand_values((n_cols, N), dt, gen)
        C = ref_spmm(data, idx, ptr, B, (n_rows, n_cols), "non")
        key = f"spmm_longrow_{name(dt)}_non"
        cases[key + "/data"] = data.numpy()
        cases[key + "/indices"] = idx.numpy()
        cases[key + "/indptr"] = ptr.numpy()
        cases[key + "/B"] = B.numpy()
        cases[key + "/C"] = C.numpy()
        print(key, flush=True)
    np.savez_compressed(OUT_DIR / "spmm_reference.npz", **cases)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/FlagSparse")
    main(sys.argv[1])
