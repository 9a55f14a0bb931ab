#!/usr/bin/env python
"""Benchmark of the CSR SpMV / SpMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Prints ONE JSON line (rank 0).  The default workload is the power-law SpMV the headline metric
is quoted on: float64 values / int64 indices, 2^24 x 2^24, Zipf(1.8) row lengths with mean 16 and
rows up to 100,000 entries, y = 1.5 * A x + 0.5 * y.  A step is one such product.

  value         effective HBM GB/s = algorithmic bytes / device time, inputs resident in HBM
  roofline      the same figure against the measured copy bandwidth of this GPU pool
  e2e           the same product through the public API with x, y0 in pinned HOST memory and
                y copied back, copies inside the timed region
  cpu_baseline  the CPU oracle (oracle/, a restatement of the reference's arithmetic) timed on
                a bounded row slice of the same matrix, all host cores
  parity        rel-L2 of one fresh product against torch's own CSR product in float64
                (cuSPARSE), computed once outside every timed region, and against the CPU
                oracle on the rows of the cpu_baseline sample; a line whose check fails is
                printed and the run exits non-zero
  extra         GFLOP/s, gathered bytes (x / B counted once per non-zero) and their rate, the
                SpMM N = 32 product on the same matrix, the measured divergent-gather ceiling
                of the GPU and the SpMV's fraction of it, and (when the unmodified FlagSparse
                package is installed under baseline/_ref) its Triton kernels timed on the same
                GPU and tensors beside this package (reference_triton_same_gpu)
  --impl reference   only that CPU measurement, as its own line
  --workload cfg2mm  the second half of the target as a line of its own: SpMM N = 32 on the
                same power-law matrix, with its own roofline / cpu_baseline / e2e / parity

With N > 1 (launched by torchrun, one rank per GPU) every rank owns one row block of the same
size (weak scaling): x is broadcast from rank 0 (NCCL), each rank multiplies its block, and y is
assembled on every rank -- by default the last kernel of each rank stores its block straight into
all ranks' symmetric-memory buffers over NVLink (--gather peer, through peer pointers; from four
GPUs on --gather mc, one multimem store per value that the NVSwitch replicates), alternatively by
an NCCL all-gather (--gather nccl); value counts the bytes all ranks processed over the slowest rank's
time.  Every rank checks its own block and the block of the next rank of the assembled y against
torch's CSR product.  The N > 1 line also carries extra.cfg5: ONE 2^26-row float32 / int64 matrix
row-partitioned by non-zeros over the ranks (RowPartitionedCsr.from_global), SpMV and SpMM
N = 16, with broadcast / kernel / gather / step times and the same check (--no-cfg5 skips it).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

NOMINAL_HBM_GBS = 8000.0

# DRAM bytes (read + written) of one step from an ncu capture of the same command
# (dram__bytes_read.sum + dram__bytes_write.sum over the kernels of a step), keyed by
# (workload, scale); to be re-captured whenever the kernels of the step change
NCU_TRAFFIC_BYTES = {("cfg2", 1): 4.76e9, ("cfg3", 1): 1.93e9}

REL_L2_TOL = {torch.float32: 1e-5, torch.complex64: 1e-5, torch.float64: 1e-12,
              torch.complex128: 1e-12}


def measured_peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# -------------------------------------------------------------------------------------------------
# clocks during the timed region
# -------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while a region runs."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index, period_s=0.002):
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.sm_max = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.sm_max,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# -------------------------------------------------------------------------------------------------
# workloads
# -------------------------------------------------------------------------------------------------
def make_problem(name, device, scale, seed):
    from flagsparse_b200 import workloads as W
    if name == "cfg1":
        return W.cfg1_uniform_spmv(device, scale, seed), "spmv"
    if name == "cfg2":
        return W.cfg2_powerlaw_spmv(device, scale, seed), "spmv"
    if name == "cfg2mm":
        p = W.cfg2_powerlaw_spmv(device, scale, seed, n_dense=32)
        p.extra["alpha"], p.extra["beta"] = 1.0, 0.0   # C = A B, as the target states it
        return p, "spmm"
    if name == "cfg3":
        return W.cfg3_banded_spmm(device, scale, seed), "spmm"
    if name == "cfg4":
        return W.cfg4_poisson_spmm(device, scale, seed), "spmm"
    if name == "cfg4c":
        return W.cfg4_poisson_spmm(device, scale, seed, dtype=torch.complex64), "spmm"
    if name == "cfg5":
        return W.cfg5_scaling(device, scale, seed, with_B=False), "spmv"
    if name == "cfg5mm":
        return W.cfg5_scaling(device, scale, seed), "spmm"
    raise SystemExit(f"unknown workload {name}")


WORKLOAD_TEXT = {
    "cfg1": "CSR SpMV float32/int32 65536x65536, 1..32 entries per row, alpha=1 beta=0",
    "cfg2": "CSR SpMV float64/int64 2^24x2^24, Zipf(1.8) row lengths mean 16 max 100000, "
            "alpha=1.5 beta=0.5",
    "cfg2mm": "CSR SpMM float64/int64 N=32 on the 2^24-row Zipf(1.8) matrix",
    "cfg3": "CSR SpMM float32/int32 op=non, banded 2^22x2^22 (band 64, 40% fill), N=32",
    "cfg4": "CSR SpMM float32/int32 op=trans, 1e6 x 5e5 Poisson(24) rows, N=64",
    "cfg4c": "CSR SpMM complex64/int32 op=conj, 1e6 x 5e5 Poisson(24) rows, N=64",
    "cfg5": "CSR SpMV float32/int64 2^26x2^26, Zipf(2.0) row lengths mean 16",
    "cfg5mm": "CSR SpMM float32/int64 N=16 on the 2^26-row Zipf(2.0) matrix",
}

DTYPE_TEXT = {torch.float32: "f32", torch.float64: "f64", torch.complex64: "c64",
              torch.complex128: "c128"}


def config_dict(args, world, rows, nnz, nbytes_per_gpu):
    """The `config` object of a line; both arms build it here so that they print the same."""
    text = WORKLOAD_TEXT[args.workload]
    if world > 1:
        text += f"; one such row block per GPU ({world} blocks, weak scaling)"
    return {"workload": text, "rows": int(rows), "nnz": int(nnz),
            "l2": "inputs_exceed_l2" if nbytes_per_gpu > 2 * 126e6 else "l2_resident_inputs",
            "seed": args.seed, "scale": args.scale}


def problem_bytes_flops(p, kind):
    """Algorithmic bytes of one product: row_ptr + col + val + x/B once + y/C written (and read
    when beta != 0), with the caller's index widths."""
    from flagsparse_b200 import workloads as W
    vb, ib, pb = p.data.element_size(), p.indices.element_size(), p.indptr.element_size()
    op = p.extra.get("op", "non")
    n_out, n_in = (p.shape[1], p.shape[0]) if op != "non" else p.shape
    beta_nz = p.extra.get("beta", 0.0) != 0.0
    if kind == "spmv":
        b = W.spmv_bytes(n_out, n_in, p.nnz, vb, ib, pb, beta_nz)
        f = W.sp_flops(p.nnz, 1, p.data.is_complex())
    else:
        n = int(p.B.shape[1])
        b = W.spmm_bytes(n_out, n_in, p.nnz, n, vb, ib, pb, beta_nz)
        f = W.sp_flops(p.nnz, n, p.data.is_complex())
    return b, f


def gathered_bytes(p, kind, nbytes):
    """Secondary diagnostic: the algorithmic bytes with the `x / B read once` term replaced by
    what the SMs pull through L1 / L2, one value (SpMV) or one row of B (SpMM) per non-zero."""
    vb = p.data.element_size()
    n_in = p.shape[0] if p.extra.get("op", "non") != "non" else p.shape[1]
    n = 1 if kind == "spmv" else int(p.B.shape[1])
    return nbytes - n_in * n * vb + p.nnz * n * vb


def make_step(p, kind):
    """Returns (step callable, output tensor, kernels launched per step)."""
    from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr
    op = p.extra.get("op", "non")
    alpha, beta = p.extra.get("alpha", 1.0), p.extra.get("beta", 0.0)
    n_out = p.shape[1] if op != "non" else p.shape[0]
    if kind == "spmv":
        out = p.extra["y0"].clone() if beta != 0.0 else torch.empty(
            n_out, dtype=p.data.dtype, device=p.data.device)

        def step():
            flagsparse_spmv_csr(p.data, p.indices, p.indptr, p.x, p.shape, out=out, op=op,
                                alpha=alpha, beta=beta)
    else:
        out = torch.empty((n_out, p.B.shape[1]), dtype=p.data.dtype, device=p.data.device)

        def step():
            flagsparse_spmm_csr(p.data, p.indices, p.indptr, p.B, p.shape, out=out, op=op,
                                alpha=alpha, beta=beta)
    return step, out, 2  # tile kernel + carry fix-up kernel (+ panel combine, see main)


def extra_launches(p, kind):
    """Kernels per step beyond the two make_step counts.  SpMV on the column-panel stack: the
    stack kernel, its fix-up and the combine (1 more), and with long rows split off the
    shared-memory kernel, its fix-up and the long-row combine (4 more).  SpMM with the long rows
    split off: a second tile kernel and fix-up for the panel stack, and the combine (3 more)."""
    from flagsparse_b200 import _plan
    key = _plan.plan_key(kind, p.data, p.indices, p.indptr, p.shape)
    plan = _plan.cache_get(key)
    if plan is None:
        return 0
    if p.extra.get("op", "non") != "non":
        plan = plan.transposed(conj=p.extra.get("op") == "conj")
    if kind == "spmv":
        lay = plan.panels()
        if lay is None:
            return 0
        return 4 if lay.long_rows is not None else 1
    row_bytes = int(p.B.shape[1]) * p.B.element_size()
    return 3 if plan.long_row_split(row_bytes) is not None else 0


def torch_product(data, indices, indptr, shape, dense, op="non"):
    """op(A) @ dense by torch's own sparse CSR multiplication in float64 / complex128: the
    independent product the parity figure is taken against."""
    wide = torch.complex128 if data.is_complex() else torch.float64
    vals = data.to(wide)
    if op == "conj":
        vals = vals.conj().resolve_conj()
    A = torch.sparse_csr_tensor(indptr.long(), indices.long(), vals, size=shape)
    if op != "non":
        A = A.to_sparse_coo().t().coalesce()
    return A @ dense.to(wide)


def rel_l2(got, want):
    diff = got.to(want.dtype) - want
    denom = float(torch.linalg.vector_norm(want))
    return float(torch.linalg.vector_norm(diff)) / (denom if denom > 0 else 1.0)


def parity_check(p, kind):
    """One fresh product through the public API against torch's CSR product (whole result)."""
    from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr
    op = p.extra.get("op", "non")
    alpha, beta = p.extra.get("alpha", 1.0), p.extra.get("beta", 0.0)
    dense = p.x if kind == "spmv" else p.B
    out = p.extra["y0"].clone() if beta != 0.0 else None
    fn = flagsparse_spmv_csr if kind == "spmv" else flagsparse_spmm_csr
    got = fn(p.data, p.indices, p.indptr, dense, p.shape, out=out, op=op, alpha=alpha, beta=beta)
    n = int(dense.shape[1]) if kind == "spmm" else 1
    err2 = ref2 = 0.0
    step = max(1, n // 4) if p.nnz > 500_000_000 else n   # bounded memory for the float64 copy
    for c0 in range(0, n, step):
        cols = slice(c0, min(n, c0 + step))
        want = torch_product(p.data, p.indices, p.indptr, p.shape,
                             dense if kind == "spmv" else dense[:, cols], op)
        want = alpha * want
        if beta != 0.0:
            want = want + beta * p.extra["y0"].to(want.dtype)
        part = got if kind == "spmv" else got[:, cols]
        err2 += float(torch.linalg.vector_norm(part.to(want.dtype) - want)) ** 2
        ref2 += float(torch.linalg.vector_norm(want)) ** 2
        del want
    err = (err2 / ref2) ** 0.5 if ref2 > 0 else err2 ** 0.5
    tol = REL_L2_TOL[p.data.dtype]
    return {"rel_l2": err, "tol": tol, "ok": bool(err <= tol),
            "against": "torch.sparse_csr_tensor @ dense in float64 (cuSPARSE), whole result"}


def time_device(step, steps, warmup, sampler=None):
    """Device time of `steps` back-to-back steps (CUDA events on the launching stream)."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ctx = sampler if sampler is not None else _Null()
    with ctx:
        start.record()
        for _ in range(steps):
            step()
        stop.record()
        torch.cuda.synchronize()
    return start.elapsed_time(stop) / 1000.0


class _Null:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


# -------------------------------------------------------------------------------------------------
# end to end through the public API with host buffers
# -------------------------------------------------------------------------------------------------
def time_e2e(p, kind, steps, warmup, depth=2):
    """The public call with the step's dense inputs in pinned HOST memory and the result copied
    back to the host, every step.  `depth` independent steps are kept in flight on separate
    streams with separate buffers, so that the upload of one step overlaps the kernel and the
    download of the previous one (A stays resident: it is the operand that persists)."""
    from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr
    op = p.extra.get("op", "non")
    alpha, beta = p.extra.get("alpha", 1.0), p.extra.get("beta", 0.0)
    dev = p.data.device
    dense_dev = p.x if kind == "spmv" else p.B
    dense_host = dense_dev.cpu().pin_memory()
    n_out = p.shape[1] if op != "non" else p.shape[0]
    out_shape = (n_out,) if kind == "spmv" else (n_out, p.B.shape[1])
    y0_host = p.extra["y0"].cpu().pin_memory() if beta != 0.0 else None
    h2d = dense_host.numel() * dense_host.element_size()
    if y0_host is not None:
        h2d += y0_host.numel() * y0_host.element_size()
    lanes = []
    for _ in range(depth):
        lanes.append({
            "stream": torch.cuda.Stream(device=dev),
            "dense": torch.empty_like(dense_dev),
            "out": torch.empty(out_shape, dtype=p.data.dtype, device=dev),
            "out_host": torch.empty(out_shape, dtype=p.data.dtype).pin_memory(),
        })
    d2h = lanes[0]["out_host"].numel() * lanes[0]["out_host"].element_size()

    def step(k):
        lane = lanes[k % depth]
        with torch.cuda.stream(lane["stream"]):
            lane["dense"].copy_(dense_host, non_blocking=True)
            if y0_host is not None:
                lane["out"].copy_(y0_host, non_blocking=True)
            if kind == "spmv":
                flagsparse_spmv_csr(p.data, p.indices, p.indptr, lane["dense"], p.shape,
                                    out=lane["out"], op=op, alpha=alpha, beta=beta)
            else:
                flagsparse_spmm_csr(p.data, p.indices, p.indptr, lane["dense"], p.shape,
                                    out=lane["out"], op=op, alpha=alpha, beta=beta)
            lane["out_host"].copy_(lane["out"], non_blocking=True)

    torch.cuda.synchronize()
    for k in range(warmup):
        step(k)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for k in range(steps):
        step(k)
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / steps, h2d, d2h


# -------------------------------------------------------------------------------------------------
# CPU baseline: the oracle port on a bounded row slice
# -------------------------------------------------------------------------------------------------
def cpu_sample(p, kind, max_nnz=40_000_000):
    """A bounded CPU-side sample of the workload: rows are independent, so the first rows of the
    matrix holding <= max_nnz entries stand in for the whole (same x / B, same arithmetic).
    Returns (callable running the oracle once, algorithmic bytes of one run, description,
    scipy callable or None)."""
    import numpy as np

    import oracle
    from flagsparse_b200 import workloads as W
    op = p.extra.get("op", "non")
    ptr_all = p.indptr
    if op != "non":
        n_slice = p.shape[0]  # the transposed product needs every row of A
    else:
        n_slice = int(torch.searchsorted(ptr_all.long(), torch.tensor(
            [max_nnz], device=ptr_all.device), right=True).item()) - 1
        n_slice = max(1, min(n_slice, p.shape[0]))
    nnz_s = int(ptr_all[n_slice].item())
    data = p.data[:nnz_s].cpu().numpy()
    idx = p.indices[:nnz_s].cpu().numpy().astype(np.int64)
    ptr = ptr_all[: n_slice + 1].cpu().numpy().astype(np.int64)
    shape = (n_slice, p.shape[1])
    vb, ib, pb = p.data.element_size(), p.indices.element_size(), p.indptr.element_size()
    if op != "non":
        data, idx, ptr, shape = oracle.transpose_csr(data, idx, ptr, shape, conj=(op == "conj"))
    n_out, n_in = shape
    if kind == "spmv":
        dense = p.x.cpu().numpy()
        fn = lambda: oracle.spmv_acc(data, idx, ptr, dense, shape)  # noqa: E731
        nbytes = W.spmv_bytes(n_out, n_in, nnz_s, vb, ib, pb, p.extra.get("beta", 0.0) != 0.0)
    else:
        dense = p.B.cpu().numpy()
        fn = lambda: oracle.spmm_acc(data, idx, ptr, dense, shape)  # noqa: E731
        nbytes = W.spmm_bytes(n_out, n_in, nnz_s, dense.shape[1], vb, ib, pb, False)
    scipy_fn = None
    try:
        import scipy.sparse as sp
        A = sp.csr_matrix((data, idx, ptr), shape=shape)
        scipy_fn = lambda: A @ dense  # noqa: E731
    except Exception:
        pass
    text = (f"first {n_slice} rows ({nnz_s} non-zeros) of the same matrix, full x/B, "
            "oracle/csr_oracle.c (OpenMP over rows)")
    return fn, nbytes, text, scipy_fn


def host_cores():
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()


def oracle_parity(p, kind, expect):
    """rel-L2 of our product (alpha = 1, beta = 0) against what the CPU oracle computed for the
    rows of its sample."""
    import numpy as np

    from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr
    op = p.extra.get("op", "non")
    dense = p.x if kind == "spmv" else p.B
    fn = flagsparse_spmv_csr if kind == "spmv" else flagsparse_spmm_csr
    got = fn(p.data, p.indices, p.indptr, dense, p.shape, op=op)
    got = got[: expect.shape[0]].cpu().numpy()
    wide = np.complex128 if np.iscomplexobj(expect) else np.float64
    diff = np.linalg.norm((got.astype(wide) - expect.astype(wide)).ravel())
    denom = np.linalg.norm(expect.astype(wide).ravel())
    return float(diff / (denom if denom > 0 else 1.0))


def cpu_baseline(p, kind, target_seconds=12.0):
    """The oracle port timed on the sample for about target_seconds (best run), plus scipy's
    single-threaded CSR product on the same sample, plus the rel-L2 of our result on the
    sample's rows against the oracle's."""
    import oracle
    threads = oracle.set_threads(host_cores())
    fn, nbytes, text, scipy_fn = cpu_sample(p, kind)
    expect = fn()  # warm the caches and the thread pool; also the checker's answer
    oracle_err = oracle_parity(p, kind, expect)
    reps, t_total, best = 0, 0.0, float("inf")
    while reps < 3 or (t_total < target_seconds and reps < 200):
        t0 = time.perf_counter()
        fn()
        dt = time.perf_counter() - t0
        best = min(best, dt)
        t_total += dt
        reps += 1
    scipy_gbs = None
    if scipy_fn is not None:
        t0 = time.perf_counter()
        for _ in range(3):
            scipy_fn()
        scipy_gbs = nbytes / ((time.perf_counter() - t0) / 3) / 1e9
    return {
        "value": nbytes / best / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
        "sample": text + f", best of {reps} runs", "scipy_1core_gbs": scipy_gbs,
        "oracle_rel_l2_on_sample": oracle_err,
    }


# -------------------------------------------------------------------------------------------------
def run_reference_arm(args, rank, world):
    """The reference has no CPU implementation of this path (its functions reject CPU tensors
    and its kernels are Triton); the arm times the CPU restatement of its arithmetic, one run of
    the bounded sample per step, all host threads."""
    if rank != 0:
        return
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    import oracle
    # all host threads, also where the launcher exported OMP_NUM_THREADS=1 for its workers
    threads = oracle.set_threads(host_cores())
    p, kind = make_problem(args.workload, dev, args.scale, args.seed)
    job_rows, job_nnz = p.shape[0], p.nnz
    full_bytes, _ = problem_bytes_flops(p, kind)
    for r in range(1, world):  # the other ranks' row blocks: only their sizes are needed here
        q, _ = make_problem(args.workload, dev, args.scale, args.seed + r)
        job_rows, job_nnz = job_rows + q.shape[0], job_nnz + q.nnz
        del q
    fn, nbytes, text, _ = cpu_sample(p, kind)
    for _ in range(max(1, args.warmup)):
        fn()
    times = []
    for _ in range(max(1, args.steps)):
        t0 = time.perf_counter()
        fn()
        times.append(time.perf_counter() - t0)
    per_step = statistics.median(times)
    value = nbytes / per_step / 1e9
    base = {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": text + f", median of {len(times)} runs"}
    line = {
        "impl": "reference", "metric": "effective HBM GB/s (algorithmic bytes / time)",
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE_TEXT[p.data.dtype],
        "data": "synthetic",
        "config": config_dict(args, world, job_rows, job_nnz, full_bytes),
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def reference_triton(p, kind, repeats=5):
    """The unmodified FlagSparse package (its Triton kernels, its public functions) on this GPU
    and on the same device tensors, beside this package on those tensors.  Context only -- the
    reference arm of this benchmark is the CPU path.  Runs when the package is installed under
    baseline/_ref (baseline/install_reference.py), else returns None.

    The reference's SpMV kernel walks ceil(longest row / 256) segments for every row of the
    matrix it is given (spmv_csr.py:183), so power-law matrices are timed on their first 2^18
    rows; SpMM on more than 2 * 10^8 non-zeros on the first 2^20 rows.  Both sides get the same
    slice, alpha = 1, beta = 0 (the reference has no alpha / beta)."""
    ref_dir = ROOT / "baseline" / "_ref"
    if not (ref_dir / "flagsparse").is_dir():
        return None
    sys.path.insert(0, str(ref_dir))
    try:
        import flagsparse as ref
        from flagsparse_b200 import flagsparse_spmm_csr, flagsparse_spmv_csr
        op = p.extra.get("op", "non")
        rows_cap = p.shape[0]
        if kind == "spmv" and p.shape[0] > (1 << 18) and op == "non":
            rows_cap = 1 << 18
        elif kind == "spmm" and p.nnz > 200_000_000 and op == "non":
            rows_cap = 1 << 20
        j1 = int(p.indptr[rows_cap])
        data, indices = p.data[:j1], p.indices[:j1]
        indptr = p.indptr[:rows_cap + 1].clone()
        shape = (rows_cap, p.shape[1])
        if kind == "spmv":
            theirs = lambda: ref.flagsparse_spmv_csr(data, indices, indptr, p.x, shape, op=op)  # noqa: E731
            ours = lambda: flagsparse_spmv_csr(data, indices, indptr, p.x, shape, op=op)  # noqa: E731
        else:
            theirs = lambda: ref.flagsparse_spmm_csr(data, indices, indptr, p.B, shape, op=op)  # noqa: E731
            ours = lambda: flagsparse_spmm_csr(data, indices, indptr, p.B, shape, op=op)  # noqa: E731

        def timed(fn):
            for _ in range(2):
                got = fn()
            torch.cuda.synchronize()
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(repeats):
                fn()
            t1.record()
            torch.cuda.synchronize()
            return t0.elapsed_time(t1) / repeats, got

        ref_ms, ref_out = timed(theirs)
        our_ms, our_out = timed(ours)
        return {"reference_ms": ref_ms, "ours_ms": our_ms, "rows": rows_cap, "nnz": j1,
                "rel_l2_ours_vs_reference": rel_l2(our_out, ref_out.to(
                    torch.complex128 if ref_out.is_complex() else torch.float64)),
                "timing": f"CUDA events over {repeats} calls of the public function after 2 "
                          "warm-up calls, plans / prepared state cached on both sides"}
    except Exception as exc:  # reported, never fatal for the bench line
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"}
    finally:
        sys.path.remove(str(ref_dir))


def gather_ceiling(device, spmv_gathers_per_s):
    """The rate of divergent 8-byte gathers from an L2-resident array (32 MB, 2^26 random
    indices), measured with the probe kernel of libb2sprobe.so (built from
    flagsparse_b200/csrc/probe/, not part of the product library): the bound the x gather of
    SpMV runs against when the column indices have no locality."""
    import ctypes

    from flagsparse_b200 import _build
    lib = ctypes.CDLL(str(_build.PROBE_LIB_PATH))
    lib.b2s_probe_gather.restype = ctypes.c_int
    lib.b2s_probe_gather.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,
                                     ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p]
    n, n_x = 1 << 26, 1 << 22
    idx = torch.randint(0, n_x, (n,), dtype=torch.int32, device=device)
    x = torch.zeros(n_x, dtype=torch.float64, device=device)
    sink = torch.zeros(1, dtype=torch.float64, device=device)
    stream = torch.cuda.current_stream(device)

    def launch():
        if lib.b2s_probe_gather(idx.data_ptr(), n, x.data_ptr(), n_x, sink.data_ptr(),
                                stream.cuda_stream) != 0:
            raise RuntimeError("b2s_probe_gather failed")

    per = time_device(launch, 10, 3) / 10
    rate = n / per
    return {"ggathers_per_s": rate / 1e9, "spmv_ggathers_per_s": spmv_gathers_per_s / 1e9,
            "frac": spmv_gathers_per_s / rate, "x_bytes": n_x * 8, "gathers": n}


def check_assembled(part, out_full, own, nxt, dense, alpha, beta):
    """Every rank compares two row blocks of the assembled result with torch's CSR product: its
    own and the next rank's.  `own` / `nxt` are (data, indices, indptr, y0 or None, rank) of
    those blocks; where a rank's rows sit in the assembled result (one slice, or one slice per
    stage) comes from part.stage_slices.  Returns the largest rel-L2."""
    worst = 0.0
    for data, indices, indptr, y0, r in (own, nxt):
        n_local = int(indptr.numel()) - 1
        want = alpha * torch_product(data, indices, indptr, (n_local, part.n_cols), dense)
        if beta != 0.0:
            want = want + beta * y0.to(want.dtype)
        got = torch.cat([out_full[first:first + rows] for first, rows in part.stage_slices(r)])
        worst = max(worst, rel_l2(got, want))
        del want
    return worst


def cfg5_extra(args, rank, world, device, timed):
    """ONE 2^26-row float32 / int64 matrix (Zipf(2.0) row lengths), row-partitioned by
    non-zeros over the ranks: SpMV and SpMM N = 16 with x / B broadcast from rank 0 and y / C
    assembled on every rank.  Every rank draws the same matrix (same seed), keeps its block,
    and checks its own and the next rank's block of the result against torch's CSR product."""
    import torch.distributed as dist

    from flagsparse_b200 import workloads as W
    from flagsparse_b200.distributed import (RowPartitionedCsr, partition_rows_by_nnz,
                                             slice_rows)
    out = {}
    g = W.cfg5_scaling(device, args.cfg5_scale, args.seed)
    bounds = partition_rows_by_nnz(g.indptr, world)
    part = RowPartitionedCsr.from_global(g.data, g.indices, g.indptr, g.shape)
    nxt_rank = (rank + 1) % world
    own = (part.data, part.indices, part.indptr, None, rank)
    nd, ni, nptr = slice_rows(g.data, g.indices, g.indptr, bounds[nxt_rank], bounds[nxt_rank + 1])
    nxt = (nd, ni, nptr, None, nxt_rank)
    n_rows, n_cols, nnz = g.shape[0], g.shape[1], g.nnz
    vb, ib = g.data.element_size(), g.indices.element_size()
    out["rows"], out["nnz"] = n_rows, nnz
    out["rows_per_rank"] = part.rows_per_rank
    for kind, dense in (("spmv", g.x), ("spmm", g.B)):
        n = 1 if kind == "spmv" else int(dense.shape[1])
        trailing = () if kind == "spmv" else (n,)
        if kind == "spmm":      # a partition object holds one assembled-result buffer
            part = RowPartitionedCsr.from_global(g.data, g.indices, g.indptr, g.shape)
        out_local = torch.empty((part.n_local, *trailing), dtype=g.data.dtype, device=device)
        out_full, mode = None, "nccl"
        if args.gather in ("peer", "dma", "mc"):
            part.peer_transfer = {"dma": "dma", "mc": "multicast"}.get(args.gather, "stores")
            try:    # collective: raises on every rank or on none
                out_full = part.enable_peer_gather(g.data.dtype, trailing,
                                                   multicast=args.gather == "mc")
                mode = args.gather
            except RuntimeError as exc:
                print(f"[rank {rank}] cfg5 {kind}: {exc}", file=sys.stderr, flush=True)
        if out_full is None:
            out_full = torch.empty((n_rows, *trailing), dtype=g.data.dtype, device=device)
        op = part.spmv if kind == "spmv" else part.spmm
        local = part.spmv_local if kind == "spmv" else part.spmm_local

        def step():
            return op(dense, src=0, out_local=out_local, out=out_full)

        full = step()
        torch.cuda.synchronize()
        err = check_assembled(part, full, own, nxt, dense, 1.0, 0.0)
        errs = torch.tensor([err], dtype=torch.float64, device=device)
        dist.all_reduce(errs, op=dist.ReduceOp.MAX)
        steps = max(3, min(args.steps, 10))
        per_step = timed(step, steps, 2) / steps
        phases = {
            "broadcast_ms": timed(lambda: part.broadcast_dense(dense, 0), 3, 1) / 3 * 1e3,
            "kernel_ms": timed(lambda: local(dense, out=out_local), 3, 1) / 3 * 1e3,
            "allgather_ms": timed(lambda: part.gather_rows(out_local, out=out_full), 3, 1)
            / 3 * 1e3,
        }
        if kind == "spmv":
            nbytes = W.spmv_bytes(n_rows, n_cols, nnz, vb, ib, ib, False)
        else:
            nbytes = W.spmm_bytes(n_rows, n_cols, nnz, n, vb, ib, ib, False)
        # per-GPU algorithmic bytes: the rank's share of the matrix and of y / C, all of x / B
        per_gpu = (nbytes - n_cols * n * vb) / world + n_cols * n * vb
        out[kind] = {
            "ms_per_step": per_step * 1e3, "job_gbs": nbytes / per_step / 1e9,
            "per_gpu_kernel_gbs": per_gpu / (phases["kernel_ms"] / 1e3) / 1e9,
            "algorithmic_bytes": nbytes, "phases": phases, "gather": mode,
            "rel_l2_vs_torch_own_and_next_block": float(errs.item()),
            "parity_ok": bool(float(errs.item()) <= REL_L2_TOL[g.data.dtype]),
        }
        del out_local, out_full, full, part, op, local
        torch.cuda.empty_cache()
    return out


def run_multi_gpu(args, rank, world, local_rank, device):
    """Weak scaling over the GPUs of one node: rank r owns the r-th row block, a matrix of the
    single-GPU workload's size drawn with seed + r; the global matrix is (world * rows) x cols.
    A step is: broadcast x (or B) from rank 0, multiply the local block, all-gather y (or C)."""
    import torch.distributed as dist

    from flagsparse_b200.distributed import RowPartitionedCsr

    dist.init_process_group("nccl", device_id=device)
    peak, peak_kind = measured_peaks()
    p, kind = make_problem(args.workload, device, args.scale, args.seed + rank)
    nbytes, flops = problem_bytes_flops(p, kind)
    if p.extra.get("op", "non") != "non":
        raise SystemExit("multi-GPU bench covers op=non workloads")
    part = RowPartitionedCsr(p.data, p.indices, p.indptr, p.shape[1])
    alpha, beta = p.extra.get("alpha", 1.0), p.extra.get("beta", 0.0)
    dense = p.x if kind == "spmv" else p.B
    trailing = () if kind == "spmv" else (int(p.B.shape[1]),)
    out_local = (p.extra["y0"].clone() if beta != 0.0 else
                 torch.empty((part.n_local, *trailing), dtype=p.data.dtype, device=device))
    out_full = torch.empty((part.n_rows, *trailing), dtype=p.data.dtype, device=device)
    local = part.spmv_local if kind == "spmv" else part.spmm_local

    def bcast():
        part.broadcast_dense(dense, 0)

    def kernel():
        local(dense, out=out_local, alpha=alpha, beta=beta)

    def gather():
        part.gather_rows(out_local, out=out_full)

    if args.gather == "auto":
        # measured (step, ms): 2 GPUs peer stores 1.68, multicast 1.72; 4 GPUs 1.96 / 1.92;
        # 8 GPUs 2.56 / 2.19 -- from four ranks on the block leaves the GPU once
        args.gather = "peer" if world < 4 else "mc"
    if args.stages <= 0:
        args.stages = 1 if world < 4 else 4
    if args.store_ctas >= 0:
        part.peer_store_ctas = args.store_ctas
    part.pipeline_broadcast = bool(args.pipelined_broadcast)
    staged = part.split_stages(args.stages if kind == "spmv" or args.gather == "nccl" else 1,
                               first_fraction=args.first_stage if args.first_stage > 0 else None)
    op = part.spmv if kind == "spmv" else part.spmm
    gather_mode = "peer" if args.gather in ("dma", "mc") else args.gather
    part.peer_transfer = {"dma": "dma", "mc": "multicast"}.get(args.gather, "stores")
    if gather_mode == "peer":
        # the last kernel of every rank stores its block into all ranks' result buffers; if
        # symmetric memory cannot be set up on any rank, every rank falls back to NCCL
        ok = torch.ones(1, dtype=torch.int32, device=device)
        try:
            peer_full = part.enable_peer_gather(p.data.dtype, trailing,
                                                multicast=args.gather == "mc")
        except Exception as exc:  # noqa: BLE001 - reported below, decided collectively
            ok.zero_()
            print(f"[rank {rank}] peer gather unavailable: {exc}", file=sys.stderr, flush=True)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1:
            out_full = peer_full
        else:
            part._peer = None
            gather_mode = "nccl"

    def step():
        if staged or gather_mode == "peer":
            # staged: the gather of stage s overlaps the kernel of stage s+1
            op(dense, src=0, out_local=out_local, out=out_full, alpha=alpha, beta=beta)
        else:
            bcast()
            kernel()
            gather()

    def timed(fn, steps, warmup, sampler=None):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with (sampler if sampler is not None else _Null()):
            start.record()
            for _ in range(steps):
                fn()
            stop.record()
            torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        t = torch.tensor([start.elapsed_time(stop) / 1000.0], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    step()  # plans, NCCL communicators
    torch.cuda.synchronize()
    # result check, outside every timed region: own block and the next rank's block
    q, _ = make_problem(args.workload, device, args.scale, args.seed + (rank + 1) % world)
    y0_of = (lambda pr: pr.extra["y0"]) if beta != 0.0 else (lambda pr: None)
    if beta != 0.0:
        out_local.copy_(p.extra["y0"])
    checked = op(dense, src=0, out_local=out_local, out=out_full, alpha=alpha, beta=beta) \
        if (staged or gather_mode == "peer") else None
    if checked is None:
        bcast()
        kernel()
        gather()
        checked = out_full
    torch.cuda.synchronize()
    worst = check_assembled(
        part, checked, (p.data, p.indices, p.indptr, y0_of(p), rank),
        (q.data, q.indices, q.indptr, y0_of(q), (rank + 1) % world), dense, alpha, beta)
    del q
    torch.cuda.empty_cache()
    errs = torch.tensor([worst], dtype=torch.float64, device=device)
    dist.all_reduce(errs, op=dist.ReduceOp.MAX)
    tol = REL_L2_TOL[p.data.dtype]
    parity = {"rel_l2": float(errs.item()), "tol": tol, "ok": bool(float(errs.item()) <= tol),
              "against": "torch.sparse_csr_tensor @ dense in float64 (cuSPARSE): every rank "
                         "checks its own block and the next rank's block of the assembled "
                         "result"}
    sampler = ClockSampler(local_rank) if rank == 0 else None
    seconds = timed(step, args.steps, args.warmup, sampler)
    per_step = seconds / args.steps
    phase_steps = max(3, args.steps // 3)
    phases = {name: timed(fn, phase_steps, 2) / phase_steps * 1e3
              for name, fn in (("broadcast_ms", bcast), ("kernel_ms", kernel),
                               ("allgather_ms", gather))}
    tot = torch.tensor([float(nbytes), float(flops), float(p.nnz)], dtype=torch.float64,
                       device=device)
    dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    job_bytes, job_flops, job_nnz = (float(v) for v in tot.tolist())

    # end to end: x from pinned host memory on rank 0, every rank's y0 block from its host
    # buffer, the assembled y copied back to the host on rank 0 (where x came from)
    dense_host = dense.cpu().pin_memory() if rank == 0 else None
    y0_host = p.extra["y0"].cpu().pin_memory() if beta != 0.0 else None
    full_host = torch.empty(out_full.shape, dtype=out_full.dtype).pin_memory() if rank == 0 \
        else None

    def e2e_step():
        if rank == 0:
            dense.copy_(dense_host, non_blocking=True)
        if y0_host is not None:
            out_local.copy_(y0_host, non_blocking=True)
        step()
        if rank == 0:
            full_host.copy_(out_full, non_blocking=True)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_s = timed(e2e_step, e2e_steps, 2) / e2e_steps
    h2d = (dense.numel() * dense.element_size()
           + world * (out_local.numel() * out_local.element_size() if y0_host is not None else 0))
    d2h = out_full.numel() * out_full.element_size()

    # kernels per rank and step: every stage launches the tile kernel and the carry fix-up, on
    # the column-panel layout also the combine; the peer route without panels adds the scatter
    from flagsparse_b200 import _plan as plan_mod
    n_stage = args.stages if staged else 1
    panels = (kind == "spmv" and plan_mod.PANEL_POLICY == "auto"
              and dense.numel() * dense.element_size() > plan_mod.PANEL_TRIGGER_BYTES
              and p.nnz // n_stage >= plan_mod.PANEL_MIN_NNZ)
    # (the count follows the plan of the whole block, which the phase timing above has built)
    per_stage = 2 + extra_launches(p, kind)
    if gather_mode == "peer" and not panels:
        per_stage += 1
    launches_per_rank_step = n_stage * per_stage
    pipelined_bcast = bool(gather_mode == "peer" and panels and part.pipeline_broadcast)
    if pipelined_bcast:   # the wide-panel kernel of the first stage runs as one launch per panel
        launches_per_rank_step += (((p.shape[1] - 1) >> plan_mod.panel_shift(p.data.dtype)) + 1) - 1
    if rank == 0:
        gbs = job_bytes / per_step / 1e9
        kernel_gbs = job_bytes / (phases["kernel_ms"] / 1e3) / 1e9
        line = {
            "metric": "effective HBM GB/s (algorithmic bytes / time)",
            "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": per_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE_TEXT[p.data.dtype],
            "data": "synthetic",
            "config": config_dict(args, world, part.n_rows, int(job_nnz), nbytes),
            "parity": parity,
            "exchange": {
                "broadcast": ("NCCL broadcast of x from rank 0, one asynchronous broadcast per "
                              "column panel; the kernel of a panel starts when its slice has "
                              "landed" if pipelined_bcast else
                              "NCCL broadcast of x / B from rank 0"),
                "gather": (("one multimem store per 16 bytes by each rank's last kernel into "
                            "an NVSwitch multicast mapping of all ranks' symmetric-memory result "
                            "buffers" if (part.peer_transfer == "multicast" and kind == "spmv"
                                          and part._peer and part._peer.get("multicast_ptr"))
                            else "each rank's last kernel writes its block into its own "
                            "symmetric-memory result buffer and the copy engines take it to "
                            "every other rank's buffer over NVLink (one asynchronous copy per "
                            "peer)" if part.peer_transfer == "dma" and kind == "spmv" else
                            "stores of each rank's last kernel into every rank's "
                            "symmetric-memory result buffer over NVLink")
                           + ", then a one-element NCCL all-reduce as the end-of-step fence"
                           if gather_mode == "peer" else "NCCL all-gather of y / C"),
                "inside_timed_step": True, "stages": args.stages if staged else 1,
                "stage_rows": list(part._stage_heights) if staged else [part.n_local],
                "mode": args.gather if gather_mode == "peer" else gather_mode,
                "multicast": bool(part._peer and part._peer.get("multicast_ptr")
                                  and part.peer_transfer == "multicast"),
                "store_ctas": part.peer_store_ctas},
            "roofline": {"bound": "hbm", "achieved": kernel_gbs / world, "peak": peak,
                         "unit": "GB/s", "frac": kernel_gbs / world / peak, "traffic": None,
                         "peak_kind": peak_kind,
                         "note": "per-GPU rate of the local kernel phase alone"},
            "e2e": {"value": job_bytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3},
            "gpu_launches": world * args.steps * launches_per_rank_step,
            "clocks": sampler.summary(),
            "extra": {"gflops": job_flops / per_step / 1e9,
                      "pct_of_8tbs_nominal_per_gpu": 100.0 * gbs / world / NOMINAL_HBM_GBS,
                      "phases": phases, "kernel_phase_gbs_all_gpus": kernel_gbs,
                      "algorithmic_bytes_per_step": job_bytes},
        }
    # the scaling configuration as stated: one 2^26-row matrix partitioned by non-zeros
    cfg5 = None
    if not args.no_cfg5:
        del part, out_local, out_full, p, dense
        torch.cuda.empty_cache()
        cfg5 = cfg5_extra(args, rank, world, device, timed)
    if cfg5 is not None:  # the same figures on every rank (all-reduced)
        parity["ok"] = bool(parity["ok"] and cfg5["spmv"]["parity_ok"]
                            and cfg5["spmm"]["parity_ok"])
    if rank == 0:
        if cfg5 is not None:
            line["extra"]["cfg5"] = cfg5
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()      # nothing of this rank in flight when the ranks part
    dist.barrier()
    dist.destroy_process_group()
    if not parity["ok"]:
        raise SystemExit(f"parity check failed: {parity}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOAD_TEXT))
    ap.add_argument("--scale", type=int, default=1, help="divide the row count (debugging)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--store-ctas", type=int, default=-1,
                    help="several GPUs, peer gather with stages: CTAs of the combine + store "
                         "kernel that runs beside the next stage (-1 = library default, "
                         "0 = one thread per row)")
    ap.add_argument("--stages", type=int, default=0,
                    help="N > 1: row sub-blocks per rank; the gather of one overlaps the kernel "
                         "of the next (1 = no overlap; 0 = 1 below four GPUs, 4 from four on)")
    ap.add_argument("--first-stage", type=float, default=0.0,
                    help="N > 1 with stages: share of a rank's rows in its first sub-block "
                         "(0 = equal sub-blocks); the exchange cannot start before the first "
                         "sub-block is done")
    ap.add_argument("--gather", default="auto", choices=["auto", "nccl", "peer", "dma", "mc"],
                    help="N > 1: how y / C is assembled (auto: peer below four GPUs, mc from four "
                         "on) -- NCCL all-gather; stores of the last "
                         "kernel into every rank's symmetric-memory buffer (peer); or the last "
                         "kernel writes this rank's buffer and the copy engines move the block "
                         "to the other ranks (dma); or it stores once into an NVSwitch multicast "
                         "mapping of all buffers (mc; falls back to peer where there is none)")
    ap.add_argument("--pipelined-broadcast", action="store_true",
                    help="N > 1: broadcast x one column panel at a time, the kernel of a panel "
                         "starting when its slice has landed (default: one broadcast first)")
    ap.add_argument("--no-cfg5", action="store_true",
                    help="N > 1: skip the partitioned 2^26-row matrix in extra.cfg5")
    ap.add_argument("--cfg5-scale", type=int, default=1,
                    help="divide the rows of the extra.cfg5 matrix (debugging)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the SpMM N=32 side measurement")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling)")
    ap.add_argument("--e2e-depth", type=int, default=2,
                    help="independent steps kept in flight in the host-buffer leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)

    if world > 1:
        run_multi_gpu(args, rank, world, local_rank, device)
        return

    peak, peak_kind = measured_peaks()
    p, kind = make_problem(args.workload, device, args.scale, args.seed)
    nbytes, flops = problem_bytes_flops(p, kind)
    step, out, launches_per_step = make_step(p, kind)
    step()  # builds the plan (validation, tiles, transpose) outside every timed region
    torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    seconds = time_device(step, args.steps, args.warmup, sampler)
    per_step = seconds / args.steps
    gbs = nbytes / per_step / 1e9

    parity = parity_check(p, kind)  # once, outside every timed region
    torch.cuda.empty_cache()

    if args.no_e2e:
        e2e_s, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_s, h2d, d2h = time_e2e(p, kind, max(6, min(args.steps, 12)), 4,
                                   depth=max(1, args.e2e_depth))

    extra = {"gflops": flops / per_step / 1e9, "pct_of_8tbs_nominal": 100.0 * gbs / NOMINAL_HBM_GBS,
             "algorithmic_bytes_per_step": nbytes,
             "gathered_bytes_per_step": gathered_bytes(p, kind, nbytes),
             "gathered_gbs": gathered_bytes(p, kind, nbytes) / per_step / 1e9}
    if args.workload == "cfg2" and not args.no_extra:
        # the second half of the target: SpMM N=32 on the same matrix
        from flagsparse_b200 import workloads as W
        g = torch.Generator(device=device)
        g.manual_seed(args.seed + 1)
        p.extra["B"] = torch.randn(p.shape[0] * 32, dtype=p.data.dtype, device=device,
                                   generator=g).view(p.shape[0], 32)
        saved = (p.extra.pop("alpha"), p.extra.pop("beta"))
        mm_bytes, mm_flops = problem_bytes_flops(p, "spmm")
        mm_step, mm_out, _ = make_step(p, "spmm")
        mm_step()
        torch.cuda.synchronize()
        mm_s = time_device(mm_step, max(3, args.steps // 5), 3) / max(3, args.steps // 5)
        mm_want = torch_product(p.data, p.indices, p.indptr, p.shape, p.extra["B"])
        mm_err = rel_l2(mm_out, mm_want)
        del mm_want
        extra["spmm_n32_same_matrix"] = {
            "rel_l2_vs_torch": mm_err, "parity_ok": bool(mm_err <= REL_L2_TOL[p.data.dtype]),
            "ms_per_step": mm_s * 1e3, "gbs": mm_bytes / mm_s / 1e9,
            "gflops": mm_flops / mm_s / 1e9, "frac_of_measured_peak": mm_bytes / mm_s / 1e9 / peak,
            "algorithmic_bytes_per_step": mm_bytes,
            "gathered_bytes_per_step": gathered_bytes(p, "spmm", mm_bytes),
            "gathered_gbs": gathered_bytes(p, "spmm", mm_bytes) / mm_s / 1e9,
        }
        if not extra["spmm_n32_same_matrix"]["parity_ok"]:
            parity["ok"] = False
        p.extra["alpha"], p.extra["beta"] = saved
        del p.extra["B"], mm_out
        torch.cuda.empty_cache()

    if kind == "spmv" and not args.no_extra:
        extra["gather_ceiling"] = gather_ceiling(device, p.nnz / per_step)

    if not args.no_extra:
        side = reference_triton(p, kind)
        if side is not None:
            extra["reference_triton_same_gpu"] = side
        torch.cuda.empty_cache()

    if nbytes < 1e9:
        # small problems are bound by launch latency: the same products replayed from a CUDA
        # graph separate the device time from the Python / launch overhead
        try:
            side = torch.cuda.Stream()
            with torch.cuda.stream(side):
                for _ in range(3):
                    step()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(20):
                        step()
            torch.cuda.synchronize()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            graph.replay()
            g0.record()
            for _ in range(20):
                graph.replay()
            g1.record()
            torch.cuda.synchronize()
            per = g0.elapsed_time(g1) / 400.0 / 1e3
            extra["cuda_graph_replay"] = {"us_per_product": per * 1e6, "gbs": nbytes / per / 1e9}
        except Exception as exc:  # reported, never fatal for the bench line
            extra["cuda_graph_replay"] = {"error": str(exc)[:200]}

    line = {
        "metric": "effective HBM GB/s (algorithmic bytes / time)",
        "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": DTYPE_TEXT[p.data.dtype], "data": "synthetic",
        "config": config_dict(args, 1, p.shape[0], p.nnz, nbytes),
        "parity": parity,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get((args.workload, args.scale)),
                     "peak_kind": peak_kind},
        "e2e": {"value": nbytes / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3,
                "steps_in_flight": max(1, args.e2e_depth),
                "note": "throughput with A resident and steps_in_flight steps overlapping their "
                        "copies; not the latency of one call from host buffers"},
        "gpu_launches": (launches_per_step + extra_launches(p, kind)) * args.steps,
        "clocks": sampler.summary(),
        "extra": extra,
    }
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(p, kind)
        sample_err = line["cpu_baseline"]["oracle_rel_l2_on_sample"]
        parity["oracle_rel_l2_on_sample"] = sample_err
        parity["ok"] = bool(parity["ok"] and sample_err <= parity["tol"])
    print(json.dumps(line), flush=True)
    if not parity["ok"]:
        raise SystemExit(f"parity check failed: {parity}")


if __name__ == "__main__":
    main()
