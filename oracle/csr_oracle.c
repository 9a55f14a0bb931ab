/*
 * csr_oracle.c -- CPU restatement of FlagSparse's CSR SpMV / SpMM arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared with (tests/,
 * the smoke test, and the CPU-baseline leg of the benchmark).  Nothing in the shipped package
 * links, imports or calls it.
 *
 * Each function restates one Triton kernel of FlagSparse together with the dtype promotion its
 * Python launcher applies (paths relative to the FlagSparse tree):
 *
 *   orc_spmv_real     _spmv_csr_real_kernel      spmv_csr.py:167-192, launcher :679-705
 *                     float32 input is promoted to float64 (spmv_csr.py:124-129); a row is
 *                     walked in segments of BLOCK_NNZ entries, each segment is summed as a
 *                     block (tl.sum, :191) and the block sums are added serially.
 *   orc_spmv_cplx     _spmv_csr_complex_kernel   spmv_csr.py:196-227, launcher :706-723
 *                     accumulates re / im in the COMPONENT dtype (float32 for complex64).
 *   orc_spmm_real     _spmm_csr_real_kernel      spmm_csr.py:135-176, launcher :2712-2759
 *                     serial over a row's entries, ACC_DTYPE float64 for float32 input.
 *   orc_spmm_cplx     _spmm_csr_complex_kernel   spmm_csr.py:181-237, launcher :2764-2789
 *                     ACC_DTYPE = component dtype.
 *   orc_transpose     _transpose_csr_for_spmv    spmv_csr.py:477-515 (== spmm_csr.py:300-338)
 *                     stable sort of the entries by column (a counting sort here, the same
 *                     permutation as the stable argsort there); optional conjugation
 *                     (spmv_csr.py:615-618, spmm_csr.py:345-348).
 *
 * Results are returned in the accumulation dtype; the Python wrapper casts them back and
 * applies alpha / beta in that same promoted precision.
 *
 * Index arrays are int64.  Rows are independent, so the row loops carry an OpenMP pragma; the
 * arithmetic inside a row is sequential and does not depend on the thread count.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Threads of the row loops.  A launcher may have exported OMP_NUM_THREADS=1 for its worker
 * processes (torch.distributed.run does); the timed CPU baseline asks for the host's cores
 * explicitly.  Returns the number of threads the next call will use. */
int orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

/* tl.sum over one block of `n` lane products: modelled as a pairwise tree over a power-of-two
 * padded block, the shape a warp-shuffle / shared-memory reduction has. */
static double block_sum_f64(double* w, int n, int block) {
  for (int i = n; i < block; ++i) w[i] = 0.0;
  for (int h = block >> 1; h > 0; h >>= 1)
    for (int i = 0; i < h; ++i) w[i] += w[i + h];
  return w[0];
}
static float block_sum_f32(float* w, int n, int block) {
  for (int i = n; i < block; ++i) w[i] = 0.0f;
  for (int h = block >> 1; h > 0; h >>= 1)
    for (int i = 0; i < h; ++i) w[i] += w[i + h];
  return w[0];
}

/* y_acc[row] (float64) = sum over the row; `is_f32` selects the input width. */
void orc_spmv_real(const void* data, int is_f32, const int64_t* idx, const int64_t* ptr,
                   const void* x, double* y_acc, int64_t n_rows, int block_nnz) {
  const float* df = (const float*)data;
  const double* dd = (const double*)data;
  const float* xf = (const float*)x;
  const double* xd = (const double*)x;
#pragma omp parallel
  {
    double* w = (double*)malloc(sizeof(double) * (size_t)block_nnz);
#pragma omp for schedule(dynamic, 256)
    for (int64_t r = 0; r < n_rows; ++r) {
      double acc = 0.0;
      for (int64_t s = ptr[r]; s < ptr[r + 1]; s += block_nnz) {
        int n = (int)((ptr[r + 1] - s) < block_nnz ? (ptr[r + 1] - s) : block_nnz);
        for (int k = 0; k < n; ++k) {
          const int64_t j = s + k;
          const double a = is_f32 ? (double)df[j] : dd[j];
          const double b = is_f32 ? (double)xf[idx[j]] : xd[idx[j]];
          w[k] = a * b;
        }
        acc = acc + block_sum_f64(w, n, block_nnz);
      }
      y_acc[r] = acc;
    }
    free(w);
  }
}

/* complex: data / x / y are interleaved (re, im).  is_c64: float components, float accumulate. */
void orc_spmv_cplx(const void* data, int is_c64, const int64_t* idx, const int64_t* ptr,
                   const void* x, void* y_acc, int64_t n_rows, int block_nnz) {
#pragma omp parallel
  {
    if (is_c64) {
      const float* d = (const float*)data;
      const float* xv = (const float*)x;
      float* y = (float*)y_acc;
      float* wr = (float*)malloc(sizeof(float) * (size_t)block_nnz);
      float* wi = (float*)malloc(sizeof(float) * (size_t)block_nnz);
#pragma omp for schedule(dynamic, 256)
      for (int64_t r = 0; r < n_rows; ++r) {
        float ar = 0.f, ai = 0.f;
        for (int64_t s = ptr[r]; s < ptr[r + 1]; s += block_nnz) {
          int n = (int)((ptr[r + 1] - s) < block_nnz ? (ptr[r + 1] - s) : block_nnz);
          for (int k = 0; k < n; ++k) {
            const int64_t j = s + k, c = idx[j];
            const float a_re = d[2 * j], a_im = d[2 * j + 1];
            const float x_re = xv[2 * c], x_im = xv[2 * c + 1];
            wr[k] = a_re * x_re - a_im * x_im;
            wi[k] = a_re * x_im + a_im * x_re;
          }
          ar = ar + block_sum_f32(wr, n, block_nnz);
          ai = ai + block_sum_f32(wi, n, block_nnz);
        }
        y[2 * r] = ar;
        y[2 * r + 1] = ai;
      }
      free(wr);
      free(wi);
    } else {
      const double* d = (const double*)data;
      const double* xv = (const double*)x;
      double* y = (double*)y_acc;
      double* wr = (double*)malloc(sizeof(double) * (size_t)block_nnz);
      double* wi = (double*)malloc(sizeof(double) * (size_t)block_nnz);
#pragma omp for schedule(dynamic, 256)
      for (int64_t r = 0; r < n_rows; ++r) {
        double ar = 0.0, ai = 0.0;
        for (int64_t s = ptr[r]; s < ptr[r + 1]; s += block_nnz) {
          int n = (int)((ptr[r + 1] - s) < block_nnz ? (ptr[r + 1] - s) : block_nnz);
          for (int k = 0; k < n; ++k) {
            const int64_t j = s + k, c = idx[j];
            const double a_re = d[2 * j], a_im = d[2 * j + 1];
            const double x_re = xv[2 * c], x_im = xv[2 * c + 1];
            wr[k] = a_re * x_re - a_im * x_im;
            wi[k] = a_re * x_im + a_im * x_re;
          }
          ar = ar + block_sum_f64(wr, n, block_nnz);
          ai = ai + block_sum_f64(wi, n, block_nnz);
        }
        y[2 * r] = ar;
        y[2 * r + 1] = ai;
      }
      free(wr);
      free(wi);
    }
  }
}

/* C_acc (float64, n_rows x n_dense, row-major) = A B;  B row-major with leading dimension ldb. */
void orc_spmm_real(const void* data, int is_f32, const int64_t* idx, const int64_t* ptr,
                   const void* B, int64_t ldb, int64_t n_dense, double* C_acc, int64_t n_rows) {
  const float* df = (const float*)data;
  const double* dd = (const double*)data;
  const float* bf = (const float*)B;
  const double* bd = (const double*)B;
#pragma omp parallel for schedule(dynamic, 64)
  for (int64_t r = 0; r < n_rows; ++r) {
    double* c = C_acc + r * n_dense;
    for (int64_t n = 0; n < n_dense; ++n) c[n] = 0.0;
    for (int64_t j = ptr[r]; j < ptr[r + 1]; ++j) {
      const double a = is_f32 ? (double)df[j] : dd[j];
      const int64_t k = idx[j];
      if (is_f32) {
        const float* b = bf + k * ldb;
        for (int64_t n = 0; n < n_dense; ++n) c[n] = c[n] + a * (double)b[n];
      } else {
        const double* b = bd + k * ldb;
        for (int64_t n = 0; n < n_dense; ++n) c[n] = c[n] + a * b[n];
      }
    }
  }
}

void orc_spmm_cplx(const void* data, int is_c64, const int64_t* idx, const int64_t* ptr,
                   const void* B, int64_t ldb, int64_t n_dense, void* C_acc, int64_t n_rows) {
  if (is_c64) {
    const float* d = (const float*)data;
    const float* bv = (const float*)B;
    float* C = (float*)C_acc;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; ++r) {
      float* c = C + 2 * r * n_dense;
      for (int64_t n = 0; n < 2 * n_dense; ++n) c[n] = 0.f;
      for (int64_t j = ptr[r]; j < ptr[r + 1]; ++j) {
        const float a_re = d[2 * j], a_im = d[2 * j + 1];
        const float* b = bv + 2 * idx[j] * ldb;
        for (int64_t n = 0; n < n_dense; ++n) {
          const float b_re = b[2 * n], b_im = b[2 * n + 1];
          c[2 * n] = c[2 * n] + a_re * b_re - a_im * b_im;
          c[2 * n + 1] = c[2 * n + 1] + a_re * b_im + a_im * b_re;
        }
      }
    }
  } else {
    const double* d = (const double*)data;
    const double* bv = (const double*)B;
    double* C = (double*)C_acc;
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t r = 0; r < n_rows; ++r) {
      double* c = C + 2 * r * n_dense;
      for (int64_t n = 0; n < 2 * n_dense; ++n) c[n] = 0.0;
      for (int64_t j = ptr[r]; j < ptr[r + 1]; ++j) {
        const double a_re = d[2 * j], a_im = d[2 * j + 1];
        const double* b = bv + 2 * idx[j] * ldb;
        for (int64_t n = 0; n < n_dense; ++n) {
          const double b_re = b[2 * n], b_im = b[2 * n + 1];
          c[2 * n] = c[2 * n] + a_re * b_re - a_im * b_im;
          c[2 * n + 1] = c[2 * n + 1] + a_re * b_im + a_im * b_re;
        }
      }
    }
  }
}

/* CSR(A) -> CSR(A^T): elem_bytes per value; conj_kind 0 none, 1 negate the second float of each
 * value (complex64), 2 negate the second double (complex128). */
void orc_transpose(const void* data, int elem_bytes, int conj_kind, const int64_t* idx,
                   const int64_t* ptr, int64_t n_rows, int64_t n_cols, void* t_data,
                   int64_t* t_idx, int64_t* t_ptr) {
  const int64_t nnz = ptr[n_rows];
  for (int64_t c = 0; c <= n_cols; ++c) t_ptr[c] = 0;
  for (int64_t j = 0; j < nnz; ++j) t_ptr[idx[j] + 1] += 1;
  for (int64_t c = 0; c < n_cols; ++c) t_ptr[c + 1] += t_ptr[c];
  int64_t* next = (int64_t*)malloc(sizeof(int64_t) * (size_t)(n_cols > 0 ? n_cols : 1));
  memcpy(next, t_ptr, sizeof(int64_t) * (size_t)n_cols);
  const char* src = (const char*)data;
  char* dst = (char*)t_data;
  for (int64_t r = 0; r < n_rows; ++r) {
    for (int64_t j = ptr[r]; j < ptr[r + 1]; ++j) { /* CSR order == ascending source position */
      const int64_t k = next[idx[j]]++;
      t_idx[k] = r;
      memcpy(dst + k * elem_bytes, src + j * elem_bytes, (size_t)elem_bytes);
      if (conj_kind == 1) ((float*)(dst + k * elem_bytes))[1] = -((float*)(dst + k * elem_bytes))[1];
      if (conj_kind == 2) ((double*)(dst + k * elem_bytes))[1] = -((double*)(dst + k * elem_bytes))[1];
    }
  }
  free(next);
}
