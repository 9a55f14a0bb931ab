// Shared device helpers: value types, warp shuffles, mbarrier + bulk-copy (TMA) wrappers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "../../include/b200sparse.h"

namespace b2s {

// ---------------------------------------------------------------------------------------------
// value types
// ---------------------------------------------------------------------------------------------
struct __align__(8) c64 {
  float re, im;
};
struct __align__(16) c128 {
  double re, im;
};

__host__ __device__ inline c64 operator+(c64 a, c64 b) { return {a.re + b.re, a.im + b.im}; }
__host__ __device__ inline c128 operator+(c128 a, c128 b) { return {a.re + b.re, a.im + b.im}; }
__host__ __device__ inline c64 operator*(c64 a, c64 b) {
  return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re};
}
__host__ __device__ inline c128 operator*(c128 a, c128 b) {
  return {a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re};
}

template <class V> struct vt;
template <> struct vt<float> {
  __host__ __device__ static float zero() { return 0.f; }
  __host__ __device__ static float one() { return 1.f; }
  __host__ __device__ static bool is_zero(float a) { return a == 0.f; }
  __host__ __device__ static float conj(float a) { return a; }
};
template <> struct vt<double> {
  __host__ __device__ static double zero() { return 0.0; }
  __host__ __device__ static double one() { return 1.0; }
  __host__ __device__ static bool is_zero(double a) { return a == 0.0; }
  __host__ __device__ static double conj(double a) { return a; }
};
template <> struct vt<c64> {
  __host__ __device__ static c64 zero() { return {0.f, 0.f}; }
  __host__ __device__ static c64 one() { return {1.f, 0.f}; }
  __host__ __device__ static bool is_zero(c64 a) { return a.re == 0.f && a.im == 0.f; }
  __host__ __device__ static c64 conj(c64 a) { return {a.re, -a.im}; }
};
template <> struct vt<c128> {
  __host__ __device__ static c128 zero() { return {0.0, 0.0}; }
  __host__ __device__ static c128 one() { return {1.0, 0.0}; }
  __host__ __device__ static bool is_zero(c128 a) { return a.re == 0.0 && a.im == 0.0; }
  __host__ __device__ static c128 conj(c128 a) { return {a.re, -a.im}; }
};

// 16-bit storage types: values, x / B and y / C are kept as float16 or bfloat16, every sum is a
// float32 sum and the result is rounded once.  to_acc widens, from_acc rounds to nearest even.
using f16 = __half;
using bf16 = __nv_bfloat16;
template <class V> __host__ __device__ inline V to_acc(V s) { return s; }
__device__ inline float to_acc(f16 s) { return __half2float(s); }
__device__ inline float to_acc(bf16 s) { return __bfloat162float(s); }
template <class S> struct storage_of {
  template <class V> __device__ static S from_acc(V v) { return v; }
};
template <> struct storage_of<f16> {
  __device__ static f16 from_acc(float v) { return __float2half_rn(v); }
};
template <> struct storage_of<bf16> {
  __device__ static bf16 from_acc(float v) { return __float2bfloat16_rn(v); }
};
__device__ inline f16 ldg_val(const f16* p) { return __ldg(p); }
__device__ inline bf16 ldg_val(const bf16* p) { return __ldg(p); }

// 2-byte payload for kernels that only move values (transpose, re-layouts): both 16-bit dtypes
struct raw16 {
  uint16_t bits;
};
template <> struct vt<raw16> {
  __host__ __device__ static raw16 conj(raw16 a) { return a; }
};
// value dtype -> the type that moves its values around (the 16-bit dtypes share one)
#define B2S_DISPATCH_MOVE(vtype, ...)                           \
  switch (vtype) {                                              \
    case B2S_F32: { using V = float; __VA_ARGS__; } break;      \
    case B2S_F64: { using V = double; __VA_ARGS__; } break;     \
    case B2S_C64: { using V = b2s::c64; __VA_ARGS__; } break;   \
    case B2S_C128: { using V = b2s::c128; __VA_ARGS__; } break; \
    case B2S_F16:                                               \
    case B2S_BF16: { using V = b2s::raw16; __VA_ARGS__; } break; \
    default: return B2S_ERR_DTYPE;                              \
  }

// acc = acc + a * b with the contraction the hardware offers
__device__ inline void fma_acc(float& acc, float a, float b) { acc = fmaf(a, b, acc); }
__device__ inline void fma_acc(double& acc, double a, double b) { acc = fma(a, b, acc); }
__device__ inline void fma_acc(c64& acc, c64 a, c64 b) {
  acc.re = fmaf(a.re, b.re, acc.re);
  acc.re = fmaf(-a.im, b.im, acc.re);
  acc.im = fmaf(a.re, b.im, acc.im);
  acc.im = fmaf(a.im, b.re, acc.im);
}
__device__ inline void fma_acc(c128& acc, c128 a, c128 b) {
  acc.re = fma(a.re, b.re, acc.re);
  acc.re = fma(-a.im, b.im, acc.re);
  acc.im = fma(a.re, b.im, acc.im);
  acc.im = fma(a.im, b.re, acc.im);
}

// read-only (non-coherent) global load of one value
__device__ inline float ldg_val(const float* p) { return __ldg(p); }
__device__ inline double ldg_val(const double* p) { return __ldg(p); }
__device__ inline c64 ldg_val(const c64* p) {
  float2 t = __ldg(reinterpret_cast<const float2*>(p));
  return {t.x, t.y};
}
__device__ inline c128 ldg_val(const c128* p) {
  double2 t = __ldg(reinterpret_cast<const double2*>(p));
  return {t.x, t.y};
}

// the same loads carrying an L2 eviction-priority descriptor
__device__ inline float ldg_val(const float* p, uint64_t pol) {
  float v;
  asm volatile("ld.global.nc.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ inline double ldg_val(const double* p, uint64_t pol) {
  double v;
  asm volatile("ld.global.nc.L2::cache_hint.f64 %0, [%1], %2;" : "=d"(v) : "l"(p), "l"(pol));
  return v;
}
__device__ inline c64 ldg_val(const c64* p, uint64_t pol) {
  c64 v;
  asm volatile("ld.global.nc.L2::cache_hint.v2.f32 {%0,%1}, [%2], %3;"
               : "=f"(v.re), "=f"(v.im)
               : "l"(p), "l"(pol));
  return v;
}
__device__ inline c128 ldg_val(const c128* p, uint64_t pol) {
  c128 v;
  asm volatile("ld.global.nc.L2::cache_hint.v2.f64 {%0,%1}, [%2], %3;"
               : "=d"(v.re), "=d"(v.im)
               : "l"(p), "l"(pol));
  return v;
}

// load of one element of a stream that is read exactly once: read-only path, no L1 allocation,
// L2 eviction priority given by `pol` (evict-first keeps the stream from displacing x)
template <class T>
__device__ inline T stream_val(const T* p, uint64_t pol) {
  T v;
  if constexpr (sizeof(T) == 4) {
    uint32_t r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b32 %0, [%1], %2;"
                 : "=r"(r) : "l"(p), "l"(pol));
    memcpy(&v, &r, 4);
  } else if constexpr (sizeof(T) == 8) {
    uint64_t r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.b64 %0, [%1], %2;"
                 : "=l"(r) : "l"(p), "l"(pol));
    memcpy(&v, &r, 8);
  } else {
    uint64_t a, b;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.b64 {%0,%1}, [%2], %3;"
                 : "=l"(a), "=l"(b) : "l"(p), "l"(pol));
    uint64_t t[2] = {a, b};
    memcpy(&v, t, 16);
  }
  return v;
}

// epilogue: alpha * s (+ beta * y0 when beta != 0; y0 is not touched otherwise)
template <class V>
__device__ inline V axpby(V alpha, V s, bool has_beta, V beta, const V* y0) {
  V r = alpha * s;
  if (has_beta) r = r + beta * (*y0);
  return r;
}

// ---------------------------------------------------------------------------------------------
// warp shuffles for 4 / 8 / 16-byte values
// ---------------------------------------------------------------------------------------------
__device__ inline float shfl_xor(float v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ inline double shfl_xor(double v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ inline c64 shfl_xor(c64 v, int m) {
  return {__shfl_xor_sync(0xffffffffu, v.re, m), __shfl_xor_sync(0xffffffffu, v.im, m)};
}
__device__ inline c128 shfl_xor(c128 v, int m) {
  return {__shfl_xor_sync(0xffffffffu, v.re, m), __shfl_xor_sync(0xffffffffu, v.im, m)};
}

// value of the lane `d` below (the caller ignores what lanes < d receive)
__device__ inline float shfl_up(float v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ inline double shfl_up(double v, int d) { return __shfl_up_sync(0xffffffffu, v, d); }
__device__ inline c64 shfl_up(c64 v, int d) {
  return {__shfl_up_sync(0xffffffffu, v.re, d), __shfl_up_sync(0xffffffffu, v.im, d)};
}
__device__ inline c128 shfl_up(c128 v, int d) {
  return {__shfl_up_sync(0xffffffffu, v.re, d), __shfl_up_sync(0xffffffffu, v.im, d)};
}

// butterfly sum over aligned groups of `width` lanes (width a power of two <= 32); every lane of
// the warp must call it.  The tree is fixed, so the result does not depend on scheduling.
template <class V>
__device__ inline V group_sum(V v, int width) {
  for (int m = width >> 1; m > 0; m >>= 1) v = v + shfl_xor(v, m);
  return v;
}

// ---------------------------------------------------------------------------------------------
// mbarrier + 1-D bulk asynchronous copy (TMA engine), CTA-local destination, no multicast
// ---------------------------------------------------------------------------------------------
__device__ inline uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ inline void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
  // make the initialised barrier visible to the async proxy that completes the copies
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)),
               "r"(bytes)
               : "memory");
}

// L2 eviction-priority descriptors
__device__ inline uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ inline uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// global -> this CTA's shared memory; src, dst 16-byte aligned, bytes a multiple of 16
__device__ inline void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes,
                                uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(smem_addr(dst_smem)),
      "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
      : "memory");
}

// Bounded wait for a barrier phase.  Each try_wait lets the hardware suspend the warp for up to
// the hinted time, so a waiting warp costs almost no issue slots; the iteration limit keeps the
// total wait finite (a lost copy ends the kernel with an error bit instead of hanging the GPU).
constexpr int kMbarSpinLimit = 1 << 18;
constexpr uint32_t kMbarSuspendNs = 2000;

__device__ inline bool mbar_wait(uint64_t* bar, uint32_t parity) {
  uint32_t a = smem_addr(bar);
  for (int it = 0; it < kMbarSpinLimit; ++it) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; "
        "selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(a), "r"(parity), "r"(kMbarSuspendNs)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// 128-bit global loads with an eviction hint for streams read exactly once
__device__ inline uint4 ldg_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

// ---------------------------------------------------------------------------------------------
// host-side dispatch helpers
// ---------------------------------------------------------------------------------------------
inline size_t vsize(int vtype) {
  switch (vtype) {
    case B2S_F32: return 4;
    case B2S_F64: return 8;
    case B2S_C64: return 8;
    case B2S_C128: return 16;
    case B2S_F16: return 2;
    case B2S_BF16: return 2;
  }
  return 0;
}
// size of the scalar alpha / beta point at: the accumulation type (float for 16-bit values)
inline size_t acc_size(int vtype) {
  return (vtype == B2S_F16 || vtype == B2S_BF16) ? 4 : vsize(vtype);
}
inline size_t isize(int itype) { return itype == B2S_I32 ? 4 : (itype == B2S_I64 ? 8 : 0); }

#define B2S_DISPATCH_V(vtype, ...)                          \
  switch (vtype) {                                          \
    case B2S_F32: { using V = float; __VA_ARGS__; } break;  \
    case B2S_F64: { using V = double; __VA_ARGS__; } break; \
    case B2S_C64: { using V = b2s::c64; __VA_ARGS__; } break;    \
    case B2S_C128: { using V = b2s::c128; __VA_ARGS__; } break;  \
    default: return B2S_ERR_DTYPE;                          \
  }
// value dtype -> accumulation type V and storage type S (S == V but for the 16-bit dtypes)
#define B2S_DISPATCH_VS(vtype, ...)                                                   \
  switch (vtype) {                                                                    \
    case B2S_F32: { using V = float; using S = float; __VA_ARGS__; } break;           \
    case B2S_F64: { using V = double; using S = double; __VA_ARGS__; } break;         \
    case B2S_C64: { using V = b2s::c64; using S = b2s::c64; __VA_ARGS__; } break;     \
    case B2S_C128: { using V = b2s::c128; using S = b2s::c128; __VA_ARGS__; } break;  \
    case B2S_F16: { using V = float; using S = b2s::f16; __VA_ARGS__; } break;        \
    case B2S_BF16: { using V = float; using S = b2s::bf16; __VA_ARGS__; } break;      \
    default: return B2S_ERR_DTYPE;                                                    \
  }
#define B2S_DISPATCH_I(itype, NAME, ...)                       \
  switch (itype) {                                             \
    case B2S_I32: { using NAME = int32_t; __VA_ARGS__; } break; \
    case B2S_I64: { using NAME = int64_t; __VA_ARGS__; } break; \
    default: return B2S_ERR_DTYPE;                             \
  }

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? B2S_OK : B2S_ERR_LAUNCH;
}

}  // namespace b2s
