// Shared device/host helpers for libssd_b200: dtype-erased loads and stores, error
// reporting for the C ABI, small math helpers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "ssd_b200.h"

namespace ssd {

// ---- error reporting -----------------------------------------------------------------
void set_error(const char* fmt, ...);            // defined in ssd_abi.cu
const char* get_error();

#define SSD_REQUIRE(cond, status, ...)                                                    \
  do {                                                                                    \
    if (!(cond)) {                                                                        \
      ::ssd::set_error(__VA_ARGS__);                                                      \
      return (status);                                                                    \
    }                                                                                     \
  } while (0)

#define SSD_CUDA_OK(expr)                                                                 \
  do {                                                                                    \
    cudaError_t e__ = (expr);                                                             \
    if (e__ != cudaSuccess) {                                                             \
      ::ssd::set_error("%s failed: %s", #expr, cudaGetErrorString(e__));                  \
      return SSD_ERR_CUDA;                                                                \
    }                                                                                     \
  } while (0)

inline bool valid_dtype(int d) { return d == SSD_F32 || d == SSD_BF16 || d == SSD_F16; }
inline int dtype_size(int d) { return d == SSD_F32 ? 4 : 2; }

// ---- dtype-erased element access -----------------------------------------------------
__device__ __forceinline__ float load_f(const void* base, int dtype, int64_t idx) {
  switch (dtype) {
    case SSD_BF16: return __bfloat162float(static_cast<const __nv_bfloat16*>(base)[idx]);
    case SSD_F16: return __half2float(static_cast<const __half*>(base)[idx]);
    default: return static_cast<const float*>(base)[idx];
  }
}

__device__ __forceinline__ void store_f(void* base, int dtype, int64_t idx, float v) {
  switch (dtype) {
    case SSD_BF16: static_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v); break;
    case SSD_F16: static_cast<__half*>(base)[idx] = __float2half_rn(v); break;
    default: static_cast<float*>(base)[idx] = v; break;
  }
}

// Round a float to `dtype` and back: the reference's "cast to the input type before the
// dot product" rounding points.
__device__ __forceinline__ float round_to(float v, int dtype) {
  switch (dtype) {
    case SSD_BF16: return __bfloat162float(__float2bfloat16_rn(v));
    case SSD_F16: return __half2float(__float2half_rn(v));
    default: return v;
  }
}

// exp(x) evaluated as 2^(x * log2 e) with the hardware ex2 approximation: the form a
// compiled Triton `tl.exp` takes on NVIDIA GPUs, so decay factors computed here carry the
// same bits as the reference's.  Every kernel of the library uses this one function for the
// decay terms, which keeps the fused and the unfused routes bit-identical to each other.
__device__ __forceinline__ float fast_exp(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}
// z * sigmoid(z), the gate of kernels/ssd_chunk_scan.py's device code (`out *= z * tl.sigmoid(z)`), with
// the operations a compiled Triton kernel uses for it: the fast exponential above and the approximate
// division.  One function for every kernel that gates, so that they agree bit for bit.
__device__ __forceinline__ float silu_gate(float z) { return z * __fdividef(1.0f, 1.0f + fast_exp(-z)); }
// 2^y with the same instruction, for callers that have already multiplied by log2 e.
__device__ __forceinline__ float ex2_approx(float y) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(y));
  return r;
}

// log(exp(x) + 1) where x <= 20, x otherwise: the reference's softplus
// (kernels/softplus.py:8-10 applied at kernels/ssd_chunk_state.py:70).  exp as everywhere in
// the library (the form a compiled `tl.exp` takes), log through the hardware lg2
// approximation: absolute error below 2e-7 on the values a softplus returns, against a
// tolerance of 1e-5 on the cumulative sums built from them.
__device__ __forceinline__ float softplus_ref(float x) {
  return x <= 20.0f ? __logf(fast_exp(x) + 1.0f) : x;
}

// dt' of one position: bias, optional softplus, clamp (kernels/ssd_chunk_state.py:66-73 of the
// reference).  One function for every kernel that produces dt', so that they agree bit for bit.
__device__ __forceinline__ float dt_transform(float raw, float bias, bool softplus, float lo, float hi) {
  float t = raw + bias;
  if (softplus) t = softplus_ref(t);
  return fminf(fmaxf(t, lo), hi);
}

// Inclusive running sum of d[i] * a over the 256 positions a warp holds as 8 consecutive ones
// per lane (position = 8 * lane + i), continued from `carry`: each lane scans its eight
// serially, the lane totals go through one shuffle scan.  s receives the sums; the return value
// is `carry` plus the total, for the next 256 positions.  Shared by the cumsum kernel and the
// state kernel that computes the cumulative sums itself: same operations, same order.
__device__ __forceinline__ float warp_cumsum8(const float (&d)[8], float a, float carry, int lane, float (&s)[8]) {
  float run = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    run += d[i] * a;
    s[i] = run;
  }
  float incl = run;                                 // inclusive scan of the lane totals
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, off);
    if (lane >= off) incl += t;
  }
  const float before = carry + (incl - run);
#pragma unroll
  for (int i = 0; i < 8; ++i) s[i] += before;
  return carry + __shfl_sync(0xffffffffu, incl, 31);
}

}  // namespace ssd
