// Adding a carried state to passed states that were computed from a zero carry-in.
// Shared by the two second-pass kernels: the one that joins the segments of a strip inside
// one GPU and the one that joins the slices of a sequence across GPUs.
//
// For a run of chunks that started from a zero state, the true passed state of its j-th
// chunk is  out0[j] + f_j * S_in,  f_j = exp(sum of the chunk decays before j).  The helpers
// here build the f_j of up to kCarryTile chunks in shared memory and apply them.
#pragma once

#include "ssd_common.cuh"

namespace ssd {

constexpr int kCarryTile = 1024;      // chunks per factor tile
constexpr int kCarryThreads = 256;    // block size the helpers assume
constexpr int kCarryQuad = 4;         // consecutive state elements per thread

// A contribution f * S_in is dropped when f is at most this.  fp32 passed states take every
// non-zero factor.  16-bit passed states carry 8 or 11 significant bits; there, factors up to
// 2^-24 (the rounding step of the fp32 recurrence itself, relative to the carried state) are
// dropped, which bounds the second pass to the few chunks after a cut that can see the carry
// instead of every chunk whose factor has not yet underflowed in fp32.
__host__ __device__ inline float carry_cutoff(int out_dtype) {
  return out_dtype == SSD_F32 ? 0.0f : 5.9604644775390625e-8f;
}

// Called by all kCarryThreads threads.  Reads tn (<= kCarryTile) chunk decays
// decay[j * stride] and leaves fac[j] = exp(cum_in + decay[0] + ... + decay[j-1]) for j < tn
// and 0 up to the next multiple of 32.  Returns cum_in + the sum of all tn decays.
__device__ inline float chunk_factors(const float* decay, int64_t stride, int tn, float cum_in, float* fac,
                                      float* cum_slot) {
  const int tid = threadIdx.x, lane = tid & 31;
  __syncthreads();                                   // earlier readers of fac are done
  for (int j = tid; j < tn; j += kCarryThreads) fac[j] = decay[(int64_t)j * stride];
  __syncthreads();
  if (tid < 32) {
    float cum = cum_in;
    for (int j0 = 0; j0 < tn; j0 += 32) {
      const int j = j0 + lane;
      const float v = (j < tn) ? fac[j] : 0.0f;
      float incl = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
      }
      fac[j] = (j < tn) ? fast_exp(cum + incl - v) : 0.0f;
      cum += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (tid == 0) *cum_slot = cum;
  }
  __syncthreads();
  return *cum_slot;
}

// Four consecutive elements of a passed state, as one 8- or 16-byte access (VEC) or one by
// one with a count of valid elements.
template <typename OT, bool VEC>
struct Quad;

template <>
struct Quad<float, true> {
  static __device__ __forceinline__ void load(const float* p, int, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  static __device__ __forceinline__ void store(float* p, int, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Quad<__nv_bfloat16, true> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, int, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, int, const float (&v)[4]) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};
template <>
struct Quad<__half, true> {
  static __device__ __forceinline__ void load(const __half* p, int, float (&v)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__half* p, int, const float (&v)[4]) {
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    uint2 t;
    t.x = *reinterpret_cast<const uint32_t*>(&a);
    t.y = *reinterpret_cast<const uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
  }
};
template <typename OT>
struct Quad<OT, false> {
  static __device__ __forceinline__ void load(const OT* p, int n, float (&v)[4]) {
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = (e < n) ? static_cast<float>(p[e]) : 0.0f;
  }
  static __device__ __forceinline__ void store(OT* p, int n, const float (&v)[4]) {
#pragma unroll
    for (int e = 0; e < 4; ++e)
      if (e < n) p[e] = static_cast<OT>(v[e]);      // round-to-nearest conversions
  }
};

// out[j * chunk_stride + 0..n) += fac[j] * carry for the chunks j < tn whose factor exceeds
// `cut` (a NaN factor counts as exceeding, so that it still propagates).  `out` points at the
// calling thread's quad in the tile's first chunk; fac is padded with zeros to a multiple of
// four.  Four chunks are in flight per thread.
template <typename OT, bool VEC>
__device__ __forceinline__ void add_carry_tile(OT* out, int64_t chunk_stride, const float* fac, int tn, float cut,
                                               const float (&carry)[4], int n) {
  for (int j = 0; j < tn; j += 4) {
    const float4 f4 = *reinterpret_cast<const float4*>(fac + j);
    const float f[4] = {f4.x, f4.y, f4.z, f4.w};
    bool on[4];
    bool any = false;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      on[u] = !(f[u] <= cut);
      any |= on[u];
    }
    if (!any) continue;
    float v[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (on[u]) Quad<OT, VEC>::load(out + (int64_t)(j + u) * chunk_stride, n, v[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (on[u]) {
#pragma unroll
        for (int e = 0; e < 4; ++e) v[u][e] = fmaf(f[u], carry[e], v[u][e]);
        Quad<OT, VEC>::store(out + (int64_t)(j + u) * chunk_stride, n, v[u]);
      }
  }
}

// The same with the element type and the access form chosen at run time.
__device__ __forceinline__ void add_carry_tile_any(void* out, int dtype, bool vec, int64_t elem_offset,
                                                   int64_t chunk_stride, const float* fac, int tn, float cut,
                                                   const float (&carry)[4], int n) {
  switch (dtype) {
    case SSD_BF16: {
      __nv_bfloat16* p = static_cast<__nv_bfloat16*>(out) + elem_offset;
      if (vec) add_carry_tile<__nv_bfloat16, true>(p, chunk_stride, fac, tn, cut, carry, n);
      else add_carry_tile<__nv_bfloat16, false>(p, chunk_stride, fac, tn, cut, carry, n);
      break;
    }
    case SSD_F16: {
      __half* p = static_cast<__half*>(out) + elem_offset;
      if (vec) add_carry_tile<__half, true>(p, chunk_stride, fac, tn, cut, carry, n);
      else add_carry_tile<__half, false>(p, chunk_stride, fac, tn, cut, carry, n);
      break;
    }
    default: {
      float* p = static_cast<float*>(out) + elem_offset;
      if (vec) add_carry_tile<float, true>(p, chunk_stride, fac, tn, cut, carry, n);
      else add_carry_tile<float, false>(p, chunk_stride, fac, tn, cut, carry, n);
      break;
    }
  }
}

}  // namespace ssd
