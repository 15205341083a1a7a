// General-shape kernels of libssd_b200: any strides, fp32 / bf16 / fp16 inputs, ragged last
// chunk, optional seq_idx.  Plain CUDA-core arithmetic in fp32.  They cover every argument
// combination the reference's Python functions accept; the tcgen05 kernels
// (ssd_fused_sm100.cu, ssd_gemm_sm100.cu) take over for the shapes they are built for.
//
// One tiled-GEMM kernel template serves the three contractions (per-chunk state, C.B^T,
// chunk scan); each is a "problem" struct that says how to fetch an operand element, what
// to do between the two accumulation phases and how to store a result element.
#include "ssd_carry.cuh"
#include "ssd_common.cuh"
#include "ssd_launch.h"

namespace ssd {

// =====================================================================================
// chunk cumsum
// =====================================================================================
constexpr int CS_HT = 16;        // heads per block
constexpr int CS_THREADS = 256;
constexpr int CS_PER = 8;        // consecutive positions per lane in the scan
constexpr int CS_ROUND = 32 * CS_PER;
static_assert(CS_PER == 8, "warp_cumsum8 scans eight positions per lane");

// 16 bytes of consecutive heads of one position, widened to fp32.
template <typename DT> struct DtVec;
template <> struct DtVec<float> {
  static constexpr int VEC = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
};
template <> struct DtVec<__nv_bfloat16> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};
template <> struct DtVec<__half> {
  static constexpr int VEC = 8;
  static __device__ __forceinline__ void load(const __half* p, float (&v)[8]) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      v[2 * i] = f.x;
      v[2 * i + 1] = f.y;
    }
  }
};

// Block (head tile, chunk, batch).  Phase 1 reads the (L x CS_HT) tile of dt with heads
// fastest (the input's contiguous dimension), applies bias / softplus / clamp / tail mask
// and parks dt' in shared memory, one row per head.  FAST: the heads of a position are
// contiguous and 16-byte aligned, a thread takes 16 bytes of them per load; otherwise any
// strides and dtype, one element per load.  Phase 2: one warp per head; a lane takes
// CS_PER consecutive positions (two 16-byte reads), scans them serially, the lane totals go
// through one shuffle scan, and both outputs are written with positions fastest (the
// outputs' contiguous dimension), 32 bytes per lane and tensor.
template <typename DT, bool FAST>
__global__ void __launch_bounds__(CS_THREADS)
chunk_cumsum_kernel(ssd_chunk_cumsum_params_t p, int nchunks, int pitch, int vec) {
  extern __shared__ __align__(16) float tile[];         // [CS_HT][pitch], pitch % 4 == 0
  const int h0 = blockIdx.x * CS_HT;
  const int c = blockIdx.y;
  const int b = blockIdx.z;
  const int L = p.chunk_size;
  const int limit = min(L, p.seqlen - c * L);
  const int Lr = (L + CS_ROUND - 1) / CS_ROUND * CS_ROUND;
  const int tid = threadIdx.x;

  if constexpr (FAST) {
    constexpr int VEC = DtVec<DT>::VEC;
    constexpr int TPP = CS_HT / VEC;                   // threads per position
    constexpr int PPP = CS_THREADS / TPP;              // positions per pass
    const int sub = tid % TPP, kk = tid / TPP;
    float bias[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j)
      bias[j] = p.dt_bias != nullptr ? load_f(p.dt_bias, p.bias_dtype, (int64_t)(h0 + sub * VEC + j) * p.bias_stride) : 0.0f;
    const DT* src = static_cast<const DT*>(p.dt) + (int64_t)b * p.dt_stride_b + (int64_t)c * L * p.dt_stride_l + h0 + sub * VEC;
    float* dst = tile + sub * VEC * pitch;
    const bool sp = p.dt_softplus != 0;
    const float lo = p.dt_min, hi = p.dt_max;
    for (int k0 = kk; k0 < Lr; k0 += PPP * 2) {
      float v[2][VEC];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int k = k0 + u * PPP;
        if (k < limit) {
          DtVec<DT>::load(src + (int64_t)k * p.dt_stride_l, v[u]);
        } else {
#pragma unroll
          for (int j = 0; j < VEC; ++j) v[u][j] = 0.0f;
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int k = k0 + u * PPP;
        if (k < Lr) {
          const bool live = k < limit;
#pragma unroll
          for (int j = 0; j < VEC; ++j) {
            const float t = dt_transform(v[u][j], bias[j], sp, lo, hi);
            dst[j * pitch + k] = live ? t : 0.0f;      // positions past the chunk hold zeros
          }
        }
      }
    }
  } else {
    // a thread always serves the same head (CS_THREADS is a multiple of CS_HT)
    const int hh_t = tid % CS_HT;
    const int h_t = h0 + hh_t;
    const bool head_ok = h_t < p.nheads;
    const float bias = (head_ok && p.dt_bias != nullptr)
                           ? load_f(p.dt_bias, p.bias_dtype, (int64_t)h_t * p.bias_stride) : 0.0f;
    const int64_t dt_base = (int64_t)b * p.dt_stride_b + (int64_t)c * L * p.dt_stride_l + (int64_t)h_t * p.dt_stride_h;
    constexpr int kRowsPerPass = CS_THREADS / CS_HT;     // 16 positions per pass
    constexpr int kUnroll = 8;                           // loads in flight per thread
    for (int k0 = tid / CS_HT; k0 < Lr; k0 += kRowsPerPass * kUnroll) {
      float v[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = k0 + u * kRowsPerPass;
        v[u] = (head_ok && k < limit) ? load_f(p.dt, p.dt_dtype, dt_base + (int64_t)k * p.dt_stride_l) : 0.0f;
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int k = k0 + u * kRowsPerPass;
        if (k < Lr) {
          float t = 0.0f;
          if (head_ok && k < limit) t = dt_transform(v[u], bias, p.dt_softplus != 0, p.dt_min, p.dt_max);
          tile[hh_t * pitch + k] = t;                    // positions past the chunk hold zeros
        }
      }
    }
  }
  __syncthreads();

  const int warp = tid >> 5, lane = tid & 31;
  for (int hh = warp; hh < CS_HT; hh += CS_THREADS / 32) {
    const int h = h0 + hh;
    if (h >= p.nheads) break;
    const float a = load_f(p.A, p.A_dtype, (int64_t)h * p.A_stride);
    const int64_t obase = (((int64_t)b * p.nheads + h) * nchunks + c) * L;
    float carry = 0.0f;
    for (int k0 = 0; k0 < Lr; k0 += CS_ROUND) {
      const int k = k0 + lane * CS_PER;
      float d[CS_PER], s[CS_PER];
      {
        const float4 lo = *reinterpret_cast<const float4*>(tile + hh * pitch + k);
        const float4 hi = *reinterpret_cast<const float4*>(tile + hh * pitch + k + 4);
        d[0] = lo.x; d[1] = lo.y; d[2] = lo.z; d[3] = lo.w;
        d[4] = hi.x; d[5] = hi.y; d[6] = hi.z; d[7] = hi.w;
      }
      carry = warp_cumsum8(d, a, carry, lane, s);
      if (vec && k + CS_PER <= L) {
        float4* o1 = reinterpret_cast<float4*>(p.dt_out + obase + k);
        float4* o2 = reinterpret_cast<float4*>(p.dA_cumsum + obase + k);
        o1[0] = make_float4(d[0], d[1], d[2], d[3]);
        o1[1] = make_float4(d[4], d[5], d[6], d[7]);
        o2[0] = make_float4(s[0], s[1], s[2], s[3]);
        o2[1] = make_float4(s[4], s[5], s[6], s[7]);
      } else {
#pragma unroll
        for (int i = 0; i < CS_PER; ++i)
          if (k + i < L) {
            p.dt_out[obase + k + i] = d[i];
            p.dA_cumsum[obase + k + i] = s[i];
          }
      }
    }
  }
}

int launch_chunk_cumsum(const ssd_chunk_cumsum_params_t& p, cudaStream_t stream) {
  const int nchunks = (p.seqlen + p.chunk_size - 1) / p.chunk_size;
  const int pitch = (p.chunk_size + CS_ROUND - 1) / CS_ROUND * CS_ROUND + 4;
  const size_t smem = (size_t)CS_HT * pitch * sizeof(float);
  SSD_REQUIRE(smem <= 200 * 1024, SSD_ERR_UNSUPPORTED, "chunk_size %d too large for the cumsum kernel",
              p.chunk_size);
  // the vector path: heads contiguous, every position's head tile 16-byte aligned, whole tiles
  const int esz = dtype_size(p.dt_dtype);
  const bool fast = p.dt_stride_h == 1 && p.nheads % CS_HT == 0 && (reinterpret_cast<uintptr_t>(p.dt) & 15) == 0 &&
                    (p.dt_stride_l * esz) % 16 == 0 && (p.dt_stride_b * esz) % 16 == 0;
  void (*kern)(ssd_chunk_cumsum_params_t, int, int, int) = chunk_cumsum_kernel<float, false>;
  if (fast) {
    kern = p.dt_dtype == SSD_F32    ? chunk_cumsum_kernel<float, true>
           : p.dt_dtype == SSD_BF16 ? chunk_cumsum_kernel<__nv_bfloat16, true>
                                    : chunk_cumsum_kernel<__half, true>;
  }
  if (smem > 48 * 1024) {
    SSD_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  }
  SSD_REQUIRE(nchunks <= 65535 && p.batch <= 65535, SSD_ERR_UNSUPPORTED,
              "cumsum grid too large (nchunks %d, batch %d)", nchunks, p.batch);
  // 16-byte stores need aligned output rows: aligned bases and a chunk size that keeps them so
  const int vec = (p.chunk_size % 4 == 0) && (reinterpret_cast<uintptr_t>(p.dt_out) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(p.dA_cumsum) & 15) == 0;
  dim3 grid((p.nheads + CS_HT - 1) / CS_HT, nchunks, p.batch);
  kern<<<grid, CS_THREADS, smem, stream>>>(p, nchunks, pitch, vec);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

// =====================================================================================
// state passing
// =====================================================================================
__global__ void __launch_bounds__(256)
state_passing_kernel(ssd_state_passing_params_t p) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  if (d >= p.dim) return;
  float s = 0.0f;
  if (p.initial_states != nullptr)
    s = load_f(p.initial_states, p.init_dtype,
               (int64_t)b * p.init_stride[0] + (int64_t)h * p.init_stride[1] +
                   (int64_t)d * p.init_stride[2]);
  const int64_t sbase = (int64_t)b * p.states_stride[0] + (int64_t)h * p.states_stride[2] +
                        (int64_t)d * p.states_stride[3];
  const int64_t obase = (int64_t)b * p.out_stride[0] + (int64_t)h * p.out_stride[2] +
                        (int64_t)d * p.out_stride[3];
  const int64_t abase = (int64_t)b * p.dA_stride[0] + (int64_t)h * p.dA_stride[1];
  int seq_prev = 0;
  // one chunk of look-ahead keeps a load in flight while the previous chunk is combined
  float nxt = load_f(p.states, p.states_dtype, sbase);
  for (int c = 0; c < p.nchunks; ++c) {
    const float cur = nxt;
    if (c + 1 < p.nchunks)
      nxt = load_f(p.states, p.states_dtype, sbase + (int64_t)(c + 1) * p.states_stride[1]);
    store_f(p.out, p.out_dtype, obase + (int64_t)c * p.out_stride[1], s);
    float scale = fast_exp(load_f(p.dA_chunk_cumsum, p.dA_dtype, abase + (int64_t)c * p.dA_stride[2]));
    if (p.seq_idx != nullptr) {
      const int pos = min((c + 1) * p.chunk_size, p.seqlen) - 1;
      const int seq_new = p.seq_idx[(int64_t)b * p.seq_idx_stride[0] + (int64_t)pos * p.seq_idx_stride[1]];
      if (seq_new != seq_prev) scale = 0.0f;
      seq_prev = seq_new;
    }
    s = fmaf(scale, s, cur);
  }
  p.final_states[(int64_t)b * p.final_stride[0] + (int64_t)h * p.final_stride[1] +
                 (int64_t)d * p.final_stride[2]] = s;
}

// The same recurrence with four consecutive state elements per thread (16-byte fp32 / 8-byte
// 16-bit accesses through the Quad helpers of the carry kernels) and the loads of kSpAhead chunks
// in flight: the kernel is a pure stream (read every chunk state once, write every passed
// state once), so what matters is memory-level parallelism.  Needs dim-contiguous, aligned
// tensors; launch_state_passing falls back to the kernel above otherwise.
constexpr int kSpAhead = 4;

template <typename ST, typename OT>
__global__ void __launch_bounds__(256)
state_passing_vec_kernel(ssd_state_passing_params_t p) {
  const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int h = blockIdx.y;
  const int b = blockIdx.z;
  if (d >= p.dim) return;
  float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  if (p.initial_states != nullptr) {
    const int64_t ib = (int64_t)b * p.init_stride[0] + (int64_t)h * p.init_stride[1] + d;
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = load_f(p.initial_states, p.init_dtype, ib + e);
  }
  const ST* src = static_cast<const ST*>(p.states) + (int64_t)b * p.states_stride[0] + (int64_t)h * p.states_stride[2] + d;
  OT* dst = static_cast<OT*>(p.out) + (int64_t)b * p.out_stride[0] + (int64_t)h * p.out_stride[2] + d;
  const int64_t abase = (int64_t)b * p.dA_stride[0] + (int64_t)h * p.dA_stride[1];
  int seq_prev = 0;
  for (int c0 = 0; c0 < p.nchunks; c0 += kSpAhead) {
    float cur[kSpAhead][4], scale[kSpAhead];
#pragma unroll
    for (int u = 0; u < kSpAhead; ++u) {
      const int c = c0 + u;
      if (c < p.nchunks) {
        Quad<ST, true>::load(src + (int64_t)c * p.states_stride[1], 4, cur[u]);
        scale[u] = fast_exp(load_f(p.dA_chunk_cumsum, p.dA_dtype, abase + (int64_t)c * p.dA_stride[2]));
      }
    }
#pragma unroll
    for (int u = 0; u < kSpAhead; ++u) {
      const int c = c0 + u;
      if (c < p.nchunks) {
        Quad<OT, true>::store(dst + (int64_t)c * p.out_stride[1], 4, s);
        float sc = scale[u];
        if (p.seq_idx != nullptr) {
          const int pos = min((c + 1) * p.chunk_size, p.seqlen) - 1;
          const int seq_new = p.seq_idx[(int64_t)b * p.seq_idx_stride[0] + (int64_t)pos * p.seq_idx_stride[1]];
          if (seq_new != seq_prev) sc = 0.0f;
          seq_prev = seq_new;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) s[e] = fmaf(sc, s[e], cur[u][e]);
      }
    }
  }
  float* fo = p.final_states + (int64_t)b * p.final_stride[0] + (int64_t)h * p.final_stride[1] + d;
  *reinterpret_cast<float4*>(fo) = make_float4(s[0], s[1], s[2], s[3]);
}

template <typename ST>
void launch_state_passing_vec(const ssd_state_passing_params_t& p, dim3 grid, cudaStream_t stream) {
  switch (p.out_dtype) {
    case SSD_BF16: state_passing_vec_kernel<ST, __nv_bfloat16><<<grid, 256, 0, stream>>>(p); break;
    case SSD_F16: state_passing_vec_kernel<ST, __half><<<grid, 256, 0, stream>>>(p); break;
    default: state_passing_vec_kernel<ST, float><<<grid, 256, 0, stream>>>(p); break;
  }
}

int launch_state_passing(const ssd_state_passing_params_t& p, cudaStream_t stream) {
  SSD_REQUIRE(p.nheads <= 65535 && p.batch <= 65535, SSD_ERR_UNSUPPORTED,
              "state passing grid too large (nheads %d, batch %d)", p.nheads, p.batch);
  auto aligned = [](const void* q, int dtype) { return (reinterpret_cast<uintptr_t>(q) % (4 * dtype_size(dtype))) == 0; };
  bool vec = p.dim % 4 == 0 && p.states_stride[3] == 1 && p.out_stride[3] == 1 && p.final_stride[2] == 1 &&
             aligned(p.states, p.states_dtype) && aligned(p.out, p.out_dtype) && aligned(p.final_states, SSD_F32) &&
             (p.initial_states == nullptr || p.init_stride[2] == 1);
  for (int i = 0; i < 3; ++i) vec = vec && p.states_stride[i] % 4 == 0 && p.out_stride[i] % 4 == 0;
  for (int i = 0; i < 2; ++i) vec = vec && p.final_stride[i] % 4 == 0;
  if (vec) {
    dim3 grid((p.dim / 4 + 255) / 256, p.nheads, p.batch);
    switch (p.states_dtype) {
      case SSD_BF16: launch_state_passing_vec<__nv_bfloat16>(p, grid, stream); break;
      case SSD_F16: launch_state_passing_vec<__half>(p, grid, stream); break;
      default: launch_state_passing_vec<float>(p, grid, stream); break;
    }
  } else {
    dim3 grid((p.dim + 255) / 256, p.nheads, p.batch);
    state_passing_kernel<<<grid, 256, 0, stream>>>(p);
  }
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

// =====================================================================================
// sequence-parallel fix-up
// =====================================================================================
// Block = one (batch, head) and one slice of 1024 state elements; a thread owns four
// consecutive ones.  The carried state is a weighted sum of the earlier ranks' slice-final
// states (weights: products of the slice decays in between).  The block turns the local chunk
// decays into per-chunk factors exp(sum of the earlier chunks' decays), 1024 chunks at a
// time, and adds factor * carried state to its elements of the chunks whose factor is above
// the cut-off of the output type, and to the local final state.
constexpr int SP_SLICE = kCarryThreads * kCarryQuad;

__global__ void __launch_bounds__(kCarryThreads)
seqpar_fixup_kernel(ssd_seqpar_fixup_params_t p, int vec) {
  __shared__ __align__(16) float fac[kCarryTile];
  __shared__ float cum_slot;
  const int tid = threadIdx.x;
  const int h = blockIdx.x, b = blockIdx.y;
  const int d0 = blockIdx.z * SP_SLICE + tid * kCarryQuad;
  const int n = max(0, min(kCarryQuad, p.dim - d0));          // owned elements that exist
  const int64_t bh = (int64_t)b * p.nheads + h;
  const int64_t zstride = p.Z_rank_stride != 0 ? p.Z_rank_stride : (int64_t)p.batch * p.nheads * p.dim;
  const int64_t lstride = p.logP_rank_stride != 0 ? p.logP_rank_stride : (int64_t)p.batch * p.nheads;
  float s_in[kCarryQuad];
#pragma unroll
  for (int e = 0; e < kCarryQuad; ++e) s_in[e] = 0.0f;
  float logw = 0.0f;                      // sum of logP_k for j < k < rank, built from the back
  for (int j = p.rank - 1; j >= 0; --j) {
    const float w = fast_exp(logw);
#pragma unroll
    for (int e = 0; e < kCarryQuad; ++e)
      if (e < n) s_in[e] = fmaf(w, p.Z_all[(int64_t)j * zstride + bh * p.dim + d0 + e], s_in[e]);
    logw += p.logP_all[(int64_t)j * lstride + bh];
  }
  const float* decay = p.dA_chunk_last + (int64_t)b * p.dA_stride[0] + (int64_t)h * p.dA_stride[1];
  const int64_t obase = (int64_t)b * p.out_stride[0] + (int64_t)h * p.out_stride[2] + d0;
  const float cut = carry_cutoff(p.out_dtype);
  float cum = 0.0f;                       // decay accumulated since the slice start
  for (int t0 = 0; t0 < p.nchunks; t0 += kCarryTile) {
    const int tn = min(kCarryTile, p.nchunks - t0);
    cum = chunk_factors(decay + (int64_t)t0 * p.dA_stride[2], p.dA_stride[2], tn, cum, fac, &cum_slot);
    if (n > 0)
      add_carry_tile_any(p.out, p.out_dtype, vec != 0 && n == kCarryQuad, obase + (int64_t)t0 * p.out_stride[1],
                         p.out_stride[1], fac, tn, cut, s_in, n);
  }
  const float ftot = fast_exp(cum);
  const int64_t fo = (int64_t)b * p.final_stride[0] + (int64_t)h * p.final_stride[1];
#pragma unroll
  for (int e = 0; e < kCarryQuad; ++e)
    if (e < n)
      p.final_states[fo + d0 + e] = fmaf(ftot, s_in[e], p.Z_all[(int64_t)p.rank * zstride + bh * p.dim + d0 + e]);
}

int launch_seqpar_fixup(const ssd_seqpar_fixup_params_t& p, cudaStream_t stream) {
  SSD_REQUIRE(p.nheads <= 65535 * 32 && p.batch <= 65535, SSD_ERR_UNSUPPORTED, "fix-up grid too large");
  dim3 grid(p.nheads, p.batch, (p.dim + SP_SLICE - 1) / SP_SLICE);
  bool vec = reinterpret_cast<uintptr_t>(p.out) % (kCarryQuad * dtype_size(p.out_dtype)) == 0;
  for (int i = 0; i < 3; ++i) vec = vec && p.out_stride[i] % kCarryQuad == 0;
  seqpar_fixup_kernel<<<grid, kCarryThreads, 0, stream>>>(p, vec ? 1 : 0);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

// =====================================================================================
// tiled contraction template
// =====================================================================================
constexpr int TG_BM = 64, TG_BN = 64, TG_BK = 16, TG_THREADS = 256;
constexpr int TG_MAX_L = 1024;   // per-chunk vectors parked in shared memory

// A problem P provides:
//   static constexpr int kPhases; static constexpr bool kAFastM[kPhases-as-bits], ...
//   __device__ bool init(Ctx&, int by, int bz, int m0, int n0, float* vec0, float* vec1)
//   __device__ int  K(const Ctx&, int phase)
//   __device__ float loadA(const Ctx&, int phase, int m, int k)
//   __device__ float loadB(const Ctx&, int phase, int k, int n)
//   __device__ float after_phase(const Ctx&, int phase, int m, float acc)   (row scaling)
//   __device__ void  store(const Ctx&, int m, int n, float acc)
//   __host__ dim3 grid()
template <class P>
__global__ void __launch_bounds__(TG_THREADS) tiled_contraction_kernel(P prob) {
  __shared__ float As[TG_BK][TG_BM + 4];
  __shared__ float Bs[TG_BK][TG_BN + 4];
  __shared__ float vec0[TG_MAX_L];
  __shared__ float vec1[TG_MAX_L];
  typename P::Ctx ctx;
  const int tiles_n = (prob.N() + TG_BN - 1) / TG_BN;
  const int m0 = (blockIdx.x / tiles_n) * TG_BM;
  const int n0 = (blockIdx.x % tiles_n) * TG_BN;
  if (!prob.init(ctx, blockIdx.y, blockIdx.z, m0, n0, vec0, vec1)) return;
  __syncthreads();

  const int tid = threadIdx.x;
  const int tm = (tid / 16) * 4;      // 4 rows of the 64x64 tile
  const int tn = (tid % 16) * 4;      // 4 columns
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  for (int phase = 0; phase < P::kPhases; ++phase) {
    const int K = prob.K(ctx, phase);
    for (int k0 = 0; k0 < K; k0 += TG_BK) {
#pragma unroll
      for (int i = 0; i < (TG_BM * TG_BK) / TG_THREADS; ++i) {
        const int e = tid + i * TG_THREADS;
        int mm, kk;
        if (P::a_fast_m(phase)) { mm = e % TG_BM; kk = e / TG_BM; }
        else { kk = e % TG_BK; mm = e / TG_BK; }
        As[kk][mm] = (k0 + kk < K) ? prob.loadA(ctx, phase, m0 + mm, k0 + kk) : 0.0f;
      }
#pragma unroll
      for (int i = 0; i < (TG_BN * TG_BK) / TG_THREADS; ++i) {
        const int e = tid + i * TG_THREADS;
        int nn, kk;
        if (P::b_fast_n(phase)) { nn = e % TG_BN; kk = e / TG_BN; }
        else { kk = e % TG_BK; nn = e / TG_BK; }
        Bs[kk][nn] = (k0 + kk < K) ? prob.loadB(ctx, phase, k0 + kk, n0 + nn) : 0.0f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TG_BK; ++kk) {
        float a[4], bv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][tm + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tn + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], bv[j], acc[i][j]);
      }
      __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = prob.after_phase(ctx, phase, m0 + tm + i, acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) prob.store(ctx, m0 + tm + i, n0 + tn + j, acc[i][j]);
}

// ---- per-chunk state -------------------------------------------------------------------
struct ChunkStateProblem {
  static constexpr int kPhases = 1;
  __device__ static bool a_fast_m(int) { return true; }    // x[k, p]: p contiguous
  __device__ static bool b_fast_n(int) { return true; }    // B[k, n]: n contiguous
  ssd_state_inputs_t in;
  void* states;
  int states_dtype;
  int64_t ss[5];
  int nchunks;
  int clamp_decay;
  struct Ctx {
    int64_t xbase, bbase, obase;
    int limit;
    const float* scale;
  };
  __host__ __device__ int N() const { return in.dstate; }
  __device__ bool init(Ctx& c, int by, int bz, int, int, float* vec0, float*) const {
    const int b = by / nchunks, ch = by % nchunks, h = bz;
    const int L = in.chunk_size;
    const int g = h / (in.nheads / in.ngroups);
    c.limit = min(L, in.seqlen - ch * L);
    c.xbase = (int64_t)b * in.x_stride[0] + (int64_t)ch * L * in.x_stride[1] + (int64_t)h * in.x_stride[2];
    c.bbase = (int64_t)b * in.B_stride[0] + (int64_t)ch * L * in.B_stride[1] + (int64_t)g * in.B_stride[2];
    c.obase = (int64_t)b * ss[0] + (int64_t)ch * ss[1] + (int64_t)h * ss[2];
    const int64_t dtb = (int64_t)b * in.dt_stride[0] + (int64_t)h * in.dt_stride[1] + (int64_t)ch * in.dt_stride[2];
    const int64_t dab = (int64_t)b * in.dA_stride[0] + (int64_t)h * in.dA_stride[1] + (int64_t)ch * in.dA_stride[2];
    const float last = in.dA_cumsum[dab + (int64_t)(L - 1) * in.dA_stride[3]];
    int seq_last = 0;
    const int64_t sib = in.seq_idx ? (int64_t)b * in.seq_idx_stride[0] + (int64_t)ch * L * in.seq_idx_stride[1] : 0;
    if (in.seq_idx) seq_last = in.seq_idx[sib + (int64_t)(c.limit - 1) * in.seq_idx_stride[1]];
    for (int k = threadIdx.x; k < L; k += blockDim.x) {
      float s = 0.0f;
      if (k < c.limit) {
        float d = last - in.dA_cumsum[dab + (int64_t)k * in.dA_stride[3]];
        if (clamp_decay) d = fminf(d, 0.0f);
        s = fast_exp(d) * in.dt[dtb + (int64_t)k * in.dt_stride[3]];
        if (in.seq_idx && in.seq_idx[sib + (int64_t)k * in.seq_idx_stride[1]] != seq_last) s = 0.0f;
      }
      vec0[k] = s;
    }
    c.scale = vec0;
    return true;
  }
  __device__ int K(const Ctx& c, int) const { return c.limit; }
  __device__ float loadA(const Ctx& c, int, int m, int k) const {
    if (m >= in.headdim) return 0.0f;
    return load_f(in.x, in.in_dtype, c.xbase + (int64_t)k * in.x_stride[1] + (int64_t)m * in.x_stride[3]);
  }
  __device__ float loadB(const Ctx& c, int, int k, int n) const {
    if (n >= in.dstate) return 0.0f;
    const float v = load_f(in.B, in.in_dtype, c.bbase + (int64_t)k * in.B_stride[1] + (int64_t)n * in.B_stride[3]);
    return round_to(v * c.scale[k], in.in_dtype);
  }
  __device__ float after_phase(const Ctx&, int, int, float acc) const { return acc; }
  __device__ void store(const Ctx& c, int m, int n, float acc) const {
    if (m < in.headdim && n < in.dstate)
      store_f(states, states_dtype, c.obase + (int64_t)m * ss[3] + (int64_t)n * ss[4], acc);
  }
};

int launch_chunk_state_general(const ssd_chunk_state_params_t& p, int clamp_decay, cudaStream_t stream) {
  ChunkStateProblem prob;
  prob.in = p.in;
  prob.states = p.states;
  prob.states_dtype = p.states_dtype;
  for (int i = 0; i < 5; ++i) prob.ss[i] = p.states_stride[i];
  prob.nchunks = (p.in.seqlen + p.in.chunk_size - 1) / p.in.chunk_size;
  prob.clamp_decay = clamp_decay;
  SSD_REQUIRE(p.in.chunk_size <= TG_MAX_L, SSD_ERR_UNSUPPORTED, "chunk_size %d > %d", p.in.chunk_size, TG_MAX_L);
  const int64_t by = (int64_t)p.in.batch * prob.nchunks;
  SSD_REQUIRE(by <= 65535 && p.in.nheads <= 65535, SSD_ERR_UNSUPPORTED,
              "chunk state grid too large (batch*nchunks %lld)", (long long)by);
  dim3 grid(((p.in.headdim + TG_BM - 1) / TG_BM) * ((p.in.dstate + TG_BN - 1) / TG_BN), (unsigned)by, p.in.nheads);
  tiled_contraction_kernel<ChunkStateProblem><<<grid, TG_THREADS, 0, stream>>>(prob);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

// ---- C . B^T per chunk ----------------------------------------------------------------
struct BmmProblem {
  static constexpr int kPhases = 1;
  __device__ static bool a_fast_m(int) { return false; }   // a[i, k]: k contiguous
  __device__ static bool b_fast_n(int) { return false; }   // b[j, k]: k contiguous
  ssd_bmm_chunk_params_t p;
  int nchunks;
  struct Ctx {
    int64_t abase, bbase, obase, sib;
    int limit, m0, n0;
  };
  __host__ __device__ int N() const { return p.chunk_size; }
  __device__ bool init(Ctx& c, int by, int bz, int m0, int n0, float*, float*) const {
    if (p.causal && n0 >= m0 + TG_BM) return false;
    const int b = by, ch = bz / p.ngroups, g = bz % p.ngroups;
    const int L = p.chunk_size;
    c.limit = min(L, p.seqlen - ch * L);
    c.abase = (int64_t)b * p.a_stride[0] + (int64_t)ch * L * p.a_stride[1] + (int64_t)g * p.a_stride[2];
    c.bbase = (int64_t)b * p.b_stride[0] + (int64_t)ch * L * p.b_stride[1] + (int64_t)g * p.b_stride[2];
    c.obase = (int64_t)b * p.out_stride[0] + (int64_t)ch * p.out_stride[1] + (int64_t)g * p.out_stride[2];
    c.sib = p.seq_idx ? (int64_t)b * p.seq_idx_stride[0] + (int64_t)ch * L * p.seq_idx_stride[1] : 0;
    return true;
  }
  __device__ int K(const Ctx&, int) const { return p.k; }
  __device__ float loadA(const Ctx& c, int, int m, int k) const {
    if (m >= c.limit) return 0.0f;
    return load_f(p.a, p.in_dtype, c.abase + (int64_t)m * p.a_stride[1] + (int64_t)k * p.a_stride[3]);
  }
  __device__ float loadB(const Ctx& c, int, int k, int n) const {
    if (n >= c.limit) return 0.0f;
    return load_f(p.b, p.in_dtype, c.bbase + (int64_t)n * p.b_stride[1] + (int64_t)k * p.b_stride[3]);
  }
  __device__ float after_phase(const Ctx&, int, int, float acc) const { return acc; }
  __device__ void store(const Ctx& c, int m, int n, float acc) const {
    if (m >= p.chunk_size || n >= p.chunk_size) return;
    if (p.seq_idx) {
      // out-of-range rows/columns carry -1 / -2 so that they never compare equal
      const int sm = m < c.limit ? p.seq_idx[c.sib + (int64_t)m * p.seq_idx_stride[1]] : -1;
      const int sn = n < c.limit ? p.seq_idx[c.sib + (int64_t)n * p.seq_idx_stride[1]] : -2;
      if (sm != sn) acc = 0.0f;
    }
    store_f(p.out, p.out_dtype, c.obase + (int64_t)m * p.out_stride[3] + (int64_t)n * p.out_stride[4], acc);
  }
};

int launch_bmm_chunk_general(const ssd_bmm_chunk_params_t& p, cudaStream_t stream) {
  BmmProblem prob;
  prob.p = p;
  prob.nchunks = (p.seqlen + p.chunk_size - 1) / p.chunk_size;
  const int tiles = (p.chunk_size + TG_BM - 1) / TG_BM;
  const int64_t bz = (int64_t)prob.nchunks * p.ngroups;
  SSD_REQUIRE(bz <= 65535 && p.batch <= 65535, SSD_ERR_UNSUPPORTED, "bmm grid too large");
  dim3 grid(tiles * tiles, p.batch, (unsigned)bz);
  tiled_contraction_kernel<BmmProblem><<<grid, TG_THREADS, 0, stream>>>(prob);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

// ---- chunk scan -----------------------------------------------------------------------
struct ChunkScanProblem {
  static constexpr int kPhases = 2;
  // phase 0: A = C[m, n] (n contiguous), B = states[p, n] (n contiguous)
  // phase 1: A = cb[m, k] (k contiguous), B = x[k, p] (p contiguous)
  __device__ static bool a_fast_m(int) { return false; }
  __device__ static bool b_fast_n(int phase) { return phase == 1; }
  ssd_chunk_scan_params_t p;
  int nchunks;
  struct Ctx {
    int64_t cbbase, xbase, zbase, obase, Cbase, sbase;
    int limit, m0, h;
    const float* dA;
    const float* dt;
    int seq_prev;
    int64_t sib;
  };
  __host__ __device__ int N() const { return p.headdim; }
  __device__ bool init(Ctx& c, int by, int bz, int m0, int, float* vec0, float* vec1) const {
    const int b = by / nchunks, ch = by % nchunks, h = bz;
    const int L = p.chunk_size;
    const int g = h / (p.nheads / p.ngroups);
    c.h = h;
    c.m0 = m0;
    c.limit = min(L, p.seqlen - ch * L);
    c.cbbase = (int64_t)b * p.cb_stride[0] + (int64_t)ch * p.cb_stride[1] + (int64_t)g * p.cb_stride[2];
    c.xbase = (int64_t)b * p.x_stride[0] + (int64_t)ch * L * p.x_stride[1] + (int64_t)h * p.x_stride[2];
    c.zbase = (int64_t)b * p.z_stride[0] + (int64_t)ch * L * p.z_stride[1] + (int64_t)h * p.z_stride[2];
    c.obase = (int64_t)b * p.out_stride[0] + (int64_t)ch * L * p.out_stride[1] + (int64_t)h * p.out_stride[2];
    c.Cbase = (int64_t)b * p.C_stride[0] + (int64_t)ch * L * p.C_stride[1] + (int64_t)g * p.C_stride[2];
    c.sbase = (int64_t)b * p.states_stride[0] + (int64_t)ch * p.states_stride[1] + (int64_t)h * p.states_stride[2];
    const int64_t dtb = (int64_t)b * p.dt_stride[0] + (int64_t)h * p.dt_stride[1] + (int64_t)ch * p.dt_stride[2];
    const int64_t dab = (int64_t)b * p.dA_stride[0] + (int64_t)h * p.dA_stride[1] + (int64_t)ch * p.dA_stride[2];
    for (int k = threadIdx.x; k < L; k += blockDim.x) {
      vec0[k] = p.dA_cumsum[dab + (int64_t)k * p.dA_stride[3]];
      vec1[k] = p.dt[dtb + (int64_t)k * p.dt_stride[3]];
    }
    c.dA = vec0;
    c.dt = vec1;
    c.sib = 0;
    c.seq_prev = 0;
    if (p.seq_idx) {
      c.sib = (int64_t)b * p.seq_idx_stride[0] + (int64_t)ch * L * p.seq_idx_stride[1];
      c.seq_prev = ch >= 1 ? p.seq_idx[c.sib - p.seq_idx_stride[1]] : 0;
    }
    return true;
  }
  __device__ int K(const Ctx& c, int phase) const {
    return phase == 0 ? p.dstate : min(c.m0 + TG_BM, c.limit);   // causal: stop at the diagonal tile
  }
  __device__ float loadA(const Ctx& c, int phase, int m, int k) const {
    if (phase == 0) {
      if (m >= c.limit) return 0.0f;
      return load_f(p.C, p.in_dtype, c.Cbase + (int64_t)m * p.C_stride[1] + (int64_t)k * p.C_stride[3]);
    }
    if (m >= p.chunk_size || k > m) return 0.0f;
    float v = load_f(p.cb, p.cb_dtype, c.cbbase + (int64_t)m * p.cb_stride[3] + (int64_t)k * p.cb_stride[4]);
    v *= fast_exp(fminf(c.dA[m] - c.dA[k], 0.0f));
    v *= c.dt[k];
    return round_to(v, p.in_dtype);
  }
  __device__ float loadB(const Ctx& c, int phase, int k, int n) const {
    if (n >= p.headdim) return 0.0f;
    if (phase == 0) {
      const float v = load_f(p.states, p.states_dtype, c.sbase + (int64_t)n * p.states_stride[3] + (int64_t)k * p.states_stride[4]);
      return round_to(v, p.in_dtype);
    }
    return load_f(p.x, p.in_dtype, c.xbase + (int64_t)k * p.x_stride[1] + (int64_t)n * p.x_stride[3]);
  }
  __device__ float after_phase(const Ctx& c, int phase, int m, float acc) const {
    if (phase != 0 || m >= p.chunk_size) return acc;
    float s = fast_exp(c.dA[m]);
    if (p.seq_idx) {
      const int sm = m < c.limit ? p.seq_idx[c.sib + (int64_t)m * p.seq_idx_stride[1]] : -1;
      if (sm != c.seq_prev) s = 0.0f;
    }
    return acc * s;
  }
  __device__ void store(const Ctx& c, int m, int n, float acc) const {
    if (m >= c.limit || n >= p.headdim) return;
    if (p.D) {
      const float d = load_f(p.D, p.D_dtype, (int64_t)c.h * p.D_stride + (p.D_has_hdim ? n : 0));
      const float xr = load_f(p.x, p.in_dtype, c.xbase + (int64_t)m * p.x_stride[1] + (int64_t)n * p.x_stride[3]);
      acc += xr * d;
    }
    const int64_t o = c.obase + (int64_t)m * p.out_stride[1] + (int64_t)n * p.out_stride[3];
    if (p.z) {
      store_f(p.out_x, p.in_dtype, o, acc);
      const float zv = load_f(p.z, p.in_dtype, c.zbase + (int64_t)m * p.z_stride[1] + (int64_t)n * p.z_stride[3]);
      acc *= silu_gate(zv);
    }
    store_f(p.out, p.in_dtype, o, acc);
  }
};

int launch_chunk_scan_general(const ssd_chunk_scan_params_t& p, cudaStream_t stream) {
  ChunkScanProblem prob;
  prob.p = p;
  prob.nchunks = (p.seqlen + p.chunk_size - 1) / p.chunk_size;
  SSD_REQUIRE(p.chunk_size <= TG_MAX_L, SSD_ERR_UNSUPPORTED, "chunk_size %d > %d", p.chunk_size, TG_MAX_L);
  const int64_t by = (int64_t)p.batch * prob.nchunks;
  SSD_REQUIRE(by <= 65535 && p.nheads <= 65535, SSD_ERR_UNSUPPORTED, "chunk scan grid too large");
  dim3 grid(((p.chunk_size + TG_BM - 1) / TG_BM) * ((p.headdim + TG_BN - 1) / TG_BN), (unsigned)by, p.nheads);
  tiled_contraction_kernel<ChunkScanProblem><<<grid, TG_THREADS, 0, stream>>>(prob);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

}  // namespace ssd
