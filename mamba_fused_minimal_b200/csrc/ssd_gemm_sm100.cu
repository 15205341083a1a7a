// Chunk-local C . B^T for sm_100a: out[b, c, g, i, j] = sum_k a[b, cL + i, g, k] * b[b, cL + j, g, k]
// (the reference's _bmm_chunk_fwd, kernels/ssd_bmm.py:31-87), one tcgen05.mma tile per CTA.
//
// CTA = (128 rows i of one chunk, all L columns j) of one (batch, chunk, group).  Both operands
// are K-major as they lie in memory (k contiguous), so TMA boxes of 64 k x rows with the
// 128-byte swizzle are MMA operands as delivered.  Warp 4: one thread issues the loads, waits
// for them, issues the K / 16 MMAs (M = 128, N = L) into a TMEM accumulator and commits;
// warps 0-3 read the accumulator in the matrix-fragment arrangement and store it, each store
// instruction covering whole 32-byte sectors of eight rows.  The contraction is tiny
// (L * L * K per tile); the kernel is bound by writing the L x L result.
#include <cuda.h>

#include <mutex>

#include "sm100_ptx.cuh"
#include "ssd_common.cuh"
#include "ssd_launch.h"

namespace ssd {
namespace {

using namespace ptx;

template <typename T> struct Pack16;
template <> struct Pack16<__nv_bfloat16> { static constexpr uint32_t kFmt = 1; };
template <> struct Pack16<__half> { static constexpr uint32_t kFmt = 0; };

// Two 16-bit values in one 32-bit word, low half first.
template <typename T> struct PackPair;
template <> struct PackPair<__nv_bfloat16> {
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
};
template <> struct PackPair<__half> {
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ static __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
};

constexpr int kSeqPad = -2147483647 - 1;   // sequence index of positions past the end: matches nothing
constexpr int kBmmRows = 128;        // rows i per CTA (the MMA's M)
constexpr int kBmmThreads = 160;     // 4 epilogue warps + 1 service warp

enum BmmWait { kBmmWaitLoad = 201, kBmmWaitAcc };

struct BmmArgs {
  void* out;
  int* status;                       // device word that takes the code of a wait that gave up
  int64_t out_s[5];                  // b, c, g, i, j (elements; j stride is 1)
  int out_dtype;
  int L, K, ngroups;
  long long wait_limit;              // SM cycles a device-side wait may last
  const int32_t* seq;                // (b, l) sequence index of each position, or NULL
  int64_t seq_s[2];
  int seqlen;
};

// Status word of the bmm kernel's bounded waits.
__device__ int g_bmm_status[4];

template <typename T>
__global__ void __launch_bounds__(kBmmThreads)
bmm_chunk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const BmmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int L = a.L, K = a.K;
  const int kboxes = K / 64;
  const uint32_t a_bytes = kBmmRows * 128, b_bytes = (uint32_t)L * 128;     // one 64-k box of each operand
  const uint32_t off_b = kboxes * a_bytes;
  const uint32_t off_ctl = off_b + kboxes * b_bytes;                          // 2 barriers, abort flag, tmem address
  const uint32_t bar_load = sbase + off_ctl, bar_acc = sbase + off_ctl + 8;
  volatile int* ctl = reinterpret_cast<volatile int*>(smem + off_ctl + 16);   // [0] abort, [1] tmem
  WaitCtx wc{ctl, a.status, a.wait_limit};
  int* seq_sm = reinterpret_cast<int*>(smem + off_ctl + 64);                   // [L], packed sequences only

  const int mt = blockIdx.x;
  const int c = blockIdx.y / a.ngroups, g = blockIdx.y % a.ngroups;
  const int b = blockIdx.z;
  const uint32_t ncols = L <= 32 ? 32u : (L <= 64 ? 64u : (L <= 128 ? 128u : 256u));
  // packed sequences (kernels/ssd_bmm.py:79-83): a product survives only between two positions of the
  // same sequence; positions past the end of the tensor match nothing
  if (a.seq != nullptr) {
    const int limit = min(L, a.seqlen - c * L);
    for (int k = tid; k < L; k += kBmmThreads)
      seq_sm[k] = k < limit ? a.seq[(int64_t)b * a.seq_s[0] + (int64_t)(c * L + k) * a.seq_s[1]] : kSeqPad;
  }

  if (tid == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_acc, 1);
    ctl[0] = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == 4) {
    tmem_alloc(sbase + off_ctl + 20, ncols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = static_cast<uint32_t>(ctl[1]);

  if (warp == 4) {
    if (lane == 0) {
      mbar_expect_tx(bar_load, kboxes * (a_bytes + b_bytes));
      for (int kb = 0; kb < kboxes; ++kb) {
        tma_load_4d(sbase + kb * a_bytes, &tmap_a, bar_load, kb * 64, g, c * L + mt * kBmmRows, b);
        tma_load_4d(sbase + off_b + kb * b_bytes, &tmap_b, bar_load, kb * 64, g, c * L, b);
      }
      if (mbar_wait(bar_load, 0, wc, kBmmWaitLoad)) {
        tc_fence_after();
        const uint32_t idesc = mma_idesc(Pack16<T>::kFmt, false, false, kBmmRows, (uint32_t)L);
        // K-major operands, 128-byte swizzle: 8 rows of 128 bytes per 1024-byte atom; a K = 16
        // step inside a 64-k box is 32 bytes further along the row.
        for (int k16 = 0; k16 < K / 16; ++k16) {
          const uint32_t koff = (k16 & 3) * 32;
          const uint64_t ad = smem_desc_sw128(sbase + (k16 >> 2) * a_bytes + koff, 16, 1024);
          const uint64_t bd = smem_desc_sw128(sbase + off_b + (k16 >> 2) * b_bytes + koff, 16, 1024);
          mma_f16_ss(tmem_base, ad, bd, idesc, k16 != 0 ? 1u : 0u);
        }
        mma_commit(bar_acc);
      }
    }
  } else {
    // epilogue: warp w owns TMEM lanes 32 w .. 32 w + 31 = rows i of the tile
    if (mbar_wait(bar_acc, 0, wc, kBmmWaitAcc, 64)) {
      tc_fence_after();
      const int gq = lane >> 2, q = lane & 3;
      const int64_t tile = (int64_t)b * a.out_s[0] + (int64_t)c * a.out_s[1] + (int64_t)g * a.out_s[2] +
                           (int64_t)(mt * kBmmRows + warp * 32) * a.out_s[3];
      for (int j0 = 0; j0 < L; j0 += 32) {
#pragma unroll
        for (int lh = 0; lh < 2; ++lh) {
          uint32_t r[16];
          tmem_ld_16x256b_x4(tmem_base + (static_cast<uint32_t>(warp * 32 + lh * 16) << 16) + j0, r);
          tmem_ld_wait();
          // registers 4j+0,1: row gq, columns 8j + 2q, +1; registers 4j+2,3: row gq + 8
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
              const int64_t e = tile + (int64_t)(lh * 16 + gq + hr * 8) * a.out_s[3] + j0 + jj * 8 + 2 * q;
              float v0 = __uint_as_float(r[4 * jj + 2 * hr]), v1 = __uint_as_float(r[4 * jj + 2 * hr + 1]);
              if (a.seq != nullptr) {
                const int si = seq_sm[mt * kBmmRows + warp * 32 + lh * 16 + gq + hr * 8];
                const int2 sj = *reinterpret_cast<const int2*>(seq_sm + j0 + jj * 8 + 2 * q);
                if (si != sj.x || si == kSeqPad) v0 = 0.0f;
                if (si != sj.y || si == kSeqPad) v1 = 0.0f;
              }
              if (a.out_dtype == SSD_F32) {
                *reinterpret_cast<float2*>(static_cast<float*>(a.out) + e) = make_float2(v0, v1);
              } else if (a.out_dtype == SSD_BF16) {
                *reinterpret_cast<__nv_bfloat162*>(static_cast<__nv_bfloat16*>(a.out) + e) = __floats2bfloat162_rn(v0, v1);
              } else {
                *reinterpret_cast<__half2*>(static_cast<__half*>(a.out) + e) = __floats2half2_rn(v0, v1);
              }
            }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ncols);
  }
}


// =====================================================================================
// chunk scan (the reference's _chunk_scan_fwd, kernels/ssd_chunk_scan.py:38-169)
// =====================================================================================
// CTA = 128 positions m of one (batch, chunk, head) x the 64 headdim columns.
//   acc1[m, p] = sum_n C[m, n] * state[p, n]            SS MMA, both operands K-major from TMA
//   acc2[m, p] = sum_{k <= m} A2[m, k] * x[k, p]        A2 from tensor memory, x as TMA delivers it
//   A2[m, k]   = cast_x(cb[m, k] * exp(min(a_m - a_k, 0)) * dt_k)   (the reference's rounding point)
//   out[m, p]  = exp(a_m) * acc1 + acc2 + D * x[m, p]
// The positions k are walked in units of 32.  A ring of three shared-memory slots takes, per
// unit, the 128 x 32 fp32 tile of cb and the 32 x 64 tile of x (TMA, 128-byte swizzle).
// Warps 0-7: a thread owns one row m (= one TMEM lane; warp w covers lanes 32 (w % 4) ..) and
// 16 of a unit's 32 positions (w / 4): it reads them from the staged cb tile, applies decay, dt
// and the k <= m mask in fp32, rounds to the input type and writes them to one of two A2 slots
// in tensor memory (tcgen05.st); afterwards it runs the epilogue for 32 of the 64 headdim
// columns.  Warp 8: one thread issues every TMA load and MMA.  Units wholly above the
// diagonal are never touched.
constexpr int kScanRows = 128;
constexpr int kScanRowWarps = 8;
constexpr int kScanThreads = (kScanRowWarps + 1) * 32;
constexpr int kScanU = 32;             // positions per unit
constexpr int kScanSlots = 3;          // ring depth
constexpr int kScanP = 64;             // headdim
constexpr int kScanN = 128;            // dstate

enum ScanWait { kScanWaitCS = 301, kScanWaitFull, kScanWaitAReady, kScanWaitFree, kScanWaitAcc };

struct ScanArgs {
  const void* x;
  const float* dt;
  const float* dA;
  const void* D;
  const void* z;                       // gate, same layout rules as x; NULL: no gating
  void* out;
  void* out_x;                         // the ungated result when z is given (strides of out)
  int* status;
  int64_t x_s[3], z_s[3];              // b, l, h (p stride is 1)
  int64_t dt_s[3], dA_s[3];            // b, h, c (L stride is 1)
  int64_t out_s[3];                    // b, l, h (p stride is 1)
  int64_t D_stride;
  int D_dtype, D_has_hdim;
  int L, seqlen, nheads, ngroups, nchunks;
  long long wait_limit;
  const int32_t* seq;                  // (b, l) sequence index of each position, or NULL
  int64_t seq_s[2];
};

__device__ int g_scan_status[4];

template <typename T>
__global__ void __launch_bounds__(kScanThreads, 2)
chunk_scan_kernel(const __grid_constant__ CUtensorMap tmap_C, const __grid_constant__ CUtensorMap tmap_S,
                  const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_cb,
                  const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_outx,
    const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int L = a.L;
  // shared-memory map
  constexpr uint32_t kCBox = kScanRows * 128, kSBox = kScanP * 128;          // one 64-n box of C / of the state
  constexpr uint32_t kCbTile = kScanRows * kScanU * 4, kXTile = kScanU * 128; // one unit: cb 16 KiB, x 4 KiB
  constexpr uint32_t kSlot = kCbTile + kXTile;
  constexpr uint32_t kOffS = 2 * kCBox, kOffRing = kOffS + 2 * kSBox, kOffVec = kOffRing + kScanSlots * kSlot;
  constexpr uint32_t kOffCtl = kOffVec + 2 * 256 * 4;
  float* dA_s = reinterpret_cast<float*>(smem + kOffVec);
  float* dt_s = dA_s + 256;
  const uint32_t bars = sbase + kOffCtl;
  const uint32_t bar_cs = bars, bar_acc = bars + 8;
  auto bar_full = [&](int i) { return bars + 16 + 8u * i; };
  auto bar_free = [&](int i) { return bars + 40 + 8u * i; };
  auto bar_a_ready = [&](int i) { return bars + 64 + 8u * i; };
  volatile int* ctl = reinterpret_cast<volatile int*>(smem + kOffCtl + 80);     // [0] abort, [1] tmem
  WaitCtx wc{ctl, a.status, a.wait_limit};

  const int mt = blockIdx.x;                       // 128-row tile inside the chunk
  const int h = blockIdx.y;
  const int b = blockIdx.z / a.nchunks, c = blockIdx.z % a.nchunks;
  const int g = h / (a.nheads / a.ngroups);
  const int limit = min(L, a.seqlen - c * L);      // valid positions of this chunk
  // units this tile needs: up to its own diagonal, and only those that hold data
  const int nu = min((kScanRows / kScanU) * (mt + 1), (limit + kScanU - 1) / kScanU);

  auto load_unit = [&](int u) {                     // service thread only
    const int s = u % kScanSlots;
    const uint32_t dst = sbase + kOffRing + s * kSlot;
    mbar_expect_tx(bar_full(s), kSlot);
    tma_load_5d(dst, &tmap_cb, bar_full(s), u * kScanU, mt * kScanRows, g, c, b);
    tma_load_4d(dst + kCbTile, &tmap_x, bar_full(s), 0, h, c * L + u * kScanU, b);
  };
  if (warp == kScanRowWarps && lane == 0) {
    mbar_init(bar_cs, 1);
    mbar_init(bar_acc, 1);
    for (int i = 0; i < kScanSlots; ++i) { mbar_init(bar_full(i), 1); mbar_init(bar_free(i), 1); }
    for (int i = 0; i < 2; ++i) mbar_init(bar_a_ready(i), kScanRowWarps);
    ctl[0] = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    // the first loads are on their way while the rest of the CTA sets up
    mbar_expect_tx(bar_cs, 2 * kCBox + 2 * kSBox);
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_4d(sbase + kb * kCBox, &tmap_C, bar_cs, kb * 64, g, c * L + mt * kScanRows, b);
      tma_load_5d(sbase + kOffS + kb * kSBox, &tmap_S, bar_cs, kb * 64, 0, h, c, b);
    }
    for (int u = 0; u < nu && u < kScanSlots; ++u) load_unit(u);
  }
  if (warp == kScanRowWarps) {
    tmem_alloc(sbase + kOffCtl + 84, 256);
    tmem_relinquish();
  } else {
    // this chunk's cumulative log-decay and dt rows
    const float* dAr = a.dA + (int64_t)b * a.dA_s[0] + (int64_t)h * a.dA_s[1] + (int64_t)c * a.dA_s[2];
    const float* dtr = a.dt + (int64_t)b * a.dt_s[0] + (int64_t)h * a.dt_s[1] + (int64_t)c * a.dt_s[2];
    for (int k = tid; k < L; k += kScanRowWarps * 32) {
      dA_s[k] = dAr[k];
      dt_s[k] = dtr[k];
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = static_cast<uint32_t>(ctl[1]);
  constexpr uint32_t kAcc1 = 0, kAcc2 = 64, kA2 = 128;       // TMEM columns; two A2 slots of 16

  if (warp == kScanRowWarps) {
    if (lane == 0) {
      bool ok = mbar_wait(bar_cs, 0, wc, kScanWaitCS);
      if (ok) {
        tc_fence_after();
        // acc1 = C . state^T: both K-major (dstate contiguous), 128-byte swizzle
        const uint32_t idesc1 = mma_idesc(Pack16<T>::kFmt, false, false, kScanRows, kScanP);
        for (int k16 = 0; k16 < kScanN / 16; ++k16) {
          const uint32_t koff = (k16 & 3) * 32;
          const uint64_t ad = smem_desc_sw128(sbase + (k16 >> 2) * kCBox + koff, 16, 1024);
          const uint64_t bd = smem_desc_sw128(sbase + kOffS + (k16 >> 2) * kSBox + koff, 16, 1024);
          mma_f16_ss(tmem_base + kAcc1, ad, bd, idesc1, k16 != 0 ? 1u : 0u);
        }
        // acc2 += A2 . x: A2 from tensor memory (K-major by construction), x MN-major as loaded
        const uint32_t idesc2 = mma_idesc(Pack16<T>::kFmt, false, true, kScanRows, kScanP);
        for (int u = 0; u < nu && ok; ++u) {
          const int s = u % kScanSlots;
          ok = mbar_wait(bar_full(s), (u / kScanSlots) & 1, wc, kScanWaitFull);
          if (!ok) break;
          ok = mbar_wait(bar_a_ready(u & 1), (u >> 1) & 1, wc, kScanWaitAReady);
          if (!ok) break;
          tc_fence_after();
          const uint64_t bd0 = smem_desc_sw128(sbase + kOffRing + s * kSlot + kCbTile, kXTile, 1024);
          for (int k16 = 0; k16 < kScanU / 16; ++k16)
            mma_f16_ts(tmem_base + kAcc2, tmem_base + kA2 + (u & 1) * 16 + k16 * 8, bd0 + (uint64_t)((k16 * 2048) >> 4),
                       idesc2, (u | k16) != 0 ? 1u : 0u);
          mma_commit(bar_free(s));
          // refill the slot of the previous unit once its MMAs are complete
          if (u >= 1 && u - 1 + kScanSlots < nu) {
            const int ps = (u - 1) % kScanSlots;
            ok = mbar_wait(bar_free(ps), ((u - 1) / kScanSlots) & 1, wc, kScanWaitFree);
            if (!ok) break;
            load_unit(u - 1 + kScanSlots);
          }
        }
        if (ok) mma_commit(bar_acc);
      }
    }
  } else {
    const int r = (warp & 3) * 32 + lane;            // row of the tile = TMEM lane
    const int half = warp >> 2;                      // which 16 positions of a unit / which 32 headdim columns
    const int m = mt * kScanRows + r;                // position inside the chunk
    const float am = dA_s[min(m, L - 1)];
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    // this thread's cb row inside a staged tile: 128 bytes, 16-byte pieces swizzled by row % 8
    const uint32_t row_off = (uint32_t)r * 128;
    const uint32_t rs = r & 7;
    bool ok = true;
    for (int u = 0; u < nu && ok; ++u) {
      const int s = u % kScanSlots;
      const int k0 = u * kScanU + half * 16;
      ok = mbar_wait(bar_full(s), (u / kScanSlots) & 1, wc, kScanWaitFull);
      if (!ok) break;
      // the A2 slot is free once the MMAs of unit u - 2 are complete, which is what frees that unit's ring slot
      if (u >= 2) {
        ok = mbar_wait(bar_free((u - 2) % kScanSlots), ((u - 2) / kScanSlots) & 1, wc, kScanWaitFree);
        if (!ok) break;
        tc_fence_after();
      }
      uint32_t o[8];
      if (k0 > m) {                                  // wholly above the diagonal
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = 0u;
      } else {
        const uint8_t* tile = smem + kOffRing + s * kSlot + row_off;
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 t = *reinterpret_cast<const float4*>(tile + (((half * 4 + i) ^ rs) << 4));
          v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
        float ak[16], dk[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 t = *reinterpret_cast<const float4*>(dA_s + k0 + 4 * i);
          const float4 d = *reinterpret_cast<const float4*>(dt_s + k0 + 4 * i);
          ak[4 * i] = t.x; ak[4 * i + 1] = t.y; ak[4 * i + 2] = t.z; ak[4 * i + 3] = t.w;
          dk[4 * i] = d.x; dk[4 * i + 1] = d.y; dk[4 * i + 2] = d.z; dk[4 * i + 3] = d.w;
        }
        // two positions per instruction (packed fp32): the same IEEE operations in the same order
        // as cb * exp(min(a_m - a_k, 0)) * dt_k one element at a time
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
          float2 dl = __ffma2_rn(make_float2(ak[i], ak[i + 1]), make_float2(-1.0f, -1.0f), make_float2(am, am));
          dl.x = fminf(dl.x, 0.0f);
          dl.y = fminf(dl.y, 0.0f);
          dl = __fmul2_rn(dl, make_float2(1.4426950408889634f, 1.4426950408889634f));
          const float2 e = make_float2(ex2_approx(dl.x), ex2_approx(dl.y));
          float2 w = __fmul2_rn(make_float2(v[i], v[i + 1]), e);
          w = __fmul2_rn(w, make_float2(dk[i], dk[i + 1]));
          v[i] = w.x;
          v[i + 1] = w.y;
        }
        if (k0 + 15 > m) {                           // the diagonal runs through this piece
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (k0 + i > m) v[i] = 0.0f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = PackPair<T>::pack(v[2 * i], v[2 * i + 1]);
      }
      tmem_st_32x32b_x8(tmem_base + lane_sel + kA2 + (u & 1) * 16 + half * 8, o);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_a_ready(u & 1));
    }
    // ---- epilogue: out = exp(a_m) * acc1 + acc2 + D * x[m]
    const bool live = m < limit;
    const int q = half;
    const int64_t pos = (int64_t)c * L + m;
    const uint8_t* xrow = static_cast<const uint8_t*>(a.x) +
                          2 * ((int64_t)b * a.x_s[0] + pos * a.x_s[1] + (int64_t)h * a.x_s[2]) + q * 64;
    uint4 xr[4];
    if (a.D != nullptr && live) {                    // requested before the wait, used after it
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) xr[pc] = __ldg(reinterpret_cast<const uint4*>(xrow) + pc);
    }
    uint4 zr[4];
    if (a.z != nullptr && live) {
      const uint8_t* zrow = static_cast<const uint8_t*>(a.z) +
                            2 * ((int64_t)b * a.z_s[0] + pos * a.z_s[1] + (int64_t)h * a.z_s[2]) + q * 64;
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) zr[pc] = __ldg(reinterpret_cast<const uint4*>(zrow) + pc);
    }
    const float dh = (a.D != nullptr && !a.D_has_hdim) ? load_f(a.D, a.D_dtype, (int64_t)h * a.D_stride) : 0.0f;
    if (ok) ok = mbar_wait(bar_acc, 0, wc, kScanWaitAcc, 64);
    if (ok) {
      tc_fence_after();
      float sm = fast_exp(am);
      // packed sequences (kernels/ssd_chunk_scan.py:104-108): the state carried into the chunk belongs to
      // the sequence of the previous chunk's last position (sequence 0 before the first chunk)
      if (a.seq != nullptr) {
        const int64_t sb = (int64_t)b * a.seq_s[0];
        const int prev = c > 0 ? a.seq[sb + (int64_t)(c * L - 1) * a.seq_s[1]] : 0;
        const int mine = live ? a.seq[sb + pos * a.seq_s[1]] : -1;
        if (mine != prev) sm = 0.0f;
      }
      uint32_t r1[32], r2[32];
      tmem_ld_32x32(tmem_base + lane_sel + kAcc1 + q * 32, r1);
      tmem_ld_32x32(tmem_base + lane_sel + kAcc2 + q * 32, r2);
      tmem_ld_wait();
      float res[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) res[i] = fmaf(__uint_as_float(r1[i]), sm, __uint_as_float(r2[i]));
      if (a.D != nullptr && live) {
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {             // 16-byte pieces = 8 headdim columns
          const uint32_t w[4] = {xr[pc].x, xr[pc].y, xr[pc].z, xr[pc].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float x0, x1;
            PackPair<T>::unpack(w[i], x0, x1);
            const int pcol = q * 32 + pc * 8 + 2 * i;
            const float d0 = a.D_has_hdim ? load_f(a.D, a.D_dtype, (int64_t)h * a.D_stride + pcol) : dh;
            const float d1 = a.D_has_hdim ? load_f(a.D, a.D_dtype, (int64_t)h * a.D_stride + pcol + 1) : dh;
            res[pc * 8 + 2 * i] = fmaf(x0, d0, res[pc * 8 + 2 * i]);        // explicit: both scan kernels round alike
            res[pc * 8 + 2 * i + 1] = fmaf(x1, d1, res[pc * 8 + 2 * i + 1]);
          }
        }
      }
      // The result leaves through shared memory as one TMA store per warp: this warp's 32 rows x 32
      // columns as a 32 x 64-byte box (64-byte swizzle: piece c of row r at piece c ^ ((r / 2) % 4)) in
      // the C tile's shared memory, which no MMA reads any more.  Rows past the sequence end are clipped
      // by the tensor map.  With a gate there are two boxes per warp: out_x, the ungated result, and
      // out = out_x * z * sigmoid(z) (ssd_chunk_scan.py device code).
      const bool rows_in_range = mt * kScanRows + (warp & 3) * 32 < limit;
      auto stage_and_store = [&](const CUtensorMap* map, uint32_t off) {
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint4 t;
          t.x = PackPair<T>::pack(res[pc * 8], res[pc * 8 + 1]);
          t.y = PackPair<T>::pack(res[pc * 8 + 2], res[pc * 8 + 3]);
          t.z = PackPair<T>::pack(res[pc * 8 + 4], res[pc * 8 + 5]);
          t.w = PackPair<T>::pack(res[pc * 8 + 6], res[pc * 8 + 7]);
          *reinterpret_cast<uint4*>(smem + off + lane * 64 + ((pc ^ ((lane >> 1) & 3)) << 4)) = t;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && rows_in_range) {
          tma_store_4d(map, sbase + off, q * 32, h, c * L + mt * kScanRows + (warp & 3) * 32, b);
          bulk_commit();
        }
      };
      if (a.z != nullptr) {
        stage_and_store(&tmap_outx, warp * (32 * 64));
        if (live) {
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            const uint32_t w[4] = {zr[pc].x, zr[pc].y, zr[pc].z, zr[pc].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float z0, z1;
              PackPair<T>::unpack(w[i], z0, z1);
              res[pc * 8 + 2 * i] *= silu_gate(z0);
              res[pc * 8 + 2 * i + 1] *= silu_gate(z1);
            }
          }
        }
        stage_and_store(&tmap_out, (8 + warp) * (32 * 64));
      } else {
        stage_and_store(&tmap_out, warp * (32 * 64));
      }
      if (lane == 0) bulk_wait_read_all();                          // the CTA's shared memory goes away with it
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kScanRowWarps) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// =====================================================================================
// chunk scan with the chunk-local C . B^T computed on chip (the reference's _bmm_chunk_fwd and
// _chunk_scan_fwd, kernels/ssd_bmm.py:64-72 and kernels/ssd_chunk_scan.py:96-143, in one kernel)
// =====================================================================================
// Same tile (128 positions m of one (batch, chunk, head) x 64 headdim columns), same two
// accumulators and the same rounding point as chunk_scan_kernel.  What differs:
//   * cb[m, k] is not read from memory.  Per unit of 64 positions k the MMA thread multiplies the
//     staged C tile (the A operand of acc1) by the unit's B tile (64 x 128, TMA, K-major) into a
//     128 x 64 fp32 block in tensor memory -- the MMA the stand-alone bmm kernel issues, so the
//     values are the same -- and a row thread fetches its 32 values with one tcgen05.ld.  The
//     (b, c, g, L, L) tensor, its TMA ring and its shared-memory reads are gone.  The block is free
//     again as soon as the row threads hold it in registers, so the next unit's product is ready
//     long before it is needed.
//   * Units are 64 positions wide (four per 256-position chunk): half as many hand-offs between the
//     row threads and the MMA thread as with 32.
//   * The decay, dt and causal mask are applied with the same operations in the same order as in
//     chunk_scan_kernel, the products accumulate in the same order of positions and the epilogues
//     use the same explicit FMAs: the result carries the same bits as _bmm_chunk_fwd followed by
//     _chunk_scan_fwd.  (Applying the decay below the diagonal as two multiplications,
//     exp(a_m - a_e) times a per-chunk vector exp(a_e - a_k) dt_k, was measured: 3 % faster, one
//     element in 10^5 a 16-bit step apart; the exact form is kept.)
//   * Epilogue: without a gate the x values of the D term come from the staged x tiles (a row's unit
//     is one of the last two this CTA loaded); every warp sends its 32 x 32 piece of the output (two
//     pieces with a gate) through shared memory as one TMA store.
//   * TMA and MMA issue are two threads in two warps: neither waits for the other's barriers.
constexpr int kFsU = 64;               // positions per unit
constexpr int kFsBSlots = 2;           // ring of B tiles (released by the cb MMAs)
constexpr int kFsXSlots = 3;           // ring of x tiles (released by the acc2 MMAs)
constexpr int kFsThreads = (kScanRowWarps + 2) * 32;
enum FusedScanWait { kFsWaitCbFull = 311, kFsWaitCbFree, kFsWaitBFull, kFsWaitBFree, kFsWaitXFull, kFsWaitXFree };

template <typename T, bool SEQ>
__global__ void __launch_bounds__(kFsThreads, 2)
chunk_scan_fused_kernel(const __grid_constant__ CUtensorMap tmap_C, const __grid_constant__ CUtensorMap tmap_S,
                        const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_B,
                        const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_outx,
    const ScanArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int L = a.L;
  constexpr uint32_t kCBox = kScanRows * 128, kSBox = kScanP * 128;          // one 64-n box of C / of the state
  constexpr uint32_t kBBox = kFsU * 128;                                      // one 64-n box of a unit's B rows
  constexpr uint32_t kBTile = 2 * kBBox, kXTile = kFsU * 128;                 // 16 KiB, 8 KiB
  constexpr uint32_t kOffS = 2 * kCBox, kOffB = kOffS + 2 * kSBox, kOffX = kOffB + kFsBSlots * kBTile;
  constexpr uint32_t kOffVec = kOffX + kFsXSlots * kXTile;
  constexpr uint32_t kOffCtl = kOffVec + 3 * 256 * 4;
  float* dA_s = reinterpret_cast<float*>(smem + kOffVec);
  float* dt_s = dA_s + 256;
  int* seq_sm = reinterpret_cast<int*>(dt_s + 256);         // packed sequences only
  const uint32_t bars = sbase + kOffCtl;
  const uint32_t bar_cs = bars, bar_acc = bars + 8, bar_cb_full = bars + 16, bar_cb_free = bars + 24;
  auto bar_b_full = [&](int i) { return bars + 32 + 8u * i; };
  auto bar_b_free = [&](int i) { return bars + 48 + 8u * i; };
  auto bar_x_full = [&](int i) { return bars + 64 + 8u * i; };
  auto bar_x_free = [&](int i) { return bars + 88 + 8u * i; };
  auto bar_a_ready = [&](int i) { return bars + 112 + 8u * i; };
  volatile int* ctl = reinterpret_cast<volatile int*>(smem + kOffCtl + 128);    // [0] abort, [1] tmem
  WaitCtx wc{ctl, a.status, a.wait_limit};

  const int mt = blockIdx.x;
  const int h = blockIdx.y;
  const int b = blockIdx.z / a.nchunks, c = blockIdx.z % a.nchunks;
  const int g = h / (a.nheads / a.ngroups);
  const int limit = min(L, a.seqlen - c * L);
  const int nu = min((kScanRows / kFsU) * (mt + 1), (limit + kFsU - 1) / kFsU);
  constexpr int kMmaWarp = kScanRowWarps, kTmaWarp = kScanRowWarps + 1;

  auto load_B = [&](int u) {                        // TMA thread only
    const int s = u % kFsBSlots;
    const uint32_t dst = sbase + kOffB + s * kBTile;
    mbar_expect_tx(bar_b_full(s), kBTile);
    tma_load_4d(dst, &tmap_B, bar_b_full(s), 0, g, c * L + u * kFsU, b);
    tma_load_4d(dst + kBBox, &tmap_B, bar_b_full(s), 64, g, c * L + u * kFsU, b);
  };
  auto load_x = [&](int u) {
    const int s = u % kFsXSlots;
    mbar_expect_tx(bar_x_full(s), kXTile);
    tma_load_4d(sbase + kOffX + s * kXTile, &tmap_x, bar_x_full(s), 0, h, c * L + u * kFsU, b);
  };
  if (warp == kTmaWarp && lane == 0) {
    mbar_init(bar_cs, 1);
    mbar_init(bar_acc, 1);
    mbar_init(bar_cb_full, 1);
    mbar_init(bar_cb_free, kScanRowWarps);
    for (int i = 0; i < kFsBSlots; ++i) { mbar_init(bar_b_full(i), 1); mbar_init(bar_b_free(i), 1); }
    for (int i = 0; i < kFsXSlots; ++i) { mbar_init(bar_x_full(i), 1); mbar_init(bar_x_free(i), 1); }
    for (int i = 0; i < 2; ++i) mbar_init(bar_a_ready(i), kScanRowWarps);
    ctl[0] = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    // the first loads are on their way while the rest of the CTA sets up
    mbar_expect_tx(bar_cs, 2 * kCBox + 2 * kSBox);
    for (int kb = 0; kb < 2; ++kb) {
      tma_load_4d(sbase + kb * kCBox, &tmap_C, bar_cs, kb * 64, g, c * L + mt * kScanRows, b);
      tma_load_5d(sbase + kOffS + kb * kSBox, &tmap_S, bar_cs, kb * 64, 0, h, c, b);
    }
    for (int u = 0; u < nu && u < kFsBSlots; ++u) load_B(u);
    for (int u = 0; u < nu && u < kFsXSlots; ++u) load_x(u);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(sbase + kOffCtl + 132, 256);
    tmem_relinquish();
  } else if (warp < kScanRowWarps) {
    const float* dAr = a.dA + (int64_t)b * a.dA_s[0] + (int64_t)h * a.dA_s[1] + (int64_t)c * a.dA_s[2];
    const float* dtr = a.dt + (int64_t)b * a.dt_s[0] + (int64_t)h * a.dt_s[1] + (int64_t)c * a.dt_s[2];
    for (int k = tid; k < L; k += kScanRowWarps * 32) {
      dA_s[k] = dAr[k];
      dt_s[k] = dtr[k];
      if constexpr (SEQ)
        seq_sm[k] = k < limit ? a.seq[(int64_t)b * a.seq_s[0] + (int64_t)(c * L + k) * a.seq_s[1]] : kSeqPad;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = static_cast<uint32_t>(ctl[1]);
  constexpr uint32_t kAcc1 = 0, kAcc2 = 64, kCB = 128, kA2 = 192;     // TMEM columns: one cb block of 64, two A2 slots of 32

  if (warp == kTmaWarp) {
    if (lane == 0) {
      bool ok = true;
      for (int u = 0; u < nu && ok; ++u) {
        if (u + kFsBSlots < nu) {
          ok = mbar_wait(bar_b_free(u % kFsBSlots), (u / kFsBSlots) & 1, wc, kFsWaitBFree);
          if (!ok) break;
          load_B(u + kFsBSlots);
        }
        if (u + kFsXSlots < nu) {
          ok = mbar_wait(bar_x_free(u % kFsXSlots), (u / kFsXSlots) & 1, wc, kFsWaitXFree);
          if (!ok) break;
          load_x(u + kFsXSlots);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      bool ok = mbar_wait(bar_cs, 0, wc, kScanWaitCS);
      if (ok) {
        tc_fence_after();
        const uint32_t idesc1 = mma_idesc(Pack16<T>::kFmt, false, false, kScanRows, kScanP);
        for (int k16 = 0; k16 < kScanN / 16; ++k16) {
          const uint32_t koff = (k16 & 3) * 32;
          const uint64_t ad = smem_desc_sw128(sbase + (k16 >> 2) * kCBox + koff, 16, 1024);
          const uint64_t bd = smem_desc_sw128(sbase + kOffS + (k16 >> 2) * kSBox + koff, 16, 1024);
          mma_f16_ss(tmem_base + kAcc1, ad, bd, idesc1, k16 != 0 ? 1u : 0u);
        }
        const uint32_t idesc_cb = mma_idesc(Pack16<T>::kFmt, false, false, kScanRows, kFsU);
        const uint32_t idesc2 = mma_idesc(Pack16<T>::kFmt, false, true, kScanRows, kScanP);
        for (int u = 0; u <= nu && ok; ++u) {
          if (u < nu) {
            // cb block of unit u: C tile (128 x 128, K-major) . B unit tile (64 x 128, K-major)^T
            const int s = u % kFsBSlots;
            ok = mbar_wait(bar_b_full(s), (u / kFsBSlots) & 1, wc, kFsWaitBFull);
            if (!ok) break;
            if (u > 0) {                               // the row threads hold unit u - 1's block in registers
              ok = mbar_wait(bar_cb_free, (u - 1) & 1, wc, kFsWaitCbFree);
              if (!ok) break;
            }
            tc_fence_after();
            for (int k16 = 0; k16 < kScanN / 16; ++k16) {
              const uint32_t koff = (k16 & 3) * 32;
              const uint64_t ad = smem_desc_sw128(sbase + (k16 >> 2) * kCBox + koff, 16, 1024);
              const uint64_t bd = smem_desc_sw128(sbase + kOffB + s * kBTile + (k16 >> 2) * kBBox + koff, 16, 1024);
              mma_f16_ss(tmem_base + kCB, ad, bd, idesc_cb, k16 != 0 ? 1u : 0u);
            }
            mma_commit(bar_cb_full);
            mma_commit(bar_b_free(s));
          }
          if (u > 0) {
            // acc2 += A2(u - 1) . x(u - 1): A2 from tensor memory (K-major by construction), x MN-major as loaded
            const int v = u - 1, sx = v % kFsXSlots;
            ok = mbar_wait(bar_x_full(sx), (v / kFsXSlots) & 1, wc, kFsWaitXFull);
            if (!ok) break;
            ok = mbar_wait(bar_a_ready(v & 1), (v >> 1) & 1, wc, kScanWaitAReady);
            if (!ok) break;
            tc_fence_after();
            const uint64_t bd0 = smem_desc_sw128(sbase + kOffX + sx * kXTile, kXTile, 1024);
            for (int k16 = 0; k16 < kFsU / 16; ++k16)
              mma_f16_ts(tmem_base + kAcc2, tmem_base + kA2 + (v & 1) * (kFsU / 2) + k16 * 8,
                         bd0 + (uint64_t)((k16 * 2048) >> 4), idesc2, (v | k16) != 0 ? 1u : 0u);
            mma_commit(bar_x_free(sx));
          }
        }
        if (ok) mma_commit(bar_acc);
      }
    }
  } else {
    const int wq = warp & 3;
    const int r = wq * 32 + lane;                    // row of the tile = TMEM lane
    const int half = warp >> 2;                      // which 32 positions of a unit / which 32 headdim columns
    const int m = mt * kScanRows + r;                // position inside the chunk
    const float am = dA_s[min(m, L - 1)];
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    const int udiag = (mt * kScanRows + wq * 32) / kFsU;   // the unit that holds this warp's rows
    // packed sequences (kernels/ssd_bmm.py:79-83): cb[m, k] counts only between positions of one sequence
    int sq_m = kSeqPad + 1;
    if constexpr (SEQ) {
      if (m < limit) sq_m = seq_sm[m];
    }
    bool ok = true;
    for (int u = 0; u < nu && ok; ++u) {
      const int k0 = u * kFsU + half * 32;
      ok = mbar_wait(bar_cb_full, u & 1, wc, kFsWaitCbFull);
      if (!ok) break;
      tc_fence_after();
      uint32_t o[16];
      float v[32];
      const bool above = u > udiag;                  // wholly above the diagonal
      if (!above) {
        uint32_t raw[32];
        tmem_ld_32x32(tmem_base + lane_sel + kCB + half * 32, raw);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_cb_free);       // the block may take the next unit
      if (above) {
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = 0u;
      } else {
        // cb * exp(min(a_m - a_k, 0)) * dt_k, two positions per instruction (packed fp32): the same IEEE
        // operations in the same order as one element at a time
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 t = *reinterpret_cast<const float4*>(dA_s + k0 + i);
          const float4 d = *reinterpret_cast<const float4*>(dt_s + k0 + i);
          const float ak[4] = {t.x, t.y, t.z, t.w}, dk[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
          for (int jj = 0; jj < 4; jj += 2) {
            float2 dl = __ffma2_rn(make_float2(ak[jj], ak[jj + 1]), make_float2(-1.0f, -1.0f), make_float2(am, am));
            dl.x = fminf(dl.x, 0.0f);
            dl.y = fminf(dl.y, 0.0f);
            dl = __fmul2_rn(dl, make_float2(1.4426950408889634f, 1.4426950408889634f));
            const float2 e = make_float2(ex2_approx(dl.x), ex2_approx(dl.y));
            float2 w = __fmul2_rn(make_float2(v[i + jj], v[i + jj + 1]), e);
            w = __fmul2_rn(w, make_float2(dk[jj], dk[jj + 1]));
            v[i + jj] = w.x;
            v[i + jj + 1] = w.y;
          }
        }
        if (u == udiag) {                              // the diagonal runs through this unit
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (k0 + i > m) v[i] = 0.0f;
        }
        if constexpr (SEQ) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const int4 sk = *reinterpret_cast<const int4*>(seq_sm + k0 + i);
            if (sk.x != sq_m) v[i] = 0.0f;
            if (sk.y != sq_m) v[i + 1] = 0.0f;
            if (sk.z != sq_m) v[i + 2] = 0.0f;
            if (sk.w != sq_m) v[i + 3] = 0.0f;
          }
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = PackPair<T>::pack(v[2 * i], v[2 * i + 1]);
      }
      // the A2 slot is free once the MMAs of unit u - 2 are complete, which is what frees that unit's x tile
      if (u >= 2) {
        ok = mbar_wait(bar_x_free((u - 2) % kFsXSlots), ((u - 2) / kFsXSlots) & 1, wc, kFsWaitXFree);
        if (!ok) break;
        tc_fence_after();
      }
      tmem_st_32x32b_x16(tmem_base + lane_sel + kA2 + (u & 1) * (kFsU / 2) + half * 16, o);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_a_ready(u & 1));
    }
    // ---- epilogue: out = exp(a_m) * acc1 + acc2 + D * x[m]
    const bool live = m < limit;
    const int q = half;
    const int64_t pos = (int64_t)c * L + m;
    // The row's x values for the D term come from the staged x tile of its unit (one of the last two
    // units this CTA loaded, still in the ring: 128-byte rows, 16-byte pieces swizzled by the row index
    // modulo 8).
    uint4 xr[4];
    if (a.D != nullptr && live) {                    // requested before the wait, used after it
      const int ux = m / kFsU;
      ok = mbar_wait(bar_x_full(ux % kFsXSlots), (ux / kFsXSlots) & 1, wc, kFsWaitXFull);
      const uint32_t xoff = kOffX + (ux % kFsXSlots) * kXTile + (m & (kFsU - 1)) * 128;
#pragma unroll
      for (int pc = 0; pc < 4; ++pc)
        xr[pc] = *reinterpret_cast<const uint4*>(smem + xoff + (((q * 4 + pc) ^ (m & 7)) << 4));
    }
    uint4 zr[4];
    if (a.z != nullptr && live) {
      const uint8_t* zrow = static_cast<const uint8_t*>(a.z) +
                            2 * ((int64_t)b * a.z_s[0] + pos * a.z_s[1] + (int64_t)h * a.z_s[2]) + q * 64;
#pragma unroll
      for (int pc = 0; pc < 4; ++pc) zr[pc] = __ldg(reinterpret_cast<const uint4*>(zrow) + pc);
    }
    const float dh = (a.D != nullptr && !a.D_has_hdim) ? load_f(a.D, a.D_dtype, (int64_t)h * a.D_stride) : 0.0f;
    if (ok) ok = mbar_wait(bar_acc, 0, wc, kScanWaitAcc, 64);
    if (ok) {
      tc_fence_after();
      float sm = fast_exp(am);
      // packed sequences (kernels/ssd_chunk_scan.py:104-108): the state carried into the chunk belongs to
      // the sequence of the previous chunk's last position (sequence 0 before the first chunk)
      if (a.seq != nullptr) {
        const int64_t sb = (int64_t)b * a.seq_s[0];
        const int prev = c > 0 ? a.seq[sb + (int64_t)(c * L - 1) * a.seq_s[1]] : 0;
        const int mine = live ? a.seq[sb + pos * a.seq_s[1]] : -1;
        if (mine != prev) sm = 0.0f;
      }
      uint32_t r1[32], r2[32];
      tmem_ld_32x32(tmem_base + lane_sel + kAcc1 + q * 32, r1);
      tmem_ld_32x32(tmem_base + lane_sel + kAcc2 + q * 32, r2);
      tmem_ld_wait();
      float res[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) res[i] = fmaf(__uint_as_float(r1[i]), sm, __uint_as_float(r2[i]));
      if (a.D != nullptr && live) {
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {             // 16-byte pieces = 8 headdim columns
          const uint32_t w[4] = {xr[pc].x, xr[pc].y, xr[pc].z, xr[pc].w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float x0, x1;
            PackPair<T>::unpack(w[i], x0, x1);
            const int pcol = q * 32 + pc * 8 + 2 * i;
            const float d0 = a.D_has_hdim ? load_f(a.D, a.D_dtype, (int64_t)h * a.D_stride + pcol) : dh;
            const float d1 = a.D_has_hdim ? load_f(a.D, a.D_dtype, (int64_t)h * a.D_stride + pcol + 1) : dh;
            res[pc * 8 + 2 * i] = fmaf(x0, d0, res[pc * 8 + 2 * i]);        // explicit: both scan kernels round alike
            res[pc * 8 + 2 * i + 1] = fmaf(x1, d1, res[pc * 8 + 2 * i + 1]);
          }
        }
      }
      // The result leaves through shared memory as one TMA store per warp: this warp's 32 rows x 32
      // columns as a 32 x 64-byte box (64-byte swizzle: piece c of row r at piece c ^ ((r / 2) % 4)) in
      // the C tile's shared memory, which no MMA reads any more.  Rows past the sequence end are clipped
      // by the tensor map.  With a gate there are two boxes per warp: out_x, the ungated result, and
      // out = out_x * z * sigmoid(z) (ssd_chunk_scan.py device code).
      const bool rows_in_range = mt * kScanRows + wq * 32 < limit;
      auto stage_and_store = [&](const CUtensorMap* map, uint32_t off) {
#pragma unroll
        for (int pc = 0; pc < 4; ++pc) {
          uint4 t;
          t.x = PackPair<T>::pack(res[pc * 8], res[pc * 8 + 1]);
          t.y = PackPair<T>::pack(res[pc * 8 + 2], res[pc * 8 + 3]);
          t.z = PackPair<T>::pack(res[pc * 8 + 4], res[pc * 8 + 5]);
          t.w = PackPair<T>::pack(res[pc * 8 + 6], res[pc * 8 + 7]);
          *reinterpret_cast<uint4*>(smem + off + lane * 64 + ((pc ^ ((lane >> 1) & 3)) << 4)) = t;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0 && rows_in_range) {
          tma_store_4d(map, sbase + off, q * 32, h, c * L + mt * kScanRows + wq * 32, b);
          bulk_commit();
        }
      };
      if (a.z != nullptr) {
        stage_and_store(&tmap_outx, warp * (32 * 64));
        if (live) {
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            const uint32_t w[4] = {zr[pc].x, zr[pc].y, zr[pc].z, zr[pc].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float z0, z1;
              PackPair<T>::unpack(w[i], z0, z1);
              res[pc * 8 + 2 * i] *= silu_gate(z0);
              res[pc * 8 + 2 * i + 1] *= silu_gate(z1);
            }
          }
        }
        stage_and_store(&tmap_out, (8 + warp) * (32 * 64));
      } else {
        stage_and_store(&tmap_out, warp * (32 * 64));
      }
      if (lane == 0) bulk_wait_read_all();                          // the CTA's shared memory goes away with it
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

}  // namespace

int gemm_wait_status(int* code) {
  int bs[4] = {0, 0, 0, 0}, ss[4] = {0, 0, 0, 0};
  SSD_CUDA_OK(cudaMemcpyFromSymbol(bs, g_bmm_status, sizeof(bs)));
  SSD_CUDA_OK(cudaMemcpyFromSymbol(ss, g_scan_status, sizeof(ss)));
  *code = bs[0] != 0 ? bs[0] : ss[0];
  if (*code != 0) {
    const int zero[4] = {0, 0, 0, 0};
    SSD_CUDA_OK(cudaMemcpyToSymbol(g_bmm_status, zero, sizeof(zero)));
    SSD_CUDA_OK(cudaMemcpyToSymbol(g_scan_status, zero, sizeof(zero)));
  }
  return SSD_OK;
}

// 1 if the tcgen05 kernel takes this problem (otherwise the plain kernel does).
int bmm_fast_ok(const ssd_bmm_chunk_params_t& p) {
  if (p.in_dtype != SSD_BF16 && p.in_dtype != SSD_F16) return 0;
  if (p.chunk_size != 128 && p.chunk_size != 256) return 0;
  if (p.k != 64 && p.k != 128) return 0;
  if (p.a_stride[3] != 1 || p.b_stride[3] != 1 || p.out_stride[4] != 1) return 0;
  if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15)) return 0;
  for (int i = 0; i < 3; ++i)
    if (p.a_stride[i] % 8 != 0 || p.b_stride[i] % 8 != 0) return 0;
  if (reinterpret_cast<uintptr_t>(p.out) & 7) return 0;
  for (int i = 0; i < 4; ++i)
    if (p.out_stride[i] % 2 != 0) return 0;
  if (p.ngroups > 65535 || p.batch > 65535) return 0;
  return 1;
}

int launch_bmm_chunk_fast(const ssd_bmm_chunk_params_t& p, cudaStream_t stream) {
  const int L = p.chunk_size;
  const int nchunks = (p.seqlen + L - 1) / L;
  SSD_REQUIRE((long long)nchunks * p.ngroups <= 65535, SSD_ERR_UNSUPPORTED, "bmm grid too large");
  CUtensorMap ma, mb;
  int rc = make_rows_map(&ma, p.a, p.in_dtype, p.k, p.ngroups, p.seqlen, p.batch, p.a_stride, kBmmRows);
  if (rc != SSD_OK) return rc;
  rc = make_rows_map(&mb, p.b, p.in_dtype, p.k, p.ngroups, p.seqlen, p.batch, p.b_stride, L);
  if (rc != SSD_OK) return rc;
  BmmArgs a{};
  a.out = p.out;
  SSD_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&a.status), g_bmm_status));
  for (int i = 0; i < 5; ++i) a.out_s[i] = p.out_stride[i];
  a.out_dtype = p.out_dtype;
  a.L = L;
  a.K = p.k;
  a.ngroups = p.ngroups;
  a.wait_limit = wait_limit_cycles();
  a.seq = p.seq_idx;
  a.seq_s[0] = p.seq_idx_stride[0];
  a.seq_s[1] = p.seq_idx_stride[1];
  a.seqlen = p.seqlen;
  const int kboxes = p.k / 64;
  const int smem = kboxes * (kBmmRows * 128 + L * 128) + 64 + L * 4 + 1024;
  auto kern = p.in_dtype == SSD_BF16 ? bmm_chunk_kernel<__nv_bfloat16> : bmm_chunk_kernel<__half>;
  SSD_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(L / kBmmRows, nchunks * p.ngroups, p.batch);
  kern<<<grid, kBmmThreads, smem, stream>>>(ma, mb, a);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}


// 1 if the tcgen05 chunk-scan kernel takes this problem (otherwise the plain kernel does).
int scan_fast_ok(const ssd_chunk_scan_params_t& p) {
  if (p.in_dtype != SSD_BF16 && p.in_dtype != SSD_F16) return 0;
  if (p.states_dtype != p.in_dtype || p.cb_dtype != SSD_F32) return 0;
  if (p.z != nullptr) {
    if (p.out_x == nullptr || p.z_stride[3] != 1 || (reinterpret_cast<uintptr_t>(p.z) & 15) ||
        (reinterpret_cast<uintptr_t>(p.out_x) & 15))
      return 0;
    for (int i = 0; i < 3; ++i)
      if (p.z_stride[i] % 8 != 0) return 0;
  }
  if (p.headdim != kScanP || p.dstate != kScanN) return 0;
  if (p.chunk_size != 128 && p.chunk_size != 256) return 0;
  if (p.x_stride[3] != 1 || p.C_stride[3] != 1 || p.states_stride[4] != 1 || p.out_stride[3] != 1 || p.cb_stride[4] != 1 ||
      p.dt_stride[3] != 1 || p.dA_stride[3] != 1)
    return 0;
  if (p.states_stride[3] != kScanN) return 0;                            // (p, n) dense
  auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (!al16(p.x) || !al16(p.C) || !al16(p.states) || !al16(p.out) || !al16(p.cb)) return 0;
  for (int i = 0; i < 3; ++i)
    if (p.x_stride[i] % 8 != 0 || p.C_stride[i] % 8 != 0 || p.out_stride[i] % 8 != 0) return 0;
  for (int i = 0; i < 3; ++i)
    if (p.states_stride[i] % 8 != 0) return 0;
  for (int i = 0; i < 4; ++i)
    if (p.cb_stride[i] % 4 != 0) return 0;
  if (p.nheads > 65535) return 0;
  return 1;
}

int launch_chunk_scan_fast(const ssd_chunk_scan_params_t& p, cudaStream_t stream) {
  const int L = p.chunk_size;
  const int nchunks = (p.seqlen + L - 1) / L;
  SSD_REQUIRE((long long)p.batch * nchunks <= 65535, SSD_ERR_UNSUPPORTED, "chunk scan grid too large");
  CUtensorMap mC, mS, mx, mcb;
  int rc = make_rows_map(&mC, p.C, p.in_dtype, p.dstate, p.ngroups, p.seqlen, p.batch, p.C_stride, kScanRows);
  if (rc != SSD_OK) return rc;
  rc = make_rows_map(&mx, p.x, p.in_dtype, p.headdim, p.nheads, p.seqlen, p.batch, p.x_stride, kScanU);
  if (rc != SSD_OK) return rc;
  rc = make_cb_map(&mcb, p.cb, L, p.ngroups, nchunks, p.batch, p.cb_stride, kScanU, kScanRows);
  if (rc != SSD_OK) return rc;
  rc = make_states_map(&mS, p.states, p.in_dtype, p.nheads, nchunks, p.batch, p.states_stride);
  if (rc != SSD_OK) return rc;
  ScanArgs a{};
  a.x = p.x;
  a.z = p.z;
  a.out_x = p.out_x;
  a.dt = p.dt;
  a.dA = p.dA_cumsum;
  a.D = p.D;
  a.out = p.out;
  SSD_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&a.status), g_scan_status));
  for (int i = 0; i < 3; ++i) {
    a.dt_s[i] = p.dt_stride[i];
    a.dA_s[i] = p.dA_stride[i];
    a.out_s[i] = p.out_stride[i];
    a.x_s[i] = p.x_stride[i];
    a.z_s[i] = p.z_stride[i];
  }
  a.D_stride = p.D_stride;
  a.D_dtype = p.D_dtype;
  a.D_has_hdim = p.D_has_hdim;
  a.L = L;
  a.seqlen = p.seqlen;
  a.nheads = p.nheads;
  a.ngroups = p.ngroups;
  a.nchunks = nchunks;
  a.wait_limit = wait_limit_cycles();
  a.seq = p.seq_idx;
  a.seq_s[0] = p.seq_idx_stride[0];
  a.seq_s[1] = p.seq_idx_stride[1];
  const int smem = 2 * kScanRows * 128 + 2 * kScanP * 128 + kScanSlots * (kScanRows * kScanU * 4 + kScanU * 128) +
                   2 * 256 * 4 + 128 + 1024;
  auto kern = p.in_dtype == SSD_BF16 ? chunk_scan_kernel<__nv_bfloat16> : chunk_scan_kernel<__half>;
  SSD_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(L / kScanRows, p.nheads, p.batch * nchunks);
  CUtensorMap mo, mox;
  rc = make_rows_store_map(&mo, p.out, p.in_dtype, p.nheads, p.seqlen, p.batch, p.out_stride);
  if (rc != SSD_OK) return rc;
  mox = mo;                             // a valid map even where the kernel never touches it
  if (p.z != nullptr) {
    rc = make_rows_store_map(&mox, p.out_x, p.in_dtype, p.nheads, p.seqlen, p.batch, p.out_stride);
    if (rc != SSD_OK) return rc;
  }
  kern<<<grid, kScanThreads, smem, stream>>>(mC, mS, mx, mcb, mo, mox, a);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

// 1 if the on-chip-cb chunk-scan kernel takes this problem: what scan_fast_ok asks of everything but
// cb, and B laid out like C.
int scan_fused_ok(const ssd_chunk_scan_fused_params_t& f) {
  ssd_chunk_scan_params_t p = f.scan;
  // (stand-ins so that the shared checks pass for the tensor this kernel does not read)
  p.cb = p.C;
  p.cb_dtype = SSD_F32;
  for (int i = 0; i < 4; ++i) p.cb_stride[i] = 4;
  p.cb_stride[4] = 1;
  if (!scan_fast_ok(p)) return 0;
  if (f.B == nullptr || f.B_stride[3] != 1 || (reinterpret_cast<uintptr_t>(f.B) & 15)) return 0;
  for (int i = 0; i < 3; ++i)
    if (f.B_stride[i] % 8 != 0) return 0;
  return 1;
}

int launch_chunk_scan_fused(const ssd_chunk_scan_fused_params_t& f, cudaStream_t stream) {
  const ssd_chunk_scan_params_t& p = f.scan;
  const int L = p.chunk_size;
  const int nchunks = (p.seqlen + L - 1) / L;
  SSD_REQUIRE((long long)p.batch * nchunks <= 65535, SSD_ERR_UNSUPPORTED, "chunk scan grid too large");
  CUtensorMap mC, mS, mx, mB;
  int rc = make_rows_map(&mC, p.C, p.in_dtype, p.dstate, p.ngroups, p.seqlen, p.batch, p.C_stride, kScanRows);
  if (rc != SSD_OK) return rc;
  rc = make_rows_map(&mx, p.x, p.in_dtype, p.headdim, p.nheads, p.seqlen, p.batch, p.x_stride, kFsU);
  if (rc != SSD_OK) return rc;
  rc = make_rows_map(&mB, f.B, p.in_dtype, p.dstate, p.ngroups, p.seqlen, p.batch, f.B_stride, kFsU);
  if (rc != SSD_OK) return rc;
  rc = make_states_map(&mS, p.states, p.in_dtype, p.nheads, nchunks, p.batch, p.states_stride);
  if (rc != SSD_OK) return rc;
  ScanArgs a{};
  a.x = p.x;
  a.z = p.z;
  a.out_x = p.out_x;
  a.dt = p.dt;
  a.dA = p.dA_cumsum;
  a.D = p.D;
  a.out = p.out;
  SSD_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&a.status), g_scan_status));
  for (int i = 0; i < 3; ++i) {
    a.dt_s[i] = p.dt_stride[i];
    a.dA_s[i] = p.dA_stride[i];
    a.out_s[i] = p.out_stride[i];
    a.x_s[i] = p.x_stride[i];
    a.z_s[i] = p.z_stride[i];
  }
  a.D_stride = p.D_stride;
  a.D_dtype = p.D_dtype;
  a.D_has_hdim = p.D_has_hdim;
  a.L = L;
  a.seqlen = p.seqlen;
  a.nheads = p.nheads;
  a.ngroups = p.ngroups;
  a.nchunks = nchunks;
  a.wait_limit = wait_limit_cycles();
  a.seq = p.seq_idx;
  a.seq_s[0] = p.seq_idx_stride[0];
  a.seq_s[1] = p.seq_idx_stride[1];
  const int smem = 2 * kScanRows * 128 + 2 * kScanP * 128 + kFsBSlots * 2 * kFsU * 128 + kFsXSlots * kFsU * 128 +
                   3 * 256 * 4 + 256 + 1024;
  auto kern = p.in_dtype == SSD_BF16 ? chunk_scan_fused_kernel<__nv_bfloat16, false> : chunk_scan_fused_kernel<__half, false>;
  if (p.seq_idx != nullptr)
    kern = p.in_dtype == SSD_BF16 ? chunk_scan_fused_kernel<__nv_bfloat16, true> : chunk_scan_fused_kernel<__half, true>;
  SSD_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(L / kScanRows, p.nheads, p.batch * nchunks);
  CUtensorMap mo, mox;
  rc = make_rows_store_map(&mo, p.out, p.in_dtype, p.nheads, p.seqlen, p.batch, p.out_stride);
  if (rc != SSD_OK) return rc;
  mox = mo;                             // a valid map even where the kernel never touches it
  if (p.z != nullptr) {
    rc = make_rows_store_map(&mox, p.out_x, p.in_dtype, p.nheads, p.seqlen, p.batch, p.out_stride);
    if (rc != SSD_OK) return rc;
  }
  kern<<<grid, kFsThreads, smem, stream>>>(mC, mS, mx, mB, mo, mox, a);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

}  // namespace ssd
