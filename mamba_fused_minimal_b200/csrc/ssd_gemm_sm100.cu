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

constexpr int kBmmRows = 128;        // rows i per CTA (the MMA's M)
constexpr int kBmmThreads = 160;     // 4 epilogue warps + 1 service warp

enum BmmWait { kBmmWaitLoad = 201, kBmmWaitAcc };

struct BmmArgs {
  void* out;
  int* status;                       // device word that takes the code of a wait that gave up
  int64_t out_s[5];                  // b, c, g, i, j (elements; j stride is 1)
  int out_dtype;
  int L, K, ngroups;
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
  WaitCtx wc{ctl, a.status};

  const int mt = blockIdx.x;
  const int c = blockIdx.y / a.ngroups, g = blockIdx.y % a.ngroups;
  const int b = blockIdx.z;
  const uint32_t ncols = L <= 32 ? 32u : (L <= 64 ? 64u : (L <= 128 ? 128u : 256u));

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
              const float v0 = __uint_as_float(r[4 * jj + 2 * hr]), v1 = __uint_as_float(r[4 * jj + 2 * hr + 1]);
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

}  // namespace

// 1 if the tcgen05 kernel takes this problem (otherwise the plain kernel does).
int bmm_fast_ok(const ssd_bmm_chunk_params_t& p) {
  if (p.in_dtype != SSD_BF16 && p.in_dtype != SSD_F16) return 0;
  if (p.seq_idx != nullptr) return 0;
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
  const int kboxes = p.k / 64;
  const int smem = kboxes * (kBmmRows * 128 + L * 128) + 64 + 1024;
  auto kern = p.in_dtype == SSD_BF16 ? bmm_chunk_kernel<__nv_bfloat16> : bmm_chunk_kernel<__half>;
  SSD_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(L / kBmmRows, nchunks * p.ngroups, p.batch);
  kern<<<grid, kBmmThreads, smem, stream>>>(ma, mb, a);
  SSD_CUDA_OK(cudaGetLastError());
  return SSD_OK;
}

}  // namespace ssd
