// Copy-engine probe for the state kernel's roofline: how fast can one persistent CTA per SM move the
// state kernel's tiles with TMA and nothing else (no tensor cores, no arithmetic)?  The access
// pattern is the state kernel's at the Mamba2-2.7B layer shape (batch 8 x 4096 x 80 heads x 64, one
// group, dstate 128, chunk 256, bf16): strip-major contiguous ranges of (head pair, chunk) items per
// CTA; per stage of `rows` positions the raw B tile (rows x 128) and the x tiles of two heads
// (rows x 64 each) into a shared-memory ring that a second thread releases at once; per chunk and
// head the 64 x 128 bf16 tile of passed states stored from shared memory.
//   merge = 0: two copies for B and two for x per stage; merge = 1: one each (the state kernel's form)
//   store  = 0: loads only; 2 / 4 / 8: stores in boxes of 2 KiB (the state kernel's), 4 KiB, 8 KiB
// The figures bound what the state kernel can reach with its traffic on this GPU; they are quoted
// in profiles/.  Every wait is bounded.  Build and run:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o tma_copy_probe tma_copy_probe.cu -lcuda
//   ./tma_copy_probe
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <algorithm>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("%s: %s\n", #x, cudaGetErrorString(e)); exit(1);} } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t c) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(c) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t b) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(b) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t par) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 20000;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(ok) : "r"(bar), "r"(par) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t par, int* err) {
  long long t0 = clock64();
  while (!mbar_try(bar, par)) {
    if (clock64() - t0 > 2000000000ll) { *err = 1; return false; }
  }
  return true;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
               ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
__device__ __forceinline__ void tma_store_5d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3, int c4) {
  asm volatile("cp.async.bulk.tensor.5d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5, %6}], [%1];"
               ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}

struct Args {
  int merge, rows, ns, store_kb, with_B;
  int batch, seqlen, nheads, L;
  int* err;
};

__global__ void __launch_bounds__(128, 1) probe(const __grid_constant__ CUtensorMap mx, const __grid_constant__ CUtensorMap mB,
                                                const __grid_constant__ CUtensorMap mxm, const __grid_constant__ CUtensorMap mBm,
                                                const __grid_constant__ CUtensorMap mo, Args a) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  const uint32_t sbase = smem_u32(smem);
  const int xb = a.rows * 128;                             // one head's x tile / half of the B tile
  const int stage_bytes = xb * (2 + (a.with_B ? 2 : 0));
  const uint32_t staging = sbase + a.ns * stage_bytes;     // 16 KB
  const uint32_t bars = staging + 16384;
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.ns; ++s) { mbar_init(bars + 8 * s, 1); mbar_init(bars + 8 * (a.ns + s), 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();
  const int nchunks = a.seqlen / a.L;
  const int spb = a.nheads / 2;
  const long long total = (long long)a.batch * spb * nchunks;
  const int ksteps = a.L / a.rows;
  const long long lo = total * blockIdx.x / gridDim.x, hi = total * (blockIdx.x + 1) / gridDim.x;
  if (threadIdx.x == 0) {
    uint32_t it = 0;
    for (long long i = lo; i < hi; ++i) {
      const int strip = (int)(i / nchunks), c = (int)(i % nchunks), b = strip / spb, h0 = (strip % spb) * 2;
      for (int ks = 0; ks < ksteps; ++ks, ++it) {
        const int s = it % a.ns;
        if (!mbar_wait(bars + 8 * (a.ns + s), ((it / a.ns) & 1) ^ 1, a.err)) return;
        const uint32_t st = sbase + s * stage_bytes;
        mbar_expect_tx(bars + 8 * s, stage_bytes);
        const int l0 = c * a.L + ks * a.rows;
        uint32_t off = 0;
        if (a.with_B) {
          if (a.merge) {
            tma_load_5d(st, &mBm, bars + 8 * s, 0, l0, 0, 0, b);
          } else {
            tma_load_4d(st, &mB, bars + 8 * s, 0, 0, l0, b);
            tma_load_4d(st + xb, &mB, bars + 8 * s, 64, 0, l0, b);
          }
          off = 2 * xb;
        }
        if (a.merge) {
          tma_load_4d(st + off, &mxm, bars + 8 * s, 0, l0, h0, b);
        } else {
          tma_load_4d(st + off, &mx, bars + 8 * s, 0, h0, l0, b);
          tma_load_4d(st + off + xb, &mx, bars + 8 * s, 0, h0 + 1, l0, b);
        }
      }
    }
  } else if (threadIdx.x == 32) {
    uint32_t it = 0;
    for (long long i = lo; i < hi; ++i) {
      const int strip = (int)(i / nchunks), c = (int)(i % nchunks), b = strip / spb, h0 = (strip % spb) * 2;
      for (int ks = 0; ks < ksteps; ++ks, ++it) {
        const int s = it % a.ns;
        if (!mbar_wait(bars + 8 * s, (it / a.ns) & 1, a.err)) return;
        mbar_arrive(bars + 8 * (a.ns + s));
      }
      if (a.store_kb) {
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        for (int hd = 0; hd < 2; ++hd) {
          if (a.store_kb == 2) {
            for (int q = 0; q < 4; ++q) for (int hq = 0; hq < 2; ++hq) tma_store_5d(&mo, staging + (q * 2 + hq) * 2048, q * 32, hq * 32, h0 + hd, c, b);
          } else if (a.store_kb == 4) {
            for (int q = 0; q < 4; ++q) tma_store_5d(&mo, staging + q * 4096, q * 32, 0, h0 + hd, c, b);
          } else {
            for (int q = 0; q < 2; ++q) tma_store_5d(&mo, staging + q * 8192, q * 64, 0, h0 + hd, c, b);
          }
        }
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
}

// plain vector read kernel (ld.global.v4), grid-stride; the sum defeats dead-code elimination
__global__ void __launch_bounds__(512) vread(const uint4* p, size_t n, uint32_t* sink) {
  uint32_t acc = 0;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i + 3 * stride < n; i += 4 * stride) {
    uint4 a = p[i], b = p[i + stride], c = p[i + 2 * stride], d = p[i + 3 * stride];
    acc += a.x ^ b.y ^ c.z ^ d.w;
  }
  for (; i < n; i += stride) acc += p[i].x;
  if (acc == 0x12345678u) *sink = acc;
}

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int main() {
  const int batch = 8, seqlen = 4096, nheads = 80, P = 64, N = 128, L = 256, nchunks = seqlen / L;
  void* fn = nullptr; cudaDriverEntryPointQueryResult q;
  CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
  EncodeFn enc = (EncodeFn)fn;
  const size_t xbytes = (size_t)batch * seqlen * nheads * P * 2, Bbytes = (size_t)batch * seqlen * N * 2;
  const size_t obytes = (size_t)batch * nchunks * nheads * P * N * 2;
  void *x, *B, *out; int* err;
  CK(cudaMalloc(&x, xbytes)); CK(cudaMalloc(&B, Bbytes)); CK(cudaMalloc(&out, obytes)); CK(cudaMalloc(&err, 4));
  CK(cudaMemset(x, 1, xbytes)); CK(cudaMemset(B, 1, Bbytes)); CK(cudaMemset(err, 0, 4));
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  auto timeit = [&](auto f, int reps) {
    f(); f();
    CK(cudaDeviceSynchronize());
    std::vector<float> ts;
    for (int r = 0; r < reps; ++r) { cudaEventRecord(e0); f(); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); float ms; cudaEventElapsedTime(&ms, e0, e1); ts.push_back(ms); }
    std::sort(ts.begin(), ts.end());
    return ts[ts.size() / 2];
  };
  {
    void* y; CK(cudaMalloc(&y, xbytes));
    float ms = timeit([&] { CK(cudaMemcpyAsync(y, x, xbytes, cudaMemcpyDeviceToDevice)); }, 10);
    printf("cudaMemcpy device to device of x: %.1f us  %.0f GB/s (read + write)\n", ms * 1e3, 2 * xbytes / ms / 1e6);
    ms = timeit([&] { vread<<<148 * 4, 512>>>((const uint4*)x, xbytes / 16, (uint32_t*)err + 0); }, 10);
    printf("plain 16-byte loads of x        : %.1f us  %.0f GB/s (read)\n", ms * 1e3, xbytes / ms / 1e6);
    CK(cudaMemset(err, 0, 4));
    CK(cudaFree(y));
  }
  const cuuint32_t es4[4] = {1, 1, 1, 1}, es5[5] = {1, 1, 1, 1, 1};
  for (int rows : {64, 128}) {
    CUtensorMap mx, mB, mxm, mBm;
    {
      cuuint64_t dims[4] = {(cuuint64_t)P, (cuuint64_t)nheads, (cuuint64_t)seqlen, (cuuint64_t)batch};
      cuuint64_t str[3] = {(cuuint64_t)P * 2, (cuuint64_t)nheads * P * 2, (cuuint64_t)seqlen * nheads * P * 2};
      cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
      CUresult r = enc(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x, dims, str, box, es4, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r) { printf("enc x %d\n", (int)r); return 1; }
      cuuint64_t dB[4] = {(cuuint64_t)N, 1, (cuuint64_t)seqlen, (cuuint64_t)batch};
      cuuint64_t sB[3] = {(cuuint64_t)N * 2, (cuuint64_t)N * 2, (cuuint64_t)seqlen * N * 2};
      r = enc(&mB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, B, dB, sB, box, es4, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r) { printf("enc B %d\n", (int)r); return 1; }
      // merged x: dims (p, l, h, b), box (64, rows, 2, 1) -> smem [head][row][p]
      cuuint64_t dxm[4] = {(cuuint64_t)P, (cuuint64_t)seqlen, (cuuint64_t)nheads, (cuuint64_t)batch};
      cuuint64_t sxm[3] = {(cuuint64_t)nheads * P * 2, (cuuint64_t)P * 2, (cuuint64_t)seqlen * nheads * P * 2};
      cuuint32_t bxm[4] = {64, (cuuint32_t)rows, 2, 1};
      r = enc(&mxm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x, dxm, sxm, bxm, es4, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r) { printf("enc xm rows %d: %d\n", rows, (int)r); }
      // merged B: dims (n_lo 64, l, n_hi 2, g, b), box (64, rows, 2, 1, 1) -> smem [n half][row][64 n]
      cuuint64_t dBm[5] = {64, (cuuint64_t)seqlen, 2, 1, (cuuint64_t)batch};
      cuuint64_t sBm[4] = {(cuuint64_t)N * 2, 128, (cuuint64_t)N * 2, (cuuint64_t)seqlen * N * 2};
      cuuint32_t bBm[5] = {64, (cuuint32_t)rows, 2, 1, 1};
      CUresult r2 = enc(&mBm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, B, dBm, sBm, bBm, es5, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r2) { printf("enc Bm rows %d: %d\n", rows, (int)r2); }
      if (r || r2) { printf("merged maps not encodable at rows %d\n", rows); continue; }
    }
    for (int store_kb : {0, 2, 4, 8}) {
      CUtensorMap mo;
      {
        cuuint64_t dims[5] = {(cuuint64_t)N, (cuuint64_t)P, (cuuint64_t)nheads, (cuuint64_t)nchunks, (cuuint64_t)batch};
        cuuint64_t str[4] = {(cuuint64_t)N * 2, (cuuint64_t)P * N * 2, (cuuint64_t)nheads * P * N * 2, (cuuint64_t)nchunks * nheads * P * N * 2};
        cuuint32_t box[5] = {32, 32, 1, 1, 1};
        CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_64B;
        if (store_kb == 4) box[1] = 64;
        if (store_kb == 8) { box[0] = 64; box[1] = 64; sw = CU_TENSOR_MAP_SWIZZLE_128B; }
        CUresult r = enc(&mo, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, out, dims, str, box, es5, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r) { printf("enc out %d\n", (int)r); return 1; }
      }
      for (int merge : {0, 1})
        for (int with_B : {1}) {
          Args a{};
          a.merge = merge; a.rows = rows; a.store_kb = store_kb; a.with_B = with_B;
          a.batch = batch; a.seqlen = seqlen; a.nheads = nheads; a.L = L; a.err = err;
          const int stage_bytes = rows * 128 * 4;
          for (int kb : {192}) {
            a.ns = kb * 1024 / stage_bytes;
            if (a.ns < 1) continue;
            const int smem = a.ns * stage_bytes + 16384 + 16 * a.ns + 1024;
            if (smem > 227 * 1024) continue;
            CK(cudaFuncSetAttribute(probe, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            float ms = timeit([&] { probe<<<148, 128, smem>>>(mx, mB, mxm, mBm, mo, a); }, 7);
            CK(cudaGetLastError());
            const double bytes = (double)xbytes + (store_kb ? (double)obytes : 0.0);
            printf("rows %3d merge %d store %d KB ns %2d (%3d KB ring): %.1f us  %.0f GB/s (x%s)\n", rows, merge, store_kb, a.ns,
                   a.ns * stage_bytes / 1024, ms * 1e3, bytes / ms / 1e6, store_kb ? " + out" : "");
          }
        }
    }
  }
  int herr = 0; CK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
  printf("err flag %d\n", herr);
  return 0;
}
