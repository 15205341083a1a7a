// ssd_fused_state_fwd_static: the fused chunk-state + state-passing entry point for callers
// that have no way to hand the library a scratch buffer.
//
// ssd_fused_state_fwd needs scratch memory (a small header, the carry slots through which a
// running state crosses from one CTA to the next, and -- on the plain-kernel route -- the
// fp32 per-chunk states), and it leaves the allocation of that scratch to the caller.  Some
// callers cannot allocate: a serving process that reserves all of its device memory once at
// start-up and forbids any later cudaMalloc, a plug-in that is invoked from inside another
// runtime's execution callback where a synchronising, possibly failing allocation call is
// not acceptable, a real-time loop that must not take the allocator's lock.  For them this
// file keeps the scratch in a file-scope device array that is part of the loaded library:
// every GPU that loads libssd_b200.so holds kStaticScratchBytes (16 MiB) of it until the
// process exits, whether or not this entry point is ever called.
#include <mutex>

#include "ssd_common.cuh"
#include "ssd_launch.h"

namespace ssd {
namespace {

constexpr size_t kStaticScratchBytes = 16u << 20;   // 16 MiB per GPU, fixed at build time

// In host code this name is only a handle for the runtime's symbol table, not a device
// address: the address a kernel can use comes from cudaGetSymbolAddress (below).
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_ptr[64] = {nullptr};   // per device ordinal, filled on first use

// Device address of the scratch array on the CURRENT device; looked up once per device.
int static_scratch_address(void** out) {
  int dev = -1;
  SSD_CUDA_OK(cudaGetDevice(&dev));
  SSD_REQUIRE(dev >= 0 && dev < 64, SSD_ERR_UNSUPPORTED, "device ordinal %d is outside 0..63", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    SSD_REQUIRE(e == cudaSuccess && p != nullptr, SSD_ERR_CUDA,
                "cudaGetSymbolAddress for the static scratch failed on device %d: %s", dev, cudaGetErrorString(e));
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return SSD_OK;
}

}  // namespace

int static_scratch_wait_status(int* code) {
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != SSD_OK) return rc;
  SSD_CUDA_OK(cudaMemcpy(code, scratch, sizeof(int), cudaMemcpyDeviceToHost));
  return SSD_OK;
}

}  // namespace ssd

using namespace ssd;

extern "C" {

size_t ssd_static_scratch_bytes(void) { return kStaticScratchBytes; }

int ssd_fused_state_fwd_static(const ssd_fused_state_params_t* prm, ssd_stream_t stream) {
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  // same arguments as ssd_fused_state_fwd; the caller's workspace fields are not read
  ssd_fused_state_params_t p = *prm;
  p.workspace = nullptr;
  p.workspace_bytes = 0;
  const size_t need = ssd_fused_state_workspace_bytes(&p);
  SSD_REQUIRE(need <= kStaticScratchBytes, SSD_ERR_WORKSPACE,
              "this problem needs %zu bytes of scratch but the static scratch holds %zu: pass the per-chunk "
              "`states` buffer yourself, split the batch, or call ssd_fused_state_fwd with your own workspace",
              need, kStaticScratchBytes);
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != SSD_OK) return rc;
  // The array keeps whatever the previous call left in it.  Only the 4 KiB header (status
  // word, launch counter, carry flags) has to start from zero; carry slots and per-chunk
  // states are written before they are read.
  SSD_CUDA_OK(cudaMemsetAsync(scratch, 0, FusedWorkspaceLayout::kCarryOffset, reinterpret_cast<cudaStream_t>(stream)));
  p.workspace = scratch;
  p.workspace_bytes = kStaticScratchBytes;
  return ssd_fused_state_fwd(&p, stream);
}

}  // extern "C"
