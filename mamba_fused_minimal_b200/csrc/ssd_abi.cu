// extern "C" entry points of libssd_b200.so: argument validation and dispatch.
// Declarations and the reference functions each one replaces: include/ssd_b200.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <nvtx3/nvToolsExt.h>

#include "ssd_common.cuh"
#include "ssd_launch.h"

namespace ssd {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
const char* get_error() { return g_error; }

// about two seconds of SM clocks
static std::atomic<long long> g_wait_limit_cycles{4000000000ll};
static std::atomic<int> g_debug_flags{0};
long long wait_limit_cycles() { return g_wait_limit_cycles.load(std::memory_order_relaxed); }
int debug_flags() { return g_debug_flags.load(std::memory_order_relaxed); }

namespace {

// One NVTX range per entry point (host side: validation, tensor maps, launches), visible in any
// tool that attaches to NVTX; without a tool the calls return at once.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};

int check_state_inputs(const ssd_state_inputs_t& in) {
  SSD_REQUIRE(in.x && in.B && in.dt && in.dA_cumsum, SSD_ERR_BAD_ARGUMENT, "x, B, dt and dA_cumsum must not be NULL");
  SSD_REQUIRE(valid_dtype(in.in_dtype), SSD_ERR_BAD_ARGUMENT, "bad in_dtype %d", in.in_dtype);
  SSD_REQUIRE(in.batch > 0 && in.seqlen > 0 && in.nheads > 0 && in.headdim > 0 && in.ngroups > 0 &&
                  in.dstate > 0 && in.chunk_size > 0,
              SSD_ERR_BAD_ARGUMENT, "sizes must be positive");
  SSD_REQUIRE(in.nheads % in.ngroups == 0, SSD_ERR_BAD_ARGUMENT, "nheads %d not a multiple of ngroups %d",
              in.nheads, in.ngroups);
  return SSD_OK;
}

// Workspace of the fused entry point: the tcgen05 kernel's header/flags/carry slots, then,
// for the plain-kernel route without a caller-supplied `states`, an fp32 per-chunk states
// buffer.
size_t general_states_bytes(const ssd_fused_state_params_t& p) {
  const ssd_state_inputs_t& in = p.in;
  const size_t nchunks = (in.seqlen + in.chunk_size - 1) / in.chunk_size;
  return (size_t)in.batch * nchunks * in.nheads * in.headdim * in.dstate * sizeof(float);
}

bool use_fast(const ssd_fused_state_params_t& p) {
  return !p.force_general && fused_fast_variant(p, nullptr) != 0;
}

}  // namespace
}  // namespace ssd

using namespace ssd;

extern "C" {

const char* ssd_last_error(void) { return get_error(); }
int ssd_abi_version(void) { return SSD_B200_ABI_VERSION; }

int ssd_chunk_cumsum_fwd(const ssd_chunk_cumsum_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_chunk_cumsum_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_chunk_cumsum_params_t& p = *prm;
  SSD_REQUIRE(p.dt && p.A && p.dt_out && p.dA_cumsum, SSD_ERR_BAD_ARGUMENT, "dt, A, dt_out and dA_cumsum must not be NULL");
  SSD_REQUIRE(valid_dtype(p.dt_dtype) && valid_dtype(p.A_dtype) && (p.dt_bias == nullptr || valid_dtype(p.bias_dtype)),
              SSD_ERR_BAD_ARGUMENT, "bad dtype");
  SSD_REQUIRE(p.batch > 0 && p.seqlen > 0 && p.nheads > 0 && p.chunk_size > 0, SSD_ERR_BAD_ARGUMENT,
              "sizes must be positive");
  return launch_chunk_cumsum(p, reinterpret_cast<cudaStream_t>(stream));
}

int ssd_chunk_state_fwd(const ssd_chunk_state_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_chunk_state_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_chunk_state_params_t& p = *prm;
  int rc = check_state_inputs(p.in);
  if (rc != SSD_OK) return rc;
  SSD_REQUIRE(p.states != nullptr && valid_dtype(p.states_dtype), SSD_ERR_BAD_ARGUMENT, "states NULL or bad dtype");
  // tcgen05 route: the fused kernel in its states-only mode
  ssd_fused_state_params_t f;
  memset(&f, 0, sizeof(f));
  f.in = p.in;
  f.states = p.states;
  f.states_dtype = p.states_dtype;
  for (int i = 0; i < 4; ++i) f.states_stride[i] = p.states_stride[i];
  f.clamp_decay = 1;
  // the states-only mode needs no carry slots; its status words live in the library
  if (p.states_stride[4] == 1 && fused_fast_variant(f, nullptr) != 0)
    return launch_fused_fast(f, 1, reinterpret_cast<cudaStream_t>(stream));
  return launch_chunk_state_general(p, 1, reinterpret_cast<cudaStream_t>(stream));
}

int ssd_state_passing_fwd(const ssd_state_passing_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_state_passing_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_state_passing_params_t& p = *prm;
  SSD_REQUIRE(p.states && p.dA_chunk_cumsum && p.out && p.final_states, SSD_ERR_BAD_ARGUMENT,
              "states, dA_chunk_cumsum, out and final_states must not be NULL");
  SSD_REQUIRE(valid_dtype(p.states_dtype) && valid_dtype(p.dA_dtype) && valid_dtype(p.out_dtype) &&
                  (p.initial_states == nullptr || valid_dtype(p.init_dtype)),
              SSD_ERR_BAD_ARGUMENT, "bad dtype");
  SSD_REQUIRE(p.batch > 0 && p.nchunks > 0 && p.nheads > 0 && p.dim > 0, SSD_ERR_BAD_ARGUMENT, "sizes must be positive");
  SSD_REQUIRE(p.seq_idx == nullptr || (p.chunk_size > 0 && p.seqlen > 0), SSD_ERR_BAD_ARGUMENT,
              "seq_idx needs seqlen and chunk_size");
  return launch_state_passing(p, reinterpret_cast<cudaStream_t>(stream));
}

size_t ssd_fused_state_workspace_bytes(const ssd_fused_state_params_t* prm) {
  if (prm == nullptr) return 0;
  size_t bytes = fused_fast_workspace_bytes(*prm);
  if (!use_fast(*prm) && prm->states == nullptr) bytes += general_states_bytes(*prm);
  return bytes;
}

int ssd_fused_state_fwd(const ssd_fused_state_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_fused_state_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_fused_state_params_t& p = *prm;
  int rc = check_state_inputs(p.in);
  if (rc != SSD_OK) return rc;
  SSD_REQUIRE(p.out && p.final_states, SSD_ERR_BAD_ARGUMENT, "out and final_states must not be NULL");
  SSD_REQUIRE(valid_dtype(p.out_dtype) && (p.initial_states == nullptr || valid_dtype(p.init_dtype)) &&
                  (p.states == nullptr || valid_dtype(p.states_dtype)),
              SSD_ERR_BAD_ARGUMENT, "bad dtype");
  SSD_REQUIRE(p.workspace != nullptr && (reinterpret_cast<uintptr_t>(p.workspace) & 255) == 0, SSD_ERR_WORKSPACE,
              "workspace is NULL or not 256-byte aligned");
  SSD_REQUIRE(p.workspace_bytes >= ssd_fused_state_workspace_bytes(prm), SSD_ERR_WORKSPACE,
              "workspace holds %zu bytes, %zu needed", p.workspace_bytes, ssd_fused_state_workspace_bytes(prm));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (use_fast(p)) return launch_fused_fast(p, 0, st);

  // plain route: per-chunk states (into the caller's buffer or the workspace), then the scan
  const ssd_state_inputs_t& in = p.in;
  const int nchunks = (in.seqlen + in.chunk_size - 1) / in.chunk_size;
  const int64_t dim = (int64_t)in.headdim * in.dstate;
  ssd_chunk_state_params_t cs;
  memset(&cs, 0, sizeof(cs));
  cs.in = in;
  if (p.states != nullptr) {
    cs.states = p.states;
    cs.states_dtype = p.states_dtype;
    for (int i = 0; i < 4; ++i) cs.states_stride[i] = p.states_stride[i];
    cs.states_stride[4] = 1;
  } else {
    cs.states = static_cast<uint8_t*>(p.workspace) + fused_fast_workspace_bytes(p);
    cs.states_dtype = SSD_F32;
    cs.states_stride[4] = 1;
    cs.states_stride[3] = in.dstate;
    cs.states_stride[2] = dim;
    cs.states_stride[1] = dim * in.nheads;
    cs.states_stride[0] = dim * in.nheads * nchunks;
  }
  // the scan addresses the flattened (p, n) index d as p * row_pitch + n, which equals
  // d * 1 only when rows are dense; the fused entry point requires that (as the reference
  // does, kernels/fused_concurrent.py:316,322-326)
  SSD_REQUIRE(cs.states_stride[3] == in.dstate && p.out_stride[3] == in.dstate && p.final_stride[2] == in.dstate &&
                  (p.initial_states == nullptr || p.init_stride[2] == in.dstate),
              SSD_ERR_UNSUPPORTED, "fused entry point needs (headdim, dstate)-contiguous states/out/final/initial");
  rc = launch_chunk_state_general(cs, p.clamp_decay, st);
  if (rc != SSD_OK) return rc;
  ssd_state_passing_params_t sp;
  memset(&sp, 0, sizeof(sp));
  sp.states = cs.states;
  sp.states_dtype = cs.states_dtype;
  sp.dA_chunk_cumsum = in.dA_cumsum + (int64_t)(in.chunk_size - 1) * in.dA_stride[3];
  sp.dA_dtype = SSD_F32;
  sp.initial_states = p.initial_states;
  sp.init_dtype = p.init_dtype;
  sp.seq_idx = in.seq_idx;
  sp.out = p.out;
  sp.out_dtype = p.out_dtype;
  sp.final_states = p.final_states;
  sp.batch = in.batch;
  sp.nchunks = nchunks;
  sp.nheads = in.nheads;
  sp.dim = (int)dim;
  sp.seqlen = in.seqlen;
  sp.chunk_size = in.chunk_size;
  sp.states_stride[0] = cs.states_stride[0];
  sp.states_stride[1] = cs.states_stride[1];
  sp.states_stride[2] = cs.states_stride[2];
  sp.states_stride[3] = 1;
  sp.dA_stride[0] = in.dA_stride[0];
  sp.dA_stride[1] = in.dA_stride[1];
  sp.dA_stride[2] = in.dA_stride[2];
  sp.init_stride[0] = p.init_stride[0];
  sp.init_stride[1] = p.init_stride[1];
  sp.init_stride[2] = 1;
  sp.out_stride[0] = p.out_stride[0];
  sp.out_stride[1] = p.out_stride[1];
  sp.out_stride[2] = p.out_stride[2];
  sp.out_stride[3] = 1;
  sp.final_stride[0] = p.final_stride[0];
  sp.final_stride[1] = p.final_stride[1];
  sp.final_stride[2] = 1;
  sp.seq_idx_stride[0] = in.seq_idx_stride[0];
  sp.seq_idx_stride[1] = in.seq_idx_stride[1];
  return launch_state_passing(sp, st);
}

// The fused parameters of a state-path call with dt / dA_cumsum pointing at the cumsum outputs.
static ssd_fused_state_params_t state_path_fused(const ssd_state_path_params_t& p) {
  ssd_fused_state_params_t f = p.fused;
  const ssd_chunk_cumsum_params_t& c = p.cumsum;
  const int64_t L = c.chunk_size, nchunks = L > 0 ? (c.seqlen + L - 1) / L : 0;
  f.in.dt = c.dt_out;
  f.in.dA_cumsum = c.dA_cumsum;
  f.in.chunk_size = c.chunk_size;
  const int64_t strides[4] = {(int64_t)c.nheads * nchunks * L, nchunks * L, L, 1};
  for (int i = 0; i < 4; ++i) f.in.dt_stride[i] = f.in.dA_stride[i] = strides[i];
  return f;
}

size_t ssd_state_path_workspace_bytes(const ssd_state_path_params_t* prm) {
  if (prm == nullptr) return 0;
  const ssd_fused_state_params_t f = state_path_fused(*prm);
  return ssd_fused_state_workspace_bytes(&f);
}

int ssd_state_path_fwd(const ssd_state_path_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_state_path_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_chunk_cumsum_params_t& c = prm->cumsum;
  SSD_REQUIRE(c.dt && c.A && c.dt_out && c.dA_cumsum, SSD_ERR_BAD_ARGUMENT, "dt, A, dt_out and dA_cumsum must not be NULL");
  SSD_REQUIRE(valid_dtype(c.dt_dtype) && valid_dtype(c.A_dtype) && (c.dt_bias == nullptr || valid_dtype(c.bias_dtype)),
              SSD_ERR_BAD_ARGUMENT, "bad dtype");
  const ssd_fused_state_params_t f = state_path_fused(*prm);
  SSD_REQUIRE(c.batch == f.in.batch && c.seqlen == f.in.seqlen && c.nheads == f.in.nheads && c.chunk_size > 0,
              SSD_ERR_BAD_ARGUMENT, "cumsum and state parameters disagree on batch / seqlen / nheads");
  int rc = check_state_inputs(f.in);
  if (rc != SSD_OK) return rc;
  if (use_fast(f) && fused_raw_ok(f, c)) {
    SSD_REQUIRE(f.out && f.final_states, SSD_ERR_BAD_ARGUMENT, "out and final_states must not be NULL");
    SSD_REQUIRE(valid_dtype(f.out_dtype) && (f.initial_states == nullptr || valid_dtype(f.init_dtype)) &&
                    (f.states == nullptr || valid_dtype(f.states_dtype)),
                SSD_ERR_BAD_ARGUMENT, "bad dtype");
    SSD_REQUIRE(f.workspace != nullptr && (reinterpret_cast<uintptr_t>(f.workspace) & 255) == 0, SSD_ERR_WORKSPACE,
                "workspace is NULL or not 256-byte aligned");
    SSD_REQUIRE(f.workspace_bytes >= ssd_fused_state_workspace_bytes(&f), SSD_ERR_WORKSPACE,
                "workspace holds %zu bytes, %zu needed", f.workspace_bytes, ssd_fused_state_workspace_bytes(&f));
    return launch_fused_fast(f, 0, reinterpret_cast<cudaStream_t>(stream), &c);
  }
  rc = ssd_chunk_cumsum_fwd(&c, stream);
  if (rc != SSD_OK) return rc;
  return ssd_fused_state_fwd(&f, stream);
}

void ssd_debug_set_wait_limit_cycles(long long cycles) {
  g_wait_limit_cycles.store(cycles > 0 ? cycles : 4000000000ll, std::memory_order_relaxed);
}
void ssd_debug_set_flags(int flags) { g_debug_flags.store(flags, std::memory_order_relaxed); }

int ssd_check_status(void* workspace, ssd_stream_t stream) {
  SSD_CUDA_OK(cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream)));
  int status = 0;
  if (workspace != nullptr) {
    SSD_CUDA_OK(cudaMemcpy(&status, workspace, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != 0) {
      set_error("a bounded device-side wait gave up (wait code %d); outputs are incomplete and the "
                "workspace header (SSD_FUSED_WORKSPACE_HEADER_BYTES) must be cleared before reuse", status);
      return SSD_ERR_TIMEOUT;
    }
  } else {
    // no workspace: the caller used ssd_fused_state_fwd_static, whose header is in the library
    const int rc = static_scratch_wait_status(&status);
    if (rc != SSD_OK) return rc;
    if (status != 0) {
      set_error("a bounded device-side wait of the last ssd_fused_state_fwd_static call gave up (wait code %d); "
                "its outputs are incomplete (the next static call clears the header)", status);
      return SSD_ERR_TIMEOUT;
    }
  }
  // ssd_chunk_state_fwd's tcgen05 route keeps its status word in the library too
  int so_code = 0;
  const int rc_so = states_only_wait_status(&so_code);
  if (rc_so != SSD_OK) return rc_so;
  if (so_code != 0) {
    set_error("a bounded device-side wait of ssd_chunk_state_fwd gave up (wait code %d); the per-chunk states "
              "are incomplete", so_code);
    return SSD_ERR_TIMEOUT;
  }
  // the chunk bmm / chunk scan kernels keep their wait status in the library (they use no workspace)
  int gemm_code = 0;
  const int rc = gemm_wait_status(&gemm_code);
  if (rc != SSD_OK) return rc;
  if (gemm_code != 0) {
    set_error("a bounded device-side wait of the chunk bmm / chunk scan kernels gave up (wait code %d); "
              "their outputs are incomplete", gemm_code);
    return SSD_ERR_TIMEOUT;
  }
  return SSD_OK;
}

int ssd_seqpar_fixup(const ssd_seqpar_fixup_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_seqpar_fixup");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_seqpar_fixup_params_t& p = *prm;
  SSD_REQUIRE(p.Z_all && p.logP_all && p.dA_chunk_last && p.out && p.final_states, SSD_ERR_BAD_ARGUMENT,
              "Z_all, logP_all, dA_chunk_last, out and final_states must not be NULL");
  SSD_REQUIRE(valid_dtype(p.out_dtype), SSD_ERR_BAD_ARGUMENT, "bad out_dtype %d", p.out_dtype);
  SSD_REQUIRE(p.world > 0 && p.rank >= 0 && p.rank < p.world, SSD_ERR_BAD_ARGUMENT, "rank %d outside world %d",
              p.rank, p.world);
  SSD_REQUIRE(p.batch > 0 && p.nheads > 0 && p.nchunks > 0 && p.dim > 0, SSD_ERR_BAD_ARGUMENT, "sizes must be positive");
  return launch_seqpar_fixup(p, reinterpret_cast<cudaStream_t>(stream));
}

int ssd_bmm_chunk_fwd(const ssd_bmm_chunk_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_bmm_chunk_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_bmm_chunk_params_t& p = *prm;
  SSD_REQUIRE(p.a && p.b && p.out, SSD_ERR_BAD_ARGUMENT, "a, b and out must not be NULL");
  SSD_REQUIRE(valid_dtype(p.in_dtype) && valid_dtype(p.out_dtype), SSD_ERR_BAD_ARGUMENT, "bad dtype");
  SSD_REQUIRE(p.batch > 0 && p.seqlen > 0 && p.ngroups > 0 && p.k > 0 && p.chunk_size > 0, SSD_ERR_BAD_ARGUMENT,
              "sizes must be positive");
  if (bmm_fast_ok(p) && !(debug_flags() & SSD_DEBUG_PLAIN_CHUNK_KERNELS)) return launch_bmm_chunk_fast(p, reinterpret_cast<cudaStream_t>(stream));
  return launch_bmm_chunk_general(p, reinterpret_cast<cudaStream_t>(stream));
}

int ssd_chunk_scan_fwd(const ssd_chunk_scan_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_chunk_scan_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_chunk_scan_params_t& p = *prm;
  SSD_REQUIRE(p.cb && p.x && p.dt && p.dA_cumsum && p.C && p.states && p.out, SSD_ERR_BAD_ARGUMENT,
              "cb, x, dt, dA_cumsum, C, states and out must not be NULL");
  SSD_REQUIRE(p.z == nullptr || p.out_x != nullptr, SSD_ERR_BAD_ARGUMENT, "out_x is required when z is given");
  SSD_REQUIRE(valid_dtype(p.cb_dtype) && valid_dtype(p.in_dtype) && valid_dtype(p.states_dtype) &&
                  (p.D == nullptr || valid_dtype(p.D_dtype)),
              SSD_ERR_BAD_ARGUMENT, "bad dtype");
  SSD_REQUIRE(p.batch > 0 && p.seqlen > 0 && p.nheads > 0 && p.headdim > 0 && p.ngroups > 0 && p.dstate > 0 &&
                  p.chunk_size > 0 && p.nheads % p.ngroups == 0,
              SSD_ERR_BAD_ARGUMENT, "bad sizes");
  if (scan_fast_ok(p) && !(debug_flags() & SSD_DEBUG_PLAIN_CHUNK_KERNELS)) return launch_chunk_scan_fast(p, reinterpret_cast<cudaStream_t>(stream));
  return launch_chunk_scan_general(p, reinterpret_cast<cudaStream_t>(stream));
}

int ssd_chunk_scan_fused_fwd(const ssd_chunk_scan_fused_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_chunk_scan_fused_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  const ssd_chunk_scan_params_t& p = prm->scan;
  SSD_REQUIRE(prm->B && p.x && p.dt && p.dA_cumsum && p.C && p.states && p.out, SSD_ERR_BAD_ARGUMENT,
              "B, x, dt, dA_cumsum, C, states and out must not be NULL");
  SSD_REQUIRE(p.z == nullptr || p.out_x != nullptr, SSD_ERR_BAD_ARGUMENT, "out_x is required when z is given");
  SSD_REQUIRE(valid_dtype(p.in_dtype) && valid_dtype(p.states_dtype) && (p.D == nullptr || valid_dtype(p.D_dtype)),
              SSD_ERR_BAD_ARGUMENT, "bad dtype");
  SSD_REQUIRE(p.batch > 0 && p.seqlen > 0 && p.nheads > 0 && p.headdim > 0 && p.ngroups > 0 && p.dstate > 0 &&
                  p.chunk_size > 0 && p.nheads % p.ngroups == 0,
              SSD_ERR_BAD_ARGUMENT, "bad sizes");
  SSD_REQUIRE(scan_fused_ok(*prm) && !(debug_flags() & SSD_DEBUG_PLAIN_CHUNK_KERNELS), SSD_ERR_UNSUPPORTED,
              "the fused chunk bmm + chunk scan kernel does not take this problem: call ssd_bmm_chunk_fwd and "
              "ssd_chunk_scan_fwd");
  return launch_chunk_scan_fused(*prm, reinterpret_cast<cudaStream_t>(stream));
}

int ssd_combined_fwd(const ssd_combined_params_t* prm, ssd_stream_t stream) {
  NvtxRange nvtx_range("ssd_combined_fwd");
  SSD_REQUIRE(prm != nullptr, SSD_ERR_BAD_ARGUMENT, "params is NULL");
  SSD_REQUIRE(prm->scan.B != nullptr && prm->scan.scan.x != nullptr && prm->scan.scan.C != nullptr, SSD_ERR_BAD_ARGUMENT,
              "B, x and C must not be NULL");
  SSD_REQUIRE(scan_fused_ok(prm->scan) && !(debug_flags() & SSD_DEBUG_PLAIN_CHUNK_KERNELS), SSD_ERR_UNSUPPORTED,
              "the fused chunk bmm + chunk scan kernel does not take this problem: make the separate calls");
  const int rc = ssd_state_path_fwd(&prm->path, stream);
  if (rc != SSD_OK) return rc;
  return ssd_chunk_scan_fused_fwd(&prm->scan, stream);
}

}  // extern "C"
