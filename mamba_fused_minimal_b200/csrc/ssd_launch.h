// Internal launch interface between the C ABI (ssd_abi.cu) and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "ssd_b200.h"

namespace ssd {

// ---- settings shared by every launch (ssd_abi.cu) --------------------------------------
// SM cycles a device-side wait may last before it gives up (ssd_debug_set_wait_limit_cycles).
long long wait_limit_cycles();
// Test hooks (ssd_debug_set_flags); 0 in normal use.
int debug_flags();

// ---- general kernels (ssd_general.cu) -------------------------------------------------
int launch_chunk_cumsum(const ssd_chunk_cumsum_params_t& p, cudaStream_t stream);
int launch_state_passing(const ssd_state_passing_params_t& p, cudaStream_t stream);
int launch_chunk_state_general(const ssd_chunk_state_params_t& p, int clamp_decay, cudaStream_t stream);
int launch_bmm_chunk_general(const ssd_bmm_chunk_params_t& p, cudaStream_t stream);
int launch_chunk_scan_general(const ssd_chunk_scan_params_t& p, cudaStream_t stream);
int launch_seqpar_fixup(const ssd_seqpar_fixup_params_t& p, cudaStream_t stream);

// ---- tcgen05 fused state kernel (ssd_fused_sm100.cu) ----------------------------------
// Layout of the caller-supplied workspace used by the fused kernel.
struct FusedWorkspaceLayout {
  static constexpr size_t kHeaderBytes = 256;      // status, epoch, done counter
  static constexpr size_t kFlagsBytes = 4096 - 256;  // one word per (CTA, head slot)
  static constexpr size_t kCarryOffset = 4096;
  static constexpr int kMaxCtas = 160;             // flags: kMaxCtas * 2 words
};

// Which heads-per-CTA variant (0 = the fast kernel cannot take this problem).
int fused_fast_variant(const ssd_fused_state_params_t& p, const char** why);
size_t fused_fast_workspace_bytes(const ssd_fused_state_params_t& p);
// mode 0: chunk state + state passing; mode 1: per-chunk states only (p.states required).
// raw != NULL: the RAW variant -- p.in.dt / p.in.dA_cumsum are OUTPUTS computed in the same launch
// from the raw dt, A and dt_bias described by *raw (mode 0, no seq_idx; see fused_raw_ok).
int launch_fused_fast(const ssd_fused_state_params_t& p, int mode, cudaStream_t stream,
                      const ssd_chunk_cumsum_params_t* raw = nullptr);
bool fused_raw_ok(const ssd_fused_state_params_t& p, const ssd_chunk_cumsum_params_t& raw);
// Reads (and clears when set) the wait status word of launches in the states-only mode, which
// have no workspace, on the current device; *code = 0 when no wait gave up.
int states_only_wait_status(int* code);
// The same for the header of the static scratch array (ssd_static_scratch.cu); the word is read,
// not cleared: the next static call clears the whole header.
int static_scratch_wait_status(int* code);

// 4-D tensor map over a 16-bit (b, l, heads, inner) tensor whose innermost dimension is
// contiguous (strides in elements: b, l, heads, inner); box = 64 inner elements x 1 head x
// box_rows positions x 1 batch element, 128-byte swizzle.
int make_rows_map(CUtensorMap* map, const void* base, int dtype, int inner, int heads, int seqlen, int batch,
                  const int64_t* stride, int box_rows);

// 5-D tensor map over 16-bit passed states (b, c, h, p, n) with (p, n) dense (strides in
// elements: b, c, h); box = 64 n x 64 p, 128-byte swizzle.
int make_rows_store_map(CUtensorMap* map, const void* base, int dtype, int heads, int seqlen, int batch,
                        const int64_t* stride /* b, l, h */);
int make_states_map(CUtensorMap* map, const void* base, int dtype, int nheads, int nchunks, int batch,
                    const int64_t* stride);

// 5-D tensor map over the fp32 chunk products cb (b, c, g, m, k) with k contiguous (strides in
// elements: b, c, g, m); box = box_k columns x box_m rows, 128-byte swizzle (box_k * 4 <= 128).
int make_cb_map(CUtensorMap* map, const void* base, int L, int ngroups, int nchunks, int batch, const int64_t* stride,
                int box_k, int box_m);

// ---- tcgen05 chunk bmm and chunk scan (ssd_gemm_sm100.cu) -----------------------------
int bmm_fast_ok(const ssd_bmm_chunk_params_t& p);
int launch_bmm_chunk_fast(const ssd_bmm_chunk_params_t& p, cudaStream_t stream);
// Reads (and clears) the wait status words of the two kernels on the current device; *code = 0
// when no wait gave up.  The caller has synchronised the stream.
int gemm_wait_status(int* code);
int scan_fast_ok(const ssd_chunk_scan_params_t& p);
int launch_chunk_scan_fast(const ssd_chunk_scan_params_t& p, cudaStream_t stream);
// The chunk scan that computes the chunk-local C . B^T itself (no cb tensor).
int scan_fused_ok(const ssd_chunk_scan_fused_params_t& f);
int launch_chunk_scan_fused(const ssd_chunk_scan_fused_params_t& f, cudaStream_t stream);

}  // namespace ssd
