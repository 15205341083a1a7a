/*
 * ssd_b200.h -- C ABI of libssd_b200.so: the Mamba2 SSD forward hot path on NVIDIA B200
 * (sm_100a): chunk cumsum of dt*A, per-chunk state, inter-chunk state passing, their
 * fused form, and the two chunk GEMM steps (C.B^T and the chunk scan) that the
 * end-to-end forward check needs.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer on the device that is current when the call is
 *     made; every call only enqueues work on `stream` and returns without synchronising.
 *   - Strides are in ELEMENTS, not bytes.  Shapes use: b batch, l seqlen, h nheads,
 *     p headdim, g ngroups, n dstate, L chunk_size, c = ceil(l / L) nchunks.
 *   - Optional tensors are NULL when absent.
 *   - Return value: SSD_OK or an ssd_status_t error; ssd_last_error() gives a message for
 *     the calling thread.  No call allocates device memory except where stated; scratch
 *     memory is supplied by the caller (see ssd_fused_state_workspace_bytes).
 *   - The library contains sm_100a code only.  On any other device the launch fails and
 *     the call returns SSD_ERR_CUDA; there is no CPU path.
 *
 * Each entry point names the function of the reference project
 * (RishiAstra/mamba-fused-minimal, paths relative to its root) whose device work it
 * replaces.
 */
#ifndef SSD_B200_H_
#define SSD_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SSD_B200_ABI_VERSION 1

#if defined(__GNUC__)
#define SSD_API __attribute__((visibility("default")))
#else
#define SSD_API
#endif

typedef struct CUstream_st* ssd_stream_t; /* a cudaStream_t / CUstream handle */

typedef enum {
  SSD_F32 = 0,
  SSD_BF16 = 1,
  SSD_F16 = 2
} ssd_dtype_t;

typedef enum {
  SSD_OK = 0,
  SSD_ERR_BAD_ARGUMENT = 1, /* null pointer, non-positive size, inconsistent shapes        */
  SSD_ERR_UNSUPPORTED = 2,  /* a combination this build has no kernel for                  */
  SSD_ERR_CUDA = 3,         /* the CUDA runtime / driver reported an error on launch       */
  SSD_ERR_WORKSPACE = 4,    /* workspace missing, misaligned or too small                  */
  SSD_ERR_TIMEOUT = 5       /* a bounded device-side wait gave up (see ssd_check_status)   */
} ssd_status_t;

/* Message for the last non-OK status returned to the calling thread ("" if none). */
SSD_API const char* ssd_last_error(void);
/* SSD_B200_ABI_VERSION the library was built with. */
SSD_API int ssd_abi_version(void);

/* ------------------------------------------------------------------------------------
 * 1. chunk cumsum.  Replaces _chunk_cumsum_fwd, kernels/ssd_chunk_state.py:176-199
 *    (device code :33-79).
 *    dt' = clamp(softplus?(dt + dt_bias), dt_min, dt_max), zero past seqlen;
 *    dA_cumsum = inclusive cumsum over each chunk of dt' * A.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* dt;        /* (b, l, h), dt_dtype */
  const void* A;         /* (h,), A_dtype */
  const void* dt_bias;   /* (h,) or NULL, bias_dtype */
  float* dt_out;         /* (b, h, c, L) contiguous fp32 */
  float* dA_cumsum;      /* (b, h, c, L) contiguous fp32 */
  int32_t dt_dtype, A_dtype, bias_dtype;
  int32_t batch, seqlen, nheads, chunk_size;
  int64_t dt_stride_b, dt_stride_l, dt_stride_h;
  int64_t A_stride, bias_stride;
  float dt_min, dt_max;
  int32_t dt_softplus;   /* non-zero: softplus where dt + bias <= 20 */
} ssd_chunk_cumsum_params_t;

SSD_API int ssd_chunk_cumsum_fwd(const ssd_chunk_cumsum_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Tensors shared by the state kernels.
 *   x (b, l, h, p), B (b, l, g, n) of in_dtype; dt, dA_cumsum (b, h, c, L) fp32 with
 *   element strides given as (b, h, c, L).  seq_idx (b, l) int32 or NULL.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* B;
  const float* dt;
  const float* dA_cumsum;
  const int32_t* seq_idx;
  int32_t in_dtype;
  int32_t batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size;
  int64_t x_stride[4];       /* b, l, h, p */
  int64_t B_stride[4];       /* b, l, g, n */
  int64_t dt_stride[4];      /* b, h, c, L */
  int64_t dA_stride[4];      /* b, h, c, L */
  int64_t seq_idx_stride[2]; /* b, l */
} ssd_state_inputs_t;

/* ------------------------------------------------------------------------------------
 * 2. per-chunk state.  Replaces _chunk_state_fwd, kernels/ssd_chunk_state.py:202-232
 *    (device code :97-173).
 *    states[b,c,h,p,n] = sum_k x[k,p] * cast_in(B[k,n] * exp(min(dA_last - dA_k, 0)) * dt_k)
 * ---------------------------------------------------------------------------------- */
typedef struct {
  ssd_state_inputs_t in;
  void* states;              /* (b, c, h, p, n) of states_dtype */
  int32_t states_dtype;
  int64_t states_stride[5];  /* b, c, h, p, n */
} ssd_chunk_state_params_t;

SSD_API int ssd_chunk_state_fwd(const ssd_chunk_state_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 3. state passing.  Replaces _state_passing_fwd, kernels/ssd_state_passing.py:87-115
 *    (device code :27-84).
 *    S = initial or 0; for each chunk: out[c] = S; S = exp(dA_chunk[c]) * S + states[c];
 *    final = S.  S stays fp32.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* states;          /* (b, c, h, dim) of states_dtype */
  const void* dA_chunk_cumsum; /* (b, h, c) of dA_dtype */
  const void* initial_states;  /* (b, h, dim) of init_dtype, or NULL */
  const int32_t* seq_idx;      /* (b, l) or NULL */
  void* out;                   /* (b, c, h, dim) of out_dtype */
  float* final_states;         /* (b, h, dim) fp32 */
  int32_t states_dtype, dA_dtype, init_dtype, out_dtype;
  int32_t batch, nchunks, nheads, dim;
  int32_t seqlen, chunk_size;  /* used with seq_idx only */
  int64_t states_stride[4];    /* b, c, h, dim */
  int64_t dA_stride[3];        /* b, h, c */
  int64_t init_stride[3];      /* b, h, dim */
  int64_t out_stride[4];       /* b, c, h, dim */
  int64_t final_stride[3];     /* b, h, dim */
  int64_t seq_idx_stride[2];
} ssd_state_passing_params_t;

SSD_API int ssd_state_passing_fwd(const ssd_state_passing_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 4. fused chunk state + state passing, one launch.  Replaces both
 *    _fused_chunk_state_state_passing_fwd_concurrent, kernels/fused_concurrent.py:255-331
 *    (device code :17-252) and _fused_chunk_state_state_passing_fwd_globalbar,
 *    kernels/fused_globalbar.py:201-266 (device code :16-198).
 *
 *    out[b,c,h,p,n]   the state entering chunk c (exclusive prefix), out_dtype
 *    final[b,h,p,n]   the state after the last chunk, fp32
 *    states           optional: the per-chunk states, written as in (2) when non-NULL
 *
 *    The fp32 per-chunk states never go to memory unless `states` is given.  The kernel
 *    is persistent (one CTA per SM); each CTA walks a contiguous range of (b, h, chunk)
 *    units and keeps the running state on chip.  Where a CTA's range starts in the middle
 *    of a (b, h) sequence the carried state comes from the CTA that owns the preceding
 *    range, through `workspace` and a flag; the wait on that flag is bounded, and a wait
 *    that gives up sets a status word (see ssd_check_status).
 *
 *    `workspace`: ssd_fused_state_workspace_bytes() bytes, 256-byte aligned, owned by the
 *    caller, used by one call at a time.  Its first SSD_FUSED_WORKSPACE_HEADER_BYTES
 *    (4096: status word, launch epoch, done counter and one flag word per CTA and head
 *    slot) must be zero on the first use -- zeroing the whole buffer once is the simple
 *    way -- and are left zero-equivalent by every call (flags carry an epoch), so one
 *    buffer can be reused by successive calls on the same stream without clearing.  After
 *    SSD_ERR_TIMEOUT from ssd_check_status the same bytes must be cleared again.
 * ---------------------------------------------------------------------------------- */
#define SSD_FUSED_WORKSPACE_HEADER_BYTES 4096
typedef struct {
  ssd_state_inputs_t in;
  const void* initial_states; /* (b, h, p, n) of init_dtype, (p, n) contiguous, or NULL */
  void* out;                  /* (b, c, h, p, n) of out_dtype, (p, n) contiguous */
  float* final_states;        /* (b, h, p, n) fp32, (p, n) contiguous */
  void* states;               /* optional (b, c, h, p, n) of states_dtype, (p, n) contiguous */
  int32_t init_dtype, out_dtype, states_dtype;
  int64_t init_stride[3];     /* b, h, p (n has stride 1) */
  int64_t out_stride[4];      /* b, c, h, p */
  int64_t final_stride[3];    /* b, h, p */
  int64_t states_stride[4];   /* b, c, h, p */
  void* workspace;
  size_t workspace_bytes;
  int32_t clamp_decay;        /* non-zero: exp(min(d, 0)) as the unfused kernel does
                                 (ssd_chunk_state.py:153); zero: exp(d) as the reference's
                                 fused kernels do (fused_concurrent.py:119).  Identical
                                 whenever dt >= 0 and A <= 0. */
  int32_t force_general;      /* non-zero: skip the tcgen05 kernel, use the plain kernels */
} ssd_fused_state_params_t;

SSD_API size_t ssd_fused_state_workspace_bytes(const ssd_fused_state_params_t* prm);
SSD_API int ssd_fused_state_fwd(const ssd_fused_state_params_t* prm, ssd_stream_t stream);

/* Reads back (synchronously, after synchronising `stream`) every bounded-wait status word
 * on the current device: the one the last ssd_fused_state_fwd on `workspace` left -- or,
 * with workspace == NULL, the one the last ssd_fused_state_fwd_static left in the library's
 * own scratch -- and the library-held words of ssd_chunk_state_fwd's tcgen05 route and of
 * the tcgen05 chunk bmm / chunk scan kernels.  Returns SSD_OK, or SSD_ERR_TIMEOUT if a
 * bounded device wait gave up (outputs are then incomplete; ssd_last_error() names the
 * kernel and the wait).  The library-held words are cleared by the call that reports them;
 * a caller's workspace header is the caller's to clear (SSD_FUSED_WORKSPACE_HEADER_BYTES),
 * and the static scratch header is cleared by the next static call, so a static caller
 * checks BEFORE its next static call.  Optional: a healthy run never sets a word.  Has no
 * counterpart in the reference, whose waits are unbounded
 * (kernels/fused_concurrent.py:82-84,205-208). */
SSD_API int ssd_check_status(void* workspace, ssd_stream_t stream);

/* Test hooks.  No counterpart in the reference.
 *   ssd_debug_set_wait_limit_cycles: SM clock cycles a device-side wait may last before it
 *     gives up (process-wide, read at launch; <= 0 restores the default of 4e9, about two
 *     seconds).  A wait that gives up never traps or spins on: the CTA records a wait code,
 *     lets its copies in flight land, frees its tensor memory and returns.
 *   ssd_debug_set_flags: SSD_DEBUG_DROP_CARRY_FLAGS makes the fused kernel skip publishing its
 *     carry flags, so that a CTA which needs a carried state waits for a flag that nothing
 *     sets, runs into the limit and the call ends with SSD_ERR_TIMEOUT from ssd_check_status.
 *     This exists to test that path with a short limit; 0 restores normal operation.
 *     SSD_DEBUG_CUT_STRIPS makes the fused kernel always cut its work into one range per SM, also
 *     where a problem has no more (batch, head pair) strips than SMs and would run one CTA per
 *     strip: small test problems then exercise the carry chain between CTAs.
 *     SSD_DEBUG_PLAIN_CHUNK_KERNELS sends ssd_bmm_chunk_fwd and ssd_chunk_scan_fwd to the plain kernels
 *     (and makes ssd_chunk_scan_fused_fwd answer SSD_ERR_UNSUPPORTED) also where the tcgen05 kernels
 *     would take the problem: the tests compare the two routes on the same inputs with it. */
#define SSD_DEBUG_DROP_CARRY_FLAGS 1
#define SSD_DEBUG_CUT_STRIPS 2
#define SSD_DEBUG_PLAIN_CHUNK_KERNELS 4
SSD_API void ssd_debug_set_wait_limit_cycles(long long cycles);
SSD_API void ssd_debug_set_flags(int flags);

/* ------------------------------------------------------------------------------------
 * 4a. the whole state path in one call: chunk cumsum (1) + fused chunk state and state
 *    passing (4).  Replaces the pair of calls the reference's pipelines make,
 *    _chunk_cumsum_fwd then _fused_chunk_state_state_passing_fwd_concurrent
 *    (main.py:96-100; kernels/ssd_chunk_state.py:176-199, kernels/fused_concurrent.py:255-331).
 *
 *    `cumsum` describes the raw dt, A, dt_bias and the two fp32 outputs dt_out and dA_cumsum
 *    ((b, h, c, L) contiguous) exactly as for ssd_chunk_cumsum_fwd; `fused` describes x, B,
 *    initial_states, out, final_states, states and the workspace exactly as for
 *    ssd_fused_state_fwd, except that fused.in.dt, fused.in.dA_cumsum and their strides are
 *    ignored: the state kernel uses cumsum.dt_out / cumsum.dA_cumsum.  All four outputs carry
 *    the same bits as the two separate calls would give.
 *
 *    When the tcgen05 kernel takes the problem and the raw dt has contiguous heads (16-bit or
 *    fp32, each position's pair of heads aligned to its size), ONE launch does everything:
 *    the persistent kernel computes each chunk's cumulative sums in the warp that needs them
 *    for the B scaling and writes dt_out / dA_cumsum as a by-product.  Otherwise the call
 *    enqueues the cumsum kernel and then the state kernels.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  ssd_chunk_cumsum_params_t cumsum;
  ssd_fused_state_params_t fused;
} ssd_state_path_params_t;

SSD_API size_t ssd_state_path_workspace_bytes(const ssd_state_path_params_t* prm);
SSD_API int ssd_state_path_fwd(const ssd_state_path_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 4b. ssd_fused_state_fwd without a caller-supplied workspace.  It has no counterpart in
 *    the reference (whose wrappers allocate with torch.empty / torch.zeros on every call,
 *    kernels/fused_concurrent.py:270-298).
 *
 *    For callers that cannot allocate device memory at the time of the call -- a server
 *    that hands out all of its device memory once at start-up, a plug-in running inside
 *    another runtime's callback, a loop that must not block on the allocator -- and so
 *    cannot provide `workspace`.  Arguments and results are those of ssd_fused_state_fwd;
 *    `workspace` and `workspace_bytes` are ignored.  The scratch lives in a device array
 *    that is part of the library image: ssd_static_scratch_bytes() = 16 MiB on EVERY GPU
 *    that loads the library, held until the process exits.
 *
 *    Limits and rules:
 *      - a problem whose scratch need (ssd_fused_state_workspace_bytes) exceeds 16 MiB is
 *        rejected with SSD_ERR_WORKSPACE and a message; the tcgen05 route always fits, the
 *        plain-kernel route fits while batch*nchunks*nheads*headdim*dstate*4 bytes stay
 *        under about 6 MiB (or without limit when `states` is passed);
 *      - the call allocates and frees nothing: it looks up the array's device address,
 *        clears its 4 KiB header with cudaMemsetAsync on `stream`, and launches;
 *      - the first call on each device looks the address up (cudaGetSymbolAddress) with
 *        that device current; make that first call before any stream capture begins;
 *      - every call on a device shares the one array: two calls whose kernels may overlap
 *        on the GPU (different streams, no dependency between them) race on it.  Calls
 *        ordered on one stream are safe.
 * ---------------------------------------------------------------------------------- */
SSD_API size_t ssd_static_scratch_bytes(void);
SSD_API int ssd_fused_state_fwd_static(const ssd_fused_state_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 5. chunk bmm.  Replaces _bmm_chunk_fwd, kernels/ssd_bmm.py:89-134 (device code :31-87).
 *    out[b,c,g,i,j] = sum_k a[b, c*L+i, g, k] * b[b, c*L+j, g, k]
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* a;             /* (b, l, g, k) of in_dtype */
  const void* b;             /* (b, l, g, k) of in_dtype */
  const int32_t* seq_idx;    /* (b, l) or NULL */
  void* out;                 /* (b, c, g, L, L) of out_dtype */
  int32_t in_dtype, out_dtype;
  int32_t batch, seqlen, ngroups, k, chunk_size;
  int32_t causal;            /* non-zero: tiles strictly above the diagonal are not written */
  int64_t a_stride[4], b_stride[4]; /* b, l, g, k */
  int64_t out_stride[5];     /* b, c, g, i, j */
  int64_t seq_idx_stride[2];
} ssd_bmm_chunk_params_t;

SSD_API int ssd_bmm_chunk_fwd(const ssd_bmm_chunk_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 6. chunk scan.  Replaces _chunk_scan_fwd, kernels/ssd_chunk_scan.py:172-221
 *    (device code :38-169).
 *    out[m] = exp(dA_m) * C[m] . cast_C(prev_state) + sum_{k<=m} cast_x(cb[m,k] *
 *             exp(min(dA_m - dA_k, 0)) * dt_k) * x[k] + D * x[m];  with z: out_x = that,
 *             out = out_x * z * sigmoid(z).
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* cb;            /* (b, c, g, L, L) of cb_dtype */
  const void* x;             /* (b, l, h, p) of in_dtype */
  const float* dt;           /* (b, h, c, L) fp32 */
  const float* dA_cumsum;    /* (b, h, c, L) fp32 */
  const void* C;             /* (b, l, g, n) of in_dtype */
  const void* states;        /* (b, c, h, p, n) of states_dtype: the PASSED states */
  const void* D;             /* (h,) or (h, p) of D_dtype, or NULL */
  const void* z;             /* (b, l, h, p) of in_dtype, or NULL */
  const int32_t* seq_idx;    /* (b, l) or NULL */
  void* out;                 /* (b, l, h, p) of in_dtype */
  void* out_x;               /* (b, l, h, p) of in_dtype; required when z is given */
  int32_t cb_dtype, in_dtype, states_dtype, D_dtype;
  int32_t batch, seqlen, nheads, headdim, ngroups, dstate, chunk_size;
  int32_t D_has_hdim;        /* non-zero: D is (h, p) */
  int64_t cb_stride[5];      /* b, c, g, m, k */
  int64_t x_stride[4], z_stride[4], out_stride[4]; /* b, l, h, p */
  int64_t dt_stride[4], dA_stride[4];              /* b, h, c, L */
  int64_t C_stride[4];       /* b, l, g, n */
  int64_t states_stride[5];  /* b, c, h, p, n */
  int64_t D_stride;          /* per head */
  int64_t seq_idx_stride[2];
} ssd_chunk_scan_params_t;

SSD_API int ssd_chunk_scan_fwd(const ssd_chunk_scan_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 6a. chunk bmm + chunk scan in one kernel.  Replaces the pair _bmm_chunk_fwd(C, B, ...) then
 *    _chunk_scan_fwd(cb, ...) of the reference's pipelines (main.py:71-73 and :95,101;
 *    kernels/ssd_bmm.py:64-72, kernels/ssd_chunk_scan.py:96-143): the chunk-local
 *    cb[m, k] = C[m] . B[k] is computed on chip, tile by tile, by the kernel that consumes it, and
 *    never exists in memory.  `scan` is read as for ssd_chunk_scan_fwd except that scan.cb, its
 *    dtype and strides are ignored; B is (b, l, g, n) of scan.in_dtype.
 *
 *    Only the tcgen05 kernel implements this: 16-bit inputs, headdim 64, dstate 128, chunk size
 *    128 or 256, 16-byte aligned tensors with contiguous innermost dimensions.  For
 *    anything else the call returns SSD_ERR_UNSUPPORTED and enqueues nothing; the caller then makes
 *    the two separate calls (5) and (6).  Same operations in the same order as the two calls: the
 *    output carries the same bits as theirs.  scan.seq_idx (packed sequences) is honoured: products
 *    between positions of different sequences are dropped on chip as _bmm_chunk_fwd drops them.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  ssd_chunk_scan_params_t scan;
  const void* B;             /* (b, l, g, n) of scan.in_dtype */
  int64_t B_stride[4];       /* b, l, g, n */
} ssd_chunk_scan_fused_params_t;

SSD_API int ssd_chunk_scan_fused_fwd(const ssd_chunk_scan_fused_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 6b. the whole forward in one call.  Replaces the body of
 *    _mamba_chunk_scan_combined_fwd_concurrent (main.py:93-103 of the reference: chunk bmm, chunk
 *    cumsum, fused chunk state + state passing, chunk scan -- four launches there): here the state
 *    path (4a) and the chunk bmm + chunk scan (6a) are enqueued back to back on `stream`, TWO
 *    launches when both tcgen05 kernels take the problem, and cb never exists.
 *    `path` and `scan` are read exactly as by ssd_state_path_fwd and ssd_chunk_scan_fused_fwd; the
 *    caller points scan.scan.dt / dA_cumsum at path.cumsum.dt_out / dA_cumsum and scan.scan.states at
 *    path.fused.out.  If the scan part is not supported (SSD_ERR_UNSUPPORTED, see 6a) nothing is
 *    enqueued.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  ssd_state_path_params_t path;
  ssd_chunk_scan_fused_params_t scan;
} ssd_combined_params_t;

SSD_API int ssd_combined_fwd(const ssd_combined_params_t* prm, ssd_stream_t stream);

/* ------------------------------------------------------------------------------------
 * 7. sequence-parallel fix-up.  No counterpart in the reference (it is single-GPU,
 *    kernels/fused_concurrent.py:289); the carry it builds on is the reference's
 *    initial_states / final_states pair (kernels/ssd_state_passing.py:61-65,81).
 *
 *    A sequence is cut into `world` chunk-aligned slices, one per rank.  Every rank first
 *    runs ssd_fused_state_fwd on its slice with a zero carry-in (rank 0: the caller's
 *    initial_states), which yields out0 (its passed states), Z_r (its final state) and
 *    logP_r[b,h] = sum over its chunks of dA_cumsum[b,h,c,L-1].  After all ranks' (Z, logP)
 *    have been gathered into local memory (NCCL all-gather or any other transport), this
 *    call adds the carried state:
 *        S_in   = sum_{j<rank} exp(sum_{j<k<rank} logP_k) * Z_j
 *        out[c] = out0[c] + exp(sum_{k<c, local} dA_last_k) * S_in      (skipped, leaving out[c]
 *                 bit-identical, where the factor is zero in fp32; for a 16-bit out also where
 *                 it is at most 2^-24, far below what that type resolves)
 *        final  = Z_rank + exp(logP_rank) * S_in
 *    Rank 0 has nothing to add and returns at once.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const float* Z_all;         /* (world, b, h, dim) fp32, dense per rank: every rank's slice-final state */
  const float* logP_all;      /* (world, b, h) fp32, dense per rank */
  const float* dA_chunk_last; /* (b, h, c) fp32: dA_cumsum[..., L-1] of the local slice */
  void* out;                  /* (b, c, h, dim) of out_dtype, dim contiguous; updated in place */
  float* final_states;        /* (b, h, dim) fp32, dim contiguous; written */
  int32_t out_dtype;
  int32_t world, rank;
  int32_t batch, nheads, nchunks, dim;
  int64_t dA_stride[3];       /* b, h, c */
  int64_t out_stride[3];      /* b, c, h */
  int64_t final_stride[2];    /* b, h */
  int64_t Z_rank_stride;      /* elements between two ranks' Z; 0 = b * h * dim (contiguous) */
  int64_t logP_rank_stride;   /* elements between two ranks' logP; 0 = b * h (contiguous) */
} ssd_seqpar_fixup_params_t;

SSD_API int ssd_seqpar_fixup(const ssd_seqpar_fixup_params_t* prm, ssd_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* SSD_B200_H_ */
