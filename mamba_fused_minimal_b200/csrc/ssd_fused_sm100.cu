// Fused per-chunk state + inter-chunk state passing for sm_100a.
//
// One persistent CTA per SM.  The (batch, head-group-of-HPC, chunk) work items, ordered
// strip-major (a "strip" is one batch element and HPC adjacent heads of one B/C group)
// and chunk-minor, are cut into one contiguous range per CTA, so a CTA walks whole strips
// chunk after chunk and keeps the running fp32 state of each head in registers.  Only
// where a range boundary falls inside a strip does a state cross CTAs, through a carry
// slot in global memory guarded by an epoch-stamped flag.  A CTA whose range ends inside a
// strip processes that (dependency-free) head segment FIRST and its own dependent tail
// segment LAST, so in the common case the carry it needs was published long before it is
// asked for; when strips are longer than a CTA's range the wait is real, but it only holds
// up the epilogue warps: the loads and MMAs of up to NBUF chunks run ahead of it.
//
// Per chunk and head: states^T[n, p] = sum_k Bs[k, n] * x[k, p] with
// Bs = cast_in(B * exp(min(dA_last - dA_k, 0)) * dt_k)   (the reference's rounding point,
// kernels/ssd_chunk_state.py:153-159), a 128 x 64 x L contraction done by tcgen05.mma with
// both the A operand (Bs, dstate on the lanes) and the accumulator (lanes = dstate index n,
// columns = headdim index p) in tensor memory; only x is an operand from shared memory.
//
// Warp roles (HPC = heads per CTA sharing one B tile), in warpgroups so that each role can be
// given its own register budget (setmaxnreg):
//   warps [0, 4*HPC)      epilogue, one warpgroup per head: tcgen05.ld the chunk state in the
//                         matrix-fragment arrangement, S <- exp(dA_last) * S + state in
//                         registers; 16-bit passed states go out through stmatrix + one TMA
//                         store per warp and 32 rows, everything else with plain stores
//   warp  4*HPC           TMA producer: per 64-position stage the raw B tile and one x tile per
//                         head into a ring of six stages
//   warps 4*HPC + 1, + 2  MMA issuers, one thread per head (the first also owns the TMEM
//                         allocation); A from tensor memory, four K = 16 steps per stage
//   warp  4*HPC + 3       loads each chunk's dt / dA_cumsum rows (bulk copies) and turns them
//                         into the per-position factors exp(min(a_last - a_k, 0)) * dt_k
//   8 further warps       B scaling: ldmatrix.trans brings the raw 16-bit B values as (k, k+1)
//                         pairs per dstate column, they are widened, multiplied by their
//                         positions' factors in fp32, rounded back to the input type and
//                         written with tcgen05.st to the head's A slot in tensor memory
// The accumulator of a chunk is complete after its last stage; up to NBUF chunks of MMAs run
// ahead of the epilogue.
//
// RAW variant (the whole state path in one launch): the kernel is given the raw dt, A and
// dt_bias instead of dt_out / dA_cumsum.  The scale-vector warp then does the chunk cumsum of
// kernels/ssd_chunk_state.py:65-79 itself -- per chunk and head it fetches the raw dt values
// (small asynchronous copies, two chunks ahead), applies bias / softplus / clamp / tail mask,
// scans dt * A with the same warp scan as the stand-alone cumsum kernel (so the results carry
// the same bits), writes the dt_out and dA_cumsum rows as a by-product and derives the
// per-position factors from the values it holds in registers.
#include <cuda.h>

#include <mutex>

#include "sm100_ptx.cuh"
#include "ssd_carry.cuh"
#include "ssd_common.cuh"
#include "ssd_launch.h"

namespace ssd {
namespace {

using namespace ptx;

constexpr int kP = 64;        // headdim
constexpr int kN = 128;       // dstate
constexpr int kKT = 64;       // sequence positions per pipeline stage
constexpr int kMaxL = 256;    // largest chunk size

enum WaitCode {
  kWaitDdEmpty = 101, kWaitStageEmpty, kWaitDdFull, kWaitStageFull, kWaitBsEmpty, kWaitBsFull,
  kWaitAccEmpty, kWaitAccFull, kWaitCarry, kWaitGroup
};

template <int HPC>
struct Cfg {
  static constexpr int NS = 6;                        // shared-memory stages (raw B tile + x tiles)
  static constexpr int NA = 2;                        // scaled-B (A operand) slots per head in TMEM
  static constexpr int ND = 3;                        // dt/dA row slots (RAW variant: raw dt tiles)
  static constexpr int NBUF = (HPC == 2) ? 3 : 4;     // TMEM accumulators per head
  static constexpr int EPI_WARPS = 4 * HPC;
  // B-scaling warps: a warp can only write the TMEM lanes of its quadrant (warp index % 4), so
  // four quadrants x two halves of a stage's 64 positions
  static constexpr int SCALE_WARPS = 8;
  // one warpgroup of service warps: TMA producer, one MMA issuer per head (the second idles at
  // HPC = 1), the scale-vector warp
  static constexpr int SERVICE_WARPS = 4;
  static constexpr int SCALE_WARP0 = EPI_WARPS + SERVICE_WARPS;
  static constexpr int WARPS = SCALE_WARP0 + SCALE_WARPS;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int RAWB_BYTES = kKT * kN * 2;     // 16 KiB: two 64-column SW128 boxes
  static constexpr int X_BYTES = kKT * kP * 2;        // 8 KiB: one SW128 box
  // a stage: the raw B tile, then one x tile per head
  static constexpr int LOAD_BYTES = RAWB_BYTES + HPC * X_BYTES;   // what TMA brings per stage
  static constexpr int OFF_XT = RAWB_BYTES;                       // x tiles inside a stage
  static constexpr int STAGE_BYTES = LOAD_BYTES;
  // tensor memory: NBUF accumulators of kP columns per head, then NA scaled-B slots of kKT / 2
  // columns per head (two 16-bit K elements per column)
  static constexpr int TMEM_A0 = HPC * NBUF * kP;
  static constexpr int A_COLS = kKT / 2;
  static constexpr int TMEM_COLS = 512;
  static_assert(TMEM_A0 + HPC * NA * A_COLS <= TMEM_COLS, "tensor memory budget");
  // shared-memory map (byte offsets from a 1024-aligned base)
  static constexpr int OFF_STAGES = 0;
  static constexpr int OFF_DTDA = OFF_STAGES + NS * STAGE_BYTES;
  // dt and dA_cumsum rows of every head -- or, in the RAW variant, one [kMaxL][16 bytes] tile of raw dt
  static constexpr int DTDA_SLOT = (HPC * 2 * kMaxL * 4 > kMaxL * 16) ? HPC * 2 * kMaxL * 4 : kMaxL * 16;
  static constexpr int OFF_SCALE = OFF_DTDA + ND * DTDA_SLOT;
  static constexpr int SCALE_SLOT = HPC * kMaxL * 4;
  static constexpr int OFF_BARS = OFF_SCALE + 2 * SCALE_SLOT;
  // mbarrier indices
  static constexpr int B_FULL = 0;                       // [NS]  stage loaded (TMA bytes)
  static constexpr int B_EMPTY = B_FULL + NS;            // [NS]  stage consumed (one commit per MMA issuer)
  static constexpr int B_BS = B_EMPTY + NS;              // [NA]  scaled B written (one arrival per scaling warp)
  static constexpr int B_DD = B_BS + NA;                 // [ND]  dt / dA rows loaded
  static constexpr int B_DDE = B_DD + ND;                // [ND]  RAW variant: raw dt tile consumed
  static constexpr int B_ACCF = B_DDE + ND;              // [HPC][NBUF] accumulator complete
  static constexpr int B_ACCE = B_ACCF + HPC * NBUF;     // [HPC][NBUF] accumulator drained (4 epilogue warps)
  static constexpr int B_SCR = B_ACCE + HPC * NBUF;      // [2]   scale vector ready
  static constexpr int B_SCF = B_SCR + 2;                // [2]   scale vector no longer needed
  static constexpr int B_EPI = B_SCF + 2;                // [HPC] epilogue warpgroup sync
  static constexpr int NUM_BARS = B_EPI + HPC;
  static constexpr int OFF_CTL = OFF_BARS + NUM_BARS * 8;
  // staging for 16-bit passed states: every epilogue warp owns 32 rows (p) x 32 columns (its
  // dstate quadrant) = 32 x 64 bytes, laid out as a TMA box with the 64-byte swizzle
  static constexpr int STAGING_BYTES = 32 * 64;
  // RAW variant: each chunk's total log-decay travels from the scale-vector warp to the epilogue
  // through a ring of RING entries per head (the epilogue lags by fewer chunks than that: two
  // scale vectors, the A slots and NBUF accumulators)
  static constexpr int RING = 8;
  static constexpr int OFF_RING = OFF_CTL + 64;
  static constexpr int OFF_STAGING = (OFF_RING + RING * HPC * 4 + 1023) / 1024 * 1024;
  static constexpr int SMEM_BYTES = OFF_STAGING + EPI_WARPS * STAGING_BYTES + 1024;   // + alignment slack
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
  // Register budget per role (setmaxnreg).  The CTA is launched with LAUNCH_REGS per thread,
  // too few for the epilogue's 64 state values at 640 threads; the scaling and service warps
  // give registers back and the epilogue warps take them.  setmaxnreg.inc waits for registers
  // that other roles release, so the per-role counts must fit in what the CTA is launched
  // with, or the wait never ends.
  static constexpr int LAUNCH_REGS = 65536 / (WARPS * 32) / 8 * 8;
  static constexpr int REGS_EPI = (HPC == 2) ? 144 : 168;
  static constexpr int REGS_SCALE = (HPC == 2) ? 72 : 96;
  static constexpr int REGS_SERVICE = (HPC == 2) ? 48 : 64;   // the cumsum of the RAW variant runs here
  static constexpr bool REBALANCE = true;
  static_assert(EPI_WARPS * REGS_EPI + SERVICE_WARPS * REGS_SERVICE + SCALE_WARPS * REGS_SCALE <= WARPS * LAUNCH_REGS,
                "per-role register counts exceed the launch allocation");
  // The register file is four files of 16 384, one per scheduler, and a warp lives in file (warp index % 4):
  // the budget has to hold in each of them.  Every role is a multiple of four consecutive warps, so each
  // file gets the same share of every role.  (This is also why a 21st warp cannot be added: the file that
  // takes a sixth warp caps all threads at 80 registers, and the compiler then builds the kernel for 80.)
  static_assert(WARPS % 4 == 0 && EPI_WARPS % 4 == 0 && SERVICE_WARPS % 4 == 0 && SCALE_WARPS % 4 == 0 &&
                    (WARPS / 4) * LAUNCH_REGS * 32 <= 16384,
                "roles must spread evenly over the four register files");
  static_assert(REGS_SCALE <= LAUNCH_REGS && REGS_SERVICE <= LAUNCH_REGS && REGS_EPI >= LAUNCH_REGS,
                "scaling and service roles give registers back, the epilogue takes them");
};

struct FusedArgs {
  const float* dt;
  const float* dA;
  const void* init;
  const int32_t* seq_idx; // (b, l) sequence index of each position, or NULL
  void* out;
  float* final_states;
  void* states;
  int* status;            // workspace header: [0] status, [1] epoch, [2] done counter
  uint32_t* flags;        // [cta][HPC]
  float* carry;           // [cta][HPC][kP * kN]
  int64_t dt_s[3], dA_s[3];                 // b, h, c strides (elements); L stride is 1
  int64_t init_s[3], out_s[4], final_s[3], states_s[4], seq_s[2];
  int batch, seqlen, nheads, ngroups, chunk_size, nchunks;
  int strips_per_batch;   // nheads / HPC
  int init_dtype, out_dtype, states_dtype;
  int clamp_decay;
  int mode;               // 0: state passing fused; 1: per-chunk states only
  int defer;              // non-zero: segments that start inside a strip start from zero; the
                          // carried state is added afterwards by segment_fixup_kernel
  // RAW variant: dt / dA above are OUTPUTS ((b, h, c, L) fp32 rows, written by the kernel), computed from
  const void* dt_raw;     // (b, l, h) of raw_dtype, heads contiguous
  const void* A;          // (h,)
  const void* bias;       // (h,) or NULL
  int64_t raw_s[2];       // b, l strides of dt_raw (elements)
  int64_t A_stride, bias_stride;
  int raw_dtype, A_dtype, bias_dtype;
  int softplus;
  float dt_min, dt_max;
  int debug;              // test hooks (ssd_debug_set_flags); 0 in normal use
  long long wait_limit;   // SM cycles a device-side wait may last
};


struct Range {
  long long lo, hi;
  int s_first, m;
  bool rot;
};

__device__ __forceinline__ Range make_range(long long total, int nchunks) {
  Range r;
  r.lo = total * (long long)blockIdx.x / gridDim.x;
  r.hi = total * (long long)(blockIdx.x + 1) / gridDim.x;
  r.s_first = (int)(r.lo / nchunks);
  const int s_last = (int)((r.hi - 1) / nchunks);
  r.m = s_last - r.s_first + 1;
  r.rot = (r.m > 1) && (r.hi % nchunks != 0);
  return r;
}

// j-th segment of this CTA in processing order: the trailing head segment (if the range
// ends inside a strip) first, whole strips next, the leading (possibly dependent) one last.
__device__ __forceinline__ void get_segment(const Range& r, int nchunks, int j, int& strip,
                                            int& c0, int& c1) {
  int k;
  if (r.m == 1) k = 0;
  else if (r.rot) k = (j == 0) ? r.m - 1 : ((j == r.m - 1) ? 0 : j);
  else k = (j == r.m - 1) ? 0 : j + 1;
  strip = r.s_first + k;
  const long long base = (long long)strip * nchunks;
  c0 = (int)((r.lo > base ? r.lo : base) - base);
  const long long end = base + nchunks;
  c1 = (int)((r.hi < end ? r.hi : end) - base);
}

template <typename T> struct Pack;
template <> struct Pack<__nv_bfloat16> {
  static constexpr uint32_t kFmt = 1;
  __device__ static __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    lo = __uint_as_float(w << 16);
    hi = __uint_as_float(w & 0xffff0000u);
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Pack<__half> {
  static constexpr uint32_t kFmt = 0;
  __device__ static __forceinline__ void unpack(uint32_t w, float& lo, float& hi) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
    lo = f.x;
    hi = f.y;
  }
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

template <typename T, int HPC, bool OUT32, bool SEQ, bool RAW>
__global__ void __launch_bounds__(Cfg<HPC>::THREADS, 1)
fused_state_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_B,
                   const __grid_constant__ CUtensorMap tmap_out, const __grid_constant__ CUtensorMap tmap_dt,
                   const FusedArgs a) {
  using C = Cfg<HPC>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  // barrier addresses
  const uint32_t bars = sbase + C::OFF_BARS;
  auto bar_full = [&](int s) { return bars + 8u * (C::B_FULL + s); };
  auto bar_empty = [&](int s) { return bars + 8u * (C::B_EMPTY + s); };
  auto bar_bs_full = [&](int t) { return bars + 8u * (C::B_BS + t); };
  auto bar_dd_full = [&](int r) { return bars + 8u * (C::B_DD + r); };
  auto bar_dd_empty = [&](int r) { return bars + 8u * (C::B_DDE + r); };
  auto bar_acc_full = [&](int hd, int b) { return bars + 8u * (C::B_ACCF + hd * C::NBUF + b); };
  auto bar_acc_empty = [&](int hd, int b) { return bars + 8u * (C::B_ACCE + hd * C::NBUF + b); };
  auto bar_sc_ready = [&](int i) { return bars + 8u * (C::B_SCR + i); };
  auto bar_sc_free = [&](int i) { return bars + 8u * (C::B_SCF + i); };
  // (an mbarrier instead of bar.sync so that the wait is bounded like the rest)
  auto bar_epi_sync = [&](int hd) { return bars + 8u * (C::B_EPI + hd); };
  volatile int* ctl = reinterpret_cast<volatile int*>(smem + C::OFF_CTL);   // [0] abort, [1] tmem, [2] epoch
  WaitCtx wc{ctl, a.status, a.wait_limit};

  if (tid == 0) {
    for (int s = 0; s < C::NS; ++s) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), HPC); }
    for (int t = 0; t < C::NA; ++t) mbar_init(bar_bs_full(t), C::SCALE_WARPS);
    for (int r = 0; r < C::ND; ++r) { mbar_init(bar_dd_full(r), 1); mbar_init(bar_dd_empty(r), 1); }
    for (int hd = 0; hd < HPC; ++hd)
      for (int b = 0; b < C::NBUF; ++b) { mbar_init(bar_acc_full(hd, b), 1); mbar_init(bar_acc_empty(hd, b), 4); }
    // group barriers take ONE arrival per warp: arrivals on one mbarrier serialise
    for (int i = 0; i < 2; ++i) { mbar_init(bar_sc_ready(i), 1); mbar_init(bar_sc_free(i), C::SCALE_WARPS); }
    for (int hd = 0; hd < HPC; ++hd) mbar_init(bar_epi_sync(hd), 4);
    ctl[0] = 0;
    ctl[2] = reinterpret_cast<volatile int*>(a.status)[1];     // epoch of the previous launch
    fence_barrier_init();
    fence_proxy_async_smem();
  }
  if (warp == C::EPI_WARPS + 1) {
    tmem_alloc(sbase + C::OFF_CTL + 4, C::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == C::EPI_WARPS && lane == 0) {
    prefetch_tensormap(&tmap_x);
    prefetch_tensormap(&tmap_B);
    if (!OUT32 && a.mode == 0) prefetch_tensormap(&tmap_out);
    if (RAW) prefetch_tensormap(&tmap_dt);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = static_cast<uint32_t>(ctl[1]);
  const uint32_t epoch_target = static_cast<uint32_t>(ctl[2]) + 1u;

  const int L = a.chunk_size;
  const int nchunks = a.nchunks;
  const long long total = (long long)a.batch * a.strips_per_batch * nchunks;
  const Range rg = make_range(total, nchunks);
  const int ratio = a.nheads / a.ngroups;

  if (warp >= C::EPI_WARPS && warp < C::SCALE_WARP0) {
    if constexpr (C::REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::REGS_SERVICE));
    if (warp == C::EPI_WARPS) {
      // ============================== TMA producer ====================================
      if (lane == 0) {
        // x is read exactly once: its lines are the first to go.  B is re-read once per head pair of
        // its group and stays in L2 by being re-used; it is NOT marked evict-last: such lines outlive
        // the launch and a long sequence's worth of them (268 MB at a million tokens) would occupy the
        // L2 for whatever runs next (measured: the next launches ran 20 % slower).
        const uint64_t keep = l2_policy_evict_normal(), stream_once = l2_policy_evict_first();
        uint32_t it = 0;
        bool ok = true;
        // RAW variant: the raw dt tile of chunk i + 1 (the 16 bytes of heads around this CTA's heads x
        // one chunk of positions, a tile [position][16 bytes]) is requested when chunk i starts; a slot
        // is reused once the cumsum warp has read it
        uint32_t ditem = 0;                                    // next raw dt tile to request
        int pj = 0, pstrip = 0, pc = 0, pc1 = 0;
        if (RAW && rg.m > 0) get_segment(rg, nchunks, 0, pstrip, pc, pc1);
        auto fetch_raw = [&]() {
          if (pj >= rg.m) return true;
          const int slot = ditem % C::ND;
          if (!mbar_wait(bar_dd_empty(slot), ((ditem / C::ND) & 1) ^ 1, wc, kWaitDdEmpty)) return false;
          const int es = a.raw_dtype == SSD_F32 ? 4 : 2;
          const int pb = pstrip / a.strips_per_batch;
          const int ph0 = (pstrip % a.strips_per_batch) * HPC;
          mbar_expect_tx(bar_dd_full(slot), L * 16);
          tma_load_3d(sbase + C::OFF_DTDA + slot * C::DTDA_SLOT, &tmap_dt, bar_dd_full(slot), ph0 & ~(16 / es - 1), pc * L, pb);
          ++ditem;
          if (++pc >= pc1 && ++pj < rg.m) get_segment(rg, nchunks, pj, pstrip, pc, pc1);
          return true;
        };
        if (RAW) ok = fetch_raw();
        for (int j = 0; j < rg.m && ok; ++j) {
          int strip, c0, c1;
          get_segment(rg, nchunks, j, strip, c0, c1);
          const int b = strip / a.strips_per_batch;
          const int h0 = (strip % a.strips_per_batch) * HPC;
          const int g = h0 / ratio;
          for (int c = c0; c < c1 && ok; ++c) {
            if (RAW) {
              ok = fetch_raw();
              if (!ok) break;
            }
            const int limit = min(L, a.seqlen - c * L);
            const int ksteps = (limit + kKT - 1) / kKT;
            for (int ks = 0; ks < ksteps; ++ks, ++it) {
              const int s = it % C::NS;
              ok = mbar_wait(bar_empty(s), ((it / C::NS) & 1) ^ 1, wc, kWaitStageEmpty);
              if (!ok) break;
              const uint32_t st = sbase + C::OFF_STAGES + s * C::STAGE_BYTES;
              const int l0 = c * L + ks * kKT;
              mbar_expect_tx(bar_full(s), C::LOAD_BYTES);
              // one copy for the raw B tile (both 64-column halves, one after the other) and one for
              // the x tiles of all the CTA's heads: few large copies keep the copy engine busier than
              // many small ones
              tma_load_5d_hint(st, &tmap_B, bar_full(s), 0, l0, 0, g, b, keep);
              tma_load_4d_hint(st + C::OFF_XT, &tmap_x, bar_full(s), 0, l0, h0, b, stream_once);
            }
          }
        }
      }
    } else if (warp <= C::EPI_WARPS + HPC) {
      // ============================== MMA issuer of head mhd ==========================
      // One issuing thread per head: the two heads' accumulators are independent, and two
      // threads keep the tensor pipe fed where one spent half its time issuing.
      const int mhd = warp - (C::EPI_WARPS + 1);
      if (lane == 0) {
        // A (the scaled B tile) comes from tensor memory, K-major by construction; B (the x
        // tile) from shared memory as TMA delivered it: headdim contiguous, i.e. MN-major.
        constexpr uint32_t idesc = mma_idesc(Pack<T>::kFmt, false, true, kN, kP);
        // Descriptor of stage 0; the address field (bits 0-13, units of 16 bytes) never carries
        // out of its field for shared-memory addresses below 256 KiB, so other stages and
        // k-steps are reached by plain 64-bit additions.
        const uint64_t bdesc0 = smem_desc_sw128(sbase + C::OFF_STAGES + C::OFF_XT + mhd * C::X_BYTES, C::X_BYTES, 1024);
        uint32_t it = 0, item = 0;
        bool ok = true;
        for (int j = 0; j < rg.m && ok; ++j) {
          int strip, c0, c1;
          get_segment(rg, nchunks, j, strip, c0, c1);
          for (int c = c0; c < c1 && ok; ++c, ++item) {
            const int buf = item % C::NBUF;
            ok = mbar_wait(bar_acc_empty(mhd, buf), ((item / C::NBUF) & 1) ^ 1, wc, kWaitAccEmpty);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (mhd * C::NBUF + buf) * kP;
            const int limit = min(L, a.seqlen - c * L);
            const int ksteps = (limit + kKT - 1) / kKT;
            for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
              const int s = it % C::NS;
              const int sa = it % C::NA;
              ok = mbar_wait(bar_full(s), (it / C::NS) & 1, wc, kWaitStageFull);
              if (!ok) break;
              ok = mbar_wait(bar_bs_full(sa), (it / C::NA) & 1, wc, kWaitBsFull);
              if (!ok) break;
              tc_fence_after();
              const uint64_t bd_s = bdesc0 + (uint64_t)((s * C::STAGE_BYTES) >> 4);
              const uint32_t a_tmem = tmem_base + C::TMEM_A0 + (mhd * C::NA + sa) * C::A_COLS;
#pragma unroll
              for (int k16 = 0; k16 < kKT / 16; ++k16)
                mma_f16_ts(d_tmem, a_tmem + k16 * 8, bd_s + (uint64_t)((k16 * 2048) >> 4), idesc, (ks | k16) != 0 ? 1u : 0u);
              mma_commit(bar_empty(s));
            }
            if (ok) mma_commit(bar_acc_full(mhd, buf));
          }
        }
      }
    } else if (warp == C::EPI_WARPS + 3 && RAW) {
      // ============================== chunk cumsum + scale vectors ====================
      // One TMA copy per chunk (issued by the producer warp, one chunk ahead) brings the raw dt of the
      // 16-byte group of heads that holds this CTA's heads (4 fp32 or 8 sixteen-bit values per position)
      // as a tile [position][16 bytes].
      // Phase A, lane = position modulo 32: bias / softplus / clamp / tail mask
      // (kernels/ssd_chunk_state.py:66-74), dt' parked in the scale-vector slot ([head][position]).
      // Phase B, lane = 8 consecutive positions: cumulative sum of dt' * A with the cumsum kernel's
      // warp scan (same operations, same order, same bits), the dt_out / dA_cumsum rows written to
      // global memory, the factors exp(min(a_last - a_k, 0)) * dt_k written over the parked dt', and
      // the chunk's total left for the epilogue.
      const int es = a.raw_dtype == SSD_F32 ? 4 : 2;
      const int hmask = 16 / es - 1;                               // heads per 16-byte group, minus one
      const bool sp = a.softplus != 0;
      // the clamp is the identity for the default limits once the softplus has made dt' non-negative
      const bool clamp = !(sp && a.dt_min <= 0.0f && a.dt_max == __int_as_float(0x7f800000));
      uint32_t item = 0;
      bool ok = true;
      for (int j = 0; j < rg.m && ok; ++j) {
        int strip, c0, c1;
        get_segment(rg, nchunks, j, strip, c0, c1);
        const int b = strip / a.strips_per_batch;
        const int h0 = (strip % a.strips_per_batch) * HPC;
        float Ah[HPC], bh[HPC];
#pragma unroll
        for (int hd = 0; hd < HPC; ++hd) {
          Ah[hd] = load_f(a.A, a.A_dtype, (int64_t)(h0 + hd) * a.A_stride);
          bh[hd] = a.bias != nullptr ? load_f(a.bias, a.bias_dtype, (int64_t)(h0 + hd) * a.bias_stride) : 0.0f;
        }
        const uint32_t in_group = (uint32_t)(h0 & hmask) * es;      // byte offset of head h0 inside a position's 16 bytes
        // element offset of (b, h0, chunk 0, position 8 * lane) in the two fp32 outputs
        const int64_t row0 = (int64_t)b * a.dt_s[0] + (int64_t)h0 * a.dt_s[1] + lane * 8;
        const int k0 = lane * 8;
        for (int c = c0; c < c1 && ok; ++c, ++item) {
          const int r = item % C::ND;
          ok = mbar_wait(bar_dd_full(r), (item / C::ND) & 1, wc, kWaitDdFull);
          if (!ok) break;
          if (item >= 2) {
            ok = mbar_wait(bar_sc_free(item & 1), ((item >> 1) - 1) & 1, wc, kWaitGroup);
            if (!ok) break;
          }
          const uint32_t rawp = sbase + C::OFF_DTDA + r * C::DTDA_SLOT + in_group;
          const uint32_t scp = sbase + C::OFF_SCALE + (item & 1) * C::SCALE_SLOT;
          const int limit = min(L, a.seqlen - c * L);
          // ---- phase A (two positions per head in flight: four independent chains)
#pragma unroll 2
          for (int kk = 0; kk < kMaxL / 32; ++kk) {
            const int k = kk * 32 + lane;
            if (k >= L) break;
            float v[HPC];
            if (a.raw_dtype == SSD_F32) {
              if (HPC == 2) lds_v2(rawp + k * 16, v[0], v[HPC - 1]);
              else v[0] = lds_f32(rawp + k * 16);
            } else {
              const uint32_t w = HPC == 2 ? lds_u32(rawp + k * 16) : (uint32_t)lds_u16(rawp + k * 16);
              if (a.raw_dtype == SSD_BF16) {
                v[0] = __uint_as_float(w << 16);
                if (HPC == 2) v[HPC - 1] = __uint_as_float(w & 0xffff0000u);
              } else {
                const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w));
                v[0] = f2.x;
                if (HPC == 2) v[HPC - 1] = f2.y;
              }
            }
#pragma unroll
            for (int hd = 0; hd < HPC; ++hd) {
              float t = v[hd] + bh[hd];
              if (sp) t = softplus_ref(t);
              if (clamp) t = fminf(fmaxf(t, a.dt_min), a.dt_max);
              sts_f32(scp + (hd * kMaxL + k) * 4, k < limit ? t : 0.0f);    // positions past the sequence hold zeros
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_dd_empty(r));     // the raw tile has been read
          // ---- phase B
#pragma unroll
          for (int hd = 0; hd < HPC; ++hd) {
            float d[8], cs[8];
            if (k0 < L) {
              lds_v4(scp + (hd * kMaxL + k0) * 4, d[0], d[1], d[2], d[3]);
              lds_v4(scp + (hd * kMaxL + k0 + 4) * 4, d[4], d[5], d[6], d[7]);
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) d[i] = 0.0f;
            }
            warp_cumsum8(d, Ah[hd], 0.0f, lane, cs);
            // the chunk's total: the sum at position L - 1 (flat over a ragged tail); L is a multiple of 64
            const float last = __shfl_sync(0xffffffffu, cs[7], (L - 1) >> 3);
            if (k0 < L) {
              const int64_t row = row0 + (int64_t)hd * a.dt_s[1] + (int64_t)c * a.dt_s[2];
              float4* o1 = reinterpret_cast<float4*>(const_cast<float*>(a.dt) + row);
              float4* o2 = reinterpret_cast<float4*>(const_cast<float*>(a.dA) + row);
              o1[0] = make_float4(d[0], d[1], d[2], d[3]);
              o1[1] = make_float4(d[4], d[5], d[6], d[7]);
              o2[0] = make_float4(cs[0], cs[1], cs[2], cs[3]);
              o2[1] = make_float4(cs[4], cs[5], cs[6], cs[7]);
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                float dl = last - cs[i];
                if (a.clamp_decay) dl = fminf(dl, 0.0f);
                d[i] = fast_exp(dl) * d[i];
              }
              sts_v4(scp + (hd * kMaxL + k0) * 4, d[0], d[1], d[2], d[3]);
              sts_v4(scp + (hd * kMaxL + k0 + 4) * 4, d[4], d[5], d[6], d[7]);
            }
            if (lane == 0) sts_f32(sbase + C::OFF_RING + ((item % C::RING) * HPC + hd) * 4, last);
          }
          __syncwarp();                       // every lane has written its factors
          if (lane == 0) mbar_arrive(bar_sc_ready(item & 1));
        }
      }
    } else if (warp == C::EPI_WARPS + 3) {
      // ============================== scale vectors ===================================
      // One warp loads each chunk's dt / dA_cumsum rows (bulk copies, ND chunks ahead) and turns
      // them into the per-position factors exp(min(a_last - a_k, 0)) * dt_k, one item ahead of
      // the B-scaling warps.
      auto load_rows = [&](int strip, int c, int slot) {          // one lane
        const int b = strip / a.strips_per_batch;
        const int h0 = (strip % a.strips_per_batch) * HPC;
        mbar_expect_tx(bar_dd_full(slot), HPC * 2 * L * 4);
#pragma unroll
        for (int hd = 0; hd < HPC; ++hd) {
          const uint32_t dst = sbase + C::OFF_DTDA + slot * C::DTDA_SLOT + hd * 2 * kMaxL * 4;
          bulk_load(dst, a.dt + (int64_t)b * a.dt_s[0] + (int64_t)(h0 + hd) * a.dt_s[1] + (int64_t)c * a.dt_s[2], L * 4,
                    bar_dd_full(slot));
          bulk_load(dst + kMaxL * 4, a.dA + (int64_t)b * a.dA_s[0] + (int64_t)(h0 + hd) * a.dA_s[1] + (int64_t)c * a.dA_s[2],
                    L * 4, bar_dd_full(slot));
        }
      };
      // look-ahead position in the CTA's item order
      int pj = 0, pstrip = 0, pc = 0, pc1 = 0;
      if (rg.m > 0) get_segment(rg, nchunks, 0, pstrip, pc, pc1);
      auto pre_valid = [&]() { return pj < rg.m; };
      auto pre_next = [&]() {
        if (++pc >= pc1 && ++pj < rg.m) get_segment(rg, nchunks, pj, pstrip, pc, pc1);
      };
      for (int i = 0; i < C::ND && pre_valid(); ++i) {
        if (lane == 0) load_rows(pstrip, pc, i);
        pre_next();
      }
      uint32_t item = 0;
      bool ok = true;
      for (int j = 0; j < rg.m && ok; ++j) {
        int strip, c0, c1;
        get_segment(rg, nchunks, j, strip, c0, c1);
        for (int c = c0; c < c1 && ok; ++c, ++item) {
          const int r = item % C::ND;
          ok = mbar_wait(bar_dd_full(r), (item / C::ND) & 1, wc, kWaitDdFull);
          if (!ok) break;
          if (item >= 2) {
            ok = mbar_wait(bar_sc_free(item & 1), ((item >> 1) - 1) & 1, wc, kWaitGroup);
            if (!ok) break;
          }
          const float* dd = reinterpret_cast<const float*>(smem + C::OFF_DTDA + r * C::DTDA_SLOT);
          float* sc = reinterpret_cast<float*>(smem + C::OFF_SCALE + (item & 1) * C::SCALE_SLOT);
          // packed sequences: a position contributes to the chunk's state only if it belongs to
          // the same sequence as the chunk's last position (kernels/ssd_chunk_state.py:147-152)
          const int limit = min(L, a.seqlen - c * L);
          const int32_t* sq = nullptr;
          int seq_last = 0;
          if constexpr (SEQ) {
            sq = a.seq_idx + (int64_t)(strip / a.strips_per_batch) * a.seq_s[0] + (int64_t)c * L * a.seq_s[1];
            seq_last = sq[(int64_t)(limit - 1) * a.seq_s[1]];
          }
#pragma unroll
          for (int hd = 0; hd < HPC; ++hd) {
            const float* row = dd + hd * 2 * kMaxL;
            const float last = row[kMaxL + L - 1];
            for (int k = lane; k < L; k += 32) {
              float d = last - row[kMaxL + k];
              if (a.clamp_decay) d = fminf(d, 0.0f);
              float f = fast_exp(d) * row[k];
              if constexpr (SEQ) {
                if (k < limit && sq[(int64_t)k * a.seq_s[1]] != seq_last) f = 0.0f;
              }
              sc[hd * kMaxL + k] = f;
            }
          }
          __syncwarp();                       // every lane has read the rows and written its factors
          if (lane == 0) {
            mbar_arrive(bar_sc_ready(item & 1));
            fence_proxy_async_smem();         // the rows were read; the slot is refilled by bulk copies
            if (pre_valid()) load_rows(pstrip, pc, r);
          }
          pre_next();
        }
      }
    }
  } else if (warp >= C::SCALE_WARP0) {
    // ============================== B scaling =========================================
    if constexpr (C::REBALANCE) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(C::REGS_SCALE));
    // Warp (qn, kh): TMEM lane quadrant qn = dstate columns 32 qn .. 32 qn + 31, and positions
    // 32 kh .. 32 kh + 31 of every 64-position stage.  For each block of 16 dstate columns two
    // ldmatrix.trans bring the raw 16-bit B values as (k, k + 1) pairs per column, which is the
    // arrangement tcgen05.st (16x128b) wants for an A operand with the dstate index on the
    // lanes; each pair is widened, multiplied by its positions' factors in fp32, rounded back
    // to the input type (the reference's rounding point) and stored to the head's A slot.
    const int sw = warp - C::SCALE_WARP0;
    const int qn = sw & 3, kh = sw >> 2;
    const int lm = lane >> 3, lr = lane & 7;              // ldmatrix: matrix and row this lane addresses
    // raw B tile: two boxes of 64 columns; a row (position) is 128 bytes, its 16-byte pieces
    // swizzled by the row index modulo 8, which here is lr
    const uint32_t ld_base = (uint32_t)((qn >> 1) * (C::RAWB_BYTES / 2) + (kh * 32 + (lm >> 1) * 8 + lr) * 128);
    const uint32_t ld_piece[2] = {(uint32_t)((((qn & 1) * 4 + (lm & 1)) ^ lr) << 4),
                                  (uint32_t)((((qn & 1) * 4 + 2 + (lm & 1)) ^ lr) << 4)};
    const uint32_t st_lane = static_cast<uint32_t>(qn * 32) << 16;
    const int sq = 2 * (lane & 3);                        // first of this lane's two positions in a block of 8
    uint32_t it = 0, item = 0;
    bool ok = true;
    for (int j = 0; j < rg.m && ok; ++j) {
      int strip, c0, c1;
      get_segment(rg, nchunks, j, strip, c0, c1);
      for (int c = c0; c < c1 && ok; ++c, ++item) {
        ok = mbar_wait(bar_sc_ready(item & 1), (item >> 1) & 1, wc, kWaitDdFull);
        if (!ok) break;
        const float* sc = reinterpret_cast<const float*>(smem + C::OFF_SCALE + (item & 1) * C::SCALE_SLOT);
        const int limit = min(L, a.seqlen - c * L);
        const int ksteps = (limit + kKT - 1) / kKT;
        for (int ks = 0; ks < ksteps && ok; ++ks, ++it) {
          const int s = it % C::NS;
          const int sa = it % C::NA;
          ok = mbar_wait(bar_full(s), (it / C::NS) & 1, wc, kWaitStageFull);
          if (!ok) break;
          // the A slot is free once the MMAs of iteration it - NA are complete, which is what
          // releases that iteration's stage
          if (it >= (uint32_t)C::NA) {
            const uint32_t pit = it - C::NA;
            ok = mbar_wait(bar_empty(pit % C::NS), (pit / C::NS) & 1, wc, kWaitBsEmpty);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t raw = sbase + C::OFF_STAGES + s * C::STAGE_BYTES + ld_base;
          // factors of this lane's positions: block i of 8 positions -> (f[k], f[k + 1])
          float2 f[HPC][4];
#pragma unroll
          for (int hd = 0; hd < HPC; ++hd)
#pragma unroll
            for (int i = 0; i < 4; ++i)
              f[hd][i] = *reinterpret_cast<const float2*>(sc + hd * kMaxL + ks * kKT + kh * 32 + i * 8 + sq);
#pragma unroll
          for (int nbk = 0; nbk < 2; ++nbk) {               // dstate columns 16 nbk .. of the quadrant
            uint32_t r[8];
            {
              uint32_t t4[4];
              ldmatrix_x4_trans(raw + ld_piece[nbk], t4);              // positions 0..15 of the half
              r[0] = t4[0]; r[1] = t4[1]; r[2] = t4[2]; r[3] = t4[3];
              ldmatrix_x4_trans(raw + 16 * 128 + ld_piece[nbk], t4);   // positions 16..31
              r[4] = t4[0]; r[5] = t4[1]; r[6] = t4[2]; r[7] = t4[3];
            }
            float2 e[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) Pack<T>::unpack(r[i], e[i].x, e[i].y);
#pragma unroll
            for (int hd = 0; hd < HPC; ++hd) {
              uint32_t o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float2 v = __fmul2_rn(e[i], f[hd][i >> 1]);
                o[i] = Pack<T>::pack(v.x, v.y);
              }
              tmem_st_16x128b_x4(tmem_base + st_lane + (static_cast<uint32_t>(nbk * 16) << 16) + C::TMEM_A0 +
                                     (hd * C::NA + sa) * C::A_COLS + kh * 16, o);
            }
          }
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_bs_full(sa));
        }
        // (the __syncwarp of the last stage ordered every lane's reads of the scale vector)
        if (ok && lane == 0) mbar_arrive(bar_sc_free(item & 1));
      }
    }
  } else {
    // ============================== epilogue ==========================================
    if constexpr (C::REBALANCE) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(C::REGS_EPI));
    // One warpgroup per head; warp wq of it owns TMEM lanes 32 wq .. 32 wq + 31 (dstate n).
    // Accumulators are read in the matrix-fragment arrangement (tmem_ld_16x256b_x4), which is
    // also the arrangement stmatrix stores transposed: a warp builds its 32 rows x 32 columns of
    // a 16-bit (p, n) tile in shared memory with four stmatrix and one lane sends it off with
    // one TMA store.  Nothing here needs another warp.
    // Element i (0..63) of a thread's fragment, with g = lane / 4 and qd = lane % 4:
    //   n = 32 wq + 16 ((i / 16) % 2) + 8 ((i / 2) % 2) + g
    //   p = 32 (i / 32) + 8 ((i / 4) % 4) + (i % 2) + 2 qd
    const int hd = warp >> 2;
    const int wq = warp & 3;
    const int nb = wq * 32 + (lane >> 2);
    const int pb = 2 * (lane & 3);
    auto fn = [](int i) { return ((i >> 4) & 1) * 16 + ((i >> 1) & 1) * 8; };
    auto fp = [](int i) { return (i >> 5) * 32 + ((i >> 2) & 3) * 8 + (i & 1); };
    const uint32_t lane_sel = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t stg = sbase + C::OFF_STAGING + warp * C::STAGING_BYTES;
    // This thread's row address for stmatrix: row (lane % 8) of matrix (lane / 8); matrices 0/1
    // are the two 8-column blocks of one 8-row block, matrices 2/3 those of the next 8 rows.
    // A staging row is 64 bytes = four 16-byte pieces; the 64-byte swizzle puts piece c of row r
    // at piece c ^ ((r / 2) % 4), which for every row this thread addresses is (lane / 2) % 4.
    const uint32_t stm_rows = stg + (((lane >> 4) & 1) * 8 + (lane & 7)) * 64;
    const uint32_t stm_swz = (lane >> 1) & 3, stm_blk = (lane >> 3) & 1;
    const uint32_t stm_row[2] = {stm_rows + ((stm_blk ^ stm_swz) << 4), stm_rows + (((2 + stm_blk) ^ stm_swz) << 4)};
    float S[kP];
    uint32_t item = 0, epi_syncs = 0;
    bool ok = true;
    // Stores 32 rows (p = 32 hq ..) of a (kP x kN) tile whose element (0, 0) is at element
    // offset `tile` of `base`, row pitch `pitch`, from the fragment values vals[0..31].
    // `map` != nullptr: 16-bit tile (b = cb, chunk = cc, head = ch) of the tensor behind the map.
    auto store_half = [&](void* base, int dtype, int64_t tile, int64_t pitch, int hq, const float (&vals)[32],
                          const CUtensorMap* map, int cb, int cc, int ch) {
      if (map == nullptr) {
        const int64_t e0 = tile + (int64_t)(hq * 32 + pb) * pitch + nb;
        if (dtype == SSD_F32) {
          float* o = static_cast<float*>(base) + e0;
#pragma unroll
          for (int i = 0; i < 32; ++i) o[(int64_t)fp(i) * pitch + fn(i)] = vals[i];
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) store_f(base, dtype, e0 + (int64_t)fp(i) * pitch + fn(i), vals[i]);
        }
        return;
      }
      uint32_t pk[16];
      if (dtype == SSD_BF16) {
#pragma unroll
        for (int k = 0; k < 16; ++k) pk[k] = Pack<__nv_bfloat16>::pack(vals[2 * k], vals[2 * k + 1]);
      } else {
#pragma unroll
        for (int k = 0; k < 16; ++k) pk[k] = Pack<__half>::pack(vals[2 * k], vals[2 * k + 1]);
      }
      // the previous TMA store of this warp has read the staging rows
      if (lane == 0) bulk_wait_read_all();
      __syncwarp();
#pragma unroll
      for (int lh = 0; lh < 2; ++lh)
#pragma unroll
        for (int jp = 0; jp < 2; ++jp)
          stmatrix_x4_trans(stm_row[lh] + jp * 16 * 64, pk[lh * 8 + 4 * jp], pk[lh * 8 + 4 * jp + 1],
                            pk[lh * 8 + 4 * jp + 2], pk[lh * 8 + 4 * jp + 3]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        tma_store_5d(map, stg, wq * 32, hq * 32, ch, cc, cb);
        bulk_commit();
      }
    };
    for (int j = 0; j < rg.m && ok; ++j) {
      int strip, c0, c1;
      get_segment(rg, nchunks, j, strip, c0, c1);
      const int b = strip / a.strips_per_batch;
      const int h = (strip % a.strips_per_batch) * HPC + hd;
      if (a.mode == 0) {
        if (c0 == 0) {
          if (a.init != nullptr) {
            const int64_t ib = (int64_t)b * a.init_s[0] + (int64_t)h * a.init_s[1] + (int64_t)pb * a.init_s[2] + nb;
#pragma unroll
            for (int i = 0; i < kP; ++i) S[i] = load_f(a.init, a.init_dtype, ib + (int64_t)fp(i) * a.init_s[2] + fn(i));
          } else {
#pragma unroll
            for (int i = 0; i < kP; ++i) S[i] = 0.0f;
          }
        } else if (a.defer) {
#pragma unroll
          for (int i = 0; i < kP; ++i) S[i] = 0.0f;
        } else {
          const int src = (int)blockIdx.x - 1;
          ok = flag_wait(a.flags + (size_t)src * HPC + hd, epoch_target, wc, kWaitCarry);
          if (!ok) break;
          const float* cin = a.carry + ((size_t)src * HPC + hd) * (kP * kN) + pb * kN + nb;
#pragma unroll
          for (int i = 0; i < kP; ++i) S[i] = __ldcg(cin + fp(i) * kN + fn(i));
        }
      }
      // packed sequences: the running state is dropped where the sequence changes between the
      // ends of two successive chunks (kernels/ssd_state_passing.py:66-76)
      const int32_t* sq = nullptr;
      int seq_prev = 0;
      if constexpr (SEQ) {
        sq = a.seq_idx + (int64_t)b * a.seq_s[0];
        if (c0 > 0) seq_prev = sq[(int64_t)(c0 * L - 1) * a.seq_s[1]];
      }
      for (int c = c0; c < c1 && ok; ++c, ++item) {
        const int buf = item % C::NBUF;
        float decay = 0.0f;
        if (a.mode == 0 && !RAW) {
          decay = fast_exp(__ldg(a.dA + (int64_t)b * a.dA_s[0] + (int64_t)h * a.dA_s[1] + (int64_t)c * a.dA_s[2] + (L - 1)));
          if constexpr (SEQ) {
            const int seq_new = sq[(int64_t)(min((c + 1) * L, a.seqlen) - 1) * a.seq_s[1]];
            if (seq_new != seq_prev) decay = 0.0f;
            seq_prev = seq_new;
          }
        }
        ok = mbar_wait(bar_acc_full(hd, buf), (item / C::NBUF) & 1, wc, kWaitAccFull, 128);
        if (!ok) break;
        tc_fence_after();
        if constexpr (RAW) {
          // written by the scale-vector warp before it released this chunk's factors; the chain of
          // barriers from there to this accumulator orders the read
          decay = fast_exp(reinterpret_cast<const volatile float*>(smem + C::OFF_RING)[(item % C::RING) * HPC + hd]);
        }
        const uint32_t taddr = tmem_base + lane_sel + (hd * C::NBUF + buf) * kP;
#pragma unroll
        for (int hq = 0; hq < 2; ++hq) {
          uint32_t raw_lo[16], raw_hi[16];
          tmem_ld_16x256b_x4(taddr + hq * 32, raw_lo);
          tmem_ld_16x256b_x4(taddr + (16u << 16) + hq * 32, raw_hi);
          tmem_ld_wait();
          if (hq == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty(hd, buf));
          }
          float v[32];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            v[i] = __uint_as_float(raw_lo[i]);
            v[16 + i] = __uint_as_float(raw_hi[i]);
          }
          if (a.states != nullptr) {
            const int64_t so = (int64_t)b * a.states_s[0] + (int64_t)c * a.states_s[1] + (int64_t)h * a.states_s[2];
            store_half(a.states, a.states_dtype, so, a.states_s[3], hq, v, nullptr, 0, 0, 0);
          }
          if (a.mode == 0) {
            float cur[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) cur[i] = S[hq * 32 + i];
            const int64_t oo = (int64_t)b * a.out_s[0] + (int64_t)c * a.out_s[1] + (int64_t)h * a.out_s[2];
            store_half(a.out, OUT32 ? (int)SSD_F32 : a.out_dtype, oo, a.out_s[3], hq, cur, OUT32 ? nullptr : &tmap_out, b,
                       c, h);
#pragma unroll
            for (int i = 0; i < 32; ++i) S[hq * 32 + i] = fmaf(decay, cur[i], v[i]);
          }
        }
      }
      if (!ok || a.mode != 0) continue;
      if (c1 == nchunks) {
        float* fo = a.final_states + (int64_t)b * a.final_s[0] + (int64_t)h * a.final_s[1] + (int64_t)pb * a.final_s[2] + nb;
#pragma unroll
        for (int i = 0; i < kP; ++i) fo[(int64_t)fp(i) * a.final_s[2] + fn(i)] = S[i];
      } else {
        float* co = a.carry + ((size_t)blockIdx.x * HPC + hd) * (kP * kN) + pb * kN + nb;
#pragma unroll
        for (int i = 0; i < kP; ++i) __stcg(co + fp(i) * kN + fn(i), S[i]);
        __threadfence();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_epi_sync(hd));
        ok = mbar_wait(bar_epi_sync(hd), epi_syncs & 1, wc, kWaitGroup);
        ++epi_syncs;
        if (!ok) break;
        // (test hook: with SSD_DEBUG_DROP_CARRY_FLAGS the flag is never published, so that the
        // next CTA's bounded wait runs out)
        if ((tid & 127) == 0 && !(a.debug & SSD_DEBUG_DROP_CARRY_FLAGS))
          st_release_gpu(a.flags + (size_t)blockIdx.x * HPC + hd, epoch_target);
      }
    }
    bulk_wait_all();            // this thread's bulk copies are complete before the CTA retires
  }

  // ================================ teardown ==========================================
  if (ctl[0] != 0) {
    // a wait gave up: give in-flight bulk copies time to land before the CTA retires
    const long long t0 = clock64();
    while (clock64() - t0 < 400000ll) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == C::EPI_WARPS + 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
  if (tid == 0) {
    __threadfence();
    const int prev = atomicAdd(a.status + 2, 1);
    if (prev == (int)gridDim.x - 1) {
      a.status[2] = 0;
      __threadfence();
      reinterpret_cast<volatile int*>(a.status)[1] = (int)epoch_target;
    }
  }
}

// Second pass of the deferred-carry mode.  When strips are longer than a CTA's range, waiting
// for the previous CTA's carry would serialise the CTAs of a strip, so every segment that
// starts inside a strip is computed from a zero state and leaves its segment-final state in
// its CTA's carry slot.  This kernel walks each (batch, head)'s segments in order, keeps the
// state that was missing at each segment start, and adds it to that segment's passed states
// (wherever the accumulated decay has not underflowed to zero) and to the final state.
struct SegFixArgs {
  const float* dA;          // dA_cumsum
  const float* carry;       // [cta][HPC][kP * kN]
  void* out;
  float* final_states;
  int64_t dA_s[3], out_s[4], final_s[3];
  int out_dtype;
  int batch, nheads, nchunks, chunk_size, hpc, strips_per_batch, grid;
  int vec;                  // passed-state rows allow 8-byte (16-bit types) / 16-byte (fp32) accesses
};

// Block = one (batch, head) and one of kSegFixSplit slices of the state; a thread owns four
// consecutive elements of the slice.  For each segment the block builds the per-chunk factors
// exp(sum of the earlier chunks' decays), 1024 chunks at a time, and adds factor * carry to
// its elements of the chunks whose factor is above the cut-off of the output type.
constexpr int kSegFixSplit = kP * kN / (kCarryThreads * kCarryQuad);

__global__ void __launch_bounds__(kCarryThreads) segment_fixup_kernel(const SegFixArgs a) {
  __shared__ __align__(16) float fac[kCarryTile];
  __shared__ float cum_slot;
  const int tid = threadIdx.x;
  const int d0 = blockIdx.z * (kCarryThreads * kCarryQuad) + tid * kCarryQuad;   // first owned element
  const int h = blockIdx.x, b = blockIdx.y;
  const int strip = b * a.strips_per_batch + h / a.hpc;
  const int hd = h % a.hpc;
  const long long total = (long long)a.batch * a.strips_per_batch * a.nchunks;
  const long long first = (long long)strip * a.nchunks;
  const float* dA_last = a.dA + (int64_t)b * a.dA_s[0] + (int64_t)h * a.dA_s[1] + (a.chunk_size - 1);
  const int64_t obase = (int64_t)b * a.out_s[0] + (int64_t)h * a.out_s[2] + (d0 / kN) * a.out_s[3] + (d0 % kN);
  const float cut = carry_cutoff(a.out_dtype);
  float carry[kCarryQuad];
#pragma unroll
  for (int e = 0; e < kCarryQuad; ++e) carry[e] = 0.0f;
  bool have = false;
  int c = 0;
  while (c < a.nchunks) {
    // the CTA of the fused kernel that owned item first + c, and where its range ends
    const long long i = first + c;
    const int k = (int)(((i + 1) * a.grid + total - 1) / total) - 1;
    const long long hi = total * (long long)(k + 1) / a.grid;
    const int seg_end = (int)min((long long)a.nchunks, hi - first);
    float cum = 0.0f;                    // decay accumulated since the segment start
    for (int t0 = c; t0 < seg_end; t0 += kCarryTile) {
      const int tn = min(kCarryTile, seg_end - t0);
      cum = chunk_factors(dA_last + (int64_t)t0 * a.dA_s[2], a.dA_s[2], tn, cum, fac, &cum_slot);
      if (have)
        add_carry_tile_any(a.out, a.out_dtype, a.vec != 0, obase + (int64_t)t0 * a.out_s[1], a.out_s[1], fac, tn, cut,
                           carry, kCarryQuad);
    }
    const float ftot = fast_exp(cum);
    if (seg_end == a.nchunks) {
      if (have) {
        float* fo = a.final_states + (int64_t)b * a.final_s[0] + (int64_t)h * a.final_s[1] +
                    (d0 / kN) * a.final_s[2] + (d0 % kN);
#pragma unroll
        for (int e = 0; e < kCarryQuad; ++e) fo[e] = fmaf(ftot, carry[e], fo[e]);
      }
    } else {
#pragma unroll
      for (int e = 0; e < kCarryQuad; ++e) {
        const float z = a.carry[((size_t)k * a.hpc + hd) * (kP * kN) + d0 + e];
        carry[e] = have ? fmaf(ftot, carry[e], z) : z;
      }
      have = true;
    }
    c = seg_end;
  }
}

// Status / epoch / done words for launches in the states-only mode, which has no workspace.
__device__ int g_states_only_header[64];

// ---- host side ------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// x (b, l, h, p) as a 4-D map with the dimensions ordered (p, l, h, b): a box of 64 x kKT x heads x 1
// lands in shared memory as one (kKT x 64) tile per head, one after the other, each in the
// 128-byte-swizzled arrangement the MMA reads.
int make_x_map(CUtensorMap* map, const void* base, int dtype, int nheads, int seqlen, int batch, const int64_t* stride,
               int heads_per_box) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[4] = {(cuuint64_t)kP, (cuuint64_t)seqlen, (cuuint64_t)nheads, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)stride[1] * 2, (cuuint64_t)stride[2] * 2, (cuuint64_t)stride[0] * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)kKT, (cuuint32_t)heads_per_box, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (x) failed with CUresult %d", (int)r);
  return SSD_OK;
}

// B (b, l, g, n = 128) as a 5-D map (n low 64, l, n high 2, g, b): a box of 64 x kKT x 2 lands as
// two (kKT x 64) tiles, columns 0-63 then 64-127.
int make_B_map(CUtensorMap* map, const void* base, int dtype, int ngroups, int seqlen, int batch, const int64_t* stride) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[5] = {64, (cuuint64_t)seqlen, 2, (cuuint64_t)ngroups, (cuuint64_t)batch};
  const cuuint64_t strides[4] = {(cuuint64_t)stride[1] * 2, 128, (cuuint64_t)stride[2] * 2, (cuuint64_t)stride[0] * 2};
  const cuuint32_t box[5] = {64, (cuuint32_t)kKT, 2, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (B) failed with CUresult %d", (int)r);
  return SSD_OK;
}

// 5-D map over the 16-bit passed states (b, c, h, p, n) with (p, n) dense; box = 32 columns (one
// epilogue warp's dstate quadrant) x 32 rows, 64-byte swizzle.
int make_out_map(CUtensorMap* map, void* base, int dtype, int nheads, int nchunks, int batch, const int64_t* stride) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[5] = {(cuuint64_t)kN, (cuuint64_t)kP, (cuuint64_t)nheads, (cuuint64_t)nchunks, (cuuint64_t)batch};
  const cuuint64_t strides[4] = {(cuuint64_t)stride[3] * 2, (cuuint64_t)stride[2] * 2, (cuuint64_t)stride[1] * 2,
                                 (cuuint64_t)stride[0] * 2};
  const cuuint32_t box[5] = {32, 32, 1, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 5, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (out) failed with CUresult %d", (int)r);
  return SSD_OK;
}

// Raw dt (b, l, h) with contiguous heads as a 3-D map (h, l, b); box = the 16 bytes of heads around
// the CTA's heads x one chunk of positions, no swizzle: a tile [position][16 bytes].
int make_dt_map(CUtensorMap* map, const void* base, int dtype, int nheads, int seqlen, int batch, int64_t stride_l,
                int64_t stride_b, int chunk_size) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const int es = dtype_size(dtype);
  const cuuint64_t dims[3] = {(cuuint64_t)nheads, (cuuint64_t)seqlen, (cuuint64_t)batch};
  const cuuint64_t strides[2] = {(cuuint64_t)stride_l * es, (cuuint64_t)stride_b * es};
  const cuuint32_t box[3] = {(cuuint32_t)(16 / es), (cuuint32_t)chunk_size, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                     : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (dt) failed with CUresult %d", (int)r);
  return SSD_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int num_sms() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (sms[dev] == 0) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    sms[dev] = v > 0 ? v : 1;
  }
  return sms[dev];
}

// How a problem is laid over the GPU: heads per CTA, CTAs, and whether the carry between the CTAs of a
// strip is deferred to a second pass.  The chunks of a strip depend on one another, so cutting a strip
// over several chained CTAs buys no time and costs the hand-offs; a CTA's time per chunk is set by its
// own pipeline, hardly by how many other CTAs run (measured: 2.6 - 3.3 us per 256-position chunk alone,
// 3.2 us with all SMs busy).  Hence, with S = SMs and H = batch x heads:
//   * H <= S: one CTA per (batch, head), whole strips, one head per CTA -- twice as many SMs busy as with
//     head pairs, no carries at all (the Mamba2-130M layer shape: 96 CTAs of 8 chunks, 29 us, where 148
//     ranges of 2.6 chunks of head pairs, chained three or four deep, took 43 us);
//   * H a little above S: one head per CTA, one range per SM (a range then holds a strip or more);
//   * head pairs <= S: one CTA per (batch, head pair), whole strips;
//   * more: head pairs, one contiguous range of (strip, chunk) items per SM, a range boundary inside a
//     strip passes its state through a carry slot (the 2.7B layer shape and everything larger).
//   * Few long strips (a range of 16 chunks or more that is still shorter than a strip): ranges per SM
//     with the carry deferred to segment_fixup_kernel, whatever the above says; never with packed
//     sequences.
// Every layout does the same arithmetic per head: the results carry the same bits.  The states-only mode
// has no recurrence: its items are independent and always cut per SM.
struct FusedPlan {
  int hpc, grid, defer;
};

FusedPlan plan_fused(const ssd_fused_state_params_t& p, int variant, int mode) {
  const ssd_state_inputs_t& in = p.in;
  const long long sms = std::min(num_sms(), FusedWorkspaceLayout::kMaxCtas);
  const long long nchunks = (in.seqlen + in.chunk_size - 1) / in.chunk_size;
  auto cut = [&](int hpc) {
    const long long total = (long long)in.batch * (in.nheads / hpc) * nchunks;
    const long long grid = std::min(total, sms);
    const long long per_cta = grid > 0 ? (total + grid - 1) / grid : 0;
    const int defer = (mode == 0 && nchunks > per_cta && per_cta >= 16 && in.seq_idx == nullptr) ? 1 : 0;
    return FusedPlan{hpc, (int)grid, defer};
  };
  const FusedPlan pairs = cut(variant);
  if (mode != 0 || pairs.defer || (debug_flags() & SSD_DEBUG_CUT_STRIPS)) return pairs;
  const long long heads = (long long)in.batch * in.nheads;
  const FusedPlan singles = cut(1);
  if (heads <= sms) return singles.defer ? pairs : FusedPlan{1, (int)heads, 0};
  if (variant == 2 && heads <= sms + sms / 8 && !singles.defer) return singles;
  if (heads / variant <= sms) return FusedPlan{variant, (int)(heads / variant), 0};
  return pairs;
}

template <typename T, int HPC>
int launch_variant(const ssd_fused_state_params_t& p, int mode, cudaStream_t stream,
                   const ssd_chunk_cumsum_params_t* raw, const FusedPlan& plan) {
  using C = Cfg<HPC>;
  const ssd_state_inputs_t& in = p.in;
  CUtensorMap mx, mB;
  int rc = make_x_map(&mx, in.x, in.in_dtype, in.nheads, in.seqlen, in.batch, in.x_stride, HPC);
  if (rc != SSD_OK) return rc;
  rc = make_B_map(&mB, in.B, in.in_dtype, in.ngroups, in.seqlen, in.batch, in.B_stride);
  if (rc != SSD_OK) return rc;
  CUtensorMap mo = mx;                  // a valid map even where the kernel never touches it
  if (mode == 0 && p.out_dtype != SSD_F32) {
    rc = make_out_map(&mo, p.out, p.out_dtype, in.nheads, (in.seqlen + in.chunk_size - 1) / in.chunk_size, in.batch,
                      p.out_stride);
    if (rc != SSD_OK) return rc;
  }

  FusedArgs a{};
  a.dt = in.dt;
  a.dA = in.dA_cumsum;
  a.init = p.initial_states;
  a.seq_idx = in.seq_idx;
  a.seq_s[0] = in.seq_idx_stride[0];
  a.seq_s[1] = in.seq_idx_stride[1];
  a.out = p.out;
  a.final_states = p.final_states;
  a.states = p.states;
  if (p.workspace != nullptr) {
    uint8_t* ws = static_cast<uint8_t*>(p.workspace);
    a.status = reinterpret_cast<int*>(ws);
    a.flags = reinterpret_cast<uint32_t*>(ws + FusedWorkspaceLayout::kHeaderBytes);
    a.carry = reinterpret_cast<float*>(ws + FusedWorkspaceLayout::kCarryOffset);
  } else {
    SSD_REQUIRE(mode == 1, SSD_ERR_WORKSPACE, "workspace is NULL");
    int* hdr = nullptr;
    SSD_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&hdr), g_states_only_header));
    a.status = hdr;
  }
  for (int i = 0; i < 3; ++i) {
    a.dt_s[i] = in.dt_stride[i];
    a.dA_s[i] = in.dA_stride[i];
    a.init_s[i] = p.init_stride[i];
    a.final_s[i] = p.final_stride[i];
  }
  for (int i = 0; i < 4; ++i) {
    a.out_s[i] = p.out_stride[i];
    a.states_s[i] = p.states_stride[i];
  }
  a.batch = in.batch;
  a.seqlen = in.seqlen;
  a.nheads = in.nheads;
  a.ngroups = in.ngroups;
  a.chunk_size = in.chunk_size;
  a.nchunks = (in.seqlen + in.chunk_size - 1) / in.chunk_size;
  a.strips_per_batch = in.nheads / HPC;
  a.init_dtype = p.init_dtype;
  a.out_dtype = p.out_dtype;
  a.states_dtype = p.states_dtype;
  a.clamp_decay = p.clamp_decay;
  a.mode = mode;
  if (raw != nullptr) {
    a.dt_raw = raw->dt;
    a.A = raw->A;
    a.bias = raw->dt_bias;
    a.raw_s[0] = raw->dt_stride_b;
    a.raw_s[1] = raw->dt_stride_l;
    a.A_stride = raw->A_stride;
    a.bias_stride = raw->bias_stride;
    a.raw_dtype = raw->dt_dtype;
    a.A_dtype = raw->A_dtype;
    a.bias_dtype = raw->bias_dtype;
    a.softplus = raw->dt_softplus;
    a.dt_min = raw->dt_min;
    a.dt_max = raw->dt_max;
  }
  a.debug = debug_flags();
  a.wait_limit = wait_limit_cycles();

  const int grid = plan.grid;
  const bool out32 = p.out_dtype == SSD_F32 && mode == 0;
  const bool seq = in.seq_idx != nullptr;
  SSD_REQUIRE(raw == nullptr || (!seq && mode == 0), SSD_ERR_UNSUPPORTED, "raw dt with seq_idx or in the states-only mode");
  auto kern = out32 ? (seq ? fused_state_kernel<T, HPC, true, true, false> : fused_state_kernel<T, HPC, true, false, false>)
                    : (seq ? fused_state_kernel<T, HPC, false, true, false> : fused_state_kernel<T, HPC, false, false, false>);
  if (raw != nullptr) kern = out32 ? fused_state_kernel<T, HPC, true, false, true> : fused_state_kernel<T, HPC, false, false, true>;
  SSD_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
  // setmaxnreg.inc waits, without a limit, for registers that the other roles give back: the per-role
  // budgets only add up if the kernel was built with exactly the register count they were planned for
  if (C::REBALANCE) {
    static std::mutex mu;
    static const void* checked[16];
    static int nchecked = 0;
    std::lock_guard<std::mutex> lock(mu);
    bool seen = false;
    for (int i = 0; i < nchecked; ++i) seen = seen || checked[i] == reinterpret_cast<const void*>(kern);
    if (!seen) {
      cudaFuncAttributes fa;
      SSD_CUDA_OK(cudaFuncGetAttributes(&fa, kern));
      SSD_REQUIRE(fa.numRegs == C::LAUNCH_REGS, SSD_ERR_CUDA,
                  "fused_state_kernel was built with %d registers per thread, its role budgets need %d", fa.numRegs,
                  C::LAUNCH_REGS);
      if (nchecked < 16) checked[nchecked++] = reinterpret_cast<const void*>(kern);
    }
  }
  // (see plan_fused: a strip longer than a CTA's range would make the CTAs of that strip wait for one
  // another in turn; with long ranges the carry is deferred to a second, small kernel instead)
  a.defer = plan.defer;
  CUtensorMap mdt = mx;                 // a valid map even where the kernel never touches it
  if (raw != nullptr) {
    rc = make_dt_map(&mdt, raw->dt, raw->dt_dtype, in.nheads, in.seqlen, in.batch, raw->dt_stride_l, raw->dt_stride_b,
                     in.chunk_size);
    if (rc != SSD_OK) return rc;
  }
  kern<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(mx, mB, mo, mdt, a);
  SSD_CUDA_OK(cudaGetLastError());
  if (a.defer) {
    SegFixArgs f{};
    f.dA = a.dA;
    f.carry = a.carry;
    f.out = a.out;
    f.final_states = a.final_states;
    for (int i = 0; i < 3; ++i) { f.dA_s[i] = a.dA_s[i]; f.final_s[i] = a.final_s[i]; }
    for (int i = 0; i < 4; ++i) f.out_s[i] = a.out_s[i];
    f.out_dtype = a.out_dtype;
    f.batch = a.batch;
    f.nheads = a.nheads;
    f.nchunks = a.nchunks;
    f.chunk_size = a.chunk_size;
    f.hpc = HPC;
    f.strips_per_batch = a.strips_per_batch;
    f.grid = grid;
    f.vec = reinterpret_cast<uintptr_t>(p.out) % (kCarryQuad * dtype_size(p.out_dtype)) == 0;
    for (int i = 0; i < 4; ++i) f.vec = f.vec && a.out_s[i] % kCarryQuad == 0;
    SSD_REQUIRE(a.nheads <= 65535 && a.batch <= 65535, SSD_ERR_UNSUPPORTED, "fix-up grid too large");
    segment_fixup_kernel<<<dim3(a.nheads, a.batch, kSegFixSplit), 256, 0, stream>>>(f);
    SSD_CUDA_OK(cudaGetLastError());
  }
  return SSD_OK;
}

}  // namespace

int make_rows_map(CUtensorMap* map, const void* base, int dtype, int inner, int heads, int seqlen, int batch,
                  const int64_t* stride /* b, l, h, inner */, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)heads, (cuuint64_t)seqlen, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)stride[2] * 2, (cuuint64_t)stride[1] * 2, (cuuint64_t)stride[0] * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return SSD_OK;
}

// A 16-bit (b, l, h, 64) tensor as the destination of per-warp stores: a box is 32 positions x 32 of
// the 64 inner elements (32 rows of 64 bytes, 64-byte swizzle).  Rows past seqlen are clipped.
int make_rows_store_map(CUtensorMap* map, const void* base, int dtype, int heads, int seqlen, int batch,
                        const int64_t* stride /* b, l, h */) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[4] = {64, (cuuint64_t)heads, (cuuint64_t)seqlen, (cuuint64_t)batch};
  const cuuint64_t strides[3] = {(cuuint64_t)stride[2] * 2, (cuuint64_t)stride[1] * 2, (cuuint64_t)stride[0] * 2};
  const cuuint32_t box[4] = {32, 1, 32, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (row stores) failed with CUresult %d", (int)r);
  return SSD_OK;
}

int make_states_map(CUtensorMap* map, const void* base, int dtype, int nheads, int nchunks, int batch,
                    const int64_t* stride /* b, c, h */) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[5] = {(cuuint64_t)kN, (cuuint64_t)kP, (cuuint64_t)nheads, (cuuint64_t)nchunks, (cuuint64_t)batch};
  const cuuint64_t strides[4] = {(cuuint64_t)kN * 2, (cuuint64_t)stride[2] * 2, (cuuint64_t)stride[1] * 2,
                                 (cuuint64_t)stride[0] * 2};
  const cuuint32_t box[5] = {64, (cuuint32_t)kP, 1, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == SSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(map, dt, 5, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (states) failed with CUresult %d", (int)r);
  return SSD_OK;
}

int make_cb_map(CUtensorMap* map, const void* base, int L, int ngroups, int nchunks, int batch, const int64_t* stride,
                int box_k, int box_m) {
  EncodeTiledFn enc = get_encode_fn();
  SSD_REQUIRE(enc != nullptr, SSD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t dims[5] = {(cuuint64_t)L, (cuuint64_t)L, (cuuint64_t)ngroups, (cuuint64_t)nchunks, (cuuint64_t)batch};
  const cuuint64_t strides[4] = {(cuuint64_t)stride[3] * 4, (cuuint64_t)stride[2] * 4, (cuuint64_t)stride[1] * 4,
                                 (cuuint64_t)stride[0] * 4};
  const cuuint32_t box[5] = {(cuuint32_t)box_k, (cuuint32_t)box_m, 1, 1, 1};
  const cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  SSD_REQUIRE(r == CUDA_SUCCESS, SSD_ERR_CUDA, "cuTensorMapEncodeTiled (cb) failed with CUresult %d", (int)r);
  return SSD_OK;
}

int states_only_wait_status(int* code) {
  int hdr[4] = {0, 0, 0, 0};
  SSD_CUDA_OK(cudaMemcpyFromSymbol(hdr, g_states_only_header, sizeof(hdr)));
  *code = hdr[0];
  if (hdr[0] != 0) {
    const int zero = 0;
    SSD_CUDA_OK(cudaMemcpyToSymbol(g_states_only_header, &zero, sizeof(zero)));
  }
  return SSD_OK;
}

int fused_fast_variant(const ssd_fused_state_params_t& p, const char** why) {
  const ssd_state_inputs_t& in = p.in;
  auto no = [&](const char* m) { if (why) *why = m; return 0; };
  if (in.in_dtype != SSD_BF16 && in.in_dtype != SSD_F16) return no("inputs are not bf16/fp16");
  if (in.headdim != kP || in.dstate != kN) return no("headdim != 64 or dstate != 128");
  if (in.chunk_size % kKT != 0 || in.chunk_size > kMaxL) return no("chunk_size not a multiple of 64 up to 256");
  if (in.x_stride[3] != 1 || in.B_stride[3] != 1) return no("x or B innermost stride != 1");
  if (!aligned16(in.x) || !aligned16(in.B)) return no("x or B not 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    if (in.x_stride[i] % 8 != 0 || in.B_stride[i] % 8 != 0) return no("x or B stride not a multiple of 16 bytes");
  if (in.dt_stride[3] != 1 || in.dA_stride[3] != 1) return no("dt or dA_cumsum innermost stride != 1");
  if (!aligned16(in.dt) || !aligned16(in.dA_cumsum)) return no("dt or dA_cumsum not 16-byte aligned");
  for (int i = 0; i < 3; ++i)
    if (in.dt_stride[i] % 4 != 0 || in.dA_stride[i] % 4 != 0) return no("dt or dA_cumsum stride not a multiple of 16 bytes");
  auto rows_ok = [&](const void* ptr, int dtype, const int64_t* s, int ns) {
    if (ptr == nullptr) return true;
    if (s[ns - 1] != kN) return false;                      // (p, n) contiguous
    if ((reinterpret_cast<uintptr_t>(ptr) & 3) != 0) return false;
    if (dtype != SSD_F32) {                                 // rows leave through 16-byte bulk copies
      if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return false;
      for (int i = 0; i < ns; ++i)
        if (s[i] % 8 != 0) return false;
    }
    return true;
  };
  if (!rows_ok(p.out, p.out_dtype, p.out_stride, 4)) return no("out layout");
  if (!rows_ok(p.states, p.states_dtype, p.states_stride, 4)) return no("states layout");
  if (p.final_states != nullptr && p.final_stride[2] != kN) return no("final_states layout");
  if (p.initial_states != nullptr && p.init_stride[2] != kN) return no("initial_states layout");
  const int ratio = in.nheads / in.ngroups;
  if (why) *why = "";
  return (ratio % 2 == 0) ? 2 : 1;
}

size_t fused_fast_workspace_bytes(const ssd_fused_state_params_t&) {
  return FusedWorkspaceLayout::kCarryOffset +
         (size_t)FusedWorkspaceLayout::kMaxCtas * 2 * kP * kN * sizeof(float);
}


int launch_fused_fast(const ssd_fused_state_params_t& p, int mode, cudaStream_t stream,
                      const ssd_chunk_cumsum_params_t* raw) {
  const int variant = fused_fast_variant(p, nullptr);
  SSD_REQUIRE(variant != 0, SSD_ERR_UNSUPPORTED, "fused tcgen05 kernel cannot take this problem");
  SSD_REQUIRE(raw == nullptr || fused_raw_ok(p, *raw), SSD_ERR_UNSUPPORTED,
              "fused tcgen05 kernel cannot compute the cumsum of this dt itself");
  const bool bf16 = p.in.in_dtype == SSD_BF16;
  const FusedPlan plan = plan_fused(p, variant, mode);
  if (plan.hpc == 2)
    return bf16 ? launch_variant<__nv_bfloat16, 2>(p, mode, stream, raw, plan)
                : launch_variant<__half, 2>(p, mode, stream, raw, plan);
  return bf16 ? launch_variant<__nv_bfloat16, 1>(p, mode, stream, raw, plan)
              : launch_variant<__half, 1>(p, mode, stream, raw, plan);
}

// The RAW variant fetches the raw dt with TMA: heads contiguous, base and the position / batch
// strides multiples of 16 bytes.
bool fused_raw_ok(const ssd_fused_state_params_t& p, const ssd_chunk_cumsum_params_t& raw) {
  const int variant = fused_fast_variant(p, nullptr);
  if (variant == 0 || p.in.seq_idx != nullptr) return false;
  // Inside the persistent kernel the cumsum is one warp's work per CTA, which makes a chunk about 6 %
  // slower than when a stand-alone cumsum kernel has run first; what the single launch saves is the
  // second launch with its ramp and tail, a fixed 5 - 7 us.  Measured on B200 (2.7B shape 120 vs
  // 122 us, 8B-style shape 987 vs 897 us) the two meet at roughly a hundred chunks per CTA; beyond
  // that the two launches are used.  The results are the same bits.
  const long long nchunks = (p.in.seqlen + p.in.chunk_size - 1) / p.in.chunk_size;
  const FusedPlan plan = plan_fused(p, variant, 0);
  const long long total = (long long)p.in.batch * (p.in.nheads / plan.hpc) * nchunks;
  if (plan.grid > 0 && (total + plan.grid - 1) / plan.grid > 96) return false;
  if (raw.dt_stride_h != 1) return false;
  const int es = dtype_size(raw.dt_dtype);
  if (reinterpret_cast<uintptr_t>(raw.dt) % 16 != 0) return false;
  if ((raw.dt_stride_l * es) % 16 != 0 || (raw.dt_stride_b * es) % 16 != 0) return false;
  if (raw.batch != p.in.batch || raw.seqlen != p.in.seqlen || raw.nheads != p.in.nheads ||
      raw.chunk_size != p.in.chunk_size)
    return false;
  return true;
}

}  // namespace ssd
