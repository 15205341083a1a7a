// PyTorch front end of libssd_b200: takes torch tensors, checks devices and dtypes,
// allocates outputs the way the reference's wrappers do (torch.empty on the input's
// device), looks up the current CUDA stream and calls the C ABI (include/ssd_b200.h).
// Shape assertions live in the Python shims so that they raise AssertionError like the
// reference; this layer raises RuntimeError for anything the C ABI rejects.
#include <c10/cuda/CUDAFunctions.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <limits>
#include <map>
#include <mutex>
#include <optional>
#include <utility>
#include <vector>

#include "ssd_b200.h"

namespace {

using torch::Tensor;
using OptTensor = std::optional<Tensor>;

int dtype_code(const Tensor& t, const char* name) {
  switch (t.scalar_type()) {
    case at::kFloat: return SSD_F32;
    case at::kBFloat16: return SSD_BF16;
    case at::kHalf: return SSD_F16;
    default: TORCH_CHECK(false, name, ": dtype ", t.scalar_type(), " is not fp32 / bf16 / fp16");
  }
}
int dtype_code(at::ScalarType st) {
  switch (st) {
    case at::kFloat: return SSD_F32;
    case at::kBFloat16: return SSD_BF16;
    case at::kHalf: return SSD_F16;
    default: TORCH_CHECK(false, "dtype ", st, " is not fp32 / bf16 / fp16");
  }
}

void check_cuda(const Tensor& t, const Tensor& like, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (libssd_b200 has no CPU path)");
  TORCH_CHECK(t.device() == like.device(), name, " is on ", t.device(), ", expected ", like.device());
}

ssd_stream_t current_stream(const Tensor& t) {
  return reinterpret_cast<ssd_stream_t>(c10::cuda::getCurrentCUDAStream(t.device().index()).stream());
}

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == SSD_OK, what, " failed (status ", rc, "): ", ssd_last_error());
}

template <int N>
void copy_strides(int64_t (&dst)[N], const Tensor& t, std::initializer_list<int> dims) {
  int i = 0;
  for (int d : dims) dst[i++] = t.stride(d);
}

Tensor as_int32(const Tensor& seq_idx) {
  return seq_idx.scalar_type() == at::kInt ? seq_idx : seq_idx.to(at::kInt);
}

void fill_state_inputs(ssd_state_inputs_t& in, const Tensor& B, const Tensor& x, const Tensor& dt,
                       const Tensor& dA, const OptTensor& seq_idx, Tensor& seq_idx_hold) {
  check_cuda(B, x, "B");
  check_cuda(dt, x, "dt");
  check_cuda(dA, x, "dA_cumsum");
  TORCH_CHECK(x.dim() == 4 && B.dim() == 4 && dt.dim() == 4 && dA.dim() == 4, "x, B, dt, dA_cumsum must be 4-D");
  TORCH_CHECK(B.scalar_type() == x.scalar_type(), "B and x must have the same dtype");
  TORCH_CHECK(dt.scalar_type() == at::kFloat && dA.scalar_type() == at::kFloat, "dt and dA_cumsum must be fp32");
  in.x = x.data_ptr();
  in.B = B.data_ptr();
  in.dt = dt.data_ptr<float>();
  in.dA_cumsum = dA.data_ptr<float>();
  in.in_dtype = dtype_code(x, "x");
  in.batch = x.size(0);
  in.seqlen = x.size(1);
  in.nheads = x.size(2);
  in.headdim = x.size(3);
  in.ngroups = B.size(2);
  in.dstate = B.size(3);
  in.chunk_size = dt.size(3);
  copy_strides(in.x_stride, x, {0, 1, 2, 3});
  copy_strides(in.B_stride, B, {0, 1, 2, 3});
  copy_strides(in.dt_stride, dt, {0, 1, 2, 3});
  copy_strides(in.dA_stride, dA, {0, 1, 2, 3});
  in.seq_idx = nullptr;
  if (seq_idx.has_value()) {
    check_cuda(*seq_idx, x, "seq_idx");
    seq_idx_hold = as_int32(*seq_idx);
    in.seq_idx = seq_idx_hold.data_ptr<int32_t>();
    in.seq_idx_stride[0] = seq_idx_hold.stride(0);
    in.seq_idx_stride[1] = seq_idx_hold.stride(1);
  }
}

// One zero-initialised workspace per (device, stream), grown on demand.  The fused kernel
// leaves its header consistent after every call, so a buffer is reused without clearing.
// Calls on different streams of one device get different buffers (their kernels may overlap
// and would otherwise share flags and carry slots); calls on one stream are ordered.
struct Workspace {
  Tensor buf;
};
std::mutex g_ws_mutex;
std::map<std::pair<int, void*>, Workspace> g_ws;

Tensor get_workspace(const Tensor& like, size_t bytes, ssd_stream_t stream) {
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  Workspace& w = g_ws[{(int)like.device().index(), (void*)stream}];
  if (!w.buf.defined() || (size_t)w.buf.numel() < bytes) {
    w.buf = torch::zeros({(int64_t)bytes}, torch::dtype(torch::kUInt8).device(like.device()));
    // the fill runs on the current stream, which is the stream the buffer serves
  }
  return w.buf;
}

// ---------------------------------------------------------------------------------------
// Guard bands (debug mode; the stand-in for a memory checker on machines where none can run).
// With debug_set_guard_bytes(n > 0) every output the front end allocates is the middle of a
// larger buffer whose first and last n bytes hold a canary pattern; debug_check_guards()
// synchronises, counts the outputs allocated since the last check whose bands no longer hold
// the pattern (a kernel wrote outside its tensor) and forgets them.  Reads outside a tensor
// are caught from the other side by the tests: inputs placed between bands of NaNs.
constexpr uint8_t kCanary = 0xA5;
std::mutex g_guard_mutex;
int64_t g_guard_bytes = 0;
struct Guarded {
  Tensor buf;
  int64_t payload;
};
std::vector<Guarded> g_guarded;

Tensor alloc_out(at::IntArrayRef sizes, const at::TensorOptions& opts) {
  int64_t guard;
  {
    std::lock_guard<std::mutex> lock(g_guard_mutex);
    guard = g_guard_bytes;
  }
  if (guard == 0) return torch::empty(sizes, opts);
  int64_t numel = 1;
  for (int64_t d : sizes) numel *= d;
  const int64_t payload = numel * (int64_t)c10::elementSize(c10::typeMetaToScalarType(opts.dtype()));
  const int64_t padded = (payload + 255) / 256 * 256;
  Tensor buf = torch::full({guard + padded + guard}, kCanary, torch::dtype(torch::kUInt8).device(opts.device()));
  Tensor out = buf.narrow(0, guard, payload).view(c10::typeMetaToScalarType(opts.dtype())).view(sizes);
  std::lock_guard<std::mutex> lock(g_guard_mutex);
  g_guarded.push_back({buf, payload});
  return out;
}

void debug_set_guard_bytes(int64_t bytes) {
  TORCH_CHECK(bytes >= 0 && bytes % 256 == 0, "guard bytes must be a non-negative multiple of 256");
  std::lock_guard<std::mutex> lock(g_guard_mutex);
  g_guard_bytes = bytes;
}

int64_t debug_check_guards() {
  std::vector<Guarded> list;
  {
    std::lock_guard<std::mutex> lock(g_guard_mutex);
    list.swap(g_guarded);
  }
  int64_t damaged = 0;
  for (Guarded& g : list) {
    c10::cuda::CUDAGuard guard(g.buf.device());
    const int64_t total = g.buf.numel();
    const int64_t band = (total - (g.payload + 255) / 256 * 256) / 2;
    const bool front = g.buf.narrow(0, 0, band).eq(kCanary).all().item<bool>();
    // the bytes between the payload's end and the next multiple of 256 belong to the back band
    const bool back = g.buf.narrow(0, band + g.payload, total - band - g.payload).eq(kCanary).all().item<bool>();
    if (!front || !back) ++damaged;
  }
  return damaged;
}

// ---------------------------------------------------------------------------------------
std::tuple<Tensor, Tensor> chunk_cumsum_fwd(const Tensor& dt, const Tensor& A, int64_t chunk_size,
                                            const OptTensor& dt_bias, bool dt_softplus, double dt_min,
                                            double dt_max) {
  TORCH_CHECK(dt.is_cuda(), "dt must be a CUDA tensor (libssd_b200 has no CPU path)");
  check_cuda(A, dt, "A");
  TORCH_CHECK(dt.dim() == 3 && A.dim() == 1, "dt must be (batch, seqlen, nheads) and A (nheads,)");
  c10::cuda::CUDAGuard guard(dt.device());
  const int64_t batch = dt.size(0), seqlen = dt.size(1), nheads = dt.size(2);
  const int64_t nchunks = (seqlen + chunk_size - 1) / chunk_size;
  auto opts = torch::dtype(torch::kFloat).device(dt.device());
  Tensor dt_out = alloc_out({batch, nheads, nchunks, chunk_size}, opts);
  Tensor dA_cumsum = alloc_out({batch, nheads, nchunks, chunk_size}, opts);
  ssd_chunk_cumsum_params_t p{};
  p.dt = dt.data_ptr();
  p.A = A.data_ptr();
  p.dt_dtype = dtype_code(dt, "dt");
  p.A_dtype = dtype_code(A, "A");
  if (dt_bias.has_value()) {
    check_cuda(*dt_bias, dt, "dt_bias");
    p.dt_bias = dt_bias->data_ptr();
    p.bias_dtype = dtype_code(*dt_bias, "dt_bias");
    p.bias_stride = dt_bias->stride(0);
  }
  p.dt_out = dt_out.data_ptr<float>();
  p.dA_cumsum = dA_cumsum.data_ptr<float>();
  p.batch = batch;
  p.seqlen = seqlen;
  p.nheads = nheads;
  p.chunk_size = chunk_size;
  p.dt_stride_b = dt.stride(0);
  p.dt_stride_l = dt.stride(1);
  p.dt_stride_h = dt.stride(2);
  p.A_stride = A.stride(0);
  p.dt_min = static_cast<float>(dt_min);
  p.dt_max = static_cast<float>(dt_max);
  p.dt_softplus = dt_softplus ? 1 : 0;
  check_rc(ssd_chunk_cumsum_fwd(&p, current_stream(dt)), "ssd_chunk_cumsum_fwd");
  return {dA_cumsum, dt_out};
}

Tensor chunk_state_fwd(const Tensor& B, const Tensor& x, const Tensor& dt, const Tensor& dA_cumsum,
                       const OptTensor& seq_idx, const OptTensor& states_in, bool states_in_fp32) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (libssd_b200 has no CPU path)");
  c10::cuda::CUDAGuard guard(x.device());
  ssd_chunk_state_params_t p{};
  Tensor hold;
  fill_state_inputs(p.in, B, x, dt, dA_cumsum, seq_idx, hold);
  const int64_t nchunks = dt.size(2);
  Tensor states;
  if (states_in.has_value()) {
    states = *states_in;
    check_cuda(states, x, "states");
  } else {
    states = alloc_out({x.size(0), nchunks, x.size(2), x.size(3), B.size(3)},
                          torch::dtype(states_in_fp32 ? at::kFloat : B.scalar_type()).device(x.device()));
  }
  p.states = states.data_ptr();
  p.states_dtype = dtype_code(states, "states");
  copy_strides(p.states_stride, states, {0, 1, 2, 3, 4});
  check_rc(ssd_chunk_state_fwd(&p, current_stream(x)), "ssd_chunk_state_fwd");
  return states;
}

std::tuple<Tensor, Tensor> state_passing_fwd(const Tensor& states, const Tensor& dA_chunk_cumsum,
                                             const OptTensor& initial_states, const OptTensor& seq_idx,
                                             int64_t chunk_size, std::optional<at::ScalarType> out_dtype) {
  TORCH_CHECK(states.is_cuda(), "states must be a CUDA tensor (libssd_b200 has no CPU path)");
  check_cuda(dA_chunk_cumsum, states, "dA_chunk_cumsum");
  TORCH_CHECK(states.dim() == 4 && dA_chunk_cumsum.dim() == 3, "states must be 4-D, dA_chunk_cumsum 3-D");
  c10::cuda::CUDAGuard guard(states.device());
  const int64_t batch = states.size(0), nchunks = states.size(1), nheads = states.size(2), dim = states.size(3);
  const at::ScalarType odt = out_dtype.value_or(states.scalar_type());
  Tensor out = alloc_out({batch, nchunks, nheads, dim}, torch::dtype(odt).device(states.device()));
  Tensor fin = alloc_out({batch, nheads, dim}, torch::dtype(at::kFloat).device(states.device()));
  ssd_state_passing_params_t p{};
  p.states = states.data_ptr();
  p.states_dtype = dtype_code(states, "states");
  p.dA_chunk_cumsum = dA_chunk_cumsum.data_ptr();
  p.dA_dtype = dtype_code(dA_chunk_cumsum, "dA_chunk_cumsum");
  Tensor hold;
  if (initial_states.has_value()) {
    check_cuda(*initial_states, states, "initial_states");
    p.initial_states = initial_states->data_ptr();
    p.init_dtype = dtype_code(*initial_states, "initial_states");
    copy_strides(p.init_stride, *initial_states, {0, 1, 2});
  }
  if (seq_idx.has_value()) {
    check_cuda(*seq_idx, states, "seq_idx");
    hold = as_int32(*seq_idx);
    p.seq_idx = hold.data_ptr<int32_t>();
    p.seq_idx_stride[0] = hold.stride(0);
    p.seq_idx_stride[1] = hold.stride(1);
    p.seqlen = hold.size(1);
    p.chunk_size = chunk_size;
  }
  p.out = out.data_ptr();
  p.out_dtype = dtype_code(odt);
  p.final_states = fin.data_ptr<float>();
  p.batch = batch;
  p.nchunks = nchunks;
  p.nheads = nheads;
  p.dim = dim;
  copy_strides(p.states_stride, states, {0, 1, 2, 3});
  copy_strides(p.dA_stride, dA_chunk_cumsum, {0, 1, 2});
  copy_strides(p.out_stride, out, {0, 1, 2, 3});
  copy_strides(p.final_stride, fin, {0, 1, 2});
  check_rc(ssd_state_passing_fwd(&p, current_stream(states)), "ssd_state_passing_fwd");
  return {out, fin};
}

std::tuple<Tensor, Tensor> fused_state_fwd(const Tensor& B, const Tensor& x, const Tensor& dt,
                                           const Tensor& dA_cumsum, std::optional<at::ScalarType> out_dtype,
                                           const OptTensor& initial_states, const OptTensor& seq_idx,
                                           const OptTensor& states_in, bool states_in_fp32, bool clamp_decay,
                                           bool force_general, const OptTensor& final_out) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (libssd_b200 has no CPU path)");
  c10::cuda::CUDAGuard guard(x.device());
  ssd_fused_state_params_t p{};
  Tensor hold;
  fill_state_inputs(p.in, B, x, dt, dA_cumsum, seq_idx, hold);
  const int64_t batch = x.size(0), nheads = x.size(2), headdim = x.size(3), dstate = B.size(3);
  const int64_t nchunks = dt.size(2);
  // The reference's fused wrappers allocate a full per-chunk states tensor when none is
  // passed and take out_dtype's default from it (kernels/fused_concurrent.py:269-282).
  // Here that intermediate is never materialised unless the caller asks for it.
  const at::ScalarType states_dt = states_in.has_value() ? states_in->scalar_type()
                                                         : (states_in_fp32 ? at::kFloat : B.scalar_type());
  const at::ScalarType odt = out_dtype.value_or(states_dt);
  Tensor out = alloc_out({batch, nchunks, nheads, headdim, dstate}, torch::dtype(odt).device(x.device()));
  // final_out: a caller-owned place for the final states (e.g. a slot of an exchange buffer)
  Tensor fin;
  if (final_out.has_value()) {
    fin = *final_out;
    check_cuda(fin, x, "final_states");
    TORCH_CHECK(fin.scalar_type() == at::kFloat && fin.dim() == 4 && fin.size(0) == batch && fin.size(1) == nheads &&
                    fin.size(2) == headdim && fin.size(3) == dstate && fin.stride(3) == 1,
                "final_states must be fp32 (b, h, p, n) with a contiguous last dimension");
  } else {
    fin = alloc_out({batch, nheads, headdim, dstate}, torch::dtype(at::kFloat).device(x.device()));
  }
  if (initial_states.has_value()) {
    check_cuda(*initial_states, x, "initial_states");
    TORCH_CHECK(initial_states->stride(3) == 1, "initial_states must be contiguous in its last dimension");
    p.initial_states = initial_states->data_ptr();
    p.init_dtype = dtype_code(*initial_states, "initial_states");
    copy_strides(p.init_stride, *initial_states, {0, 1, 2});
  }
  if (states_in.has_value()) {
    check_cuda(*states_in, x, "states");
    TORCH_CHECK(states_in->stride(4) == 1, "states must be contiguous in its last dimension");
    p.states = states_in->data_ptr();
    p.states_dtype = dtype_code(*states_in, "states");
    copy_strides(p.states_stride, *states_in, {0, 1, 2, 3});
  }
  p.out = out.data_ptr();
  p.out_dtype = dtype_code(odt);
  copy_strides(p.out_stride, out, {0, 1, 2, 3});
  p.final_states = fin.data_ptr<float>();
  copy_strides(p.final_stride, fin, {0, 1, 2});
  p.clamp_decay = clamp_decay ? 1 : 0;
  p.force_general = force_general ? 1 : 0;
  const size_t need = ssd_fused_state_workspace_bytes(&p);
  const ssd_stream_t stream = current_stream(x);
  Tensor ws = get_workspace(x, need, stream);
  p.workspace = ws.data_ptr();
  p.workspace_bytes = ws.numel();
  check_rc(ssd_fused_state_fwd(&p, stream), "ssd_fused_state_fwd");
  return {out, fin};
}

// ssd_state_path_fwd: chunk cumsum + fused chunk state / state passing in one call (one launch
// when the tcgen05 kernel takes the problem).  Returns (dA_cumsum, dt_out, out, final_states).
std::tuple<Tensor, Tensor, Tensor, Tensor> state_path_fwd(
    const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& x, int64_t chunk_size,
    std::optional<at::ScalarType> out_dtype, const OptTensor& dt_bias, bool dt_softplus, double dt_min, double dt_max,
    const OptTensor& initial_states, const OptTensor& seq_idx, const OptTensor& states_in, bool states_in_fp32,
    bool clamp_decay, bool force_general, const OptTensor& final_out) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (libssd_b200 has no CPU path)");
  check_cuda(dt, x, "dt");
  check_cuda(A, x, "A");
  check_cuda(B, x, "B");
  TORCH_CHECK(dt.dim() == 3 && A.dim() == 1 && x.dim() == 4 && B.dim() == 4,
              "dt must be (b, l, h), A (h,), x (b, l, h, p), B (b, l, g, n)");
  TORCH_CHECK(B.scalar_type() == x.scalar_type(), "B and x must have the same dtype");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t batch = x.size(0), seqlen = x.size(1), nheads = x.size(2), headdim = x.size(3), dstate = B.size(3);
  TORCH_CHECK(dt.size(0) == batch && dt.size(1) == seqlen && dt.size(2) == nheads && A.size(0) == nheads &&
                  B.size(0) == batch && B.size(1) == seqlen,
              "dt, A, B and x disagree on batch / seqlen / nheads");
  const int64_t nchunks = (seqlen + chunk_size - 1) / chunk_size;
  auto f32 = torch::dtype(torch::kFloat).device(x.device());
  Tensor dt_out = alloc_out({batch, nheads, nchunks, chunk_size}, f32);
  Tensor dA_cumsum = alloc_out({batch, nheads, nchunks, chunk_size}, f32);
  ssd_state_path_params_t p{};
  ssd_chunk_cumsum_params_t& c = p.cumsum;
  c.dt = dt.data_ptr();
  c.A = A.data_ptr();
  c.dt_dtype = dtype_code(dt, "dt");
  c.A_dtype = dtype_code(A, "A");
  if (dt_bias.has_value()) {
    check_cuda(*dt_bias, x, "dt_bias");
    TORCH_CHECK(dt_bias->dim() == 1 && dt_bias->size(0) == nheads, "dt_bias must be (h,)");
    c.dt_bias = dt_bias->data_ptr();
    c.bias_dtype = dtype_code(*dt_bias, "dt_bias");
    c.bias_stride = dt_bias->stride(0);
  }
  c.dt_out = dt_out.data_ptr<float>();
  c.dA_cumsum = dA_cumsum.data_ptr<float>();
  c.batch = batch;
  c.seqlen = seqlen;
  c.nheads = nheads;
  c.chunk_size = chunk_size;
  c.dt_stride_b = dt.stride(0);
  c.dt_stride_l = dt.stride(1);
  c.dt_stride_h = dt.stride(2);
  c.A_stride = A.stride(0);
  c.dt_min = static_cast<float>(dt_min);
  c.dt_max = static_cast<float>(dt_max);
  c.dt_softplus = dt_softplus ? 1 : 0;

  ssd_fused_state_params_t& f = p.fused;
  Tensor hold;
  fill_state_inputs(f.in, B, x, dt_out, dA_cumsum, seq_idx, hold);
  const at::ScalarType states_dt = states_in.has_value() ? states_in->scalar_type()
                                                         : (states_in_fp32 ? at::kFloat : B.scalar_type());
  const at::ScalarType odt = out_dtype.value_or(states_dt);
  Tensor out = alloc_out({batch, nchunks, nheads, headdim, dstate}, torch::dtype(odt).device(x.device()));
  Tensor fin;
  if (final_out.has_value()) {
    fin = *final_out;
    check_cuda(fin, x, "final_states");
    TORCH_CHECK(fin.scalar_type() == at::kFloat && fin.dim() == 4 && fin.size(0) == batch && fin.size(1) == nheads &&
                    fin.size(2) == headdim && fin.size(3) == dstate && fin.stride(3) == 1,
                "final_states must be fp32 (b, h, p, n) with a contiguous last dimension");
  } else {
    fin = alloc_out({batch, nheads, headdim, dstate}, f32);
  }
  if (initial_states.has_value()) {
    check_cuda(*initial_states, x, "initial_states");
    TORCH_CHECK(initial_states->dim() == 4 && initial_states->stride(3) == 1 && initial_states->size(0) == batch &&
                    initial_states->size(1) == nheads && initial_states->size(2) == headdim &&
                    initial_states->size(3) == dstate,
                "initial_states must be (b, h, p, n) with a contiguous last dimension");
    f.initial_states = initial_states->data_ptr();
    f.init_dtype = dtype_code(*initial_states, "initial_states");
    copy_strides(f.init_stride, *initial_states, {0, 1, 2});
  }
  if (states_in.has_value()) {
    check_cuda(*states_in, x, "states");
    TORCH_CHECK(states_in->dim() == 5 && states_in->stride(4) == 1 && states_in->size(0) == batch &&
                    states_in->size(1) == nchunks && states_in->size(2) == nheads && states_in->size(3) == headdim &&
                    states_in->size(4) == dstate,
                "states must be (b, c, h, p, n) with a contiguous last dimension");
    f.states = states_in->data_ptr();
    f.states_dtype = dtype_code(*states_in, "states");
    copy_strides(f.states_stride, *states_in, {0, 1, 2, 3});
  }
  f.out = out.data_ptr();
  f.out_dtype = dtype_code(odt);
  copy_strides(f.out_stride, out, {0, 1, 2, 3});
  f.final_states = fin.data_ptr<float>();
  copy_strides(f.final_stride, fin, {0, 1, 2});
  f.clamp_decay = clamp_decay ? 1 : 0;
  f.force_general = force_general ? 1 : 0;
  const size_t need = ssd_state_path_workspace_bytes(&p);
  const ssd_stream_t stream = current_stream(x);
  Tensor ws = get_workspace(x, need, stream);
  f.workspace = ws.data_ptr();
  f.workspace_bytes = ws.numel();
  check_rc(ssd_state_path_fwd(&p, stream), "ssd_state_path_fwd");
  return {dA_cumsum, dt_out, out, fin};
}

// ssd_fused_state_fwd_static: the caller brings `out` and `final_states`; nothing is
// allocated here or in the library (the scratch is the library's own static device array).
void fused_state_fwd_static(const Tensor& B, const Tensor& x, const Tensor& dt, const Tensor& dA_cumsum,
                            Tensor out, Tensor fin, const OptTensor& initial_states, const OptTensor& states_in,
                            bool clamp_decay, bool force_general) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (libssd_b200 has no CPU path)");
  c10::cuda::CUDAGuard guard(x.device());
  ssd_fused_state_params_t p{};
  Tensor hold;
  fill_state_inputs(p.in, B, x, dt, dA_cumsum, std::nullopt, hold);
  check_cuda(out, x, "out");
  check_cuda(fin, x, "final_states");
  // every caller-provided tensor is written (or read) by the kernels at these exact sizes
  const int64_t batch = x.size(0), nheads = x.size(2), headdim = x.size(3), dstate = B.size(3);
  const int64_t nchunks = dt.size(2);
  TORCH_CHECK(B.size(0) == batch && B.size(1) == x.size(1) && nheads % B.size(2) == 0, "B must be (b, l, g, n) with g dividing h");
  TORCH_CHECK(dt.size(0) == batch && dt.size(1) == nheads && nchunks == (x.size(1) + dt.size(3) - 1) / dt.size(3) &&
                  dA_cumsum.sizes() == dt.sizes(),
              "dt and dA_cumsum must be (b, h, ceil(l / L), L)");
  TORCH_CHECK(out.dim() == 5 && out.stride(4) == 1 && out.size(0) == batch && out.size(1) == nchunks &&
                  out.size(2) == nheads && out.size(3) == headdim && out.size(4) == dstate,
              "out must be (b, c, h, p, n) = (", batch, ", ", nchunks, ", ", nheads, ", ", headdim, ", ", dstate,
              ") with a contiguous last dimension");
  TORCH_CHECK(fin.dim() == 4 && fin.stride(3) == 1 && fin.scalar_type() == at::kFloat && fin.size(0) == batch &&
                  fin.size(1) == nheads && fin.size(2) == headdim && fin.size(3) == dstate,
              "final_states must be fp32 (b, h, p, n) with a contiguous last dimension");
  if (initial_states.has_value()) {
    check_cuda(*initial_states, x, "initial_states");
    TORCH_CHECK(initial_states->dim() == 4 && initial_states->stride(3) == 1 && initial_states->size(0) == batch &&
                    initial_states->size(1) == nheads && initial_states->size(2) == headdim &&
                    initial_states->size(3) == dstate,
                "initial_states must be (b, h, p, n) with a contiguous last dimension");
    p.initial_states = initial_states->data_ptr();
    p.init_dtype = dtype_code(*initial_states, "initial_states");
    copy_strides(p.init_stride, *initial_states, {0, 1, 2});
  }
  if (states_in.has_value()) {
    check_cuda(*states_in, x, "states");
    TORCH_CHECK(states_in->dim() == 5 && states_in->stride(4) == 1 && states_in->size(0) == batch &&
                    states_in->size(1) == nchunks && states_in->size(2) == nheads && states_in->size(3) == headdim &&
                    states_in->size(4) == dstate,
                "states must be (b, c, h, p, n) with a contiguous last dimension");
    p.states = states_in->data_ptr();
    p.states_dtype = dtype_code(*states_in, "states");
    copy_strides(p.states_stride, *states_in, {0, 1, 2, 3});
  }
  p.out = out.data_ptr();
  p.out_dtype = dtype_code(out, "out");
  copy_strides(p.out_stride, out, {0, 1, 2, 3});
  p.final_states = fin.data_ptr<float>();
  copy_strides(p.final_stride, fin, {0, 1, 2});
  p.clamp_decay = clamp_decay ? 1 : 0;
  p.force_general = force_general ? 1 : 0;
  check_rc(ssd_fused_state_fwd_static(&p, current_stream(x)), "ssd_fused_state_fwd_static");
}

// Adds the state carried in from the earlier sequence slices (ssd_seqpar_fixup).  `out` and
// `final_states` are updated in place.
void seqpar_fixup(const Tensor& Z_all, const Tensor& logP_all, int64_t rank, const Tensor& dA_chunk_last, Tensor out,
                  Tensor final_states) {
  TORCH_CHECK(out.is_cuda(), "out must be a CUDA tensor (libssd_b200 has no CPU path)");
  check_cuda(Z_all, out, "Z_all");
  check_cuda(logP_all, out, "logP_all");
  check_cuda(dA_chunk_last, out, "dA_chunk_last");
  check_cuda(final_states, out, "final_states");
  TORCH_CHECK(Z_all.dim() == 5 && logP_all.dim() == 3 && Z_all[0].is_contiguous() && logP_all[0].is_contiguous(),
              "gathered Z (world, b, h, p, n) and logP (world, b, h) must be dense per rank");
  TORCH_CHECK(Z_all.scalar_type() == at::kFloat && logP_all.scalar_type() == at::kFloat &&
                  dA_chunk_last.scalar_type() == at::kFloat && final_states.scalar_type() == at::kFloat,
              "Z, logP, dA_chunk_last and final_states must be fp32");
  TORCH_CHECK(out.dim() == 5 && out.stride(4) == 1 && out.stride(3) == out.size(4), "out must be (b, c, h, p, n) with dense (p, n)");
  TORCH_CHECK(final_states.dim() == 4 && final_states.stride(3) == 1 && final_states.stride(2) == final_states.size(3),
              "final_states must be (b, h, p, n) with dense (p, n)");
  TORCH_CHECK(final_states.size(0) == out.size(0) && final_states.size(1) == out.size(2) &&
                  final_states.size(2) == out.size(3) && final_states.size(3) == out.size(4),
              "final_states must be (b, h, p, n) of the same b, h, p, n as out (b, c, h, p, n)");
  TORCH_CHECK(rank >= 0 && rank < Z_all.size(0), "rank ", rank, " outside world ", Z_all.size(0));
  c10::cuda::CUDAGuard guard(out.device());
  ssd_seqpar_fixup_params_t p{};
  p.Z_all = Z_all.data_ptr<float>();
  p.logP_all = logP_all.data_ptr<float>();
  p.dA_chunk_last = dA_chunk_last.data_ptr<float>();
  p.out = out.data_ptr();
  p.final_states = final_states.data_ptr<float>();
  p.out_dtype = dtype_code(out, "out");
  p.world = Z_all.size(0);
  p.Z_rank_stride = Z_all.stride(0);
  p.logP_rank_stride = logP_all.stride(0);
  p.rank = rank;
  p.batch = out.size(0);
  p.nchunks = out.size(1);
  p.nheads = out.size(2);
  p.dim = out.size(3) * out.size(4);
  TORCH_CHECK(Z_all.numel() == (int64_t)p.world * p.batch * p.nheads * p.dim, "Z_all has the wrong size");
  TORCH_CHECK(logP_all.numel() == (int64_t)p.world * p.batch * p.nheads, "logP_all has the wrong size");
  TORCH_CHECK(dA_chunk_last.dim() == 3 && dA_chunk_last.size(0) == p.batch && dA_chunk_last.size(1) == p.nheads &&
                  dA_chunk_last.size(2) == p.nchunks, "dA_chunk_last must be (b, h, c)");
  copy_strides(p.dA_stride, dA_chunk_last, {0, 1, 2});
  copy_strides(p.out_stride, out, {0, 1, 2});
  copy_strides(p.final_stride, final_states, {0, 1});
  check_rc(ssd_seqpar_fixup(&p, current_stream(out)), "ssd_seqpar_fixup");
}

// Synchronises the current stream and reports whether a device-side wait of any call made so
// far on this device gave up: the cached workspaces of the fused entry point (a workspace whose
// status word is set is cleared for reuse before the error is raised), the static scratch of
// fused_state_fwd_static, and the status words the library keeps for its other tcgen05 kernels.
void check_status(const Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  std::vector<Tensor> bufs;
  {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    for (auto& kv : g_ws)
      if (kv.first.first == (int)like.device().index() && kv.second.buf.defined()) bufs.push_back(kv.second.buf);
  }
  const ssd_stream_t stream = current_stream(like);
  if (bufs.size() > 1) c10::cuda::device_synchronize();     // other streams' calls as well
  for (Tensor& ws : bufs) {
    const int rc = ssd_check_status(ws.data_ptr(), stream);
    if (rc == SSD_ERR_TIMEOUT) ws.zero_();
    check_rc(rc, "ssd_check_status");
  }
  check_rc(ssd_check_status(nullptr, stream), "ssd_check_status (static scratch)");
}

Tensor bmm_chunk_fwd(const Tensor& a, const Tensor& b, int64_t chunk_size, const OptTensor& seq_idx, bool causal,
                     std::optional<at::ScalarType> output_dtype) {
  TORCH_CHECK(a.is_cuda(), "a must be a CUDA tensor (libssd_b200 has no CPU path)");
  check_cuda(b, a, "b");
  TORCH_CHECK(a.dim() == 3 || a.dim() == 4, "a must be (batch, seqlen, k) or (batch, seqlen, ngroups, k)");
  TORCH_CHECK(a.scalar_type() == b.scalar_type(), "a and b must have the same dtype");
  c10::cuda::CUDAGuard guard(a.device());
  const bool has_groups = a.dim() == 4;
  const Tensor a4 = has_groups ? a : a.unsqueeze(2);
  const Tensor b4 = has_groups ? b : b.unsqueeze(2);
  const int64_t batch = a4.size(0), seqlen = a4.size(1), ngroups = a4.size(2), k = a4.size(3);
  const int64_t nchunks = (seqlen + chunk_size - 1) / chunk_size;
  const at::ScalarType odt = output_dtype.value_or(a.scalar_type());
  Tensor out = alloc_out({batch, nchunks, ngroups, chunk_size, chunk_size}, torch::dtype(odt).device(a.device()));
  ssd_bmm_chunk_params_t p{};
  p.a = a4.data_ptr();
  p.b = b4.data_ptr();
  p.out = out.data_ptr();
  p.in_dtype = dtype_code(a, "a");
  p.out_dtype = dtype_code(odt);
  p.batch = batch;
  p.seqlen = seqlen;
  p.ngroups = ngroups;
  p.k = k;
  p.chunk_size = chunk_size;
  p.causal = causal ? 1 : 0;
  copy_strides(p.a_stride, a4, {0, 1, 2, 3});
  copy_strides(p.b_stride, b4, {0, 1, 2, 3});
  copy_strides(p.out_stride, out, {0, 1, 2, 3, 4});
  Tensor hold;
  if (seq_idx.has_value()) {
    check_cuda(*seq_idx, a, "seq_idx");
    hold = as_int32(*seq_idx);
    p.seq_idx = hold.data_ptr<int32_t>();
    p.seq_idx_stride[0] = hold.stride(0);
    p.seq_idx_stride[1] = hold.stride(1);
  }
  check_rc(ssd_bmm_chunk_fwd(&p, current_stream(a)), "ssd_bmm_chunk_fwd");
  return has_groups ? out : out.squeeze(2);
}

std::tuple<Tensor, OptTensor> chunk_scan_fwd(const Tensor& cb, const Tensor& x, const Tensor& dt,
                                             const Tensor& dA_cumsum, const Tensor& C, const Tensor& states,
                                             const OptTensor& D, const OptTensor& z, const OptTensor& seq_idx) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (libssd_b200 has no CPU path)");
  for (const Tensor* t : {&cb, &dt, &dA_cumsum, &C, &states}) check_cuda(*t, x, "chunk_scan input");
  TORCH_CHECK(C.scalar_type() == x.scalar_type(), "C and x must have the same dtype");
  TORCH_CHECK(dt.scalar_type() == at::kFloat && dA_cumsum.scalar_type() == at::kFloat, "dt and dA_cumsum must be fp32");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = alloc_out({x.size(0), x.size(1), x.size(2), x.size(3)}, x.options());
  OptTensor out_x;
  ssd_chunk_scan_params_t p{};
  p.cb = cb.data_ptr();
  p.x = x.data_ptr();
  p.dt = dt.data_ptr<float>();
  p.dA_cumsum = dA_cumsum.data_ptr<float>();
  p.C = C.data_ptr();
  p.states = states.data_ptr();
  p.out = out.data_ptr();
  p.cb_dtype = dtype_code(cb, "cb");
  p.in_dtype = dtype_code(x, "x");
  p.states_dtype = dtype_code(states, "states");
  p.batch = x.size(0);
  p.seqlen = x.size(1);
  p.nheads = x.size(2);
  p.headdim = x.size(3);
  p.ngroups = C.size(2);
  p.dstate = C.size(3);
  p.chunk_size = dt.size(3);
  copy_strides(p.cb_stride, cb, {0, 1, 2, 3, 4});
  copy_strides(p.x_stride, x, {0, 1, 2, 3});
  copy_strides(p.out_stride, out, {0, 1, 2, 3});
  copy_strides(p.dt_stride, dt, {0, 1, 2, 3});
  copy_strides(p.dA_stride, dA_cumsum, {0, 1, 2, 3});
  copy_strides(p.C_stride, C, {0, 1, 2, 3});
  copy_strides(p.states_stride, states, {0, 1, 2, 3, 4});
  Tensor Dh, zh, sh;
  if (D.has_value()) {
    check_cuda(*D, x, "D");
    Dh = D->dim() == 2 && D->stride(1) != 1 ? D->contiguous() : *D;
    p.D = Dh.data_ptr();
    p.D_dtype = dtype_code(Dh, "D");
    p.D_has_hdim = Dh.dim() == 2 ? 1 : 0;
    p.D_stride = Dh.stride(0);
  }
  if (z.has_value()) {
    check_cuda(*z, x, "z");
    TORCH_CHECK(z->scalar_type() == x.scalar_type(), "z and x must have the same dtype");
    zh = *z;
    p.z = zh.data_ptr();
    copy_strides(p.z_stride, zh, {0, 1, 2, 3});
    out_x = alloc_out(out.sizes(), out.options());
    p.out_x = out_x->data_ptr();
  }
  if (seq_idx.has_value()) {
    check_cuda(*seq_idx, x, "seq_idx");
    sh = as_int32(*seq_idx);
    p.seq_idx = sh.data_ptr<int32_t>();
    p.seq_idx_stride[0] = sh.stride(0);
    p.seq_idx_stride[1] = sh.stride(1);
  }
  check_rc(ssd_chunk_scan_fwd(&p, current_stream(x)), "ssd_chunk_scan_fwd");
  return {out, out_x};
}

// Chunk bmm + chunk scan behind one call: (out, out_x) from C, B instead of a cb tensor.  One
// kernel where the tcgen05 kernel takes the problem (cb never exists in memory); otherwise
// ssd_bmm_chunk_fwd into a temporary and ssd_chunk_scan_fwd.
std::tuple<Tensor, OptTensor> chunk_scan_combined_fwd(const Tensor& C, const Tensor& B, const Tensor& x, const Tensor& dt,
                                                     const Tensor& dA_cumsum, const Tensor& states, const OptTensor& D,
                                                     const OptTensor& z, const OptTensor& seq_idx) {
  TORCH_CHECK(x.is_cuda(), "x must be a CUDA tensor (libssd_b200 has no CPU path)");
  for (const Tensor* t : {&B, &dt, &dA_cumsum, &C, &states}) check_cuda(*t, x, "chunk_scan input");
  TORCH_CHECK(C.scalar_type() == x.scalar_type() && B.scalar_type() == x.scalar_type(), "B, C and x must have the same dtype");
  TORCH_CHECK(dt.scalar_type() == at::kFloat && dA_cumsum.scalar_type() == at::kFloat, "dt and dA_cumsum must be fp32");
  TORCH_CHECK(x.dim() == 4 && B.dim() == 4 && C.dim() == 4 && dt.dim() == 4 && states.dim() == 5 && B.sizes() == C.sizes(),
              "x (b, l, h, p), B and C (b, l, g, n), dt (b, h, c, L), states (b, c, h, p, n)");
  const int64_t chunk_size = dt.size(3);
  {
    c10::cuda::CUDAGuard guard(x.device());
    Tensor out = alloc_out({x.size(0), x.size(1), x.size(2), x.size(3)}, x.options());
    OptTensor out_x;
    ssd_chunk_scan_fused_params_t f{};
    ssd_chunk_scan_params_t& p = f.scan;
    p.x = x.data_ptr();
    p.dt = dt.data_ptr<float>();
    p.dA_cumsum = dA_cumsum.data_ptr<float>();
    p.C = C.data_ptr();
    p.states = states.data_ptr();
    p.out = out.data_ptr();
    p.cb_dtype = SSD_F32;
    p.in_dtype = dtype_code(x, "x");
    p.states_dtype = dtype_code(states, "states");
    p.batch = x.size(0);
    p.seqlen = x.size(1);
    p.nheads = x.size(2);
    p.headdim = x.size(3);
    p.ngroups = C.size(2);
    p.dstate = C.size(3);
    p.chunk_size = chunk_size;
    copy_strides(p.x_stride, x, {0, 1, 2, 3});
    copy_strides(p.out_stride, out, {0, 1, 2, 3});
    copy_strides(p.dt_stride, dt, {0, 1, 2, 3});
    copy_strides(p.dA_stride, dA_cumsum, {0, 1, 2, 3});
    copy_strides(p.C_stride, C, {0, 1, 2, 3});
    copy_strides(p.states_stride, states, {0, 1, 2, 3, 4});
    f.B = B.data_ptr();
    copy_strides(f.B_stride, B, {0, 1, 2, 3});
    Tensor Dh, zh;
    if (D.has_value()) {
      check_cuda(*D, x, "D");
      Dh = D->dim() == 2 && D->stride(1) != 1 ? D->contiguous() : *D;
      p.D = Dh.data_ptr();
      p.D_dtype = dtype_code(Dh, "D");
      p.D_has_hdim = Dh.dim() == 2 ? 1 : 0;
      p.D_stride = Dh.stride(0);
    }
    if (z.has_value()) {
      check_cuda(*z, x, "z");
      TORCH_CHECK(z->scalar_type() == x.scalar_type(), "z and x must have the same dtype");
      zh = *z;
      p.z = zh.data_ptr();
      copy_strides(p.z_stride, zh, {0, 1, 2, 3});
      out_x = alloc_out(out.sizes(), out.options());
      p.out_x = out_x->data_ptr();
    }
    Tensor sih;
    if (seq_idx.has_value()) {
      check_cuda(*seq_idx, x, "seq_idx");
      TORCH_CHECK(seq_idx->dim() == 2, "seq_idx must be (batch, seqlen)");
      sih = as_int32(*seq_idx);
      p.seq_idx = sih.data_ptr<int32_t>();
      p.seq_idx_stride[0] = sih.stride(0);
      p.seq_idx_stride[1] = sih.stride(1);
    }
    const int rc = ssd_chunk_scan_fused_fwd(&f, current_stream(x));
    if (rc == SSD_OK) return {out, out_x};
    TORCH_CHECK(rc == SSD_ERR_UNSUPPORTED, "ssd_chunk_scan_fused_fwd failed (status ", rc, "): ", ssd_last_error());
  }
  Tensor cb = bmm_chunk_fwd(C, B, chunk_size, seq_idx, false, at::kFloat);
  return chunk_scan_fwd(cb, x, dt, dA_cumsum, C, states, D, z, seq_idx);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "PyTorch front end of libssd_b200 (Mamba2 SSD forward hot path on sm_100a)";
  m.def("abi_version", []() { return ssd_abi_version(); });
  m.def("chunk_cumsum_fwd", &chunk_cumsum_fwd, py::arg("dt"), py::arg("A"), py::arg("chunk_size"),
        py::arg("dt_bias") = py::none(), py::arg("dt_softplus") = false, py::arg("dt_min") = 0.0,
        py::arg("dt_max") = std::numeric_limits<double>::infinity());
  m.def("chunk_state_fwd", &chunk_state_fwd, py::arg("B"), py::arg("x"), py::arg("dt"), py::arg("dA_cumsum"),
        py::arg("seq_idx") = py::none(), py::arg("states") = py::none(), py::arg("states_in_fp32") = true);
  m.def("state_passing_fwd", &state_passing_fwd, py::arg("states"), py::arg("dA_chunk_cumsum"),
        py::arg("initial_states") = py::none(), py::arg("seq_idx") = py::none(), py::arg("chunk_size") = 0,
        py::arg("out_dtype") = py::none());
  m.def("fused_state_fwd", &fused_state_fwd, py::arg("B"), py::arg("x"), py::arg("dt"), py::arg("dA_cumsum"),
        py::arg("out_dtype") = py::none(), py::arg("initial_states") = py::none(), py::arg("seq_idx") = py::none(),
        py::arg("states") = py::none(), py::arg("states_in_fp32") = true, py::arg("clamp_decay") = true,
        py::arg("force_general") = false, py::arg("final_states") = py::none());
  m.def("state_path_fwd", &state_path_fwd, py::arg("dt"), py::arg("A"), py::arg("B"), py::arg("x"), py::arg("chunk_size"),
        py::arg("out_dtype") = py::none(), py::arg("dt_bias") = py::none(), py::arg("dt_softplus") = false,
        py::arg("dt_min") = 0.0, py::arg("dt_max") = std::numeric_limits<double>::infinity(),
        py::arg("initial_states") = py::none(), py::arg("seq_idx") = py::none(), py::arg("states") = py::none(),
        py::arg("states_in_fp32") = true, py::arg("clamp_decay") = true, py::arg("force_general") = false,
        py::arg("final_states") = py::none());
  m.def("fused_state_fwd_static", &fused_state_fwd_static, py::arg("B"), py::arg("x"), py::arg("dt"),
        py::arg("dA_cumsum"), py::arg("out"), py::arg("final_states"), py::arg("initial_states") = py::none(),
        py::arg("states") = py::none(), py::arg("clamp_decay") = true, py::arg("force_general") = false);
  m.def("static_scratch_bytes", []() { return ssd_static_scratch_bytes(); });
  m.def("seqpar_fixup", &seqpar_fixup, py::arg("Z_all"), py::arg("logP_all"), py::arg("rank"),
        py::arg("dA_chunk_last"), py::arg("out"), py::arg("final_states"));
  m.def("check_status", &check_status, py::arg("like"));
  m.def("debug_set_wait_limit_cycles", [](int64_t cycles) { ssd_debug_set_wait_limit_cycles((long long)cycles); });
  m.def("debug_set_flags", [](int64_t flags) { ssd_debug_set_flags((int)flags); });
  m.def("debug_set_guard_bytes", &debug_set_guard_bytes, py::arg("bytes"));
  m.def("debug_check_guards", &debug_check_guards);
  m.def("bmm_chunk_fwd", &bmm_chunk_fwd, py::arg("a"), py::arg("b"), py::arg("chunk_size"),
        py::arg("seq_idx") = py::none(), py::arg("causal") = false, py::arg("output_dtype") = py::none());
  m.def("chunk_scan_combined_fwd", &chunk_scan_combined_fwd, py::arg("C"), py::arg("B"), py::arg("x"), py::arg("dt"),
        py::arg("dA_cumsum"), py::arg("states"), py::arg("D") = py::none(), py::arg("z") = py::none(),
        py::arg("seq_idx") = py::none());
  m.def("chunk_scan_fwd", &chunk_scan_fwd, py::arg("cb"), py::arg("x"), py::arg("dt"), py::arg("dA_cumsum"),
        py::arg("C"), py::arg("states"), py::arg("D") = py::none(), py::arg("z") = py::none(),
        py::arg("seq_idx") = py::none());
}
