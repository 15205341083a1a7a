"""Out-of-bounds accesses, looked for without a memory checker.

The reference has no sanitizer run and the pool's GPUs offer none, so the kernels' index
arithmetic is checked from the outside on ragged shapes (a last chunk that is cut short, odd
batch and head counts), on both the tcgen05 route and the plain kernels:

* every INPUT lies between two bands of NaNs (all-ones bit patterns for integers) inside a larger
  allocation: a kernel that reads before or behind a tensor and uses the value poisons its outputs;
* every OUTPUT the front end allocates lies between two bands of a canary byte pattern
  (`debug_set_guard_bytes`): a kernel that writes before or behind a tensor damages a band, which
  `debug_check_guards` counts;
* the results must be bit-identical to the same calls on ordinary tensors.

Nothing here can fault: the bands are part of the test's own allocations."""
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

BAND = 1 << 16          # bytes on either side of every tensor


def banded(t):
    """A copy of `t` in the middle of a larger allocation filled with NaNs / all-ones."""
    if t is None:
        return None
    es = t.element_size()
    pad = BAND // es
    n = t.numel()
    if t.dtype.is_floating_point:
        buf = torch.full((pad + n + pad,), float("nan"), dtype=t.dtype, device=t.device)
    else:
        buf = torch.full((pad + n + pad,), -1, dtype=t.dtype, device=t.device)
    view = buf[pad:pad + n].view(t.shape)
    view.copy_(t)
    assert view.data_ptr() % 16 == 0
    return view


def _finite(*tensors):
    return all(t is None or bool(torch.isfinite(t.float()).all()) for t in tensors)


def _same(a, b):
    if a is None or b is None:
        return a is None and b is None
    return torch.equal(a, b)


def _pipeline(d, L, out_dtype, init, with_z):
    """Every entry point of the path once; returns all outputs in a flat list."""
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd, _chunk_scan_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd, _chunk_state_fwd
    from mamba_fused_minimal_b200.kernels.ssd_state_passing import _state_passing_fwd
    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd
    dA, dt = _chunk_cumsum_fwd(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    states = _chunk_state_fwd(d["B"], d["x"], dt, dA, states_in_fp32=True)
    b, c, h, p, n = states.shape
    passed, fin = _state_passing_fwd(states.view(b, c, h, p * n), dA[:, :, :, -1],
                                     initial_states=None if init is None else init.view(b, h, p * n),
                                     chunk_size=L, out_dtype=out_dtype)
    out_f, fin_f = fused(d["B"], d["x"], dt, dA, out_dtype, initial_states=init)
    dA2, dt2, out_p, fin_p = _state_path_fwd(d["dt"], d["A"], d["B"], d["x"], L, out_dtype, dt_bias=d["dt_bias"],
                                             dt_softplus=True, initial_states=init)
    cb = _bmm_chunk_fwd(d["C"], d["B"], L, output_dtype=torch.float32)
    z = d["z"] if with_z else None
    y, yx = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], out_f, D=d["D"], z=z)
    y2, yx2 = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt, dA, out_f, D=d["D"], z=z)
    torch.cuda.synchronize()
    return [dA, dt, states, passed, fin, out_f, fin_f, dA2, dt2, out_p, fin_p, cb, y, yx, y2, yx2]


CASES = [
    # batch, seqlen, heads, headdim, groups, dstate, chunk, dtype, z
    pytest.param((3, 868, 6, 64, 1, 128, 256, torch.bfloat16, False), id="tcgen05_ragged_last_chunk"),
    pytest.param((1, 1024, 10, 64, 2, 128, 128, torch.bfloat16, False), id="tcgen05_whole_chunks_odd_head_pairs"),
    pytest.param((2, 200, 3, 64, 1, 128, 64, torch.float16, False), id="tcgen05_one_head_per_cta"),
    pytest.param((2, 330, 4, 32, 2, 16, 64, torch.float32, True), id="plain_kernels_ragged_with_gate"),
    pytest.param((1, 77, 5, 48, 5, 24, 32, torch.float32, False), id="plain_kernels_odd_sizes"),
]


@pytest.mark.parametrize("case", CASES)
def test_inputs_between_nan_bands_and_outputs_between_canaries(cuda_device, case):
    from mamba_fused_minimal_b200._ext import C
    b, l, h, p, g, n, L, dtype, with_z = case
    inp = O.make_inputs(b, l, h, p, g, n, dtype=dtype, seed=77)
    gen = torch.Generator().manual_seed(78)
    inp["z"] = torch.randn(b, l, h, p, generator=gen).to(dtype)
    init = torch.randn(b, h, p, n, generator=gen).to(cuda_device)
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    ref = _pipeline(d, L, dtype, init, with_z)
    C.check_status(d["x"])
    assert _finite(*ref)
    guarded = {k: banded(v) for k, v in d.items()}
    try:
        C.debug_set_guard_bytes(BAND)
        got = _pipeline(guarded, L, dtype, banded(init), with_z)
        C.check_status(d["x"])
        damaged = C.debug_check_guards()
    finally:
        C.debug_set_guard_bytes(0)
        C.debug_check_guards()
    assert damaged == 0, f"{damaged} outputs were written outside their bounds"
    assert _finite(*got), "an output depends on bytes outside an input tensor"
    for i, (a, r) in enumerate(zip(got, ref)):
        assert _same(a, r), f"output {i} differs between banded and ordinary tensors"


def test_a_damaged_band_is_counted(cuda_device):
    """The checker itself: a byte written behind an output (by the test, inside the test's own
    allocation) must be reported, an untouched allocation must not."""
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    inp = O.make_inputs(1, 128, 4, 64, 1, 128, dtype=torch.bfloat16, seed=5)
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    try:
        C.debug_set_guard_bytes(4096)
        dA, dt = _chunk_cumsum_fwd(d["dt"], d["A"], 64)
        assert C.debug_check_guards() == 0
        dA, dt = _chunk_cumsum_fwd(d["dt"], d["A"], 64)
        whole = torch.empty(0, dtype=torch.uint8, device=cuda_device).set_(dA.untyped_storage())
        assert whole.numel() >= dA.numel() * 4 + 2 * 4096
        behind = dA.storage_offset() * 4 + dA.numel() * 4       # first byte after the tensor
        assert int(whole[behind]) == 0xA5
        whole[behind] = 0
        assert C.debug_check_guards() == 1
        assert C.debug_check_guards() == 0                      # the list was forgotten
    finally:
        C.debug_set_guard_bytes(0)
        C.debug_check_guards()
