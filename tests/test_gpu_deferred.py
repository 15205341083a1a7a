"""The deferred-carry branch of the fused state kernel: few, long strips.

When a (batch, head-pair) strip is longer than one CTA's range of work items and that range
is at least 16 chunks, the kernel scans every segment that starts inside a strip from a zero
state and a second kernel (segment fix-up) adds the carried state afterwards.  This is the
branch a single long sequence takes (one 1 M-token sequence with 80 heads is 40 strips of
4096 chunks on 148 SMs).  The cases here force it on small tensors and compare with

  * the CPU oracle over the whole tensor (the recurrence of kernels/ssd_state_passing.py:61-84
    of the reference), at the tolerances of the other parity tests;
  * the plain-kernel route of this library (no segments, no second pass);
  * bit-exact properties of the second pass: with 16-bit passed states a chunk whose
    accumulated decay factor since the cut is at most 2^-24 is left exactly as the zero-carry
    scan wrote it; with fp32 passed states every chunk with a non-zero factor is touched.

Decay rates are set per case: with the benchmark's A in [-16, -1] a carry dies inside one
chunk and the second pass would have nothing to do, so the slow cases use A close to zero,
which keeps a carry alive across several segments (the composition of segment carries)."""
import math

import pytest
import torch

from conftest import rel_err
from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu


def _fns():
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd as fused
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    return fused, _chunk_cumsum_fwd


def _inputs(b, l, h, g, seed, a_lo, a_hi, dtype=torch.bfloat16):
    inp = O.make_inputs(b, l, h, 64, g, 128, dtype=dtype, seed=seed)
    gen = torch.Generator().manual_seed(seed + 1000)
    inp["A"] = -(a_lo + (a_hi - a_lo) * torch.rand(h, generator=gen))
    return inp


def _segments(total, nchunks, grid):
    """Chunk ranges [c0, c1) per strip as the kernel cuts them: CTA k owns work items
    [total * k / grid, total * (k + 1) / grid) of the strip-major item order."""
    cuts = sorted({total * k // grid for k in range(grid + 1)})
    segs = {}
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        while lo < hi:
            strip = lo // nchunks
            end = min(hi, (strip + 1) * nchunks)
            segs.setdefault(strip, []).append((lo - strip * nchunks, end - strip * nchunks))
            lo = end
    return segs


def _deferred(total, nchunks, sms):
    grid = min(sms, total, 160)
    per_cta = (total + grid - 1) // grid
    return nchunks > per_cta and per_cta >= 16, grid


def _close16(a, b, what):
    a, b = a.float().cpu(), b.float().cpu()
    scale = max(b.abs().max().item(), 1e-30)
    torch.testing.assert_close(a / scale, b / scale, atol=1e-2, rtol=1e-2, msg=lambda m: what + ": " + m)


CASES = [
    # b, l, h, g, L, (|A| range), initial states, caller's states buffer
    dict(id="one_strip_slow", b=1, l=262144, h=2, g=1, L=64, a=(0.01, 0.05), init=False, states_buf=False),
    dict(id="one_strip_bench_decay", b=1, l=196608, h=2, g=1, L=64, a=(1.0, 16.0), init=True, states_buf=False),
    dict(id="hpc1_groups_ragged", b=1, l=64 * 512 + 37, h=6, g=2, L=64, a=(0.02, 0.2), init=True, states_buf=False),
    dict(id="two_batches_L256", b=2, l=256 * 1200 + 100, h=2, g=1, L=256, a=(0.002, 0.01), init=False, states_buf=True),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["id"])
def test_deferred_carry_against_oracle_and_plain_route(cuda_device, case):
    fused, cumsum = _fns()
    b, l, h, g, L = (case[k] for k in ("b", "l", "h", "g", "L"))
    hpc = 2 if (h // g) % 2 == 0 else 1
    nchunks = (l + L - 1) // L
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    on, _ = _deferred(b * (h // hpc) * nchunks, nchunks, sms)
    assert on, "this case is meant to take the deferred-carry branch"
    inp = _inputs(b, l, h, g, 41, *case["a"])
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    init = torch.randn(b, h, 64, 128, generator=torch.Generator().manual_seed(6)) if case["init"] else None
    init_d = None if init is None else init.to(cuda_device)
    dA, dt = cumsum(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    buf = torch.full((b, nchunks, h, 64, 128), float("nan"), device=cuda_device) if case["states_buf"] else None
    out, fin = fused(d["B"], d["x"], dt, dA, torch.bfloat16, initial_states=init_d, states=buf)
    out32, fin32 = fused(d["B"], d["x"], dt, dA, torch.float32, initial_states=init_d)
    torch.cuda.synchronize()
    from mamba_fused_minimal_b200._ext import C
    C.check_status(d["x"])

    # the oracle on the same dt / dA_cumsum, whole tensor
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.float32,
                                         initial_states=init, exp_impl="ex2")
    assert rel_err(fin.cpu(), ref_fin) <= 1e-3
    assert rel_err(fin32.cpu(), ref_fin) <= 1e-3
    assert rel_err(out32.cpu(), ref_out) <= 1e-3
    _close16(out, ref_out.to(torch.bfloat16), "passed states (bf16)")
    # first and last 64 chunks element by element.  The second pass reads the 16-bit zero-carry
    # value, adds the carried term in fp32 and rounds again: one rounding of the result (relative
    # to the element) plus one of the zero-carry value (relative to ITS size, which is bounded
    # by the tensor's scale, not by the element: the two terms may cancel).
    for sl in (slice(0, 64), slice(nchunks - 64, nchunks)):
        a = out[:, sl].float().cpu()
        r = ref_out[:, sl]
        assert ((a - r).abs() <= 2.0 ** -7 * r.abs() + 2.0 ** -8 * ref_out.abs().max()).all()
    if buf is not None:
        ref_states = O.chunk_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), exp_impl="ex2")
        assert rel_err(buf.cpu(), ref_states) <= 1e-3

    # the plain kernels (one scan per (batch, head), no segments) on the same inputs
    out_p, fin_p = fused(d["B"], d["x"], dt, dA, torch.float32, initial_states=init_d, force_general=True)
    assert rel_err(out32, out_p) <= 1e-4
    assert rel_err(fin32, fin_p) <= 1e-4
    assert rel_err(fin, fin_p) <= 1e-4


def test_second_pass_skip_rule(cuda_device):
    """Which chunks the second pass touches.  Per segment that starts inside a strip at chunk s,
    chunk j carries the factor f_j = exp(sum of the chunk decays s .. j-1).  16-bit passed
    states: where f_j <= 2^-24 the chunk must be bit-identical to a scan of the sub-sequence
    that starts at s from a zero state.  fp32 passed states have no such cut-off: chunks whose
    factor lies a little under 2^-24 still differ from that zero-carry scan (f_j * S_in exceeds
    the rounding step of the elements near zero)."""
    fused, cumsum = _fns()
    b, l, h, g, L = 1, 64 * 4096, 2, 1, 64
    nchunks = l // L
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    on, grid = _deferred(nchunks, nchunks, sms)
    assert on
    # decay per chunk around -1.3: the factor falls under 2^-24 (e^-16.6) some 13 chunks after a cut
    inp = _inputs(b, l, h, g, 43, 0.25, 0.35)
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    dA, dt = cumsum(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    out, fin = fused(d["B"], d["x"], dt, dA, torch.bfloat16)
    out32, fin32 = fused(d["B"], d["x"], dt, dA, torch.float32)
    torch.cuda.synchronize()
    decay = dA[0, :, :, -1].double().cpu()                       # (h, c)
    segs = _segments(nchunks, nchunks, grid)[0]
    assert len(segs) == grid and segs[1][0] > 0
    checked_skipped = checked_touched = checked_under = 0
    for s, e in segs[1:9] + segs[-3:]:
        # the zero-carry scan of this segment: the same kernel on the sub-sequence (short enough
        # not to be deferred itself)
        sl = slice(s * L, e * L)
        z16, _ = fused(d["B"][:, sl], d["x"][:, sl], dt[:, :, s:e], dA[:, :, s:e], torch.bfloat16)
        z32, _ = fused(d["B"][:, sl], d["x"][:, sl], dt[:, :, s:e], dA[:, :, s:e], torch.float32)
        for hh in range(h):
            f = torch.exp(torch.cumsum(decay[hh, s:e], 0) - decay[hh, s:e])      # f_j, j = s .. e-1
            for j in range(e - s):
                a16, b16 = out[0, s + j, hh], z16[0, j, hh]
                a32, b32 = out32[0, s + j, hh], z32[0, j, hh]
                if f[j].item() <= 2.0 ** -24 * 0.99:
                    assert torch.equal(a16, b16), (s, j, hh, f[j].item())
                    checked_skipped += 1
                    if f[j].item() > 2.0 ** -27:
                        assert not torch.equal(a32, b32), (s, j, hh, f[j].item())
                        checked_under += 1
                if f[j].item() > 1e-4:
                    # the carried state is O(1) here, so such a factor shows in both output types
                    assert not torch.equal(a32, b32), (s, j, hh, f[j].item())
                    assert not torch.equal(a16, b16), (s, j, hh, f[j].item())
                    checked_touched += 1
    assert checked_skipped > 50 and checked_touched > 50 and checked_under > 5
    # and the touched result is the right one
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.float32, exp_impl="ex2")
    assert rel_err(out32.cpu(), ref_out) <= 1e-3
    assert rel_err(fin.cpu(), ref_fin) <= 1e-3
    _close16(out, ref_out.to(torch.bfloat16), "passed states (bf16)")


def test_mamba2_130m_layer_shape_against_oracle(cuda_device):
    """batch 4 x 2048 x 24 heads x 64, one group, dstate 128, chunk 256, bf16: the whole problem
    against the oracle (cumsum at 1e-5; states on identical dt / dA_cumsum)."""
    fused, cumsum = _fns()
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_state_fwd
    b, l, h, g, L = 4, 2048, 24, 1, 256
    inp = O.make_inputs(b, l, h, 64, g, 128, dtype=torch.bfloat16, seed=0)
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    dA, dt = cumsum(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    ref_dA, ref_dt = O.chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
    assert rel_err(dA.cpu(), ref_dA) <= 1e-5 and rel_err(dt.cpu(), ref_dt) <= 1e-5
    out, fin = fused(d["B"], d["x"], dt, dA, torch.bfloat16)
    st = _chunk_state_fwd(d["B"], d["x"], dt, dA)
    ref_out, ref_fin = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.bfloat16, exp_impl="ex2")
    ref_st = O.chunk_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), exp_impl="ex2")
    _close16(out, ref_out, "passed states")
    assert rel_err(fin.cpu(), ref_fin) <= 1e-3
    assert rel_err(st.cpu(), ref_st) <= 1e-3
    assert math.isfinite(fin.abs().max().item())
