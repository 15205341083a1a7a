"""A bounded device-side wait that runs out.

The reference's fused kernels spin without a limit (kernels/fused_concurrent.py:82-84,205-208
there).  Here every wait has a limit, after which the CTA records a wait code, lets its copies
in flight land, frees its tensor memory and returns; the host reads the code with
ssd_check_status.  The tests make such a wait run out WITHOUT faulting or hanging anything:
the wait limit is shortened to about a millisecond and a test hook makes the fused kernel skip
the publication of its carry flags, so the CTAs that need a carried state wait for a flag that
nothing sets.  The kernel must return, the status must say SSD_ERR_TIMEOUT, and the next
normal call on the same scratch must be correct."""
import pytest
import torch

from conftest import rel_err
from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

SHORT_LIMIT = 2_000_000          # SM cycles, about one millisecond
# SSD_DEBUG_DROP_CARRY_FLAGS | SSD_DEBUG_CUT_STRIPS: a problem this small would otherwise run one CTA
# per head with no carries between CTAs at all
DROP_CARRY_FLAGS = 1 | 2


def _problem(device):
    """One strip cut over 64 CTAs: every CTA but the first needs the previous one's carry."""
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    b, l, h, p, g, n, L = 1, 4096, 2, 64, 1, 128, 64
    inp = O.make_inputs(b, l, h, p, g, n, dtype=torch.bfloat16, seed=3)
    d = {k: v.to(device) for k, v in inp.items()}
    dA, dt = _chunk_cumsum_fwd(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    ref = O.fused_state_fwd(inp["B"], inp["x"], dt.cpu(), dA.cpu(), torch.bfloat16, exp_impl="ex2")
    return d, dA, dt, ref


def _check_good(out, fin, ref):
    scale = ref[0].float().abs().max().item()
    torch.testing.assert_close(out.float().cpu() / scale, ref[0].float() / scale, atol=1e-2, rtol=1e-2)
    assert rel_err(fin.cpu(), ref[1]) <= 1e-3


def test_wait_limit_ends_in_timeout_status_and_the_workspace_recovers(cuda_device):
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    d, dA, dt, ref = _problem(cuda_device)
    out, fin = fused(d["B"], d["x"], dt, dA, torch.bfloat16)          # healthy call first
    C.check_status(d["x"])
    _check_good(out, fin, ref)
    try:
        C.debug_set_wait_limit_cycles(SHORT_LIMIT)
        C.debug_set_flags(DROP_CARRY_FLAGS)
        fused(d["B"], d["x"], dt, dA, torch.bfloat16)
        torch.cuda.synchronize()                                       # the kernel returned
    finally:
        C.debug_set_flags(0)
        C.debug_set_wait_limit_cycles(0)
    with pytest.raises(RuntimeError, match="wait gave up"):
        C.check_status(d["x"])
    # check_status cleared the header of the workspace that reported the timeout
    C.check_status(d["x"])
    out, fin = fused(d["B"], d["x"], dt, dA, torch.bfloat16)
    C.check_status(d["x"])
    _check_good(out, fin, ref)


def test_static_scratch_reports_a_timeout_too(cuda_device):
    from mamba_fused_minimal_b200._ext import C
    d, dA, dt, ref = _problem(cuda_device)
    out = torch.empty_like(ref[0], device=cuda_device)
    fin = torch.empty_like(ref[1], device=cuda_device)
    try:
        C.debug_set_wait_limit_cycles(SHORT_LIMIT)
        C.debug_set_flags(DROP_CARRY_FLAGS)
        C.fused_state_fwd_static(d["B"], d["x"], dt, dA, out, fin)
        torch.cuda.synchronize()
    finally:
        C.debug_set_flags(0)
        C.debug_set_wait_limit_cycles(0)
    with pytest.raises(RuntimeError, match="ssd_fused_state_fwd_static call gave up"):
        C.check_status(d["x"])
    # the next static call clears the header itself
    C.fused_state_fwd_static(d["B"], d["x"], dt, dA, out, fin)
    C.check_status(d["x"])
    _check_good(out, fin, ref)
