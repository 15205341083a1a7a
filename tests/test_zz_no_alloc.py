"""The entry point that brings its own scratch memory: ssd_fused_state_fwd_static.

It exists for callers that cannot allocate device memory when they call the library (a
server whose device memory is handed out once at start-up, a plug-in invoked from another
runtime's callback) and therefore cannot give ssd_fused_state_fwd the workspace it asks
for.  Here it is called through the C ABI (the PyTorch front end only forwards pointers of
tensors this test allocated) and compared with ssd_fused_state_fwd on the same inputs: the
two run the same kernels, so the results must agree bit for bit, which is inside every
tolerance the other tests use.  Each case makes two calls in a row on one stream, because
all calls share one scratch array that keeps the previous call's contents.

This file is named so that pytest collects it last."""
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("both_layouts")]


def _run_pair(cuda_device, shape, dtype, init, force_general, seeds=(31, 32)):
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd as fused
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    b, l, h, p, g, n, L = shape
    for seed in seeds:                     # two calls in a row, different data each time
        inp = {k: v.to(cuda_device) for k, v in O.make_inputs(b, l, h, p, g, n, dtype=dtype, seed=seed).items()}
        dA, dt = _chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
        init_d = torch.randn(b, h, p, n, device=cuda_device) if init else None
        ref_out, ref_fin = fused(inp["B"], inp["x"], dt, dA, dtype, initial_states=init_d,
                                 force_general=force_general)
        nchunks = dt.shape[2]
        out = torch.full((b, nchunks, h, p, n), float("nan"), dtype=dtype, device=cuda_device)
        fin = torch.full((b, h, p, n), float("nan"), dtype=torch.float32, device=cuda_device)
        C.fused_state_fwd_static(inp["B"], inp["x"], dt, dA, out, fin, initial_states=init_d,
                                 force_general=force_general)
        torch.cuda.synchronize()
        # no bounded wait gave up, neither on the cached workspace nor on the static scratch
        # (its status word is read before the next static call clears the header)
        C.check_status(inp["x"])
        assert torch.equal(out, ref_out), f"seed {seed}: out differs"
        assert torch.equal(fin, ref_fin), f"seed {seed}: final_states differs"


def test_static_scratch_tcgen05_route(cuda_device):
    # several strips per CTA and strips cut between CTAs: carry slots and flags in use
    _run_pair(cuda_device, (2, 2048, 8, 64, 1, 128, 256), torch.bfloat16, init=True, force_general=False)
    # one strip spread over many CTAs: every CTA waits on the previous one's carry slot
    _run_pair(cuda_device, (1, 4096, 2, 64, 1, 128, 64), torch.bfloat16, init=False, force_general=False)


def test_static_scratch_plain_route(cuda_device):
    # fp32 inputs take the plain kernels, whose fp32 per-chunk states live in the scratch
    _run_pair(cuda_device, (2, 320, 4, 32, 2, 16, 64), torch.float32, init=True, force_general=False)
    _run_pair(cuda_device, (1, 512, 4, 64, 1, 128, 128), torch.bfloat16, init=False, force_general=True)


def test_static_scratch_rejects_what_does_not_fit(cuda_device):
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    assert C.static_scratch_bytes() == 16 << 20
    b, l, h, p, g, n, L = 2, 2048, 8, 64, 1, 128, 64          # plain route would need 16.8 MB of states
    inp = {k: v.to(cuda_device) for k, v in O.make_inputs(b, l, h, p, g, n, dtype=torch.bfloat16, seed=1).items()}
    dA, dt = _chunk_cumsum_fwd(inp["dt"], inp["A"], L, dt_bias=inp["dt_bias"], dt_softplus=True)
    out = torch.empty((b, dt.shape[2], h, p, n), dtype=torch.bfloat16, device=cuda_device)
    fin = torch.empty((b, h, p, n), dtype=torch.float32, device=cuda_device)
    with pytest.raises(RuntimeError, match="static scratch holds"):
        C.fused_state_fwd_static(inp["B"], inp["x"], dt, dA, out, fin, force_general=True)
    # the same problem on the tcgen05 route needs only the fixed-size header and carry slots
    C.fused_state_fwd_static(inp["B"], inp["x"], dt, dA, out, fin)
    torch.cuda.synchronize()
    assert torch.isfinite(fin).all()
