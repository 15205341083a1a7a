"""The layouts the fused state kernel chooses between give the same bits.

A problem with no more (batch, head) pairs than SMs runs one CTA per head over whole strips; a few
more, one head per CTA in one range per SM; no more head pairs than SMs, one CTA per head pair;
larger ones (the benchmark shape) head pairs cut into one range per SM with carries chained
between CTAs.  The test hook SSD_DEBUG_CUT_STRIPS forces the last layout on any problem, which is
also how small problems still exercise the carry chain.  Every layout does the same arithmetic
per head, so all outputs must be identical bit for bit (the reference has one layout only:
kernels/fused_concurrent.py:255-331)."""
import pytest
import torch

from conftest import rel_err
from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu

CUT_STRIPS = 2                   # SSD_DEBUG_CUT_STRIPS

CASES = [
    # batch, seqlen, heads, groups, chunk
    pytest.param((4, 2048, 24, 1, 256), id="one_cta_per_head_130m_layer_shape"),
    pytest.param((8, 1024, 20, 1, 256), id="one_head_per_cta_ranges"),
    pytest.param((2, 1100, 120, 2, 256), id="one_cta_per_head_pair_ragged"),
    pytest.param((2, 640, 6, 2, 128), id="three_heads_per_group"),
    pytest.param((1, 4096, 2, 1, 64), id="two_strips_of_64_chunks"),
]


@pytest.mark.parametrize("case", CASES)
def test_layouts_agree_bit_for_bit(cuda_device, case):
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd
    b, l, h, g, L = case
    inp = O.make_inputs(b, l, h, 64, g, 128, dtype=torch.bfloat16, seed=l + h)
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    init = torch.randn(b, h, 64, 128, generator=torch.Generator().manual_seed(1)).to(cuda_device)

    def run():
        dA, dt, out, fin = _state_path_fwd(d["dt"], d["A"], d["B"], d["x"], L, torch.bfloat16, dt_bias=d["dt_bias"],
                                           dt_softplus=True)
        out_i, fin_i = fused(d["B"], d["x"], dt, dA, torch.bfloat16, initial_states=init)
        out32, fin32 = fused(d["B"], d["x"], dt, dA, torch.float32)
        torch.cuda.synchronize()
        C.check_status(d["x"])
        return dA, dt, out, fin, out_i, fin_i, out32, fin32

    chosen = run()
    try:
        C.debug_set_flags(CUT_STRIPS)
        cut = run()
    finally:
        C.debug_set_flags(0)
    for i, (a, r) in enumerate(zip(chosen, cut)):
        assert torch.equal(a, r), f"output {i} differs between the chosen layout and ranges per SM"
    # and the chosen layout against the oracle (heads are independent: a slice is enough for the large case)
    hs = slice(0, min(h, 4))
    g_hs = slice(0, 1) if g < h else slice(0, g)
    ref_out, ref_fin = O.fused_state_fwd(inp["B"][:1, :, g_hs] if g == 1 else inp["B"][:1], inp["x"][:1, :, hs],
                                         chosen[1][:1, hs].cpu(), chosen[0][:1, hs].cpu(), torch.bfloat16,
                                         exp_impl="ex2") if g == 1 else (None, None)
    if ref_out is not None:
        scale = ref_out.float().abs().max().item()
        torch.testing.assert_close(chosen[2][:1, :, hs].float().cpu() / scale, ref_out.float() / scale, atol=1e-2, rtol=1e-2)
        assert rel_err(chosen[3][:1, hs].cpu(), ref_fin) <= 1e-3
