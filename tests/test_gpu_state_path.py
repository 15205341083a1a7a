"""`_state_path_fwd`: chunk cumsum + chunk state + state passing behind one call.

Its four outputs (dA_cumsum, dt_out, passed states, final states) must carry the same BITS as
`_chunk_cumsum_fwd` followed by the fused entry point (the pair of calls the reference's
pipelines make, main.py:96-100 there): where the tcgen05 kernel computes the cumulative sums
itself it uses the same operations in the same order as the stand-alone cumsum kernel.  The
cases cover the one-launch route (fp32 and 16-bit raw dt, one and two heads per CTA, ragged last
chunk, chunk sizes 64 / 128 / 256, dt limits, initial states, fp32 passed states, a caller's
states buffer, a strip long enough for the deferred carry) and the two-launch fallback (strided
dt, seq_idx, shapes the tcgen05 kernel does not take)."""
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("both_layouts")]


def _fns():
    from mamba_fused_minimal_b200.kernels._fused import _fused_chunk_state_state_passing_fwd as fused
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    from mamba_fused_minimal_b200.kernels.state_path import _state_path_fwd
    return _state_path_fwd, _chunk_cumsum_fwd, fused


CASES = [
    # b, l, h, p, g, n, L, x dtype, dt dtype, options
    dict(id="two_heads_fp32_dt", s=(2, 2048, 8, 64, 1, 128, 256), xd=torch.bfloat16, dd=torch.float32),
    dict(id="two_heads_bf16_dt_init", s=(2, 1024, 8, 64, 2, 128, 128), xd=torch.bfloat16, dd=torch.bfloat16, init=True),
    dict(id="one_head_fp32_dt_ragged", s=(1, 1000, 12, 64, 4, 128, 256), xd=torch.bfloat16, dd=torch.float32, init=True),
    dict(id="one_head_fp16_dt", s=(2, 700, 24, 64, 8, 128, 128), xd=torch.float16, dd=torch.float16),
    dict(id="fp16_L64_limits", s=(3, 64 * 5 + 9, 4, 64, 2, 128, 64), xd=torch.float16, dd=torch.float32,
         limit=(0.01, 0.2)),
    dict(id="fp32_out_states_buf", s=(2, 512, 4, 64, 1, 128, 128), xd=torch.bfloat16, dd=torch.float32,
         out32=True, states_buf=True),
    dict(id="no_softplus_no_bias", s=(1, 768, 4, 64, 1, 128, 256), xd=torch.bfloat16, dd=torch.float32,
         softplus=False, bias=False),
    dict(id="long_strip_deferred", s=(1, 64 * 4096, 2, 64, 1, 128, 64), xd=torch.bfloat16, dd=torch.float32, slow=True),
    dict(id="chained_over_many_ctas", s=(1, 8192, 2, 64, 1, 128, 64), xd=torch.bfloat16, dd=torch.float32),
    # two-launch fallbacks
    dict(id="fallback_one_head_bf16_dt", s=(1, 512, 3, 64, 3, 128, 128), xd=torch.bfloat16, dd=torch.bfloat16),
    dict(id="fallback_plain_kernels_fp32", s=(2, 320, 4, 32, 2, 16, 64), xd=torch.float32, dd=torch.float32, init=True),
    dict(id="fallback_strided_dt", s=(2, 512, 4, 64, 1, 128, 128), xd=torch.bfloat16, dd=torch.float32, strided_dt=True),
    dict(id="fallback_seq_idx", s=(2, 512, 4, 64, 1, 128, 128), xd=torch.bfloat16, dd=torch.float32, seq_idx=True),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c["id"])
def test_state_path_matches_the_two_calls_bit_for_bit(cuda_device, case):
    state_path, cumsum, fused = _fns()
    b, l, h, p, g, n, L = case["s"]
    inp = O.make_inputs(b, l, h, p, g, n, dtype=case["xd"], seed=51)
    if case.get("slow"):
        inp["A"] = inp["A"] * 0.01                       # carries that outlive a CTA's segment
    d = {k: v.to(cuda_device) for k, v in inp.items()}
    dt = d["dt"].to(case["dd"])
    if case.get("strided_dt"):
        big = torch.zeros(b, l, 2 * h, device=cuda_device, dtype=case["dd"])
        big[..., ::2] = dt
        dt = big[..., ::2]
    bias = d["dt_bias"] if case.get("bias", True) else None
    softplus = case.get("softplus", True)
    if not softplus:
        dt = dt.abs() * 0.1                              # without softplus dt must already be positive
    limit = case.get("limit", (0.0, float("inf")))
    init = torch.randn(b, h, p, n, device=cuda_device) if case.get("init") else None
    out_dtype = torch.float32 if case.get("out32") else case["xd"]
    seq_idx = None
    if case.get("seq_idx"):
        seq_idx = torch.zeros(b, l, dtype=torch.int32, device=cuda_device)
        seq_idx[:, 200:] = 1
    nchunks = (l + L - 1) // L
    mk = lambda: torch.full((b, nchunks, h, p, n), float("nan"), device=cuda_device) if case.get("states_buf") else None

    dA0, dt0 = cumsum(dt, d["A"], L, dt_bias=bias, dt_softplus=softplus, dt_limit=limit)
    buf0 = mk()
    out0, fin0 = fused(d["B"], d["x"], dt0, dA0, out_dtype, initial_states=init, seq_idx=seq_idx, states=buf0)
    buf1 = mk()
    dA1, dt1, out1, fin1 = state_path(dt, d["A"], d["B"], d["x"], L, out_dtype, dt_bias=bias, dt_softplus=softplus,
                                      dt_limit=limit, initial_states=init, seq_idx=seq_idx, states=buf1)
    torch.cuda.synchronize()
    from mamba_fused_minimal_b200._ext import C
    C.check_status(d["x"])
    assert dA1.shape == dA0.shape and dt1.shape == dt0.shape and out1.dtype == out0.dtype
    assert torch.equal(dt1, dt0), "dt_out differs"
    assert torch.equal(dA1, dA0), "dA_cumsum differs"
    assert torch.equal(out1, out0), "passed states differ"
    assert torch.equal(fin1, fin0), "final states differ"
    if buf0 is not None:
        assert torch.equal(buf1, buf0), "per-chunk states differ"
    # and the cumsum is the oracle's
    r_dA, r_dt = O.chunk_cumsum_fwd(dt.cpu(), inp["A"], L, dt_bias=None if bias is None else inp["dt_bias"],
                                    dt_softplus=softplus, dt_limit=limit)
    assert (dA1.cpu() - r_dA).abs().max().item() <= 1e-5 * max(r_dA.abs().max().item(), 1e-30)
    assert (dt1.cpu() - r_dt).abs().max().item() <= 1e-5 * max(r_dt.abs().max().item(), 1e-30)


def test_state_path_runs_twice_on_one_workspace(cuda_device):
    state_path, _, _ = _fns()
    b, l, h, p, g, n, L = 2, 2048, 8, 64, 1, 128, 256
    inp = {k: v.to(cuda_device) for k, v in O.make_inputs(b, l, h, p, g, n, dtype=torch.bfloat16, seed=52).items()}
    r1 = state_path(inp["dt"], inp["A"], inp["B"], inp["x"], L, torch.bfloat16, dt_bias=inp["dt_bias"], dt_softplus=True)
    r2 = state_path(inp["dt"], inp["A"], inp["B"], inp["x"], L, torch.bfloat16, dt_bias=inp["dt_bias"], dt_softplus=True)
    torch.cuda.synchronize()
    for a, c in zip(r1, r2):
        assert torch.equal(a, c)
