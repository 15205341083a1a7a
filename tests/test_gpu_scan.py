"""_chunk_scan_fwd on the GPU against the oracle: the shapes the tcgen05 kernels take (16-bit
inputs and passed states, fp32 cb, headdim 64, dstate 128, chunk 128 / 256; with and without D,
z and seq_idx) and the same data through the plain kernels."""
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu


def _case(device, dtype, b, l, h, g, L, seed, d_hdim=False, with_d=True):
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_state import _chunk_cumsum_fwd
    inp = O.make_inputs(b, l, h, 64, g, 128, dtype=dtype, seed=seed)
    d = {k: v.to(device) for k, v in inp.items()}
    dA, dt = _chunk_cumsum_fwd(d["dt"], d["A"], L, dt_bias=d["dt_bias"], dt_softplus=True)
    passed, _ = fused(d["B"], d["x"], dt, dA, dtype)
    cb = _bmm_chunk_fwd(d["C"], d["B"], L, output_dtype=torch.float32)
    D = None
    if with_d:
        D = torch.randn(h, 64) if d_hdim else inp["D"]
    return inp, d, dA, dt, passed, cb, D


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,l,h,g,L,d_hdim,with_d", [(2, 1024, 4, 1, 256, False, True), (1, 700, 6, 2, 256, True, True),
                                                      (2, 384, 2, 2, 128, False, False), (1, 130, 2, 1, 128, False, True)])
def test_chunk_scan_against_oracle(cuda_device, dtype, b, l, h, g, L, d_hdim, with_d):
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _chunk_scan_fwd
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, dtype, b, l, h, g, L, seed=l + h, d_hdim=d_hdim, with_d=with_d)
    out, _ = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], passed, D=None if D is None else D.to(cuda_device))
    ref, _ = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], passed.cpu(), D=D, exp_impl="ex2")
    scale = ref.float().abs().max()
    torch.testing.assert_close(out.float().cpu() / scale, ref.float() / scale, atol=1e-2, rtol=1e-2)
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_chunk_scan_with_gate(cuda_device, dtype):
    """z gating: out_x is the ungated result, out = out_x * z * sigmoid(z)."""
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _chunk_scan_fwd
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, dtype, 2, 700, 4, 2, 256, seed=11)
    z = torch.randn(2, 700, 4, 64, generator=torch.Generator().manual_seed(12)).to(dtype)
    out, out_x = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], passed, D=D.to(cuda_device), z=z.to(cuda_device))
    ref, ref_x = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], passed.cpu(), D=D, z=z, exp_impl="ex2")
    for got, want in ((out, ref), (out_x, ref_x)):
        scale = want.float().abs().max()
        torch.testing.assert_close(got.float().cpu() / scale, want.float() / scale, atol=1e-2, rtol=1e-2)


PLAIN_CHUNK_KERNELS = 4          # SSD_DEBUG_PLAIN_CHUNK_KERNELS


def test_chunk_scan_fast_and_plain_kernels_agree(cuda_device):
    """The same data through the tcgen05 kernel and, forced by the test hook, through the plain kernel."""
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _chunk_scan_fwd
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, torch.bfloat16, 2, 1024, 8, 1, 256, seed=3)
    D = D.to(cuda_device)
    out_f, _ = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], passed, D=D)
    try:
        C.debug_set_flags(PLAIN_CHUNK_KERNELS)
        out_p, _ = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], passed, D=D)
    finally:
        C.debug_set_flags(0)
    scale = out_p.float().abs().max()
    # identical rounding points; only the order of the fp32 additions differs
    assert ((out_f.float() - out_p.float()).abs().max() / scale).item() <= 1e-2
    assert (out_f == out_p).float().mean().item() > 0.99


def _packed_seq_idx(b, l, device, seed):
    """Sequence indices of packed sequences: boundaries inside chunks, on a chunk edge (position 256)
    and a one-position sequence."""
    gen = torch.Generator().manual_seed(seed)
    si = torch.zeros(b, l, dtype=torch.int32)
    for bi in range(b):
        cuts = sorted(set([256, 257] + torch.randint(1, l, (4,), generator=gen).tolist()))
        for ci, cut in enumerate(c for c in cuts if c < l):
            si[bi, cut:] = ci + 1
    return si.to(device)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,l,h,g,L", [(2, 1024, 4, 1, 256), (1, 700, 6, 2, 256), (2, 600, 2, 2, 128)])
def test_packed_sequences_on_the_tcgen05_kernels(cuda_device, dtype, b, l, h, g, L):
    """seq_idx through the tcgen05 chunk bmm, chunk scan and one-kernel chunk bmm + scan, against the
    oracle (kernels/ssd_bmm.py:79-83, kernels/ssd_chunk_scan.py:104-108 of the reference) and against
    the plain kernels on the same inputs."""
    from mamba_fused_minimal_b200._ext import C
    from mamba_fused_minimal_b200.kernels.fused_concurrent import _fused_chunk_state_state_passing_fwd_concurrent as fused
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd, _chunk_scan_fwd
    inp, d, dA, dt, _, _, D = _case(cuda_device, dtype, b, l, h, g, L, seed=l + 7 * h)
    si = _packed_seq_idx(b, l, cuda_device, seed=l)
    Dd = D.to(cuda_device)
    passed, _ = fused(d["B"], d["x"], dt, dA, dtype, seq_idx=si)

    def run():
        cb = _bmm_chunk_fwd(d["C"], d["B"], L, seq_idx=si, output_dtype=torch.float32)
        two, _ = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], passed, D=Dd, seq_idx=si)
        one, _ = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt, dA, passed, D=Dd, seq_idx=si)
        torch.cuda.synchronize()
        C.check_status(d["x"])
        return cb, two, one

    cb, two, one = run()
    try:
        C.debug_set_flags(PLAIN_CHUNK_KERNELS)
        cb_p, two_p, one_p = run()
    finally:
        C.debug_set_flags(0)
    ref_cb = O.bmm_chunk_fwd(inp["C"], inp["B"], L, seq_idx=si.cpu(), output_dtype=torch.float32)
    torch.testing.assert_close(cb.cpu(), ref_cb, atol=1e-3, rtol=1e-3)
    torch.testing.assert_close(cb_p.cpu(), ref_cb, atol=1e-3, rtol=1e-3)
    assert ((cb == 0) == (ref_cb.to(cuda_device) == 0)).all()      # exactly the masked pairs are zero
    ref, _ = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], passed.cpu(), D=D, seq_idx=si.cpu(),
                              exp_impl="ex2")
    scale = ref.float().abs().max()
    for got in (two, one, two_p, one_p):
        torch.testing.assert_close(got.float().cpu() / scale, ref.float() / scale, atol=1e-2, rtol=1e-2)
        assert torch.isfinite(got).all()
    assert torch.equal(one, two)                          # the one-kernel route: same bits as the two calls
    assert torch.equal(one_p, two_p)                      # (with the hook the call falls back to the two plain kernels)


# ---- chunk bmm + chunk scan in one kernel (`_bmm_chunk_scan_fwd`) --------------------------------

@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("b,l,h,g,L,d_hdim,with_d", [(2, 1024, 4, 1, 256, False, True), (1, 700, 6, 2, 256, True, True),
                                                      (2, 384, 2, 2, 128, False, False), (1, 130, 2, 1, 128, False, True)])
def test_bmm_chunk_scan_one_kernel_against_oracle_and_two_calls(cuda_device, dtype, b, l, h, g, L, d_hdim, with_d):
    """The kernel that computes C . B^T on chip against the oracle (atol = rtol = 1e-2 of the tensor's
    max) and against `_bmm_chunk_fwd` + `_chunk_scan_fwd`: same products, same operations in the same
    order, bit-identical results."""
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd, _chunk_scan_fwd
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, dtype, b, l, h, g, L, seed=l + h, d_hdim=d_hdim, with_d=with_d)
    Dd = None if D is None else D.to(cuda_device)
    out, _ = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt, dA, passed, D=Dd)
    two, _ = _chunk_scan_fwd(cb, d["x"], dt, dA, d["C"], passed, D=Dd)
    ref, _ = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], passed.cpu(), D=D, exp_impl="ex2")
    scale = ref.float().abs().max()
    torch.testing.assert_close(out.float().cpu() / scale, ref.float() / scale, atol=1e-2, rtol=1e-2)
    assert torch.isfinite(out).all()
    # same operations in the same order, explicit FMAs in both epilogues: the same bits
    assert torch.equal(out, two)
    from mamba_fused_minimal_b200._ext import C
    C.check_status(d["x"])


def test_bmm_chunk_scan_one_kernel_gate_and_fast_decay(cuda_device):
    """z gating through the one-kernel route, and decays so fast that the factors underflow
    (nothing may turn into NaN or infinity)."""
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd
    dtype = torch.bfloat16
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, dtype, 2, 700, 4, 2, 256, seed=11)
    z = torch.randn(2, 700, 4, 64, generator=torch.Generator().manual_seed(12)).to(dtype)
    out, out_x = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt, dA, passed, D=D.to(cuda_device), z=z.to(cuda_device))
    ref, ref_x = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA.cpu(), inp["C"], passed.cpu(), D=D, z=z, exp_impl="ex2")
    for got, want in ((out, ref), (out_x, ref_x)):
        scale = want.float().abs().max()
        torch.testing.assert_close(got.float().cpu() / scale, want.float() / scale, atol=1e-2, rtol=1e-2)
    # very fast decay: A = -200, dt up to 4 -> per-position exponents of several hundred
    dA_fast = dA * 40.0
    dt_big = dt * 10.0
    out_f, _ = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt_big, dA_fast, passed, D=D.to(cuda_device))
    ref_f, _ = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt_big.cpu(), dA_fast.cpu(), inp["C"], passed.cpu(), D=D, exp_impl="ex2")
    assert torch.isfinite(out_f).all()
    scale = ref_f.float().abs().max()
    torch.testing.assert_close(out_f.float().cpu() / scale, ref_f.float() / scale, atol=1e-2, rtol=1e-2)


def test_bmm_chunk_scan_one_kernel_increasing_cumsum(cuda_device):
    """Positive A makes the cumulative sums increase; the clamp exp(min(a_m - a_k, 0)) then matters."""
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd
    dtype = torch.bfloat16
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, dtype, 1, 512, 2, 1, 256, seed=5)
    dA_pos = -dA * 0.05
    out, _ = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt, dA_pos, passed, D=D.to(cuda_device))
    ref, _ = O.chunk_scan_fwd(cb.cpu(), inp["x"], dt.cpu(), dA_pos.cpu(), inp["C"], passed.cpu(), D=D, exp_impl="ex2")
    scale = ref.float().abs().max()
    torch.testing.assert_close(out.float().cpu() / scale, ref.float() / scale, atol=1e-2, rtol=1e-2)


def test_bmm_chunk_scan_falls_back_to_two_kernels(cuda_device):
    """Chunk size 64: no one-kernel route; the call makes the two separate calls itself."""
    from mamba_fused_minimal_b200.kernels.ssd_chunk_scan import _bmm_chunk_scan_fwd, _chunk_scan_fwd
    inp, d, dA, dt, passed, cb, D = _case(cuda_device, torch.bfloat16, 1, 512, 4, 1, 64, seed=9)
    si = torch.zeros(1, 512, dtype=torch.int32, device=cuda_device)
    si[:, 300:] = 1
    a, _ = _bmm_chunk_scan_fwd(d["C"], d["B"], d["x"], dt, dA, passed, D=D.to(cuda_device), seq_idx=si)
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    cb_si = _bmm_chunk_fwd(d["C"], d["B"], 64, seq_idx=si, output_dtype=torch.float32)
    b2, _ = _chunk_scan_fwd(cb_si, d["x"], dt, dA, d["C"], passed, D=D.to(cuda_device), seq_idx=si)
    assert torch.equal(a, b2)
