"""_bmm_chunk_fwd on the GPU against the oracle: the shapes the tcgen05 kernel takes (16-bit
inputs, chunk 128 / 256, inner dimension 64 / 128) and their neighbours that go to the plain kernel."""
import pytest
import torch

from oracle import ssd_oracle as O

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float().cpu() - b.float().cpu()).abs().max() / b.float().abs().max().clamp_min(1e-30)).item()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("L,k,groups,seqlen", [(256, 128, 1, 1024), (128, 64, 2, 640), (256, 64, 3, 700),
                                               (128, 128, 1, 130), (64, 128, 1, 256), (256, 96, 1, 512)])
def test_bmm_against_oracle(cuda_device, dtype, L, k, groups, seqlen):
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    gen = torch.Generator().manual_seed(L + k + seqlen)
    a = torch.randn(2, seqlen, groups, k, generator=gen).to(dtype)
    b = torch.randn(2, seqlen, groups, k, generator=gen).to(dtype)
    ref = O.bmm_chunk_fwd(a, b, L, output_dtype=torch.float32)
    out = _bmm_chunk_fwd(a.to(cuda_device), b.to(cuda_device), L, output_dtype=torch.float32)
    assert out.shape == ref.shape
    # products of 16-bit values are exact in fp32; only the order of the fp32 additions differs
    assert _rel(out, ref) <= 1e-5
    out16 = _bmm_chunk_fwd(a.to(cuda_device), b.to(cuda_device), L, output_dtype=dtype)
    scale = ref.abs().max()
    torch.testing.assert_close(out16.float().cpu() / scale, ref / scale, atol=1e-2, rtol=1e-2)


def test_bmm_strided_views_and_causal(cuda_device):
    """Operands that are column slices of one projection buffer (the way a model holds B and C),
    and causal=True, where only the lower triangle is specified."""
    from mamba_fused_minimal_b200.kernels.ssd_bmm import _bmm_chunk_fwd
    gen = torch.Generator().manual_seed(5)
    L, k = 256, 128
    buf = torch.randn(2, 768, 1, 2 * k + 64, generator=gen).to(torch.bfloat16)
    dbuf = buf.to(cuda_device)
    a, b = buf[..., :k], buf[..., k:2 * k]
    da, db = dbuf[..., :k], dbuf[..., k:2 * k]
    ref = O.bmm_chunk_fwd(a, b, L, output_dtype=torch.float32)
    out = _bmm_chunk_fwd(da, db, L, output_dtype=torch.float32)
    assert _rel(out, ref) <= 1e-5
    outc = _bmm_chunk_fwd(da, db, L, causal=True, output_dtype=torch.float32)
    tri = torch.tril(torch.ones(L, L, dtype=torch.bool))
    assert _rel(outc.cpu()[..., tri], ref[..., tri]) <= 1e-5
