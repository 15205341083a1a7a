"""`_bmm_chunk_fwd` with the reference's signature (kernels/ssd_bmm.py:89-134)."""
from .._ext import C as _C


def _bmm_chunk_fwd(a, b, chunk_size, seq_idx=None, causal=False, output_dtype=None):
    """a, b (batch, seqlen, k) or (batch, seqlen, ngroups, k) ->
    out (batch, nchunks, chunk_size, chunk_size) or (batch, nchunks, ngroups, chunk_size, chunk_size).
    With causal=True entries above the diagonal tiles are unspecified."""
    has_groups = a.dim() == 4
    if not has_groups:
        batch, seqlen, k = a.shape
    else:
        batch, seqlen, ngroups, k = a.shape
    assert b.shape == a.shape
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
    return _C.bmm_chunk_fwd(a, b, int(chunk_size), seq_idx, bool(causal), output_dtype)
