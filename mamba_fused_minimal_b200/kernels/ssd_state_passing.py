"""`_state_passing_fwd` with the reference's signature (kernels/ssd_state_passing.py:87-115)."""
from .._ext import C as _C


def _state_passing_fwd(states, dA_chunk_cumsum, initial_states=None, seq_idx=None, chunk_size=None,
                       out_dtype=None):
    """states (batch, nchunks, nheads, dim), dA_chunk_cumsum (batch, nheads, nchunks) ->
    (out (batch, nchunks, nheads, dim) in out_dtype, final_states (batch, nheads, dim) fp32)."""
    batch, nchunks, nheads, dim = states.shape
    assert dA_chunk_cumsum.shape == (batch, nheads, nchunks)
    if initial_states is not None:
        assert initial_states.shape == (batch, nheads, dim)
    if seq_idx is not None:
        assert chunk_size is not None
        seqlen = seq_idx.shape[-1]
        assert seq_idx.shape == (batch, seqlen)
    return _C.state_passing_fwd(states, dA_chunk_cumsum, initial_states, seq_idx,
                                int(chunk_size) if chunk_size is not None else 0, out_dtype)
