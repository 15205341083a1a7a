"""`_chunk_cumsum_fwd` and `_chunk_state_fwd` with the reference's signatures
(kernels/ssd_chunk_state.py:176-199 and :202-232 there)."""
import math

from .._ext import C as _C


def _chunk_cumsum_fwd(dt, A, chunk_size, dt_bias=None, dt_softplus=False, dt_limit=(0.0, float("inf"))):
    """dt (batch, seqlen, nheads), A (nheads,) -> (dA_cumsum, dt_out), both
    (batch, nheads, nchunks, chunk_size) fp32.  Note the order of the returned pair."""
    batch, seqlen, nheads = dt.shape
    assert A.shape == (nheads,)
    if dt_bias is not None:
        assert dt_bias.shape == (nheads,)
    assert math.ceil(seqlen / chunk_size) >= 1
    return _C.chunk_cumsum_fwd(dt, A, int(chunk_size), dt_bias, bool(dt_softplus),
                               float(dt_limit[0]), float(dt_limit[1]))


def _chunk_state_fwd(B, x, dt, dA_cumsum, seq_idx=None, states=None, states_in_fp32=True):
    """Per-chunk states (batch, nchunks, nheads, headdim, dstate); fills `states` in place
    when it is given."""
    batch, seqlen, nheads, headdim = x.shape
    _, _, nchunks, chunk_size = dt.shape
    _, _, ngroups, dstate = B.shape
    assert nheads % ngroups == 0
    assert B.shape == (batch, seqlen, ngroups, dstate)
    assert dt.shape == (batch, nheads, nchunks, chunk_size)
    assert dA_cumsum.shape == dt.shape
    if seq_idx is not None:
        assert seq_idx.shape == (batch, seqlen)
    if states is not None:
        assert states.shape == (batch, nchunks, nheads, headdim, dstate)
    return _C.chunk_state_fwd(B, x, dt, dA_cumsum, seq_idx, states, bool(states_in_fp32))
