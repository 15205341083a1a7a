"""Shared body of the two fused entry points."""
from .._ext import C as _C


def _fused_chunk_state_state_passing_fwd(B, x, dt, dA_cumsum, out_dtype, initial_states=None, seq_idx=None,
                                         states=None, states_in_fp32=True, clamp_decay=True,
                                         force_general=False, final_states=None):
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
    if initial_states is not None:
        assert initial_states.shape == (batch, nheads, headdim, dstate)
    return _C.fused_state_fwd(B, x, dt, dA_cumsum, out_dtype, initial_states, seq_idx, states,
                              bool(states_in_fp32), bool(clamp_decay), bool(force_general), final_states)
